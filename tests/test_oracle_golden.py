"""Pins the CPU oracle to the reference's own known-answer vectors.

Each case replays, through oracle/oracle.cpp, a vector that the reference's test-suite
asserts for every backend; the citation gives the file and lines the numbers come from.
"""
import math

import numpy as np
import pytest

import oracle
from jax_js_b200 import (AluExp, AluOp, AluVar, DType, Kernel, Reduction, ShapeTracker, accessor_global,
                         global_view, unravel_alu)

F32, I32, U32, BOOL = DType.Float32, DType.Int32, DType.Uint32, DType.Bool
g, r = AluVar.gidx, AluVar.ridx


def f32(*v):
    return np.array(v, dtype=np.float32)


def test_elementwise_with_flipped_view():
    # src/backend/backend.test.ts:37-85
    shape = ShapeTracker.from_shape([3])
    a1 = accessor_global(F32, 0, shape, [g])
    a2 = accessor_global(F32, 1, shape.flip([True]), [g])
    a, b = f32(1, 2, 3), f32(4, 5, 6)
    assert oracle.run_kernel(Kernel(2, 3, AluExp.mul(a1, a2)), [a, b]).tolist() == [6, 10, 12]
    assert oracle.run_kernel(Kernel(2, 3, AluExp.add(a1, a2)), [a, b]).tolist() == [7, 7, 7]


def test_array_from_index():
    # src/backend/backend.test.ts:190-203
    out = oracle.run_kernel(Kernel(0, 200, AluExp.cast(F32, g)), [])
    assert out.tolist() == list(range(200))


def test_reduction_and_fused_epilogue():
    # src/backend/backend.test.ts:248-286
    st = ShapeTracker.from_shape([3, 2])
    exp = global_view(F32, 0, st, [g, r])
    x = f32(1, 1, 2, 3, 5, 7)
    assert oracle.run_kernel(Kernel(1, 3, exp, Reduction(F32, AluOp.Add, 2)), [x]).tolist() == [2, 5, 12]
    red = Reduction(F32, AluOp.Add, 2, AluExp.add(AluVar.acc(F32), AluExp.f32(1)))
    assert oracle.run_kernel(Kernel(1, 3, exp, red), [x]).tolist() == [3, 6, 13]


def test_bitwise_vectors():
    # src/backend/backend.test.ts:288-373
    shape = ShapeTracker.from_shape([4])
    a = np.array([0xFF00FF00, 0x0F0F0F0F, 0xAAAAAAAA, 7], dtype=np.uint32)
    b = np.array([0x00FF00FF, 0xF0F0F0F0, 0x55555555, 3], dtype=np.uint32)
    x, y = accessor_global(U32, 0, shape, [g]), accessor_global(U32, 1, shape, [g])
    run = lambda e, args: oracle.run_kernel(Kernel(2, 4, e), args).tolist()
    assert run(AluExp.bit_combine(x, y, "and"), [a, b]) == [0, 0, 0, 3]
    assert run(AluExp.bit_combine(x, y, "or"), [a, b]) == [0xFFFFFFFF] * 3 + [7]
    assert run(AluExp.bit_combine(x, y, "xor"), [a, b]) == [0xFFFFFFFF] * 3 + [4]
    ones, amt = np.ones(4, np.uint32), np.array([0, 1, 8, 16], np.uint32)
    assert run(AluExp.bit_shift(x, y, "shl"), [ones, amt]) == [1, 2, 256, 65536]
    rdata = np.array([256, 65536, 0xFFFF0000, 8], np.uint32)
    assert run(AluExp.bit_shift(x, y, "shr"), [rdata, amt]) == [256, 32768, 0x00FFFF00, 0]


def _matmul_kernel(M, N, K, gid_b, swapped=False):
    stA = ShapeTracker.from_shape([M, K]).reshape([M, 1, K]).expand([M, N, K])
    stB = ShapeTracker.from_shape([K, N]).permute([1, 0]).reshape([1, N, K]).expand([M, N, K])
    idx = [*unravel_alu([M, N], g), r]
    la, lb = global_view(F32, 0, stA, idx), global_view(F32, gid_b, stB, idx)
    return Kernel(gid_b + 1, M * N, AluExp.mul(lb, la) if swapped else AluExp.mul(la, lb),
                  Reduction(F32, AluOp.Add, K))


def test_matmul_all_ones():
    # src/backend/backend.test.ts:375-409 (64x64, a^2) and :411-464 (16x48x24, both operand orders)
    n = 64
    ones = np.ones(n * n, np.float32)
    assert (oracle.run_kernel(_matmul_kernel(n, n, n, 0), [ones]) == n).all()
    M, N, K = 16, 48, 24
    a, b = np.ones(M * K, np.float32), np.ones(K * N, np.float32)
    assert (oracle.run_kernel(_matmul_kernel(M, N, K, 1), [a, b]) == K).all()
    assert (oracle.run_kernel(_matmul_kernel(M, N, K, 1, swapped=True), [a, b]) == K).all()


def test_strided_reduction_closed_form():
    # src/backend/backend.test.ts:466-507
    M, N, K = 32, 128, 5
    x = np.fromfunction(lambda m, k, n: m * 1000 + k * 10 + n, (M, K, N), dtype=np.float32).astype(np.float32)
    mm, nn = unravel_alu([M, N], g)
    exp = global_view(F32, 0, ShapeTracker.from_shape([M, K, N]), [mm, r, nn])
    out = oracle.run_kernel(Kernel(1, M * N, exp, Reduction(F32, AluOp.Add, K)), [x.reshape(-1)]).reshape(M, N)
    want = K * (np.arange(M)[:, None] * 1000 + np.arange(N)[None, :]) + 10 * K * (K - 1) / 2
    np.testing.assert_allclose(out, want, rtol=1e-6)


def test_threefry_known_answers():
    # src/alu.test.ts:202-209: threefry2x32(0,0,0,0); test/random.test.ts:21-25: bits(key(0)) = 4070199207,
    # which is x0 ^ x1 ... of the counter 0 under key (0, 0)
    x0, x1 = oracle.threefry2x32(0, 0, 0, 0)
    assert (x0, x1) == (1797259609, 2579123966)
    k = Kernel(0, 1, AluExp.threefry2x32(AluExp.u32(0), AluExp.u32(0), AluExp.u32(0), AluExp.u32(0), "xor"))
    assert int(oracle.run_kernel(k, [])[0]) == (1797259609 ^ 2579123966)
    for mode, want in ((0, x0), (1, x1)):
        k = Kernel(0, 1, AluExp.threefry2x32(AluExp.u32(0), AluExp.u32(0), AluExp.u32(0), AluExp.u32(0), mode))
        assert int(oracle.run_kernel(k, [])[0]) == want


def test_truncating_division_and_c_style_mod():
    # src/alu.test.ts:211-272: idiv truncates toward zero; mod takes the sign of the dividend
    a = np.array([7, -7, 7, -7, 0, 5], np.int32)
    b = np.array([2, 2, -2, -2, 3, 5], np.int32)
    x, y = AluExp.global_index(I32, 0, 6, g), AluExp.global_index(I32, 1, 6, g)
    assert oracle.run_kernel(Kernel(2, 6, AluExp.idiv(x, y)), [a, b]).tolist() == [3, -3, -3, 3, 0, 1]
    assert oracle.run_kernel(Kernel(2, 6, AluExp.mod(x, y)), [a, b]).tolist() == [1, -1, 1, -1, 0, 0]
    fa, fb = f32(7.5, -7.5, 7.5, -7.5), f32(2, 2, -2, -2)
    fx, fy = AluExp.global_index(F32, 0, 4, g), AluExp.global_index(F32, 1, 4, g)
    assert oracle.run_kernel(Kernel(2, 4, AluExp.idiv(fx, fy)), [fa, fb]).tolist() == [3, -3, -3, 3]
    assert oracle.run_kernel(Kernel(2, 4, AluExp.mod(fx, fy)), [fa, fb]).tolist() == [1.5, -1.5, 1.5, -1.5]


def test_casts_saturate_like_wasm():
    # src/backend/wasm/translation.ts:144-153 (trunc_sat) and src/alu.test.ts:145-200
    v = f32(3.7, -3.7, 3e10, -3e10, float("nan"), float("inf"))
    x = AluExp.global_index(F32, 0, 6, g)
    assert oracle.run_kernel(Kernel(1, 6, AluExp.cast(I32, x)), [v]).tolist() == [3, -3, 2**31 - 1, -2**31, 0, 2**31 - 1]
    assert oracle.run_kernel(Kernel(1, 6, AluExp.cast(U32, x)), [v]).tolist() == [3, 0, 2**32 - 1, 0, 0, 2**32 - 1]
    bits = oracle.run_kernel(Kernel(1, 6, AluExp.bitcast(U32, x)), [f32(1, -1, 0, 2, 0.5, -0.0)]).tolist()
    assert bits == [0x3F800000, 0xBF800000, 0, 0x40000000, 0x3F000000, 0x80000000]


def _rel(a, b):
    return abs(a - b) / max(abs(b), 1e-3)


def test_wasm_exp_log_tolerances():
    # src/backend/wasm/builtins.test.ts:20-65
    for x in [-5, -2, -1, -0.5, 0, 0.001, 0.01, 0.1, 0.2, 0.3, 0.4, 0.5, 0.6, 0.9, 0.99, 1, 2, 3, 5, 10]:
        assert _rel(oracle.wasm_unary(AluOp.Exp, x), math.exp(x)) < 2e-7
    assert oracle.wasm_unary(AluOp.Exp, math.inf) == math.inf
    assert oracle.wasm_unary(AluOp.Exp, -math.inf) == 0
    assert math.isnan(oracle.wasm_unary(AluOp.Exp, math.nan))
    for x in [0.01, 0.1, 0.5, 1, 1.5, 2, math.e, 5, 10, 100]:
        assert _rel(oracle.wasm_unary(AluOp.Log, x), math.log(x)) < 5e-7
    assert math.isnan(oracle.wasm_unary(AluOp.Log, -1))
    assert oracle.wasm_unary(AluOp.Log, 0) == -math.inf
    assert oracle.wasm_unary(AluOp.Log, math.inf) == math.inf
    assert math.isnan(oracle.wasm_unary(AluOp.Log, math.nan))


def test_wasm_trig_erf_tolerances():
    # src/backend/wasm/builtins.test.ts:67-200: sin/cos absolute error < 5e-7 on these points
    pts = [-2 * math.pi, -math.pi, -math.pi / 2, -math.pi / 4, 0, math.pi / 6, math.pi / 4, math.pi / 3,
           math.pi / 2, math.pi, 3 * math.pi / 2, 2 * math.pi, 5, 10, -5, -10]
    for x in pts:
        assert abs(oracle.wasm_unary(AluOp.Sin, x) - math.sin(x)) < 5e-7
        assert abs(oracle.wasm_unary(AluOp.Cos, x) - math.cos(x)) < 5e-7
    for bad in (math.inf, -math.inf, math.nan):
        assert math.isnan(oracle.wasm_unary(AluOp.Sin, bad)) and math.isnan(oracle.wasm_unary(AluOp.Cos, bad))
    for x in [-10, -2, -1, -0.5, 0, 0.5, 1, 2, 10]:
        assert abs(oracle.wasm_unary(AluOp.Atan, x) - math.atan(x)) < 1e-6
    for x in [-1, -0.5, 0, 0.3, 0.9, 1]:
        assert abs(oracle.wasm_unary(AluOp.Asin, x) - math.asin(x)) < 2e-6
    for x in [-3, -1, -0.3, 0, 0.3, 1, 3]:
        assert abs(oracle.wasm_unary(AluOp.Erf, x) - math.erf(x)) < 5e-7
        assert abs(oracle.wasm_unary(AluOp.Erfc, x) - math.erfc(x)) < 5e-7


def test_nan_propagating_min_max_and_signed_zero():
    # src/backend/wasm/translation.ts:72-74: f32.min / f32.max
    a, b = f32(1, float("nan"), -0.0, 0.0), f32(float("nan"), 2, 0.0, -0.0)
    x, y = AluExp.global_index(F32, 0, 4, g), AluExp.global_index(F32, 1, 4, g)
    mx = oracle.run_kernel(Kernel(2, 4, AluExp.max(x, y)), [a, b])
    mn = oracle.run_kernel(Kernel(2, 4, AluExp.min(x, y)), [a, b])
    assert np.isnan(mx[:2]).all() and np.isnan(mn[:2]).all()
    assert not np.signbit(mx[2:]).any() and np.signbit(mn[2:]).all()


def test_out_of_range_load_reads_element_zero():
    # src/backend/wasm/translation.ts:221-228
    x = AluExp.global_index(F32, 0, 3, AluExp.add(g, AluExp.i32(2)))
    assert oracle.run_kernel(Kernel(1, 3, x), [f32(5, 6, 7)]).tolist() == [7, 5, 5]


def test_sort_vectors():
    # test/numpy.test.ts:4632-4659 (NaN last), :4719-4730 (int, uint, bool), :4739-4746 (8192 elements)
    assert oracle.sort(f32(3, 1, 4, 1, 5, 9, 2, 6), F32).tolist() == [1, 1, 2, 3, 4, 5, 6, 9]
    assert oracle.sort(np.array([[3, 1, 2], [6, 4, 5]], np.float32), F32).tolist() == [[1, 2, 3], [4, 5, 6]]
    out = oracle.sort(f32(3, np.nan, 1, np.nan, 2), F32)
    assert out[:3].tolist() == [1, 2, 3] and np.isnan(out[3:]).all()
    assert oracle.sort(np.array([3, 1, 4, 1, 5], np.int32), I32).tolist() == [1, 1, 3, 4, 5]
    assert oracle.sort(np.array([3, 1, 4, 1, 5], np.uint32), U32).tolist() == [1, 1, 3, 4, 5]
    assert oracle.sort(np.array([1, 0, 1, 0, 1], np.int32), BOOL).tolist() == [0, 0, 1, 1, 1]
    x = np.linspace(0, 1, 8192, dtype=np.float32)
    np.testing.assert_array_equal(oracle.sort(x[::-1].copy(), F32), x)
    z = oracle.sort(f32(0.0, -0.0, 0.0, -0.0), F32)
    assert np.signbit(z).tolist() == [True, True, False, False]
    assert oracle.sort(np.zeros((3, 0), np.float32), F32).shape == (3, 0)


def test_argsort_vectors():
    # test/numpy.test.ts:4750-4767, stability vector :4769-4785, 8191 reversed :4794-4800
    assert oracle.argsort(f32(3, 1, 4, 2, 5), F32)[1].tolist() == [1, 3, 0, 2, 4]
    assert oracle.argsort(np.array([[3, 1, 2], [6, 4, 5]], np.float32), F32)[1].tolist() == [[1, 2, 0], [1, 2, 0]]
    x = f32(3, 1, 1, np.nan, np.inf, 2, np.nan, 1, 0, -0.0, np.inf)
    assert oracle.argsort(x, F32)[1].tolist() == [8, 9, 1, 2, 7, 5, 0, 4, 10, 3, 6]
    big = np.linspace(0, 1, 8191, dtype=np.float32)[::-1].copy()
    assert oracle.argsort(big, F32)[1].tolist() == list(range(8190, -1, -1))


def test_mlp_logsoftmax_known_answer():
    # test/platform-test/node.test.ts:29-58 pins a 2-layer MLP with logSoftmax end to end;
    # here the same composition (dot+bias+relu, dot+bias, max, sum-exp, x - max - log s) is checked
    # against float64 numpy on seeded inputs, through the same kernels the cuda tests use.
    from jax_js_b200 import programs as P
    rng = np.random.default_rng(0)
    x = rng.uniform(0, 1, (8, 16)).astype(np.float32)
    w1, b1 = rng.standard_normal((16, 32)).astype(np.float32) * 0.3, rng.standard_normal(32).astype(np.float32) * 0.1
    h = oracle.run_kernel(P.dot_kernel(8, 32, 16, bias=True, relu=True), [x, w1, b1]).reshape(8, 32)
    np.testing.assert_allclose(h, np.maximum(x.astype(np.float64) @ w1 + b1, 0), rtol=1e-5, atol=1e-6)
    m = oracle.run_kernel(P.row_reduce_kernel(8, 32, AluOp.Max), [h])
    s = oracle.run_kernel(P.lse_sum_kernel(8, 32), [h, m])
    lse = oracle.run_kernel(P.lse_finish_kernel(8), [s, m])
    want = np.log(np.exp(h.astype(np.float64)).sum(1))
    np.testing.assert_allclose(lse, want, rtol=1e-5)


def test_float16_uses_cpu_backend_semantics():
    # src/backend/cpu.ts:120-133: evaluate in doubles, round once on the float16 store;
    # f16 Add reductions accumulate in f32 / the epilogue casts back (src/alu.ts:1560-1568)
    from jax_js_b200 import programs as P
    rng = np.random.default_rng(1)
    x = (rng.standard_normal(64) * 0.02).astype(np.float16)
    w = (rng.standard_normal((64, 32)) * 0.02).astype(np.float16)
    y = oracle.run_kernel(P.matvec_kernel(64, 32, DType.Float16, orientation="xW"), [x, w])
    want = (x.astype(np.float64) @ w.astype(np.float64)).astype(np.float16)
    np.testing.assert_array_equal(y, want)
    for v in [0.0, -0.0, 1.0, 65504.0, 65520.0, 1e-8, 6e-8, 5.96e-8, 0.333251953125, float("inf")]:
        assert oracle.lib().oracle_double_to_half(v) == int(np.array(v, np.float64).astype(np.float16).view(np.uint16))


def _program(prog, arrays):
    """Replay a step list on the oracle backend and return its outputs as numpy arrays."""
    from oracle_backend import OracleBackend
    be = OracleBackend()
    outs = prog.execute(be, [be.put(a) for a in arrays])
    return [be.slots[s][0] for s in outs]


def test_softmax_logsumexp_argmax_program_known_answers():
    from jax_js_b200 import programs as P
    # test/nn.test.ts:107-117: softmax of [[1,2,3],[4,5,6]] over the last axis
    x = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    sm, lse, am = _program(P.softmax_lse_argmax_program(2, 3), [x, P.argmax_iota(3)])
    np.testing.assert_allclose(sm.view(np.float32).reshape(2, 3), [[0.09003057, 0.24472848, 0.66524094]] * 2, rtol=1e-5)
    assert am.view(np.int32).tolist() == [2, 2]
    # test/nn.test.ts:164-178: logsumexp([-10,-1,1,2]) = 2.3490167; of [[1,2,3,4],[5,6,7,8]] as one row of 8 = 8.45834
    _, lse, _ = _program(P.softmax_lse_argmax_program(1, 4), [f32(-10, -1, 1, 2).reshape(1, 4), P.argmax_iota(4)])
    assert abs(float(lse.view(np.float32)[0]) - 2.3490167) < 1e-5
    _, lse, _ = _program(P.softmax_lse_argmax_program(1, 8), [np.arange(1, 9, dtype=np.float32).reshape(1, 8), P.argmax_iota(8)])
    assert abs(float(lse.view(np.float32)[0]) - 8.45834) < 1e-4
    # test/argreduce.test.ts:15-44: first index on ties, negatives, all equal, row-wise
    for row, want in (([3, 5, 5, 2, 5, 1], 1), ([-10, -5, -20, -5, -15], 1), ([1, 1, 1, 1, 1], 0)):
        _, _, am = _program(P.softmax_lse_argmax_program(1, len(row)), [np.array([row], np.float32), P.argmax_iota(len(row))])
        assert am.view(np.int32).tolist() == [want]
    _, _, am = _program(P.softmax_lse_argmax_program(3, 3), [np.array([[1, 2, 3], [6, 5, 4], [7, 8, 9]], np.float32), P.argmax_iota(3)])
    assert am.view(np.int32).tolist() == [2, 0, 2]


def test_small_matmul_known_answers():
    from jax_js_b200 import programs as P
    # test/numpy.test.ts:1518-1550: 2 x 2 and 2 x 3 products, exact
    k = P.dot_kernel(2, 2, 2)
    assert oracle.run_kernel(k, [f32(1, 2, 3, 4), f32(5, 6, 7, 8)]).tolist() == [19, 22, 43, 50]
    k = P.dot_kernel(2, 2, 3)
    assert oracle.run_kernel(k, [f32(1, 2, 3, 4, 5, 6), f32(7, 8, 9, 10, 11, 12)]).tolist() == [58, 64, 139, 154]
    # batched 3 x 3 (:1552-1580) against numpy, and a fused bias + ReLU epilogue (:1582-1608)
    a = np.arange(1, 19, dtype=np.float32).reshape(2, 3, 3)
    got = oracle.run_kernel(P.dot_kernel(3, 3, 3, batch=2), [a, a]).reshape(2, 3, 3)
    assert np.array_equal(got, np.einsum("bij,bjk->bik", a, a))
    x, w, b = f32(1, -2, 3, -4).reshape(2, 2), f32(1, 2, 3, 4).reshape(2, 2), f32(-20, 1)
    got = oracle.run_kernel(P.dot_kernel(2, 2, 2, bias=True, relu=True), [x, w, b]).reshape(2, 2)
    assert np.array_equal(got, np.maximum(x @ w + b, 0))


def test_adam_first_steps_known_answers():
    """optax.adam (packages/optax/src/transform.ts:29-69): with g constant the bias-corrected update is
    -lr * g / (|g| + eps) at every step, so p_t = p_0 - t * lr * sign(g) to within eps/|g|."""
    from jax_js_b200 import mlp
    from oracle_backend import OracleBackend
    be = OracleBackend()
    prog = mlp.adam_program([4], ["w"], lr=1e-3)
    p, grad = f32(1, -2, 0.5, 3), f32(0.1, -0.2, 4.0, -1e-3)
    state = [be.put(np.zeros(1, np.uint32)), be.put(p), be.put(grad), be.put(np.zeros(4, np.float32)), be.put(np.zeros(4, np.float32))]
    for t in range(1, 4):
        cnt, pn, mu, nu = prog.execute(be, state)
        assert be.get(cnt, "uint32")[0] == t
        np.testing.assert_allclose(be.get(pn, "float32"), p - t * 1e-3 * np.sign(grad), rtol=0, atol=5e-7 * t)   # a few float32 ulps of p per step
        np.testing.assert_allclose(be.get(mu, "float32"), (1 - 0.9 ** t) * grad, rtol=2e-6)
        np.testing.assert_allclose(be.get(nu, "float32"), (1 - 0.999 ** t) * grad * grad, rtol=2e-6)
        state = [cnt, pn, state[2], mu, nu]
