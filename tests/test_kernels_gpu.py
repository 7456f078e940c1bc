"""Parity of the CUDA skeletons with the CPU oracle on seeded inputs, through the C ABI.

Bars: bit-exact for integer, comparison, argmax and sort outputs;
within 1e-5 relative for f32 elementwise and reduce kernels; f32 GEMM within 1e-4 and f16
GEMM/matvec within 2e-3 per element after normalising by K.  Where a result can cancel to
nearly zero (sums, dot products) "relative" is taken against the sum of absolute terms.
"""
import numpy as np
import pytest

import oracle
from jax_js_b200 import AluExp, AluOp, AluVar, DType, Kernel, Reduction, np_dtype
from jax_js_b200 import programs as P
from jax_js_b200.backend import UnsupportedOpError

from util import assert_close, assert_same_bits, run_cuda

pytestmark = pytest.mark.gpu
F32, I32, U32, BOOL, F16, F64 = (DType.Float32, DType.Int32, DType.Uint32, DType.Bool, DType.Float16, DType.Float64)
g, r = AluVar.gidx, AluVar.ridx
SPECIAL = np.array([0.0, -0.0, 1.0, -1.0, np.inf, -np.inf, np.nan, 1e-40, -1e-40, 3.4e38, 88.8, -104.0, 0.5, 2.0,
                    1.9999999, 1e-3], np.float32)


def _inputs(n, seed, lo=-4.0, hi=4.0, special=True):
    rng = np.random.default_rng(seed)
    x = rng.uniform(lo, hi, n).astype(np.float32)
    if special:
        x[: len(SPECIAL)] = SPECIAL
    return x


N = 4099  # odd on purpose: exercises the scalar tail after the 128-bit body


@pytest.mark.parametrize("op,lo,hi,rtol,scale", [
    (AluOp.Exp, -100, 90, 1e-5, 0), (AluOp.Log, 0, 50, 1e-5, 1e-3), (AluOp.Sin, -30, 30, 1e-5, 1.0),
    (AluOp.Cos, -30, 30, 1e-5, 1.0), (AluOp.Asin, -1, 1, 1e-5, 1e-3), (AluOp.Atan, -50, 50, 1e-5, 1e-3),
    (AluOp.Erf, -4, 4, 1e-5, 1.0), (AluOp.Erfc, -4, 4, 1e-5, 1.0), (AluOp.Sqrt, 0, 100, 0, 0),
    (AluOp.Floor, -9, 9, 0, 0), (AluOp.Ceil, -9, 9, 0, 0), (AluOp.Reciprocal, -9, 9, 0, 0)])
def test_unary_float_ops_match_wasm_semantics(backend, op, lo, hi, rtol, scale):
    x = _inputs(N, int(op), lo, hi)
    if op in (AluOp.Sin, AluOp.Cos):
        x[x == np.float32(3.4e38)] = 1000.0   # beyond ~1e30 the reference's own reduction overflows to garbage
    k = Kernel(1, N, AluExp(op, F32, [AluExp.global_index(F32, 0, N, g)]))
    got, want = run_cuda(backend, k, [x]), oracle.run_kernel(k, [x])
    if rtol == 0:
        assert_same_bits(got, want, op.name)   # IEEE operations: identical on both sides
    else:
        assert_close(got, want, rtol, scale or None, op.name)


@pytest.mark.parametrize("op", [AluOp.Add, AluOp.Sub, AluOp.Mul, AluOp.Idiv, AluOp.Mod, AluOp.Min, AluOp.Max])
@pytest.mark.parametrize("dtype", [F32, I32, U32])
def test_binary_ops(backend, op, dtype):
    rng = np.random.default_rng(int(op) * 7 + int(dtype))
    if dtype == F32:
        a, b = _inputs(N, 1), np.roll(_inputs(N, 2), 3)
    else:
        a = rng.integers(-2**31, 2**31, N).astype(np.int64).astype(np_dtype(dtype))
        b = rng.integers(-50, 50, N).astype(np.int64).astype(np_dtype(dtype))
        a[:4] = np.array([2**31 - 1, -2**31, 0, -1]).astype(np_dtype(dtype))
        b[:4] = np.array([-1, -1, 0, 0]).astype(np_dtype(dtype))
    k = Kernel(2, N, AluExp(op, dtype, [AluExp.global_index(dtype, 0, N, g), AluExp.global_index(dtype, 1, N, g)]))
    got, want = run_cuda(backend, k, [a, b]), oracle.run_kernel(k, [a, b])
    if dtype == F32 and op == AluOp.Mod:
        # a - trunc(a/b)*b: the GPU may fuse the multiply-subtract; bounded by one rounding of |a|
        assert_close(got, want, 1e-6, np.abs(a), "f32 Mod")
    else:
        assert_same_bits(got, want, f"{op.name}<{dtype.name}>")


def test_compare_where_cast_bitcast_bool_logic(backend):
    a, b = _inputs(N, 5), np.roll(_inputs(N, 6), 1)
    x, y = AluExp.global_index(F32, 0, N, g), AluExp.global_index(F32, 1, N, g)
    lt, ne = AluExp.cmplt(x, y), AluExp.cmpne(x, y)
    cases = {
        "cmplt": lt, "cmpne": ne, "and": AluExp.mul(lt, ne), "or": AluExp.add(lt, ne.not_()),
        "where": AluExp.where(lt, x, y), "cast_i32": AluExp.cast(I32, AluExp.mul(x, AluExp.f32(1e9))),
        "cast_u32": AluExp.cast(U32, AluExp.mul(x, AluExp.f32(1e9))), "cast_bool": AluExp.cast(BOOL, x),
        "bool_to_f32": AluExp.cast(F32, lt), "bitcast": AluExp.bitcast(U32, x),
        "u32_to_f32": AluExp.cast(F32, AluExp.bitcast(U32, x)), "i32_to_f32": AluExp.cast(F32, AluExp.bitcast(I32, x)),
        "bit_invert": AluExp.bit_invert(AluExp.bitcast(I32, x)),
        "shr_int32_is_logical": AluExp.bit_shift(AluExp.bitcast(I32, x), AluExp.i32(35), "shr"),
    }
    for name, e in cases.items():
        k = Kernel(2, N, e)
        assert_same_bits(run_cuda(backend, k, [a, b]), oracle.run_kernel(k, [a, b]), name)


def test_threefry_bits_are_exact(backend):
    n = 10007
    key = np.array([0, 42], np.uint32)
    k0, k1 = AluExp.global_index(U32, 0, 2, AluExp.i32(0)), AluExp.global_index(U32, 0, 2, AluExp.i32(1))
    c = AluExp.cast(U32, g)
    for mode in ("xor", 0, 1):
        k = Kernel(1, n, AluExp.threefry2x32(k0, k1, AluExp.u32(0), c, mode))
        assert_same_bits(run_cuda(backend, k, [key]), oracle.run_kernel(k, [key]), f"threefry {mode}")
    k = Kernel(0, 1, AluExp.threefry2x32(AluExp.u32(0), AluExp.u32(0), AluExp.u32(0), AluExp.u32(0), 0))
    assert int(run_cuda(backend, k, [])[0]) == 1797259609   # src/alu.test.ts:202-209


def test_gather_kernels_are_exact(backend):
    """`jitRules[Gather]` (src/frontend/jit.ts:716-763): the data index is built from loaded int32
    indices.  Rows of a table (an embedding lookup), elements along an axis (takeAlongAxis), and
    indices outside the table, which read element 0 (src/backend/wasm/translation.ts:221-228)."""
    rng = np.random.default_rng(5)
    V, D, B = 1000, 96, 777
    table = rng.standard_normal((V, D)).astype(np.float32)
    idx = rng.integers(0, V, B).astype(np.int32)
    idx[:4] = [0, V - 1, V + 5, -3]                      # the last two are out of range
    row = AluExp.global_index(I32, 1, B, AluExp.idiv(g, AluExp.i32(D)))
    k = Kernel(2, B * D, AluExp.global_index(F32, 0, V * D, AluExp.add(AluExp.mul(row, AluExp.i32(D)), AluExp.mod(g, AluExp.i32(D)))))
    got, want = run_cuda(backend, k, [table, idx]), oracle.run_kernel(k, [table, idx])
    assert_same_bits(got, want, "row gather")
    assert np.array_equal(got.reshape(B, D)[4:], table[idx[4:]])
    assert (got.reshape(B, D)[2:4, 1:] == table[0, 0]).all()   # out of range: element 0 of the table
    R, C, T = 513, 300, 7
    x = rng.standard_normal((R, C)).astype(np.float32)
    along = rng.integers(0, C, (R, T)).astype(np.int32)
    i = AluExp.idiv(g, AluExp.i32(T))
    k = Kernel(2, R * T, AluExp.global_index(F32, 0, R * C, AluExp.add(AluExp.mul(i, AluExp.i32(C)), AluExp.global_index(I32, 1, R * T, g))))
    got = run_cuda(backend, k, [x, along])
    assert_same_bits(got, oracle.run_kernel(k, [x, along]), "take along axis")
    assert np.array_equal(got.reshape(R, T), np.take_along_axis(x, along, 1))
    # gathered rows under a reduction: sum_j table[idx[g], j]
    k = Kernel(2, B, AluExp.global_index(F32, 0, V * D, AluExp.add(AluExp.mul(AluExp.global_index(I32, 1, B, g), AluExp.i32(D)), r)),
               Reduction(F32, AluOp.Add, D))
    assert_close(run_cuda(backend, k, [table, idx]), oracle.run_kernel(k, [table, idx]), 1e-5, np.abs(table).sum(1).max(), "gathered row sums")


def test_random_bits_kernel_is_exact(backend):
    """`jitRules[RandomBits]` (src/frontend/jit.ts:698-714): keys broadcast over the trailing shape,
    counter = gidx mod the trailing size; 5 keys x 1001 draws, every mode."""
    keys = np.random.default_rng(6).integers(0, 2**32, (5, 2), dtype=np.uint64).astype(np.uint32)
    k0s, k1s = np.ascontiguousarray(keys[:, 0]), np.ascontiguousarray(keys[:, 1])
    n = 1001
    which = AluExp.idiv(g, AluExp.i32(n))
    c1 = AluExp.mod(AluExp.cast(U32, g), AluExp.u32(n))
    for mode in ("xor", 0, 1):
        k = Kernel(2, 5 * n, AluExp.threefry2x32(AluExp.global_index(U32, 0, 5, which), AluExp.global_index(U32, 1, 5, which),
                                                 AluExp.u32(0), c1, mode))
        assert_same_bits(run_cuda(backend, k, [k0s, k1s]), oracle.run_kernel(k, [k0s, k1s]), f"random bits {mode}")


def test_out_of_range_and_guarded_loads(backend):
    # a padded view: Where(valid, load, 0) with the load clamped to element 0 when invalid
    from jax_js_b200 import ShapeTracker, accessor_global
    n = 1000
    x = _inputs(n, 9, special=False)
    st = ShapeTracker.from_shape([n]).pad([(3, 5)])
    k = Kernel(1, n + 8, accessor_global(F32, 0, st, [g]))
    got = run_cuda(backend, k, [x])
    assert_same_bits(got, oracle.run_kernel(k, [x]))
    assert (got[:3] == 0).all() and (got[-5:] == 0).all() and (got[3:-5] == x).all()
    k = Kernel(1, 3, AluExp.global_index(F32, 0, 3, AluExp.add(g, AluExp.i32(2))))
    assert run_cuda(backend, k, [np.array([5, 6, 7], np.float32)]).tolist() == [7, 5, 5]


def test_float64_and_float16_elementwise(backend):
    rng = np.random.default_rng(3)
    d = rng.standard_normal(N)
    x = AluExp.global_index(F64, 0, N, g)
    k = Kernel(1, N, AluExp.add(AluExp.mul(x, x), AluExp.f64(0.25)))
    assert_close(run_cuda(backend, k, [d]), oracle.run_kernel(k, [d], mode=oracle.MODE_WASM), 1e-15, 1.0)
    h = (rng.standard_normal(N) * 3).astype(np.float16)
    hx = AluExp.global_index(F16, 0, N, g)
    k = Kernel(1, N, AluExp.exp(AluExp.mul(hx, AluExp.f16(0.5))))
    assert_close(run_cuda(backend, k, [h]), oracle.run_kernel(k, [h]), 2e-3, 1e-4, "f16 exp")


def test_unsupported_op_is_reported_not_emulated(backend):
    # UnsupportedOpError wording of src/backend.ts:228-234; nothing falls back to the host
    bad = Kernel(1, 4, AluExp(AluOp.Sub, BOOL, [AluExp.global_index(BOOL, 0, 4, g), AluExp.bool(False)]))
    with pytest.raises(UnsupportedOpError, match=r"Sub<bool> not supported in cuda backend"):
        backend.prepare_kernel(bad)


# ---- reductions ---------------------------------------------------------------------------

def _row_kernel(rows, cols, dtype, op, body=None, epilogue=None):
    x = AluExp.global_index(dtype, 0, rows * cols, AluExp.add(AluExp.mul(g, AluExp.i32(cols)), r))
    return Kernel(1, rows, body(x) if body else x, Reduction(dtype, op, cols, epilogue))


def _col_kernel(rows, cols, dtype, op):
    x = AluExp.global_index(dtype, 0, rows * cols, AluExp.add(g, AluExp.mul(r, AluExp.i32(cols))))
    return Kernel(1, cols, x, Reduction(dtype, op, rows))


@pytest.mark.parametrize("rows,cols", [(1, 7), (5, 33), (37, 130), (64, 1000), (19, 4096), (3, 70001), (1, 300000)])
@pytest.mark.parametrize("op", [AluOp.Add, AluOp.Max, AluOp.Min, AluOp.Mul])
def test_row_reductions_f32(backend, rows, cols, op):
    rng = np.random.default_rng(rows * 131 + cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    if op == AluOp.Mul:
        x = (1 + x * 1e-3).astype(np.float32)
    if op in (AluOp.Max, AluOp.Min) and cols > 8:
        x[0, 5] = np.nan   # NaN propagates through f32.max/min
    k = _row_kernel(rows, cols, F32, op)
    got, want = run_cuda(backend, k, [x]), oracle.run_kernel(k, [x])
    if op in (AluOp.Max, AluOp.Min):
        assert_same_bits(got, want, f"{op.name} {rows}x{cols}")
    else:
        scale = np.abs(x).sum(1) if op == AluOp.Add else None
        # a product of n factors carries ~sqrt(n) roundings whatever the order: the bar widens past 10^4 terms
        rtol = 1e-5 if op == AluOp.Add or cols <= 10000 else 1e-5 * (cols / 10000) ** 0.5 * 2
        assert_close(got, want, rtol, scale, f"{op.name} {rows}x{cols}")


@pytest.mark.parametrize("rows,cols", [(7, 1), (33, 5), (1000, 64), (4096, 19), (70001, 6), (65536, 2048)])
def test_column_reductions_f32(backend, rows, cols):
    rng = np.random.default_rng(rows + cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    k = _col_kernel(rows, cols, F32, AluOp.Add)
    assert_close(run_cuda(backend, k, [x]), oracle.run_kernel(k, [x]), 1e-5, np.abs(x).sum(0))


@pytest.mark.parametrize("dtype", [I32, U32, BOOL])
@pytest.mark.parametrize("op", [AluOp.Add, AluOp.Mul, AluOp.Min, AluOp.Max])
@pytest.mark.parametrize("shape", [(9, 513), (513, 9), (2, 40000)])
def test_integer_and_bool_reductions_are_exact(backend, dtype, op, shape):
    rows, cols = shape
    rng = np.random.default_rng(int(dtype) * 100 + int(op))
    if dtype == BOOL:
        x = (rng.random((rows, cols)) < (0.999 if op in (AluOp.Mul, AluOp.Min) else 0.001)).astype(np.int32)
    else:
        x = rng.integers(-2**31, 2**31, (rows, cols)).astype(np.int64).astype(np_dtype(dtype))
        if op == AluOp.Mul:
            x |= 1
    for k in (_row_kernel(rows, cols, dtype, op), _col_kernel(rows, cols, dtype, op)):
        assert_same_bits(run_cuda(backend, k, [x]), oracle.run_kernel(k, [x]), f"{op.name}<{dtype.name}> {shape}")


def test_forced_skeletons_agree(backend, monkeypatch):
    # the same kernel through both reduce skeletons (and odd sizes that defeat vector loads)
    from jax_js_b200.backend import CudaBackend
    rows, cols = 257, 1031
    x = np.random.default_rng(0).standard_normal((rows, cols)).astype(np.float32)
    k = _row_kernel(rows, cols, F32, AluOp.Add, epilogue=AluExp.mul(AluVar.acc(F32), AluExp.f32(0.5)))
    want = oracle.run_kernel(k, [x])
    for sk in ("1", "2"):
        monkeypatch.setenv("JAXCUDA_FORCE_SKELETON", sk)
        be = CudaBackend(backend.device)
        try:
            got, exe = run_cuda(be, k, [x], keep=True)
            assert ("reduce-row" if sk == "1" else "reduce-col") in exe.describe
            assert_close(got, want, 1e-5, 0.5 * np.abs(x).sum(1), f"skeleton {sk}")
        finally:
            be.close()


# ---- config 2: softmax, log-sum-exp, argmax over f32[8192, 4096] ------------------------

@pytest.mark.parametrize("rows,cols", [(64, 1000), (8192, 4096)])
def test_softmax_lse_argmax_kernels(backend, rows, cols):
    x = np.random.default_rng(0).standard_normal((rows, cols)).astype(np.float32)
    x[1, 7] = x[1, 3] = x[1].max() + 1      # a tie: argmax takes the first index
    iota = P.argmax_iota(cols)
    prog = P.softmax_lse_argmax_program(rows, cols)
    sx, si = backend.put(x), backend.put(iota)
    outs = prog.execute(backend, [sx, si])
    sm, lse, am = backend.get(outs[0], F32, (rows, cols)), backend.get(outs[1], F32), backend.get(outs[2], I32)
    for s in outs + [sx, si]:
        backend.dec_ref(s)
    # the oracle replays the same kernels in the same order
    m = oracle.run_kernel(P.row_reduce_kernel(rows, cols, AluOp.Max), [x])
    u = oracle.run_kernel(P.softmax_exp_kernel(rows, cols), [x, m])
    s = oracle.run_kernel(P.row_reduce_kernel(rows, cols, AluOp.Add), [u])
    want_sm = oracle.run_kernel(P.softmax_scale_kernel(rows, cols), [u, s]).reshape(rows, cols)
    s2 = oracle.run_kernel(P.lse_sum_kernel(rows, cols), [x, m])
    want_lse = oracle.run_kernel(P.lse_finish_kernel(rows), [s2, m])
    want_am = oracle.run_kernel(P.argmax_index_kernel(rows, cols), [x, m, iota])
    assert_close(sm, want_sm, 1e-5, None, "softmax")
    assert_close(lse, want_lse, 1e-5, None, "logsumexp")
    assert_same_bits(am, want_am, "argmax")
    assert am[1] == 3 and (am == x.argmax(1)).all()
    np.testing.assert_allclose(sm.sum(1), 1.0, rtol=1e-5)           # size-independent properties
    assert (sm[np.arange(rows), am] == sm.max(1)).all()


# ---- config 3a: f16 matvec ---------------------------------------------------------------------

@pytest.mark.parametrize("K,Nout,orientation", [(4096, 11008, "xW"), (4096, 11008, "Wx"), (300, 70, "xW"), (70, 300, "Wx")])
def test_matvec_f16(backend, K, Nout, orientation):
    rng = np.random.default_rng(0)
    if orientation == "xW":
        W, x = (rng.standard_normal((K, Nout)) * 0.02).astype(np.float16), (rng.standard_normal(K) * 0.02).astype(np.float16)
        k, args = P.matvec_kernel(K, Nout, F16, orientation="xW"), [x, W]
        scale = np.abs(x.astype(np.float64)) @ np.abs(W.astype(np.float64))
    else:
        W, x = (rng.standard_normal((Nout, K)) * 0.02).astype(np.float16), (rng.standard_normal(K) * 0.02).astype(np.float16)
        k, args = P.matvec_kernel(Nout, K, F16, orientation="Wx"), [W, x]
        scale = np.abs(W.astype(np.float64)) @ np.abs(x.astype(np.float64))
    got, want = run_cuda(backend, k, args), oracle.run_kernel(k, args)
    # 2e-3 relative per element after normalising by K; the f16 store itself rounds by 2^-11 of the value
    assert_close(got.astype(np.float64) / K, want.astype(np.float64) / K, 2e-3, scale / K, "matvec f16")


# ---- convolution and pooling: Dot / Reduce over pooled views (src/frontend/jit.ts:620-660) --------------

def _conv_kernel(N, Ci, H, W, Co, KH, KW, stride, pad, dt=F32):
    OH, OW = (H + 2 * pad - KH) // stride + 1, (W + 2 * pad - KW) // stride + 1
    return P.conv2d_kernel(N, Ci, H, W, Co, KH, KW, stride, pad, dt), (OH, OW)


@pytest.mark.parametrize("N,Ci,H,W,Co,KH,KW,stride,pad", [(2, 3, 17, 19, 5, 3, 3, 1, 1), (1, 8, 32, 32, 16, 5, 5, 2, 2), (3, 4, 9, 9, 6, 1, 1, 1, 0)])
def test_convolution_kernel_through_the_generic_skeletons(backend, N, Ci, H, W, Co, KH, KW, stride, pad):
    rng = np.random.default_rng(3)
    x, w = rng.standard_normal((N, Ci, H, W)).astype(np.float32), rng.standard_normal((Co, Ci, KH, KW)).astype(np.float32)
    k, (OH, OW) = _conv_kernel(N, Ci, H, W, Co, KH, KW, stride, pad)
    got = run_cuda(backend, k, [x, w]).reshape(N, Co, OH, OW)
    want = oracle.run_kernel(k, [x, w], fma=True).reshape(N, Co, OH, OW)
    xp = np.pad(x.astype(np.float64), ((0, 0), (0, 0), (pad, pad), (pad, pad)))
    ref = np.zeros((N, Co, OH, OW))
    for kh in range(KH):
        for kw in range(KW):
            patch = xp[:, :, kh: kh + stride * OH: stride, kw: kw + stride * OW: stride]
            ref += np.einsum("nchw,oc->nohw", patch, w[:, :, kh, kw].astype(np.float64))
    K = Ci * KH * KW
    assert_close(got / K, want / K, 1e-4, np.abs(x).max() * np.abs(w).max(), "conv vs oracle")
    assert_close(got, ref, 1e-5, np.abs(ref).max(), "conv vs float64")


@pytest.mark.parametrize("N,Ci,H,W,Co,KH,KW,pad,dt,stride", [
    (32, 64, 56, 56, 128, 3, 3, 1, F32, 1), (8, 32, 30, 30, 96, 5, 5, 0, F32, 1), (16, 64, 28, 28, 128, 3, 3, 1, F16, 1),
    (8, 32, 30, 30, 96, 5, 5, 0, F16, 1),      # 676 pixels: not a multiple of the 8 a gather thread owns
    (8, 64, 56, 56, 128, 3, 3, 1, F32, 2),     # stride 2: neighbouring pixels read every other input column
    (6, 48, 31, 29, 80, 3, 3, 1, F32, 1)])     # 899 pixels: odd, runs cross image rows, K = 432 is no multiple of BK tail-free
def test_convolution_kernel_on_the_tensor_pipe(backend, N, Ci, H, W, Co, KH, KW, pad, dt, stride):
    """A convolution large enough to be worth it runs as a gather of the patch operand followed by the
    tcgen05 GEMM (3xTF32 for float32): same Kernel, same oracle, GEMM tolerances."""
    rng = np.random.default_rng(11)
    npdt = np.float32 if dt == F32 else np.float16
    x = (rng.standard_normal((N, Ci, H, W)) * (1.0 if dt == F32 else 0.25)).astype(npdt)
    w = (rng.standard_normal((Co, Ci, KH, KW)) * (1.0 if dt == F32 else 0.05)).astype(npdt)
    k, (OH, OW) = _conv_kernel(N, Ci, H, W, Co, KH, KW, stride, pad, dt)
    assert backend.prepare_kernel(k).describe.startswith("conv as gemm-tcgen05"), backend.prepare_kernel(k).describe
    got = run_cuda(backend, k, [x, w]).astype(np.float64).reshape(N, Co, OH, OW)
    K = Ci * KH * KW
    # the oracle on a sample of output ranges (whole images of a few channels, first and last batch)
    want = np.zeros(k.size, npdt)
    P = OH * OW
    ranges = [(0, 3 * P), ((N * Co - 2) * P, N * Co * P), ((Co + 5) * P + 17, (Co + 6) * P + 17)]
    for b, e in ranges:
        oracle.run_kernel(k, [x, w], begin=b, end=e, fma=True, out=want)
    sel = np.concatenate([np.arange(b, e) for b, e in ranges])
    tol = 1e-4 if dt == F32 else 2e-3
    assert_close(got.reshape(-1)[sel] / K, want.astype(np.float64)[sel] / K, tol, np.abs(x).max() * np.abs(w).max(), "conv vs oracle")
    # and all of it against float64
    xp = np.pad(x.astype(np.float64), ((0, 0), (0, 0), (pad, pad), (pad, pad)))
    ref = np.zeros((N, Co, OH, OW))
    for kh in range(KH):
        for kw in range(KW):
            ref += np.einsum("nchw,oc->nohw", xp[:, :, kh: kh + stride * OH: stride, kw: kw + stride * OW: stride],
                             w[:, :, kh, kw].astype(np.float64), optimize=True)
    assert_close(got, ref, 1e-5 if dt == F32 else 2e-3, np.abs(ref).max(), "conv vs float64")


def _random_conv_shapes(n, seed):
    rng = np.random.default_rng(seed)
    out = []
    while len(out) < n:
        N, Ci = int(rng.choice([2, 4, 6, 8, 12, 16])), int(rng.choice([8, 24, 32, 40, 64, 72, 96, 128]))
        H, W, Co = int(rng.integers(8, 40)), int(rng.integers(8, 40)), int(rng.choice([32, 64, 80, 128, 136, 200, 256]))
        KH, KW, stride, pad = int(rng.integers(1, 6)), int(rng.integers(1, 6)), int(rng.choice([1, 1, 2, 3])), int(rng.integers(0, 3))
        if H + 2 * pad >= KH and W + 2 * pad >= KW:
            out.append((N, Ci, H, W, Co, KH, KW, stride, pad, F32 if rng.random() < 0.6 else F16))
    return out


@pytest.mark.parametrize("N,Ci,H,W,Co,KH,KW,stride,pad,dt", _random_conv_shapes(24, 10))
def test_random_convolutions_against_float64(backend, N, Ci, H, W, Co, KH, KW, stride, pad, dt):
    """Random shapes, filters that are not square, strides 1..3 and paddings 0..2, on whichever skeleton
    the planner takes (generic reductions or the implicit GEMM), against the sum in float64."""
    rng = np.random.default_rng(1)
    npdt = np.float32 if dt == F32 else np.float16
    x = (rng.standard_normal((N, Ci, H, W)) * (1.0 if dt == F32 else 0.25)).astype(npdt)
    w = (rng.standard_normal((Co, Ci, KH, KW)) * (1.0 if dt == F32 else 0.05)).astype(npdt)
    k, (OH, OW) = _conv_kernel(N, Ci, H, W, Co, KH, KW, stride, pad, dt)
    got = run_cuda(backend, k, [x, w]).astype(np.float64).reshape(N, Co, OH, OW)
    xp = np.pad(x.astype(np.float64), ((0, 0), (0, 0), (pad, pad), (pad, pad)))
    ref = np.zeros((N, Co, OH, OW))
    for kh in range(KH):
        for kw in range(KW):
            ref += np.einsum("nchw,oc->nohw", xp[:, :, kh: kh + stride * (OH - 1) + 1: stride, kw: kw + stride * (OW - 1) + 1: stride],
                             w[:, :, kh, kw].astype(np.float64), optimize=True)
    assert_close(got, ref, 1e-5 if dt == F32 else 2e-3, np.abs(ref).max(), backend.prepare_kernel(k).describe)


def test_convolution_gather_routes_agree_and_repeat(backend):
    """The patch operand is gathered inside the GEMM kernel (the default) or by a stage of its own
    through global memory (JAXCUDA_CONV_IMPLICIT=0): the same values enter the same MMAs, so the
    results are the same bits; and forty launches in a row of the in-kernel gather (stages refilled by
    alternating warp groups) reproduce them."""
    import os
    from jax_js_b200.backend import CudaBackend
    rng = np.random.default_rng(3)
    x = rng.standard_normal((8, 64, 28, 28)).astype(np.float32)
    w = rng.standard_normal((128, 64, 3, 3)).astype(np.float32)
    k, _ = _conv_kernel(8, 64, 28, 28, 128, 3, 3, 1, 1, F32)
    exe = backend.prepare_kernel(k)
    assert exe.describe.endswith("patches gathered in the kernel"), exe.describe
    sx, sw, so = backend.put(x), backend.put(w), backend.malloc(k.bytes)
    backend.dispatch(exe, [sx, sw], [so])
    first = backend.read_sync(so).copy()
    for _ in range(40):
        backend.dispatch(exe, [sx, sw], [so])
    assert np.array_equal(backend.read_sync(so), first)
    for s_ in (sx, sw, so):
        backend.dec_ref(s_)
    old = os.environ.get("JAXCUDA_CONV_IMPLICIT")
    os.environ["JAXCUDA_CONV_IMPLICIT"] = "0"
    try:
        other = CudaBackend(backend.device)
    finally:
        if old is None:
            os.environ.pop("JAXCUDA_CONV_IMPLICIT")
        else:
            os.environ["JAXCUDA_CONV_IMPLICIT"] = old
    try:
        assert other.prepare_kernel(k).describe.endswith("patches gathered first")
        assert np.array_equal(run_cuda(other, k, [x, w]).view(np.uint8).reshape(-1), first.reshape(-1))
    finally:
        other.close()


def test_remainder_tiles_made_in_the_kernel_match_the_split_pass(backend):
    """3xTF32: the remainder tiles lo = x - tf32(x) come from a split pass through global memory or
    are derived inside the GEMM kernel from the loaded operands; the MMAs see the same values, so the
    results are the same bits (several waves of tiles, a K tail, a bias epilogue)."""
    import os
    from jax_js_b200.backend import CudaBackend
    rng = np.random.default_rng(21)
    m, n, kk = 1536, 1280, 1000
    a = rng.uniform(-1, 1, (m, kk)).astype(np.float32)
    b = rng.uniform(-1, 1, (kk, n)).astype(np.float32)
    k = P.dot_kernel(m, n, kk)
    got = {}
    for mode in ("0", "2"):
        old = os.environ.get("JAXCUDA_TC_LO_IN_KERNEL")
        os.environ["JAXCUDA_TC_LO_IN_KERNEL"] = mode
        try:
            other = CudaBackend(backend.device)
        finally:
            if old is None:
                os.environ.pop("JAXCUDA_TC_LO_IN_KERNEL")
            else:
                os.environ["JAXCUDA_TC_LO_IN_KERNEL"] = old
        try:
            assert ("lo-in-kernel" in other.prepare_kernel(k).describe) == (mode == "2")
            for _ in range(3):
                got[mode] = run_cuda(other, k, [a, b])
        finally:
            other.close()
    assert np.array_equal(got["0"].view(np.uint32), got["2"].view(np.uint32))
    want = a.astype(np.float64) @ b.astype(np.float64)
    assert_close(got["2"].reshape(m, n) / kk, want / kk, 1e-5, 1.0, "3xTF32 with in-kernel remainder tiles")


def _random_dot_shapes(n, seed):
    rng = np.random.default_rng(seed)
    dims = [8, 24, 77, 250, 1001, 130, 64, 96, 128, 136, 200, 256, 320, 384, 512, 520, 768, 1000, 1024, 1536, 2048, 3000, 4096]
    ks = [8, 20, 33, 100, 1001, 32, 40, 64, 72, 96, 128, 136, 256, 520, 1024, 2048, 4096, 8192]
    out = []
    while len(out) < n:
        M, N, K, batch = int(rng.choice(dims)), int(rng.choice(dims)), int(rng.choice(ks)), int(rng.choice([1, 1, 1, 2, 3, 8]))
        if batch * M * N * K <= 2 ** 32 and batch * (M * K + K * N + M * N) <= 2 ** 26:
            out.append((M, N, K, F32 if rng.random() < 0.55 else F16, str(rng.choice(["mk", "km"])), str(rng.choice(["kn", "nk"])), batch,
                        bool(rng.random() < 0.3), bool(rng.random() < 0.3), bool(rng.random() < 0.15)))
    return out


@pytest.mark.parametrize("M,N,K,dt,al,bl,batch,bias,relu,swap", _random_dot_shapes(40, 3))
def test_random_dots_against_float64(backend, M, N, K, dt, al, bl, batch, bias, relu, swap):
    """Random extents (tails in M, N and K, strides that rule TMA out), layouts, batches and epilogues, on
    whichever skeleton the planner takes for them, against the product in float64."""
    rng = np.random.default_rng(1)
    npdt = np.float32 if dt == F32 else np.float16
    a = (rng.standard_normal((batch, M, K)) * (1.0 if dt == F32 else 0.25)).astype(npdt)
    b = (rng.standard_normal((batch, K, N)) / np.sqrt(K)).astype(npdt)
    ins = [a if al == "mk" else np.ascontiguousarray(a.transpose(0, 2, 1)), b if bl == "kn" else np.ascontiguousarray(b.transpose(0, 2, 1))]
    bv = rng.standard_normal(N).astype(npdt)
    if bias:
        ins.append(bv)
    k = P.dot_kernel(M, N, K, dt, a_layout=al, b_layout=bl, batch=batch, bias=bias, relu=relu, swap=swap)
    got = run_cuda(backend, k, ins).astype(np.float64).reshape(batch, M, N)
    ref = np.matmul(a.astype(np.float64), b.astype(np.float64))
    scale = np.abs(ref).max()
    if bias:
        ref = ref + bv.astype(np.float64)
    if relu:
        ref = np.maximum(ref, 0)
    assert_close(got, ref, 2e-5 if dt == F32 else 3e-3, scale, backend.prepare_kernel(k).describe)


@pytest.mark.parametrize("m,n,kk,dt,layout", [
    (2304, 2304, 192, F16, "mk-kn"),     # 9 x 9 tiles of 256 x 256 on 74 pairs: two waves, the second ragged
    (2200, 2120, 200, F16, "mk-kn"),     # M, N and K tails: the odd CTA of the last pair row holds 24 valid rows
    (2304, 2304, 160, F16, "km-nk"),     # A read as [K, M], B as [N, K]
    (4864, 1100, 96, F32, "mk-kn"),      # 3xTF32 pairs on 256 x 256 tiles (two groups of epilogue warps), N tail
    (2048, 2048, 544, F32, "km-kn"),     # the weight-gradient shape: A read as [K, M], 64 pair tiles, three chunks of K
    (6912, 1024, 96, F32, "mk-kn"),      # 27 x 4 = 108 pair tiles on 74 pairs: the last 34 run as 68 half-width tiles
    (6912, 1024, 96, F32, "mk-nk")])     # the same with B read as [N, K]: a half tile uses the first half of its box of B
def test_gemm_on_cta_pairs_matches_single_ctas(backend, m, n, kk, dt, layout):
    """Two CTAs of a cluster on one 256-row tile (tcgen05 cta_group::2, each CTA loading half of B's
    columns): every output accumulates the same products in the same order as on single CTAs, so the
    bits agree; and both agree with float64 within the GEMM tolerance."""
    import os
    from jax_js_b200.backend import CudaBackend
    rng = np.random.default_rng(m + kk)
    npdt = np.float32 if dt == F32 else np.float16
    a = (rng.standard_normal((m, kk)) * 0.5).astype(npdt)
    b = (rng.standard_normal((kk, n)) * 0.5).astype(npdt)
    a_t, b_t = layout.split("-")
    k = P.dot_kernel(m, n, kk, dt, a_layout=a_t, b_layout=b_t)
    args = [a if a_t == "mk" else np.ascontiguousarray(a.T), b if b_t == "kn" else np.ascontiguousarray(b.T)]
    got = {}
    for mode in ("0", "2"):
        old = os.environ.get("JAXCUDA_TC_PAIR")
        os.environ["JAXCUDA_TC_PAIR"] = mode
        try:
            other = CudaBackend(backend.device)
        finally:
            if old is None:
                os.environ.pop("JAXCUDA_TC_PAIR")
            else:
                os.environ["JAXCUDA_TC_PAIR"] = old
        try:
            assert ("cta-pairs" in other.prepare_kernel(k).describe) == (mode == "2"), other.prepare_kernel(k).describe
            for _ in range(3):
                got[mode] = run_cuda(other, k, args)
        finally:
            other.close()
    assert np.array_equal(got["0"].view(np.uint8), got["2"].view(np.uint8))
    want = a.astype(np.float64) @ b.astype(np.float64)
    assert_close(got["2"].astype(np.float64).reshape(m, n) / kk, want / kk, 1e-5 if dt == F32 else 2e-3, 0.25, "GEMM on CTA pairs")


def test_max_pool_kernel(backend):
    """`jitRules[Pool]` then a Max reduction: 2 x 2 windows, stride 2, over [N, C, H, W]."""
    N, C, H, W = 3, 5, 16, 20
    x = np.random.default_rng(4).standard_normal((N, C, H, W)).astype(np.float32)
    i = AluExp.i32
    OH, OW = H // 2, W // 2
    ow, oh, nc = AluExp.mod(g, i(OW)), AluExp.mod(AluExp.idiv(g, i(OW)), i(OH)), AluExp.idiv(g, i(OW * OH))
    ih, iw = AluExp.add(AluExp.mul(oh, i(2)), AluExp.idiv(r, i(2))), AluExp.add(AluExp.mul(ow, i(2)), AluExp.mod(r, i(2)))
    ix = AluExp.add(AluExp.mul(AluExp.add(AluExp.mul(nc, i(H)), ih), i(W)), iw)
    k = Kernel(1, N * C * OH * OW, AluExp.global_index(F32, 0, x.size, ix), Reduction(F32, AluOp.Max, 4))
    got = run_cuda(backend, k, [x]).reshape(N, C, OH, OW)
    assert_same_bits(got.reshape(-1), oracle.run_kernel(k, [x]), "max pool")
    assert np.array_equal(got, x.reshape(N, C, OH, 2, OW, 2).max(axis=(3, 5)))


# ---- GEMM-shaped kernels -------------------------------------------------------------------------

def _gemm_case(backend, kernel, args, K, tol, dtype, rows=None):
    got = run_cuda(backend, kernel, args).astype(np.float64)
    if rows is None:
        want = oracle.run_kernel(kernel, args, fma=True).astype(np.float64)
        sel = slice(None)
    else:  # full-size case: the oracle evaluates a sample of output ranges
        want = np.zeros(kernel.size, np_dtype(kernel.dtype))
        for b, e in rows:
            oracle.run_kernel(kernel, args, begin=b, end=e, fma=True, out=want)
        sel = np.concatenate([np.arange(b, e) for b, e in rows])
        want = want.astype(np.float64)
    a, b = args[0].astype(np.float64), args[1].astype(np.float64)
    bound = np.abs(a).max() * np.abs(b).max()
    assert_close(got[sel] / K, want[sel] / K, tol, bound, "gemm")
    return got


@pytest.mark.parametrize("M,N,K,al,bl", [(1024, 1024, 1024, "mk", "kn"), (100, 130, 70, "mk", "kn"),
                                         (256, 192, 520, "km", "kn"), (192, 256, 136, "mk", "nk"), (130, 100, 64, "km", "nk"),
                                         (1024, 32, 784, "km", "nk"), (512, 48, 200, "mk", "kn")])   # 32-column tiles (a vmapped batch of 32)
def test_gemm_f32(backend, M, N, K, al, bl):
    rng = np.random.default_rng(0)
    A = rng.uniform(-1, 1, (M, K) if al == "mk" else (K, M)).astype(np.float32)
    B = rng.uniform(-1, 1, (K, N) if bl == "kn" else (N, K)).astype(np.float32)
    k = P.dot_kernel(M, N, K, F32, a_layout=al, b_layout=bl)
    got = _gemm_case(backend, k, [A, B], K, 1e-4, F32).reshape(M, N)
    Am = A if al == "mk" else A.T
    Bm = B if bl == "kn" else B.T
    ref = Am.astype(np.float64) @ Bm.astype(np.float64)
    # tighter than the bar: against float64, relative to the sum of absolute products
    assert_close(got, ref, 2e-6, np.abs(Am).astype(np.float64) @ np.abs(Bm).astype(np.float64), "gemm f32 vs f64")


def test_gemm_f32_bias_relu_batched_and_swapped(backend):
    rng = np.random.default_rng(1)
    M, N, K = 96, 160, 200
    A, B, bias = (rng.standard_normal(s).astype(np.float32) for s in ((M, K), (K, N), (N,)))
    for kw in (dict(bias=True, relu=True), dict(swap=True), dict(bias=True)):
        k = P.dot_kernel(M, N, K, F32, **kw)
        _gemm_case(backend, k, [A, B, bias][: k.nargs], K, 1e-4, F32)
    Ab, Bb = rng.standard_normal((5, 64, 40)).astype(np.float32), rng.standard_normal((5, 40, 48)).astype(np.float32)
    k = P.dot_kernel(64, 48, 40, F32, batch=5)
    got = _gemm_case(backend, k, [Ab, Bb], 40, 1e-4, F32).reshape(5, 64, 48)
    np.testing.assert_allclose(got, np.einsum("bmk,bkn->bmn", Ab, Bb), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("M,N,K,al,bl,kw", [
    (2048, 10, 8192, "km", "kn", {}),                      # weight gradient of a 10-class layer: dot-skinny-t
    (1000, 16, 777, "km", "kn", {}),                       # ragged K and M, widest N
    (512, 3, 4100, "km", "kn", dict(bias=True)),           # epilogue after the split fold
    (260, 8, 300, "km", "kn", dict(relu=True)),
    (8192, 2048, 10, "mk", "nk", dict(bias=True, relu=True)),   # K = 10: dot-small-k, both operands k-contiguous
    (300, 512, 7, "mk", "kn", dict(bias=True)),            # B read [K, N]
    (65, 1028, 16, "km", "nk", {}),                        # odd row count, last column block ragged
])
def test_skinny_and_small_k_dots(backend, M, N, K, al, bl, kw):
    rng = np.random.default_rng(7)
    A = rng.uniform(-1, 1, (M, K) if al == "mk" else (K, M)).astype(np.float32)
    B = rng.uniform(-1, 1, (K, N) if bl == "kn" else (N, K)).astype(np.float32)
    bias = rng.uniform(-1, 1, N).astype(np.float32)
    k = P.dot_kernel(M, N, K, F32, a_layout=al, b_layout=bl, **kw)
    exe = backend.prepare_kernel(k)
    assert exe.describe.startswith("dot-skinny-t" if N <= 16 else "dot-small-k"), exe.describe
    got = _gemm_case(backend, k, [A, B, bias][: k.nargs], K, 1e-4, F32).reshape(M, N)
    Am, Bm = (A if al == "mk" else A.T), (B if bl == "kn" else B.T)
    ref = Am.astype(np.float64) @ Bm.astype(np.float64)
    if kw.get("bias"):
        ref = ref + bias.astype(np.float64)
    if kw.get("relu"):
        ref = np.maximum(ref, 0)
    assert_close(got, ref, 2e-6, np.abs(Am).astype(np.float64) @ np.abs(Bm).astype(np.float64) + 1, "dot vs f64")
    # a second dispatch re-uses the persistent scratch (arrival counters re-armed by the first)
    assert np.array_equal(run_cuda(backend, k, [A, B, bias][: k.nargs]), got.reshape(-1).astype(np.float32))


def test_small_k_dot_with_a_gate_in_its_epilogue(backend):
    """dz[b, j] = (sum_k dz_next[b, k] W[j, k]) gated by a third array a[b, j] > 0: a K = 10 dot whose
    epilogue reads contiguously in gidx."""
    B, H, C = 515, 2048, 10
    rng = np.random.default_rng(8)
    dz, W = rng.standard_normal((B, C)).astype(np.float32), rng.standard_normal((H, C)).astype(np.float32)
    a = np.maximum(rng.standard_normal((B, H)), 0).astype(np.float32)
    k = P.dot_kernel(B, H, C, b_layout="nk")
    gate = AluExp.cmplt(AluExp.f32(0), AluExp.global_index(F32, 2, B * H, AluVar.gidx))
    k.reduction.epilogue = AluExp.where(gate, AluVar.acc(F32), AluExp.f32(0))
    k = Kernel(3, k.size, k.exp, k.reduction)
    assert backend.prepare_kernel(k).describe.startswith("dot-small-k")
    got = run_cuda(backend, k, [dz, W, a]).reshape(B, H)
    want = oracle.run_kernel(k, [dz, W, a], fma=True).reshape(B, H)
    assert np.array_equal(got == 0, want == 0)
    assert_close(got, want, 1e-5, np.abs(dz).astype(np.float64) @ np.abs(W.T).astype(np.float64), "gated dot")


@pytest.mark.parametrize("M,N,K,al,bl,skeleton", [(2048, 10, 4096, "km", "kn", "dot-skinny-t"), (4096, 512, 10, "mk", "nk", "dot-small-k"),
                                                   (8192, 10, 1024, "mk", "kn", "dot-skinny")])
def test_skinny_dots_f16(backend, M, N, K, al, bl, skeleton):
    # float16 operands, float32 accumulation, float16 result: `cpu`-backend semantics (2e-3 per element after / K)
    rng = np.random.default_rng(12)
    A = (rng.standard_normal((M, K) if al == "mk" else (K, M)) * 0.05).astype(np.float16)
    B = (rng.standard_normal((K, N) if bl == "kn" else (N, K)) * 0.05).astype(np.float16)
    k = P.dot_kernel(M, N, K, F16, a_layout=al, b_layout=bl)
    assert backend.prepare_kernel(k).describe.startswith(skeleton + " "), backend.prepare_kernel(k).describe
    got = _gemm_case(backend, k, [A, B], K, 2e-3, F16).reshape(M, N)
    Am, Bm = (A if al == "mk" else A.T), (B if bl == "kn" else B.T)
    ref = Am.astype(np.float64) @ Bm.astype(np.float64)
    assert_close(got, ref, 1e-3, np.abs(ref).max(), "f16 dot vs float64")


@pytest.mark.parametrize("n", [256, 4096])
def test_gemm_f16(backend, n):
    rng = np.random.default_rng(0)
    A = (rng.standard_normal((n, n)) * 0.02).astype(np.float16)
    B = (rng.standard_normal((n, n)) * 0.02).astype(np.float16)
    k = P.dot_kernel(n, n, n, F16)
    rows = None if n <= 256 else [(0, 2 * n), (n * n // 2 + 17, n * n // 2 + 17 + n), (n * n - 3 * n, n * n)]
    got = _gemm_case(backend, k, [A, B], n, 2e-3, F16, rows).reshape(n, n)
    # linearity (size independent): (2A)B == 2(AB) exactly in binary floating point, wherever the
    # float16 result is a normal number (doubling a subnormal changes its rounding)
    got2 = run_cuda(backend, k, [(A * np.float16(2)), B]).astype(np.float64).reshape(n, n)
    normal = np.abs(got) >= 2.0 ** -13
    np.testing.assert_array_equal(got2[normal], 2 * got[normal])


# ---- skeletons added for the Kernels `jit` emits around dots: transposing copies, unit reductions ----------

@pytest.mark.parametrize("shape,perm", [((2048, 784), (1, 0)), ((1000, 333), (1, 0)), ((64, 50, 130), (2, 1, 0)), ((7, 600, 520), (0, 2, 1))])
def test_materialised_transposes_use_the_tiled_skeleton_and_are_exact(backend, shape, perm):
    from jax_js_b200 import ShapeTracker, accessor_global, unravel_alu
    rng = np.random.default_rng(2)
    x = rng.standard_normal(shape).astype(np.float32)
    st = ShapeTracker.from_shape(shape).permute(perm)
    n = x.size
    k = Kernel(1, n, AluExp.mul(accessor_global(F32, 0, st, unravel_alu(st.shape, g)), AluExp.f32(2)))
    assert backend.prepare_kernel(k).describe.startswith("elementwise transposed"), backend.prepare_kernel(k).describe
    got = run_cuda(backend, k, [x])
    assert np.array_equal(got, (x.transpose(perm) * 2).reshape(-1))
    assert_same_bits(got, oracle.run_kernel(k, [x]), "transpose")


def test_reduction_over_one_element_runs_as_elementwise(backend):
    # an outer product written as a Dot with K = 1 (what vmap makes of a per-example weight gradient),
    # with an epilogue that reads a third array
    M, N = 300, 520
    rng = np.random.default_rng(6)
    a, b, c = rng.standard_normal(M).astype(np.float32), rng.standard_normal(N).astype(np.float32), rng.standard_normal(M * N).astype(np.float32)
    k = P.dot_kernel(M, N, 1)
    k.reduction.epilogue = AluExp.add(AluVar.acc(F32), AluExp.global_index(F32, 2, M * N, g))
    k = Kernel(3, k.size, k.exp, k.reduction)
    assert "unit reduction folded" in backend.prepare_kernel(k).describe
    got = run_cuda(backend, k, [a, b, c])
    # elementwise f32: 1e-5 (the product and the sum may be contracted into one fused multiply-add)
    scale = np.abs(np.outer(a, b)).reshape(-1) + np.abs(c)      # the sum may cancel: relative to its terms
    assert_close(got, oracle.run_kernel(k, [a, b, c]), 1e-5, scale, "K = 1 dot")
    assert_close(got, (np.outer(a.astype(np.float64), b) + c.reshape(M, N)).reshape(-1), 1e-6, scale, "vs float64")


def test_skinny_dot_with_few_rows_and_many_columns(backend):
    # C[10, 2048] = sum_b dz[b, 10] * a[b, 2048]: the weight gradient of the class layer as `transposeDot` writes it
    M, N, K = 10, 2048, 5000
    rng = np.random.default_rng(13)
    A, B = rng.standard_normal((K, M)).astype(np.float32), rng.standard_normal((K, N)).astype(np.float32)
    k = P.dot_kernel(M, N, K, a_layout="km", b_layout="kn")
    assert backend.prepare_kernel(k).describe.startswith("dot-skinny-t (operands swapped)"), backend.prepare_kernel(k).describe
    got = _gemm_case(backend, k, [A, B], K, 1e-4, F32).reshape(M, N)
    assert_close(got, A.T.astype(np.float64) @ B.astype(np.float64), 1e-5, np.abs(A).max() * np.abs(B).max() * np.sqrt(K), "vs float64")


@pytest.mark.parametrize("M,N,K,dt,al,bl", [(512, 512, 4096, F32, "mk", "kn"), (300, 200, 4100, F32, "mk", "nk"), (520, 1000, 6000, F32, "km", "kn"),
                                            (256, 256, 8192, F16, "mk", "kn"), (130, 700, 5000, F16, "mk", "nk")])
def test_gemm_with_few_tiles_and_a_long_k_is_split_along_k(backend, M, N, K, dt, al, bl):
    """Outputs with at most half as many tiles as SMs: the tiles' K ranges are sliced over otherwise idle
    CTAs, the slices' accumulators added up in k order by whichever CTA finishes a tile last."""
    rng = np.random.default_rng(M + N)
    npdt = np.float32 if dt == F32 else np.float16
    sc = 1.0 if dt == F32 else 0.05
    A = (rng.standard_normal((M, K) if al == "mk" else (K, M)) * sc).astype(npdt)
    B = (rng.standard_normal((K, N) if bl == "kn" else (N, K)) * sc).astype(npdt)
    k = P.dot_kernel(M, N, K, dt, a_layout=al, b_layout=bl, bias=True, relu=True)
    bias = (rng.standard_normal(N) * sc).astype(npdt)
    assert backend.prepare_kernel(k).describe.endswith("split-k"), backend.prepare_kernel(k).describe
    first = run_cuda(backend, k, [A, B, bias])
    got = _gemm_case(backend, k, [A, B, bias], K, 1e-4 if dt == F32 else 2e-3, dt)
    assert np.array_equal(first.astype(np.float64), got)          # slices are added in a fixed order: bit-reproducible
