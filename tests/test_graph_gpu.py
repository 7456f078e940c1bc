"""Captured step lists: a training step replayed as one CUDA graph gives the bits of the same step
dispatched kernel by kernel, and calls that cannot be recorded are refused inside a capture."""
import numpy as np
import pytest

from jax_js_b200 import AluExp, AluVar, DType, Kernel, mlp

pytestmark = pytest.mark.gpu


def test_captured_training_step_equals_eager_steps(backend):
    dims, B = [784, 256, 256, 10], 512
    rng = np.random.default_rng(0)
    x, y = rng.uniform(0, 1, (B, 784)).astype(np.float32), rng.integers(0, 10, B).astype(np.int32)
    sx, sy = backend.put(x), backend.put(y)
    eager, graphed = mlp.MlpTrainer(backend, dims, B, B), mlp.MlpTrainer(backend, dims, B, B)
    losses = [[], []]
    for step in range(6):
        if step == 2:
            graphed.capture(sx, sy)            # two eager steps first, then replay
        for i, tr in enumerate((eager, graphed)):
            s = tr.step(sx, sy)
            losses[i].append(backend.get(s, "float32")[0])
            backend.dec_ref(s)
    launches = backend.launch_count()
    s = graphed.step(sx, sy)
    backend.dec_ref(s)
    assert backend.launch_count() - launches >= 20      # a replay still counts its kernels (fewer than the Kernels: fused runs)
    assert np.array_equal(np.array(losses[0]).view(np.uint32), np.array(losses[1]).view(np.uint32)), losses
    eager_s = eager.step(sx, sy)
    backend.dec_ref(eager_s)
    for a, b in zip(eager.params, graphed.params):
        assert np.array_equal(backend.read_sync(a), backend.read_sync(b))
    eager.close()
    graphed.close()
    backend.dec_ref(sx)
    backend.dec_ref(sy)
    # memory that belonged to the graph is usable again afterwards
    z = backend.malloc(1 << 20)
    backend.dec_ref(z)


def test_calls_that_cannot_be_recorded_are_refused(backend):
    n = 4096
    k = Kernel(1, n, AluExp.add(AluExp.global_index(DType.Float32, 0, n, AluVar.gidx), AluExp.f32(1)))
    a, b = backend.put(np.zeros(n, np.float32)), backend.malloc(n * 4)
    exe = backend.prepare_kernel(k)
    backend.dispatch(exe, [a], [b])
    backend.capture_begin()
    with pytest.raises(ValueError, match="inside a capture"):
        backend.read_sync(b)
    with pytest.raises(ValueError, match="inside a capture"):
        backend.malloc(16, np.zeros(16, np.uint8))
    backend.dispatch(exe, [a], [b])
    backend.dispatch(exe, [b], [a])
    g = backend.capture_end()
    assert (backend.get(a, "float32") == 0).all()       # recording runs nothing
    for _ in range(3):
        backend.graph_launch(g)
    assert (backend.get(a, "float32") == 6).all()
    backend.graph_destroy(g)
    backend.dec_ref(a)
    backend.dec_ref(b)


def _softmax_parts(be, prog, slots):
    outs = prog.execute(be, slots)
    res = [be.get(outs[0], "float32"), be.get(outs[1], "float32"), be.get(outs[2], "int32")]
    for s in outs:
        be.dec_ref(s)
    return res


@pytest.mark.parametrize("rows,cols", [(8192, 4096), (37, 1000), (5, 16), (3, 16384)])
def test_captured_softmax_program_runs_as_one_row_kernel(backend, rows, cols):
    """Inside a capture the ten Kernels of softmax + logsumexp + argmax become one row-resident
    kernel; its results match the unfused oracle replay (f32 1e-5, argmax exact)."""
    import oracle
    from jax_js_b200 import AluOp
    from jax_js_b200 import programs as P
    rng = np.random.default_rng(rows)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    x[0, : min(cols, 7)] = x[0].max() + 1.0          # a tie for the row maximum: the first index wins
    if rows > 2:
        x[2, 3] = np.nan                             # NaN propagates through max, sum and the equality test
    iota = P.argmax_iota(cols)
    prog = P.softmax_lse_argmax_program(rows, cols)
    sx, si = backend.put(x), backend.put(iota)
    eager = _softmax_parts(backend, prog, [sx, si])
    graph, outs = prog.capture(backend, [sx, si])
    launches, nbytes, groups = backend.graph_cost(graph)
    assert (launches, groups) == (1, 1), (launches, groups)
    assert nbytes == 2 * rows * cols * 4 + 2 * rows * 4 + cols * 4        # x in, softmax out, lse and argmax, iota
    for _ in range(2):
        backend.graph_launch(graph)
    got = [backend.get(outs[0], "float32"), backend.get(outs[1], "float32"), backend.get(outs[2], "int32")]
    m = oracle.run_kernel(P.row_reduce_kernel(rows, cols, AluOp.Max), [x])
    u = oracle.run_kernel(P.softmax_exp_kernel(rows, cols), [x, m])
    s = oracle.run_kernel(P.row_reduce_kernel(rows, cols, AluOp.Add), [u])
    want = [oracle.run_kernel(P.softmax_scale_kernel(rows, cols), [u, s]),
            oracle.run_kernel(P.lse_finish_kernel(rows), [oracle.run_kernel(P.lse_sum_kernel(rows, cols), [x, m]), m]),
            oracle.run_kernel(P.argmax_index_kernel(rows, cols), [x, m, iota])]
    from util import assert_close
    for g, e, w, name in zip(got, eager, want, ("softmax", "lse", "argmax")):
        if name == "argmax":
            assert np.array_equal(g, w) and np.array_equal(e, w), name
        else:
            assert_close(g, w, 1e-5, 1e-30, name + " fused vs oracle")
            assert_close(g, e, 1e-5, 1e-30, name + " fused vs eager")
    backend.graph_destroy(graph)
    for s_ in list(outs) + [sx, si]:
        backend.dec_ref(s_)


def test_row_fusion_keeps_what_stays_alive_and_leaves_other_kernels_alone(backend):
    """Intermediates that outlive the capture are still written; a Kernel that is no row stage cuts
    the run; a second launch after the inputs changed recomputes everything."""
    from jax_js_b200 import AluOp
    from jax_js_b200 import programs as P
    rows, cols = 64, 512
    rng = np.random.default_rng(5)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    k_max, k_exp = P.row_reduce_kernel(rows, cols, AluOp.Max), P.softmax_exp_kernel(rows, cols)
    k_sum = P.row_reduce_kernel(rows, cols, AluOp.Add)
    k_tr = Kernel(1, rows * cols, AluExp.global_index(DType.Float32, 0, rows * cols,   # a transposing copy: not a row stage
                  AluExp.add(AluExp.idiv(AluVar.gidx, AluExp.i32(rows)), AluExp.mul(AluExp.mod(AluVar.gidx, AluExp.i32(rows)), AluExp.i32(cols)))))
    exes = [backend.prepare_kernel(k) for k in (k_max, k_exp, k_sum, k_tr)]
    sx = backend.put(x)
    m, u, s, t = backend.malloc(rows * 4), backend.malloc(x.nbytes), backend.malloc(rows * 4), backend.malloc(x.nbytes)

    def run():
        backend.dispatch(exes[0], [sx], [m])
        backend.dispatch(exes[1], [sx, m], [u])
        backend.dispatch(exes[3], [u], [t])
        backend.dispatch(exes[2], [u], [s])
    run()
    want = [backend.get(z, "float32").copy() for z in (m, u, s, t)]
    backend.capture_begin()
    run()
    g = backend.capture_end()
    launches, _, groups = backend.graph_cost(g)
    assert groups == 1 and launches == 3            # {max, exp} fused; transpose; sum
    for z, w in zip((m, u, s, t), want):
        backend.write(z, np.zeros(w.nbytes, np.uint8))
    backend.graph_launch(g)
    for z, w in zip((m, u, s, t), want):
        np.testing.assert_allclose(backend.get(z, "float32"), w, rtol=1e-6)
    x2 = (x * 0.5).astype(np.float32)
    backend.write(sx, x2)
    backend.graph_launch(g)
    np.testing.assert_array_equal(backend.get(m, "float32"), x2.max(1))
    backend.graph_destroy(g)
    for z in (sx, m, u, s, t):
        backend.dec_ref(z)


def test_runs_of_small_kernels_replay_as_one_launch(backend):
    """A chain of small Kernels (elementwise, a reduction, one that overwrites an array an earlier one
    read, one that rereads what the previous wrote) is recorded as one single-CTA kernel; the replay
    gives the bits of the Kernels one by one, again after the input changed."""
    from jax_js_b200 import AluOp, Reduction
    n, rows, cols = 1200, 120, 10
    F32 = DType.Float32
    g, r, i32 = AluVar.gidx, AluVar.ridx, AluExp.i32
    ld = lambda a, length, ix: AluExp.global_index(F32, a, length, ix)
    k_exp = Kernel(1, n, AluExp.exp(AluExp.mul(ld(0, n, g), AluExp.f32(0.5))))                       # y = exp(x / 2)
    k_rev = Kernel(1, n, ld(0, n, AluExp.add(AluExp.mul(g, i32(-1)), i32(n - 1))))                    # z = reverse(y): reads what another thread wrote
    k_sum = Kernel(1, rows, ld(0, n, AluExp.add(AluExp.mul(g, i32(cols)), r)), Reduction(F32, AluOp.Add, cols))   # s[row] = sum z[row, :]
    k_div = Kernel(2, n, AluExp.mul(ld(0, n, g), AluExp.reciprocal(ld(1, rows, AluExp.idiv(g, i32(cols))))))      # w = z / s[row]
    k_add = Kernel(2, n, AluExp.add(ld(0, n, g), ld(1, n, g)))                                         # y' = w + z, written over y
    exes = [backend.prepare_kernel(k) for k in (k_exp, k_rev, k_sum, k_div, k_add)]
    rng = np.random.default_rng(9)
    x = rng.standard_normal(n).astype(np.float32)
    sx = backend.put(x)
    y, z, s_, w = backend.malloc(n * 4), backend.malloc(n * 4), backend.malloc(rows * 4), backend.malloc(n * 4)

    def run():
        backend.dispatch(exes[0], [sx], [y])
        backend.dispatch(exes[1], [y], [z])
        backend.dispatch(exes[2], [z], [s_])
        backend.dispatch(exes[3], [z, s_], [w])
        backend.dispatch(exes[4], [w, z], [y])
    run()
    want = [backend.read_sync(b).copy() for b in (y, z, s_, w)]
    backend.capture_begin()
    run()
    graph = backend.capture_end()
    launches, _, groups = backend.graph_cost(graph)
    assert (launches, groups) == (1, 1), (launches, groups)
    for b, wv in zip((y, z, s_, w), want):
        backend.write(b, np.zeros(wv.nbytes, np.uint8))
    backend.graph_launch(graph)
    for b, wv, name in zip((y, z, s_, w), want, "yzsw"):
        assert np.array_equal(backend.read_sync(b), wv), name
    x2 = (x * 0.25 + 1).astype(np.float32)
    backend.write(sx, x2)
    backend.graph_launch(graph)
    zz = np.exp(x2.astype(np.float64) * 0.5)[::-1].reshape(rows, cols)
    np.testing.assert_allclose(backend.get(w, "float32").reshape(rows, cols), zz / zz.sum(1, keepdims=True), rtol=2e-6)
    backend.graph_destroy(graph)
    for b in (sx, y, z, s_, w):
        backend.dec_ref(b)
