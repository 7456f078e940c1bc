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
    assert backend.launch_count() - launches >= 40      # a replay still counts its kernels
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
