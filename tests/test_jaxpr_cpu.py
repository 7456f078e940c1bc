"""The Jaxpr cutter (`jax_js_b200/jaxpr.py`) against what the reference's frontend is known to produce:
its own Jaxpr snapshot for the transposition of a Dot, the Kernel forms of the softmax / logsumexp /
argmax program, the materialisation decisions of `splitGraphDataflow`, and the ReLU cotangent at a
pre-activation of exactly zero."""
import numpy as np

from jax_js_b200 import AluOp, DType, mlp
from jax_js_b200 import programs as P
from jax_js_b200.jaxpr import Builder, Lit, jit_compile, split_graph_dataflow, vmap_jaxpr

from oracle_backend import OracleBackend

F32 = DType.Float32


def test_transposed_dots_have_the_shape_of_the_reference_snapshot():
    """test/tracing.test.ts:79-121 ("grad of dot transposes to dots"): grad of sum(dot(x[2,3], w[3,4]))
    with respect to both.  The snapshot's equations after `c = transpose b; d = reshape a; e = reshape c;
    f = broadcast 1`, per operand: broadcast, transpose, transpose, dot, reshape, reshape (, transpose)."""
    b = Builder()
    x, w = b.input("a", (2, 3)), b.input("b", (3, 4))
    _, xr, wr = mlp.np_dot(b, x, w)
    f = b.broadcast(Lit(1.0), (2, 4), [0, 1])
    n0 = len(b.eqns)
    dx = b.reshape(mlp.transpose_dot(b, f, wr, xr.shape), (2, 3))
    dw = b.transpose(b.reshape(mlp.transpose_dot(b, f, xr, wr.shape), (4, 3)), (1, 0))
    got = [(e.prim, tuple(e.out.shape)) for e in b.eqns[n0:]]
    # reshapes that change nothing are dropped by `simplify`, as in the snapshot
    got = [(p, s) for (p, s), e in zip(got, b.eqns[n0:]) if not (p == "reshape" and tuple(e.inputs[0].shape) == s)]
    want = [("broadcast", (2, 4, 3)), ("transpose", (2, 3, 4)), ("transpose", (1, 3, 4)), ("dot", (2, 3)),
            ("reshape", (2, 1, 3)), ("reshape", (2, 3)),
            ("broadcast", (2, 4, 3)), ("transpose", (4, 3, 2)), ("transpose", (1, 3, 2)), ("dot", (4, 3)),
            ("reshape", (1, 4, 3)), ("reshape", (4, 3)), ("transpose", (3, 4))]
    assert got == want
    assert dx.shape == (2, 3) and dw.shape == (3, 4)


def test_softmax_program_is_cut_into_the_known_kernels():
    """The Kernels the cutter derives equal the forms written out by hand from the same rules
    (`programs.py`), plus the copy of the stop-gradient row max that logsumexp uses twice."""
    rows, cols = 64, 256
    prog = jit_compile(P.softmax_lse_argmax_jaxpr(rows, cols))
    got = {s.name: s.kernel.serialize() for s in prog.steps if s.kind == "execute"}
    k1 = P.row_reduce_kernel(rows, cols, AluOp.Max).serialize()
    assert got["m1"] == got["m2"] == got["m3"] == k1
    assert got["u"] == P.softmax_exp_kernel(rows, cols).serialize()
    assert got["s"] == P.row_reduce_kernel(rows, cols, AluOp.Add).serialize()
    assert got["softmax"] == P.softmax_scale_kernel(rows, cols).serialize()
    assert got["s2"] == P.lse_sum_kernel(rows, cols).serialize()
    assert got["argmax"] == P.argmax_index_kernel(rows, cols).serialize()
    assert [s.name for s in prog.steps if s.kind == "execute"] == ["m1", "u", "s", "softmax", "m2", "m2k", "s2", "lse", "m3", "argmax"]
    # every intermediate is freed right after its last reader
    order = [(s.kind, s.name) for s in prog.steps]
    assert order.index(("free", "m1")) == order.index(("execute", "u")) + 1
    assert ("free", "softmax") not in order and ("free", "x") not in order


def test_what_the_gradient_program_materialises():
    jaxpr = mlp.mlp_grad_jaxpr(32, [12, 16, 8, 5], -1 / 32).simplify()
    black = split_graph_dataflow(jaxpr)
    names = {e.out.name for e in jaxpr.eqns if id(e.out) in black}
    # pre-activations (two consumers: max and less), activations (inputs of the next Dot), the
    # stop-gradient copy of x, per-layer cotangents, and both forms of every weight gradient
    for n in ["x_sg", "z1", "a1", "z2", "a2", "z3", "m", "shifted", "e", "s", "onehot", "loss",
              "dz3", "dz2", "dz1", "db1", "db2", "db3", "dW1_nk", "dW1", "dW2_nk", "dW2", "dW3_nk", "dW3"]:
        assert n in names, n
    prog = jit_compile(jaxpr)
    by_name = {s.name: s.kernel for s in prog.steps if s.kind == "execute"}
    # no Where in a reduction epilogue, and the forward epilogue stops at dot + bias
    for n in ("z1", "z2"):
        ops = {e.op for e in by_name[n].reduction.epilogue.toposort()}
        assert AluOp.Where not in ops and AluOp.Max not in ops
    assert AluOp.Where in {e.op for e in by_name["dz1"].exp.toposort()}
    # without a backward pass bias and ReLU do fuse
    fwd = jit_compile(mlp.mlp_predict_jaxpr(32, [12, 16, 5]))
    a1 = next(s.kernel for s in fwd.steps if s.kind == "execute" and s.name == "a1")
    assert AluOp.Max in {e.op for e in a1.reduction.epilogue.toposort()}


def _run(prog, arrays):
    be = OracleBackend()
    outs = prog.execute(be, [be.put(a) for a in arrays])
    return [be.slots[s][0].view(np.float32) for s in outs]


def test_relu_cotangent_passes_where_the_pre_activation_is_exactly_zero():
    """jvp.ts:205-207: the tangent of max(z, 0) is where(z < 0, 0, dz), so z == 0 passes."""
    dims, B = [4, 3, 2], 5
    rng = np.random.default_rng(0)
    x = rng.uniform(0, 1, (B, dims[0])).astype(np.float32)
    y = rng.integers(0, 2, B).astype(np.int32)
    W1 = rng.standard_normal((4, 3)).astype(np.float32)
    W1[:, 1] = 0                      # unit 1: z = x . 0 + 0 == 0 exactly for every example
    b1 = np.array([0.3, 0.0, -0.2], np.float32)
    W2, b2 = rng.standard_normal((3, 2)).astype(np.float32), np.zeros(2, np.float32)
    prog = mlp.mlp_grad_program(B, dims, global_batch=B)
    loss, dW1, db1, dW2, db2 = _run(prog, [x, y, np.eye(2, dtype=np.float32), W1, b1, W2, b2])
    z1 = x.astype(np.float64) @ W1 + b1
    assert (z1[:, 1] == 0).all()
    a1 = np.maximum(z1, 0)
    logits = a1 @ W2 + b2
    p = np.exp(logits - logits.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    dz2 = p.copy()
    dz2[np.arange(B), y] -= 1
    dz2 /= B
    dz1 = (dz2 @ W2.T) * (z1 >= 0)    # the reference's rule; (a1 > 0) would zero unit 1
    np.testing.assert_allclose(db1, dz1.sum(0), rtol=1e-5, atol=1e-7)
    assert abs(db1[1]) > 1e-3
    np.testing.assert_allclose(dW1.reshape(4, 3), x.T.astype(np.float64) @ dz1, rtol=1e-5, atol=1e-7)


def test_vmap_moves_batch_axes_as_the_batching_rules_say():
    # Dot: the batch axis ends up last (vmap.ts:297-303); outputs get it moved to the front
    b = Builder()
    x, w = b.input("x", (3,)), b.input("w", (3, 4))
    d = b.dot(b.reshape(x, (1, 3)), b.transpose(w, (1, 0)), "d")
    j = vmap_jaxpr(b.build([d]), 7, [0, None])
    dot = next(e for e in j.eqns if e.prim == "dot")
    assert tuple(dot.out.shape) == (4, 7) and tuple(j.outs[0].shape) == (7, 4)
    rng = np.random.default_rng(1)
    xs, ws = rng.standard_normal((7, 3)).astype(np.float32), rng.standard_normal((3, 4)).astype(np.float32)
    (got,) = _run(jit_compile(j), [xs, ws])
    np.testing.assert_allclose(got.reshape(7, 4), xs @ ws, rtol=1e-5, atol=1e-6)
