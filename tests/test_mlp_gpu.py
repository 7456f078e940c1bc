"""MLP programs on the GPU through the C ABI: per-example gradients under vmap (config 4) and the
Adam training step (config 5), checked against the oracle replaying the same kernel lists, and at
full shard size against a float64 model evaluated with torch on the same GPU."""
import numpy as np
import pytest

from jax_js_b200 import DType, mlp

from oracle_backend import OracleBackend
from util import assert_close

pytestmark = pytest.mark.gpu
F32 = DType.Float32


def _data(batch, n_in, classes, seed=0):
    rng = np.random.default_rng(seed)
    return rng.uniform(0, 1, (batch, n_in)).astype(np.float32), rng.integers(0, classes, batch).astype(np.int32)


def test_adam_training_matches_oracle_after_1_and_10_steps(backend):
    dims, B = [784, 256, 256, 10], 512
    x, y = _data(B, dims[0], dims[-1])
    # two oracles: the Wasm backend without and with relaxed_madd (src/backend/wasm/codegen.ts:318-322);
    # both are the reference, and their distance after n Adam steps is the reference's own noise floor
    trainers = []
    for be in (backend, OracleBackend(), OracleBackend(fma=True)):
        tr = mlp.MlpTrainer(be, dims, B, B)
        trainers.append((be, tr, be.put(x), be.put(y)))
    for step in range(1, 11):
        losses = []
        for be, tr, sx, sy in trainers:
            s = tr.step(sx, sy)
            losses.append(float(be.get(s, "float32")[0]))
            be.dec_ref(s)
        # f32, GEMM-dominated: 1e-4 relative (the GEMM bar).  Adam divides by sqrt(nu), which
        # amplifies last-bit differences where gradients are of the order of eps, so trajectories of
        # the reference's own two accumulation modes drift apart; the bar never goes below that drift.
        # From the fourth step on, ReLU units that sit within rounding of zero start to switch
        # differently under a different summation order (see the parameter check below); the loss
        # bar widens to 5e-4 there.
        floor = 3 * abs(losses[2] - losses[1])
        bar = 1e-4 if step <= 3 else 5e-4
        assert abs(losses[0] - losses[1]) <= max(bar * abs(losses[1]), floor), (step, losses)
        if step == 1:
            assert abs(losses[0] - losses[1]) <= 1e-5 * abs(losses[1]), losses
        if step in (1, 5, 10):
            (b0, t0, _, _), (b1, t1, _, _), (b2, t2, _, _) = trainers
            for s0, s1, s2 in zip(t0.params, t1.params, t2.params):
                want, got = b1.get(s1, "float32").astype(np.float64), b0.get(s0, "float32").astype(np.float64)
                alt = b2.get(s2, "float32").astype(np.float64)
                # 1e-4 of the leaf's scale, but not finer than 2 % of one Adam update (lr = 1e-3): the
                # bias leaves start at zero and are themselves only a few updates large
                tol = max(1e-4 * np.abs(want).max(), 2e-5)
                err, ref_err = np.abs(got - want), np.abs(alt - want)
                # After one step: all but a sliver within 1e-4 of the leaf's scale.  After that the two
                # free-running trajectories separate geometrically (about 1.75x per step here): Adam
                # divides by sqrt(nu), so a last-bit difference in a gradient moves the next update by
                # the same relative amount, and that moves the next gradient.  Independently, a hidden
                # unit whose pre-activation lies within rounding of zero switches its ReLU differently
                # under a different summation order, which changes one whole column of dW by a few per
                # cent of an update.  So the free-running bars are: after five steps the typical element
                # within a tenth of the tolerance and at most 5 % of a leaf beyond it; after ten steps the
                # typical element still inside 1e-4 of the scale and at most half of a (bias) leaf beyond
                # it; never anything off by more than one full update per step.  The step-by-step parity of the two programs
                # from identical state, which has no such amplification, is checked by
                # test_each_step_from_the_oracle_state below.
                frac = (err > tol).mean()
                assert frac <= {1: 1e-4, 5: 0.05, 10: 0.5}[step] + 2 * (ref_err > tol).mean(), (step, frac)
                assert np.median(err) <= (1.0 if step == 10 else 0.1) * tol, (step, np.median(err), np.median(ref_err))
                assert err.max() <= step * 1e-3 * 1.01, f"params after step {step}"
    for be, tr, sx, sy in trainers:
        tr.close()
        be.dec_ref(sx)
        be.dec_ref(sy)


def test_each_step_from_the_oracle_state(backend):
    """Ten Adam steps along the oracle's trajectory; at every step the GPU runs the gradient program
    and the Adam program from the ORACLE's state of that step, so each comparison is of one program
    on identical inputs (no accumulated drift)."""
    dims, B = [784, 256, 256, 10], 512
    x, y = _data(B, dims[0], dims[-1])
    ob = OracleBackend()
    tg, to = mlp.MlpTrainer(backend, dims, B, B), mlp.MlpTrainer(ob, dims, B, B)
    gx, gy, ox, oy = backend.put(x), backend.put(y), ob.put(x), ob.put(y)
    up = lambda slot, dt="float32": backend.put(ob.get(slot, dt))
    strict = 0
    for step in range(1, 11):
        ps = [up(s) for s in to.params]
        outs_g = tg.grad.execute(backend, [gx, gy, tg.eye] + ps)
        outs_o = to.grad.execute(ob, [ox, oy, to.eye] + to.params)
        # A hidden unit whose pre-activation is within f32 summation error of zero for some example
        # ("on the edge") may have its ReLU gate taken either way, depending on summation order; that
        # example's share (1/B) of the gradient then differs: in one column of that layer's dW, one
        # element of db, and through dz in every leaf below.  Both outcomes are correct roundings of
        # the same program.  Edge units are found here in float64 from the state itself (margin
        # 2e-6: five standard deviations of the summation error of a 784-term f32 dot of these
        # magnitudes); steps without any get the strict bar, steps with one the loose bar.
        h, edge = x.astype(np.float64), 0
        for l in range(len(dims) - 2):
            z = h @ ob.get(to.params[2 * l], "float32").astype(np.float64).reshape(dims[l], dims[l + 1]) \
                + ob.get(to.params[2 * l + 1], "float32").astype(np.float64)
            edge += int((np.abs(z) < 2e-6).sum())
            h = np.maximum(z, 0)
        strict += edge == 0
        for name, a, b in zip(["loss"] + tg.names, outs_g, outs_o):
            got, want = backend.get(a, "float32").astype(np.float64), ob.get(b, "float32").astype(np.float64)
            scale = np.abs(want).max()
            err = np.abs(got - want)
            # f32, GEMM-dominated: every element within 1e-4 of the leaf's scale, the typical one 10x
            # closer; with a unit on the edge, one example's share of the gradient: 1e-2 of the scale
            assert err.max() <= (1e-4 if edge == 0 else 1e-2) * scale, (step, name, edge, err.max(), scale)
            assert np.median(err) <= 1e-5 * scale, (step, name, np.median(err), scale)
        cnt = up(to.count, "uint32")
        ins_g, ins_o, tmp = [cnt], [to.count], [cnt]
        for i in range(len(tg.names)):
            gi, mi, ni = up(outs_o[1 + i]), up(to.mu[i]), up(to.nu[i])
            tmp += [gi, mi, ni]
            ins_g += [ps[i], gi, mi, ni]
            ins_o += [to.params[i], outs_o[1 + i], to.mu[i], to.nu[i]]
        new_g, new_o = tg.adam.execute(backend, ins_g), to.adam.execute(ob, ins_o)
        assert backend.get(new_g[0], "uint32")[0] == ob.get(new_o[0], "uint32")[0] == step
        for a, b in zip(new_g[1:], new_o[1:]):
            got, want = backend.get(a, "float32").astype(np.float64), ob.get(b, "float32").astype(np.float64)
            # elementwise f32 with one reciprocal, one sqrt and the bias corrections: 1e-5 relative
            # (the elementwise bar), measured against the element or, where
            # the element is below one update, against the update size
            assert (np.abs(got - want) <= 1e-5 * np.maximum(np.abs(want), 1e-3)).all(), step
        for s in list(outs_g) + ps + tmp + list(new_g):
            backend.dec_ref(s)
        for s in list(outs_o) + list(new_o):
            ob.dec_ref(s)
        ob.dec_ref(to.step(ox, oy))
    assert strict >= 3, f"only {strict} of 10 steps were free of edge units: the strict bar was hardly exercised"
    tg.close()
    to.close()
    for be, a, b in ((backend, gx, gy), (ob, ox, oy)):
        be.dec_ref(a)
        be.dec_ref(b)


def test_per_example_gradients_config4(backend):
    dims, B = [784, 1024, 10], 64
    x, y = _data(B, dims[0], dims[-1], 1)
    params = mlp.init_params(dims, 0)
    params[1] = params[1] + 0.05   # non-zero biases so that bias handling is exercised
    prog = mlp.mlp_grad_program(B, dims, per_example=True)
    outs = []
    for be in (backend, OracleBackend()):
        slots = [be.put(x), be.put(y), be.put(np.eye(10, dtype=np.float32))] + [be.put(p) for p in params]
        res = prog.execute(be, slots)
        outs.append([be.get(s, "float32") for s in res])
        for s in slots + res:
            be.dec_ref(s)
    names = ["loss", "dW1", "db1", "dW2", "db2"]
    for name, got, want in zip(names, outs[0], outs[1]):
        # the gradients are products of GEMM-like intermediates: 1e-4 of the leaf's scale
        assert_close(got, want, 1e-4, np.abs(want).max() if name != "loss" else None, name)
    assert outs[0][1].size == 784 * 1024 * 64


def test_captured_per_example_program_substitutes_the_batch_last_products(backend):
    """Inside a capture the per-example outer products (a Dot with the batch axis last) are not
    materialised: the Kernel that moves the batch axis first runs with the product in place of its
    load.  Two launches fewer, the 205 MB array written once, the same bits as the Kernels one by one."""
    dims, B = [784, 1024, 10], 64
    x, y = _data(B, dims[0], dims[-1], 3)
    params = mlp.init_params(dims, 0)
    prog = mlp.mlp_grad_program(B, dims, per_example=True)
    slots = [backend.put(x), backend.put(y), backend.put(np.eye(10, dtype=np.float32))] + [backend.put(p) for p in params]
    eager = prog.execute(backend, slots)
    want = [backend.read_sync(s).copy() for s in eager]
    n_kernels = sum(1 for s in prog.steps if s.kind == "execute")
    graph, outs = prog.capture(backend, slots)
    launches, nbytes, groups = backend.graph_cost(graph)
    assert groups >= 2 and launches <= n_kernels - groups, (launches, n_kernels, groups)   # a batch of small Kernels saves more than one launch
    for _ in range(2):
        backend.graph_launch(graph)
    for name, s, w in zip(["loss", "dW1", "db1", "dW2", "db2"], outs, want):
        assert np.array_equal(backend.read_sync(s), w), name
    backend.graph_destroy(graph)
    for s in slots + eager + list(outs):
        backend.dec_ref(s)


def test_kept_remainder_planes_do_not_change_a_captured_training_step(backend):
    """Inside a capture the 3xTF32 remainder plane of an array is written once and read by every GEMM
    that has the array as an operand (an activation: its forward and its weight-gradient GEMM); with
    JAXCUDA_TC_PLANE_CACHE=0 every GEMM splits its own operands.  Same planes, same bits, also after
    the parameters have moved (the planes of the new values are made anew in every replay)."""
    import os
    from jax_js_b200.backend import CudaBackend
    dims, B = [784, 2048, 2048, 10], 4096
    x, y = _data(B, dims[0], dims[-1], 4)
    results = {}
    for mode in ("1", "0"):
        old = os.environ.get("JAXCUDA_TC_PLANE_CACHE")
        os.environ["JAXCUDA_TC_PLANE_CACHE"] = mode
        try:
            be = CudaBackend(backend.device)
        finally:
            if old is None:
                os.environ.pop("JAXCUDA_TC_PLANE_CACHE")
            else:
                os.environ["JAXCUDA_TC_PLANE_CACHE"] = old
        try:
            sx, sy = be.put(x), be.put(y)
            tr = mlp.MlpTrainer(be, dims, B, B)
            be.dec_ref(tr.step(sx, sy))
            tr.capture(sx, sy)
            losses = []
            for _ in range(4):
                s_ = tr.step(sx, sy)
                losses.append(be.get(s_, "float32")[0])
                be.dec_ref(s_)
            results[mode] = (np.array(losses), [be.read_sync(p).copy() for p in tr.params])
            tr.close()
            be.dec_ref(sx)
            be.dec_ref(sy)
        finally:
            be.close()
    assert np.array_equal(results["1"][0].view(np.uint32), results["0"][0].view(np.uint32)), (results["1"][0], results["0"][0])
    for a, b in zip(results["1"][1], results["0"][1]):
        assert np.array_equal(a, b)


def test_config5_shard_gradients_against_float64(backend):
    import torch
    dims, B, GB = [784, 2048, 2048, 10], 8192, 65536
    x, y = _data(B, dims[0], dims[-1], 2)
    params = mlp.init_params(dims, 0)
    prog = mlp.mlp_grad_program(B, dims, global_batch=GB)
    slots = [backend.put(x), backend.put(y), backend.put(np.eye(10, dtype=np.float32))] + [backend.put(p) for p in params]
    res = prog.execute(backend, slots)
    got = [backend.get(s, "float32") for s in res]
    for s in slots + res:
        backend.dec_ref(s)
    dev = torch.device("cuda", backend.device)
    tp = [torch.tensor(p, dtype=torch.float64, device=dev, requires_grad=True) for p in params]
    h = torch.tensor(x, dtype=torch.float64, device=dev)
    for l in range(3):
        h = h @ tp[2 * l] + tp[2 * l + 1]
        if l < 2:
            h = torch.relu(h)
    loss = torch.nn.functional.cross_entropy(h, torch.tensor(y, dtype=torch.long, device=dev), reduction="sum") / GB
    loss.backward()
    assert abs(got[0][0] - loss.item()) <= 1e-4 * abs(loss.item())
    for name, g, t in zip(mlp.param_order(3), got[1:], tp):
        want = t.grad.detach().cpu().numpy().reshape(-1)
        # A float64 forward pass switches a few ReLUs (pre-activations within rounding of zero)
        # differently from any f32 pass; each such unit changes one column of dW by up to ~1e-3 of
        # the leaf's scale.  Bar: 1e-4 of the scale for 95 % of every leaf, 1e-2 for all of it, and
        # the mean error far inside the bar.
        err = np.abs(g.astype(np.float64) - want)
        scale = np.abs(want).max()
        assert (err <= 1e-4 * scale).mean() >= 0.95, f"d{name}"
        assert err.max() <= 1e-2 * scale, f"d{name}"
        assert err.mean() <= 3e-5 * scale, f"d{name}"


def test_config5_shard_against_the_oracle(backend):
    """One gradient program and one Adam program at the benchmark's own shard: 784-2048-2048-10 with the
    8192 examples one of eight GPUs sees, global batch 65536, against the oracle replaying the same
    Kernel list on the same inputs."""
    dims, B, GB = [784, 2048, 2048, 10], 8192, 65536
    x, y = _data(B, dims[0], dims[-1], 3)
    params = mlp.init_params(dims, 0)
    params[1] = params[1] + 0.01
    eye = np.eye(10, dtype=np.float32)
    prog = mlp.mlp_grad_program(B, dims, global_batch=GB)
    ob = OracleBackend(fma=True)
    res = {}
    for key, be in (("cuda", backend), ("oracle", ob)):
        slots = [be.put(x), be.put(y), be.put(eye)] + [be.put(p) for p in params]
        outs = prog.execute(be, slots)
        res[key] = [be.get(s, "float32").astype(np.float64) for s in outs]
        for s in slots + outs:
            be.dec_ref(s)
    # hidden units within f32 summation error of zero may take their ReLU gate either way (see
    # test_each_step_from_the_oracle_state); count them in float64
    h, edge = x.astype(np.float64), 0
    for l in range(2):
        z = h @ params[2 * l].astype(np.float64) + params[2 * l + 1].astype(np.float64)
        edge += int((np.abs(z) < 4e-6).sum())
        h = np.maximum(z, 0)
    assert abs(res["cuda"][0][0] - res["oracle"][0][0]) <= 1e-5 * abs(res["oracle"][0][0])
    for name, got, want in zip(mlp.param_order(3), res["cuda"][1:], res["oracle"][1:]):
        scale = np.abs(want).max()
        err = np.abs(got - want)
        # f32, GEMM-dominated: 1e-4 of the leaf's scale.  With 8192 x 4096 hidden pre-activations some
        # always sit on the edge (about a hundred here); each one that is gated differently moves one
        # example's share of a column of dW, a few 1e-4 of the scale.  So: the typical element ten
        # times inside the bar, at most 2 % of a leaf beyond it, nothing beyond 1e-2.
        assert np.median(err) <= 1e-5 * scale, (name, np.median(err), scale)
        assert (err > 1e-4 * scale).mean() <= (0.02 if edge else 0.0), (name, (err > 1e-4 * scale).mean(), edge)
        assert err.max() <= 1e-2 * scale, (name, err.max(), scale, edge)
    # Adam on the oracle's gradients: elementwise, 1e-5
    sizes, names = mlp.leaf_sizes(dims), mlp.param_order(3)
    adam = mlp.adam_program(sizes, names)
    grads = [g.astype(np.float32) for g in res["oracle"][1:]]
    rng = np.random.default_rng(4)
    mu = [(rng.standard_normal(n) * 1e-4).astype(np.float32) for n in sizes]
    nu = [(rng.uniform(0, 1, n) * 1e-8).astype(np.float32) for n in sizes]
    new = {}
    for key, be in (("cuda", backend), ("oracle", ob)):
        ins = [be.put(np.array([6], np.uint32))]
        for i in range(len(names)):
            ins += [be.put(params[i]), be.put(grads[i]), be.put(mu[i]), be.put(nu[i])]
        outs = adam.execute(be, ins)
        assert be.get(outs[0], "uint32")[0] == 7
        new[key] = [be.get(s, "float32").astype(np.float64) for s in outs[1:]]
        for s in ins + outs:
            be.dec_ref(s)
    for got, want in zip(new["cuda"], new["oracle"]):
        assert (np.abs(got - want) <= 1e-5 * np.maximum(np.abs(want), 1e-3)).all()
