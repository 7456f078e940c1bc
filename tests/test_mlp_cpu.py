"""Host logic of the MLP programs on CPU: the kernel lists against a float64 numpy model, the
planner on every kernel of configs 4 and 5, and the data-parallel step as two gloo ranks."""
import os

import numpy as np
import pytest

from jax_js_b200 import mlp
from jax_js_b200.backend import check_kernel

from oracle_backend import OracleBackend


def numpy_mlp_step(params, x, y, state, lr=1e-3):
    """float64 reference: mean softmax cross-entropy, gradients, one Adam step."""
    p = [a.astype(np.float64) for a in params]
    L = len(p) // 2
    acts = [x.astype(np.float64)]
    for l in range(L):
        z = acts[-1] @ p[2 * l] + p[2 * l + 1]
        acts.append(np.maximum(z, 0) if l < L - 1 else z)
    logits = acts[-1]
    m = logits.max(1, keepdims=True)
    e = np.exp(logits - m)
    s = e.sum(1, keepdims=True)
    B = x.shape[0]
    loss = -(logits - m - np.log(s))[np.arange(B), y].mean()
    dz = e / s
    dz[np.arange(B), y] -= 1
    dz /= B
    grads = [None] * (2 * L)
    for l in range(L - 1, -1, -1):
        grads[2 * l], grads[2 * l + 1] = acts[l].T @ dz, dz.sum(0)
        if l > 0:
            dz = (dz @ p[2 * l].T) * (acts[l] > 0)
    t = state["t"] = state["t"] + 1
    new = []
    for i, (w, g) in enumerate(zip(p, grads)):
        state["mu"][i] = 0.9 * state["mu"][i] + 0.1 * g
        state["nu"][i] = 0.999 * state["nu"][i] + 0.001 * g * g
        mhat, vhat = state["mu"][i] / (1 - 0.9**t), state["nu"][i] / (1 - 0.999**t)
        new.append(w - lr * mhat / (np.sqrt(vhat) + 1e-8))
    return loss, grads, new


DIMS, B = [20, 32, 24, 10], 64


def _data(seed=0):
    rng = np.random.default_rng(seed)
    return rng.uniform(0, 1, (B, DIMS[0])).astype(np.float32), rng.integers(0, DIMS[-1], B).astype(np.int32)


def test_training_steps_match_float64_model():
    x, y = _data()
    be = OracleBackend()
    tr = mlp.MlpTrainer(be, DIMS, B, B)
    params = mlp.init_params(DIMS)
    state = {"t": 0, "mu": [0.0] * len(params), "nu": [0.0] * len(params)}
    sx, sy = be.put(x), be.put(y)
    for _ in range(3):
        loss_slot = tr.step(sx, sy)
        want_loss, _, params = numpy_mlp_step(params, x, y, state)
        got = be.get(loss_slot, "float32")[0]
        be.dec_ref(loss_slot)
        assert abs(got - want_loss) <= 1e-5 * abs(want_loss)
        for slot, want in zip(tr.params, params):
            np.testing.assert_allclose(be.get(slot, "float32"), want.reshape(-1), rtol=1e-4, atol=1e-6)


def test_per_example_program_matches_float64_model():
    x, y = _data(1)
    dims = [20, 16, 10]
    be = OracleBackend()
    prog = mlp.mlp_grad_program(B, dims, per_example=True)
    params = mlp.init_params(dims, 3)
    params[1] += 0.1
    slots = [be.put(x), be.put(y), be.put(np.eye(10, dtype=np.float32))] + [be.put(p) for p in params]
    outs = prog.execute(be, slots)
    loss = be.get(outs[0], "float32")
    dW1 = be.get(outs[1], "float32", (B, dims[0], dims[1]))      # vmap puts the batch axis first
    db2 = be.get(outs[4], "float32", (B, dims[2]))
    for b in (0, 7, B - 1):
        state = {"t": 0, "mu": [0.0] * 4, "nu": [0.0] * 4}
        want_loss, grads, _ = numpy_mlp_step(params, x[b:b + 1], y[b:b + 1], state)
        assert abs(loss[b] - want_loss) <= 1e-5 * max(abs(want_loss), 1e-3)
        np.testing.assert_allclose(dW1[b], grads[0], rtol=1e-4, atol=1e-6)
        np.testing.assert_allclose(db2[b], grads[3], rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("which", ["config4", "config5", "adam"])
def test_every_kernel_of_the_mlp_configs_plans_and_compiles(lib, which):
    if which == "config4":
        prog = mlp.mlp_grad_program(64, [784, 1024, 10], per_example=True)
    elif which == "config5":
        prog = mlp.mlp_grad_program(8192, [784, 2048, 2048, 10], global_batch=65536)
    else:
        dims = [784, 2048, 2048, 10]
        prog = mlp.adam_program(mlp.leaf_sizes(dims), mlp.param_order(3))
    seen = set()
    kinds = []
    for k in prog.kernels():
        if k.fingerprint() in seen:
            continue
        seen.add(k.fingerprint())
        kinds.append(check_kernel(k, compile=True)[0])
    if which == "config5":
        assert sum("gemm-tcgen05 3xtf32" in d for d in kinds) >= 5, kinds
    assert kinds


def _rank_main(rank, world, port, out):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x, y = _data()
    lo, hi = rank * B // world, (rank + 1) * B // world
    be = OracleBackend(dist=dist, threads=1)
    tr = mlp.MlpTrainer(be, DIMS, hi - lo, B)
    sx, sy = be.put(x[lo:hi]), be.put(y[lo:hi])
    losses = []
    for _ in range(2):
        s = tr.step(sx, sy, world=world)
        losses.append(float(be.get(s, "float32")[0]))
        be.dec_ref(s)
    # each step summed loss and bias gradients as one group, then every weight gradient as it appeared
    assert tr.overlap and be.joined and be.async_calls == [5, 1, 1] * 2, be.async_calls   # loss + biases ride with dW1
    # with dW3 and dW2 hoisted to where their inputs exist, whatever small outputs came before a weight
    # gradient ride with its sum: (loss, dW3), (db3, dW2), (db2, db1, dW1); the step is the same step
    be.async_calls.clear()
    th = mlp.MlpTrainer(be, DIMS, hi - lo, B, hoist=True)
    s = th.step(sx, sy, world=world)
    assert th.hoist and be.async_calls == [2, 2, 3], be.async_calls
    assert abs(float(be.get(s, "float32")[0]) - losses[0]) <= 1e-6 * abs(losses[0])
    be.dec_ref(s)
    if rank == 0:
        np.savez(out, losses=np.array(losses), **{f"p{i}": be.get(s, "float32") for i, s in enumerate(tr.params)})
    dist.destroy_process_group()


def test_two_gloo_ranks_train_like_one(tmp_path):
    import torch.multiprocessing as mp
    out = str(tmp_path / "rank0.npz")
    mp.spawn(_rank_main, args=(2, 29631, out), nprocs=2, join=True)
    got = np.load(out)
    x, y = _data()
    be = OracleBackend()
    tr = mlp.MlpTrainer(be, DIMS, B, B)
    sx, sy = be.put(x), be.put(y)
    losses = []
    for _ in range(2):
        s = tr.step(sx, sy)
        losses.append(float(be.get(s, "float32")[0]))
    np.testing.assert_allclose(got["losses"], losses, rtol=1e-5)
    for i, s in enumerate(tr.params):
        np.testing.assert_allclose(got[f"p{i}"], be.get(s, "float32"), rtol=1e-4, atol=1e-6)


def test_step_list_hooks_and_caller_owned_outputs():
    """`JitProgram.execute`: outputs written into slots the caller owns, and the two hooks (after a
    program output is dispatched, before each kernel) fire in dispatch order."""
    from jax_js_b200 import programs as P
    be = OracleBackend()
    rows, cols = 4, 6
    x = np.arange(rows * cols, dtype=np.float32).reshape(rows, cols) / 7
    prog = P.softmax_lse_argmax_program(rows, cols)
    sx, si = be.put(x), be.put(P.argmax_iota(cols))
    want = [be.slots[s][0].copy() for s in prog.execute(be, [sx, si])]
    mine = {"lse": be.malloc(rows * 4), "argmax": be.malloc(rows * 4)}
    events = []
    outs = prog.execute(be, [sx, si], on_output=lambda name, slot: events.append(("out", name)),
                        out_slots=mine, before_step=lambda step: events.append(("run", step.name)))
    assert outs[1] == mine["lse"] and outs[2] == mine["argmax"] and outs[0] not in mine.values()
    for got, w in zip(outs, want):
        assert np.array_equal(be.slots[got][0], w)
    runs = [n for kind, n in events if kind == "run"]
    assert runs == ["m1", "u", "s", "softmax", "m2", "m2k", "s2", "lse", "m3", "argmax"]
    assert [n for kind, n in events if kind == "out"] == ["softmax", "lse", "argmax"]
    assert events.index(("out", "softmax")) == events.index(("run", "softmax")) + 1


def test_hoisted_program_is_a_permutation_with_the_same_bits():
    """JitProgram.hoisted moves the weight-gradient Kernels of layers 2.. to where their inputs exist:
    the same Kernels, every intermediate released after its last reader, and on the oracle backend
    the same outputs bit for bit; nothing is read after it was released (the backend would raise)."""
    prog = mlp.mlp_grad_program(B, DIMS, global_batch=2 * B)
    hoisted = prog.hoisted(["dW2", "dW3"])
    names = [s.name for s in prog.steps if s.kind == "execute"]
    moved = [s.name for s in hoisted.steps if s.kind == "execute"]
    assert sorted(names) == sorted(moved) and names != moved
    assert moved.index("dW3") < moved.index("dz2") < moved.index("dW2") < moved.index("dz1") < moved.index("dW1") == len(moved) - 1
    assert {id(s.kernel) for s in prog.steps if s.kind == "execute"} == {id(s.kernel) for s in hoisted.steps if s.kind == "execute"}
    frees = [s.name for s in hoisted.steps if s.kind == "free"]
    assert sorted(frees) == sorted(s.name for s in prog.steps if s.kind == "free") and len(set(frees)) == len(frees)
    assert prog.hoisted([]).steps and [s.name for s in prog.hoisted([]).steps if s.kind == "execute"] == names
    x, y = _data()
    be = OracleBackend()
    params = [be.put(a) for a in mlp.init_params(DIMS, 0)]
    ins = [be.put(x), be.put(y), be.put(np.eye(DIMS[-1], dtype=np.float32))] + params
    a = [be.get(s, "float32").copy() for s in prog.execute(be, ins)]
    b = [be.get(s, "float32").copy() for s in hoisted.execute(be, ins)]
    for u, v in zip(a, b):
        assert np.array_equal(u.view(np.uint32), v.view(np.uint32))
