"""Scatter routine (src/routine.ts:44-48, :226-296): the oracle against the reference's backend test
vector on CPU, and the CUDA routine against the oracle on the GPU."""
import numpy as np
import pytest

import oracle
from jax_js_b200 import DType
from jax_js_b200.routine import Routine, Routines, RoutineType

F32, I32, BOOL = DType.Float32, DType.Int32, DType.Bool


def _params(op, shape, axis, out_dim, unique):
    return {"op": op, "shape": list(shape), "axis": list(axis), "outDim": out_dim, "uniqueIndices": unique}


def test_oracle_scatter_reference_vector():
    # src/backend/backend.test.ts:118-187: update of one element, then an empty update: the output is cleared
    p = _params("update", [4], [0], 0, True)
    assert oracle.scatter(np.array([7], np.float32), [np.array([1], np.int32)], p, F32).tolist() == [0, 7, 0, 0]
    assert oracle.scatter(np.array([7], np.float32), [np.array([2], np.int32)], p, F32).tolist() == [0, 0, 7, 0]
    assert oracle.scatter(np.zeros(0, np.float32), [np.zeros(0, np.int32)], p, F32).tolist() == [0, 0, 0, 0]


def test_oracle_scatter_add_and_last_update_wins():
    idx = np.array([1, 3, 1, 9, -1], np.int32)       # out-of-range coordinates drop the update
    upd = np.array([1, 2, 3, 4, 5], np.float32)
    assert oracle.scatter(upd, [idx], _params("add", [4], [0], 0, False), F32).tolist() == [0, 4, 0, 2]
    assert oracle.scatter(upd, [idx], _params("update", [4], [0], 0, False), F32).tolist() == [0, 3, 0, 2]
    # rows of a [5, 3] output addressed by an index over axis 0, updates [2, 3]: np.add.at semantics
    u = np.arange(6, dtype=np.float32).reshape(2, 3)
    got = oracle.scatter(u, [np.array([4, 4], np.int32)], _params("add", [5, 3], [0], 0, False), F32)
    want = np.zeros((5, 3), np.float32)
    np.add.at(want, np.array([4, 4]), u)
    assert (got == want).all()


def _cuda_scatter(backend, upd, indices, params, dtype):
    t = RoutineType([list(upd.shape)] + [list(i.shape) for i in indices], [dtype] + [I32] * len(indices),
                    [params["shape"]], [dtype])
    exe = backend.prepare_routine(Routine(Routines.Scatter, t, params))
    ins = [backend.put(upd)] + [backend.put(i) for i in indices]
    out = backend.put(np.full(params["shape"], 9, dtype=upd.dtype))     # stale contents must be cleared
    backend.dispatch(exe, ins, [out])
    res = backend.read_sync(out).view(upd.dtype).reshape(params["shape"])
    for s in ins + [out]:
        backend.dec_ref(s)
    return res


@pytest.mark.gpu
def test_cuda_scatter_reference_vector(backend):
    p = _params("update", [4], [0], 0, True)
    assert _cuda_scatter(backend, np.array([7], np.float32), [np.array([1], np.int32)], p, F32).tolist() == [0, 7, 0, 0]
    assert _cuda_scatter(backend, np.zeros(0, np.float32), [np.zeros(0, np.int32)], p, F32).tolist() == [0, 0, 0, 0]


@pytest.mark.gpu
@pytest.mark.parametrize("op,unique", [("update", True), ("update", False), ("add", False), ("add", True)])
def test_cuda_scatter_matches_oracle(backend, op, unique):
    rng = np.random.default_rng(0)
    n, rows, cols = 20000, 300, 7
    idx = rng.permutation(n)[:rows].astype(np.int32) if unique else rng.integers(-3, n + 3, rows).astype(np.int32)
    # embedding-gradient shape: rows of `cols` values scattered into [n, cols] along axis 0
    upd = rng.integers(-1000, 1000, (rows, cols)).astype(np.int32)
    p = _params(op, [n, cols], [0], 0, unique)
    assert (_cuda_scatter(backend, upd, [idx], p, I32) == oracle.scatter(upd, [idx], p, I32)).all()
    updf = rng.standard_normal((rows, cols)).astype(np.float32)
    got, want = _cuda_scatter(backend, updf, [idx], p, F32), oracle.scatter(updf, [idx], p, F32)
    if op == "add" and not unique:   # float sums: arrival order differs, within rounding of the few terms per slot
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)
    else:
        assert (got.view(np.uint32) == want.view(np.uint32)).all()
    # two indexed axes with the index dimensions inserted in the middle of the updates (outDim = 1)
    i0, i1 = rng.integers(0, 5, (4, 1)).astype(np.int32), rng.integers(0, 6, (1, 3)).astype(np.int32)
    upd3 = rng.integers(0, 100, (8, 4, 3)).astype(np.int32)
    p3 = _params(op, [5, 8, 6], [0, 2], 1, False)
    assert (_cuda_scatter(backend, upd3, [i0, i1], p3, I32) == oracle.scatter(upd3, [i0, i1], p3, I32)).all()
    b = (rng.random(50) < 0.5).astype(np.int32)
    pb = _params("add", [10], [0], 0, False)
    ib = rng.integers(0, 10, 50).astype(np.int32)
    assert (_cuda_scatter(backend, b, [ib], pb, BOOL) == oracle.scatter(b, [ib], pb, BOOL)).all()
