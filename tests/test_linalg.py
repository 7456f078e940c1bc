"""TriangularSolve, Cholesky and LU routines (src/routine.ts:44-78, CPU reference :298-432): the oracle
against the reference's own test vectors and defining properties on CPU, and the CUDA routines
against the oracle on the GPU.

Bars: the routines keep the reference's arithmetic (double intermediates, one rounding per store), so
float32 outputs are compared at 2e-6 of the output's scale (a few ulp: only the order of a double
sum differs) and pivots / permutations must be identical."""
import numpy as np
import pytest

import oracle
from jax_js_b200 import DType
from jax_js_b200.routine import Routine, Routines, RoutineType

F32, F64, I32 = DType.Float32, DType.Float64, DType.Int32
DT = {np.dtype(np.float32): F32, np.dtype(np.float64): F64}


def _spd(rng, batch, n, dtype=np.float32):
    a = rng.standard_normal((batch, n, n))
    return (a @ a.transpose(0, 2, 1) + n * np.eye(n)).astype(dtype)


# ---- the oracle against the reference's vectors (CPU) ---------------------------------------------

def test_oracle_lu_reference_vector():
    # test/lax-linalg.test.ts:277-290
    lu, piv, perm = oracle.lu(np.array([[4, 3], [6, 3]], np.float32))
    np.testing.assert_allclose(lu, [[6, 3], [0.6666667, 1.0]], rtol=1e-6)
    assert piv.tolist() == [1, 1] and perm.tolist() == [1, 0]


def test_oracle_lu_reconstructs_with_permutation():
    # test/lax-linalg.test.ts:292-305: P @ A = L @ U for a 30 x 30 uniform matrix, rtol 1e-5 / atol 1e-6
    rng = np.random.default_rng(0)
    for m, n in ((30, 30), (7, 12), (12, 7)):
        A = rng.uniform(0, 1, (m, n)).astype(np.float32)
        lu, piv, perm = oracle.lu(A)
        r = min(m, n)
        L = np.tril(lu, -1)[:, :r] + np.eye(m, r)
        U = np.triu(lu)[:r]
        np.testing.assert_allclose(A[perm], L @ U, rtol=1e-5, atol=1e-6)
        assert sorted(perm.tolist()) == list(range(m)) and (piv >= np.arange(r)).all()


def test_oracle_cholesky_reference_cases():
    # test/lax-linalg.test.ts:24-52: 2 x 2 and 3 x 3; L lower triangular, L @ L^T = x
    for x in ([[2.0, 1.0], [1.0, 2.0]], [[4.0, 2.0, 1.0], [2.0, 5.0, 3.0], [1.0, 3.0, 6.0]]):
        x = np.array(x, np.float32)
        L = oracle.cholesky(x)
        assert (np.triu(L, 1) == 0).all() and L[1, 0] != 0
        np.testing.assert_allclose(L @ L.T, x, rtol=1e-5, atol=1e-6)
    L = oracle.cholesky(np.array([[2.0, 1.0], [1.0, 2.0]], np.float32))
    np.testing.assert_allclose(L, [[np.sqrt(2), 0], [1 / np.sqrt(2), np.sqrt(1.5)]], rtol=1e-6)


def test_oracle_triangular_solve():
    # a x = b with a upper triangular, one row of b per system (src/routine.ts:44-53)
    a = np.array([[2, 1], [0, 3]], np.float32)
    np.testing.assert_allclose(oracle.triangular_solve(a, np.array([[4, 7]], np.float32)), [[5 / 6, 7 / 3]], rtol=1e-6)
    np.testing.assert_allclose(oracle.triangular_solve(a, np.array([[4, 7]], np.float32), unit_diagonal=True), [[-3, 7]])
    rng = np.random.default_rng(1)
    a = np.triu(rng.standard_normal((3, 40, 40))).astype(np.float32) + 5 * np.eye(40, dtype=np.float32)
    b = rng.standard_normal((3, 9, 40)).astype(np.float32)
    x = oracle.triangular_solve(a, b)
    np.testing.assert_allclose(np.einsum("cij,ctj->cti", a.astype(np.float64), x.astype(np.float64)), b, rtol=1e-4, atol=1e-5)


# ---- the CUDA routines against the oracle (GPU) ---------------------------------------------------

def _run(backend, name, ins, out_shapes, out_dtypes, params=None):
    t = RoutineType([list(a.shape) for a in ins], [DT[a.dtype] for a in ins], [list(s) for s in out_shapes], out_dtypes)
    exe = backend.prepare_routine(Routine(name, t, params))
    in_slots = [backend.put(a) for a in ins]
    np_of = {F32: np.float32, F64: np.float64, I32: np.int32}
    outs = [backend.put(np.full(s, 7, np_of[d])) for s, d in zip(out_shapes, out_dtypes)]   # stale contents
    backend.dispatch(exe, in_slots, outs)
    res = [backend.read_sync(o).view(np_of[d]).reshape(s) for o, s, d in zip(outs, out_shapes, out_dtypes)]
    for s in in_slots + outs:
        backend.dec_ref(s)
    return res


def _close(got, want, tol=2e-6):
    got, want = got.astype(np.float64), want.astype(np.float64)
    assert (np.isnan(got) == np.isnan(want)).all()
    ok = ~np.isnan(want)
    assert (np.abs(got - want)[ok] <= tol * max(1.0, np.abs(want[ok]).max(initial=0))).all(), np.abs(got - want)[ok].max()


@pytest.mark.gpu
@pytest.mark.parametrize("batch,n", [(1, 1), (1, 2), (5, 3), (3, 33), (2, 130), (1, 512)])
def test_cuda_cholesky(backend, batch, n):
    x = _spd(np.random.default_rng(n), batch, n)
    (L,) = _run(backend, Routines.Cholesky, [x], [x.shape], [F32])
    _close(L, oracle.cholesky(x))
    assert (np.triu(L, 1) == 0).all()                      # the upper triangle is cleared, not left stale
    # the reference's own large case: residual of the reconstruction below 1e-5 of max|x|
    Ld = L.astype(np.float64)
    assert np.abs(Ld @ Ld.transpose(0, 2, 1) - x).max() / np.abs(x).max() < 1e-5


@pytest.mark.gpu
def test_cuda_cholesky_float64_and_indefinite_input(backend):
    x = _spd(np.random.default_rng(3), 2, 40, np.float64)
    (L,) = _run(backend, Routines.Cholesky, [x], [x.shape], [F64])
    _close(L, oracle.cholesky(x), 1e-13)
    bad = np.array([[[1.0, 2.0], [2.0, 1.0]]], np.float32)  # not positive definite: sqrt of a negative number
    (L,) = _run(backend, Routines.Cholesky, [bad], [bad.shape], [F32])
    want = oracle.cholesky(bad)
    assert np.isnan(want[0, 1, 1]) and np.isnan(L[0, 1, 1]) and L[0, 0, 0] == 1 and L[0, 1, 0] == 2


@pytest.mark.gpu
@pytest.mark.parametrize("mats,rows,n,unit", [(1, 1, 1, False), (1, 1, 2, True), (3, 9, 40, False), (2, 70, 257, False),
                                              (1, 1024, 64, True), (1, 3, 1500, False)])
def test_cuda_triangular_solve(backend, mats, rows, n, unit):
    rng = np.random.default_rng(n + rows)
    a = (np.triu(rng.standard_normal((mats, n, n))) / np.sqrt(n) + 2 * np.eye(n)).astype(np.float32)
    a += np.tril(rng.standard_normal((mats, n, n)), -1).astype(np.float32)   # below the diagonal: must be ignored
    b = rng.standard_normal((mats, rows, n)).astype(np.float32)
    (x,) = _run(backend, Routines.TriangularSolve, [a, b], [b.shape], [F32], {"unitDiagonal": unit})
    _close(x, oracle.triangular_solve(a, b, unit))
    au = np.triu(a).astype(np.float64)
    if unit:
        au = au - au * np.eye(n) + np.eye(n)
    resid = np.einsum("cij,ctj->cti", au, x.astype(np.float64)) - b
    assert np.abs(resid).max() <= 1e-4 * max(1.0, np.abs(x).max())


@pytest.mark.gpu
@pytest.mark.parametrize("batch,m,n", [(1, 2, 2), (4, 30, 30), (3, 7, 12), (3, 12, 7), (2, 129, 200), (1, 512, 512), (1, 1, 5), (1, 5, 1)])
def test_cuda_lu(backend, batch, m, n):
    rng = np.random.default_rng(m * 1000 + n)
    A = rng.uniform(-1, 1, (batch, m, n)).astype(np.float32)
    if m == 2:
        A[0] = [[4, 3], [6, 3]]                               # test/lax-linalg.test.ts:277-290
    r = min(m, n)
    lu, piv, perm = _run(backend, Routines.LU, [A], [A.shape, (batch, r), (batch, m)], [F32, I32, I32])
    wlu, wpiv, wperm = oracle.lu(A)
    assert np.array_equal(piv, wpiv) and np.array_equal(perm, wperm)
    _close(lu, wlu)
    if m == 2:
        np.testing.assert_allclose(lu[0], [[6, 3], [0.6666667, 1.0]], rtol=1e-6)
        assert piv[0].tolist() == [1, 1] and perm[0].tolist() == [1, 0]
    for bi in range(batch):
        L = np.tril(lu[bi].astype(np.float64), -1)[:, :r] + np.eye(m, r)
        U = np.triu(lu[bi].astype(np.float64))[:r]
        np.testing.assert_allclose(A[bi][perm[bi]], L @ U, rtol=1e-4, atol=1e-5 * max(1, r / 30))


@pytest.mark.gpu
def test_cuda_lu_singular_ties_and_float64(backend):
    # a zero column (no elimination for it), equal candidates (the first wins), float64
    A = np.array([[[0, 2, 1], [0, -2, 3], [0, 2, 5]], [[1, 2, 3], [-1, 5, 6], [1, 8, 9]]], np.float32)
    lu, piv, perm = _run(backend, Routines.LU, [A], [A.shape, (2, 3), (2, 3)], [F32, I32, I32])
    wlu, wpiv, wperm = oracle.lu(A)
    assert np.array_equal(piv, wpiv) and np.array_equal(perm, wperm) and np.array_equal(lu, wlu)
    assert piv[1, 0] == 0                                    # |1|, |-1|, |1|: no strictly greater value, row 0 stays
    A64 = np.random.default_rng(9).standard_normal((2, 50, 50))
    lu, piv, perm = _run(backend, Routines.LU, [A64], [A64.shape, (2, 50), (2, 50)], [F64, I32, I32])
    wlu, wpiv, wperm = oracle.lu(A64)
    assert np.array_equal(piv, wpiv) and np.array_equal(perm, wperm)
    _close(lu, wlu, 1e-13)


@pytest.mark.gpu
def test_cuda_linalg_shape_errors(backend):
    # src/routine.ts:305-313, :341-346: the reference throws on these shapes
    t = RoutineType([[2, 3]], [F32], [[2, 3]], [F32])
    with pytest.raises(ValueError, match="cholesky: input must be square"):
        backend.prepare_routine(Routine(Routines.Cholesky, t))
    t = RoutineType([[3]], [F32], [[3]], [F32])
    with pytest.raises(ValueError, match="cholesky: input must be at least 2D"):
        backend.prepare_routine(Routine(Routines.Cholesky, t))
    t = RoutineType([[3, 3], [2, 4]], [F32, F32], [[2, 4]], [F32])
    with pytest.raises(ValueError, match="triangular_solve: incompatible shapes"):
        backend.prepare_routine(Routine(Routines.TriangularSolve, t, {"unitDiagonal": False}))
