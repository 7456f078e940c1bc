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


def test_oracle_routines_against_lapack_in_float64():
    """The restatements against independent implementations (LAPACK through numpy / scipy) in float64:
    same pivoting rule as getrf (largest magnitude, first occurrence), same factors to rounding."""
    import scipy.linalg as sl
    rng = np.random.default_rng(21)
    a = rng.standard_normal((60, 60))
    lu, piv, perm = oracle.lu(a)
    ref_lu, ref_piv = sl.lu_factor(a)
    assert np.array_equal(piv, ref_piv)
    np.testing.assert_allclose(lu, ref_lu, rtol=1e-10, atol=1e-12)
    x = _spd(rng, 3, 40, np.float64)
    np.testing.assert_allclose(oracle.cholesky(x), np.linalg.cholesky(x), rtol=1e-12, atol=1e-13)
    u = np.triu(rng.standard_normal((50, 50))) + 8 * np.eye(50)
    b = rng.standard_normal((7, 50))
    np.testing.assert_allclose(oracle.triangular_solve(u, b), sl.solve_triangular(u, b.T).T, rtol=1e-11, atol=1e-12)
    np.testing.assert_allclose(oracle.triangular_solve(u, b, unit_diagonal=True),
                               sl.solve_triangular(u, b.T, unit_diagonal=True).T, rtol=1e-9, atol=1e-9)
    s = _sym(rng, 2, 24, np.float64)
    d, v = oracle.jacobi_eigh(s, max_sweeps=48, tolerance=1e-12)
    full = np.tril(s) + np.tril(s, -1).transpose(0, 2, 1)
    np.testing.assert_allclose(np.sort(np.diagonal(d, axis1=1, axis2=2)), np.linalg.eigvalsh(full), rtol=1e-9, atol=1e-9)
    np.testing.assert_allclose(v.transpose(0, 2, 1) @ v, np.broadcast_to(np.eye(24), (2, 24, 24)), atol=1e-10)


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
@pytest.mark.parametrize("batch,n", [(1, 1), (1, 2), (5, 3), (3, 33), (2, 130), (2, 255), (1, 256), (3, 300), (1, 512), (1, 1500)])   # 256 and up: blocked over many CTAs
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
    for n in (40, 321):
        x = _spd(np.random.default_rng(3), 2, n, np.float64)
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


# ---- JacobiEigh and Fft ----------------------------------------------------------------------------

def _sym(rng, batch, n, dtype=np.float32):
    a = rng.standard_normal((batch, n, n))
    return ((a + a.transpose(0, 2, 1)) / 2).astype(dtype)


def _eigh_params(n, dtype=np.float32):
    # src/library/lax-linalg.ts:78-79
    return {"maxSweeps": max(8, 2 * n), "tolerance": 1e-12 if dtype == np.float64 else 1e-6}


def factor_fft_size(n):
    """`factorFftSize` (src/library/numpy-fft.ts:50-66): radices 4, 2, 3, 5, 7, then odd trial division."""
    f = []
    for radix in (4, 2, 3, 5, 7):
        while n % radix == 0:
            f.append(radix)
            n //= radix
    radix = 11
    while radix * radix <= n:
        while n % radix == 0:
            f.append(radix)
            n //= radix
        radix += 2
    if n > 1:
        f.append(n)
    return f


def test_oracle_jacobi_eigh_reference_cases():
    # test/lax-linalg.test.ts:153-165: a diagonal matrix is left alone (values 3, 1, 2; vectors = identity)
    x = np.diag([3.0, 1.0, 2.0]).astype(np.float32)
    a, v = oracle.jacobi_eigh(x, **{"max_sweeps": 8, "tolerance": 1e-6})
    assert np.array_equal(np.diag(a), [3, 1, 2]) and np.array_equal(v, np.eye(3))
    # :167-183: V diag(values) V^T reconstructs x and V is orthogonal, rtol = atol = 1e-3
    x = np.array([[4.0, 1.0, 2.0], [1.0, 3.0, 0.5], [2.0, 0.5, 5.0]], np.float32)
    a, v = oracle.jacobi_eigh(x, 8, 1e-6)
    np.testing.assert_allclose(v @ np.diag(np.diag(a)) @ v.T, x, rtol=1e-3, atol=1e-3)
    np.testing.assert_allclose(v.T @ v, np.eye(3), rtol=1e-3, atol=1e-3)
    # :185-203: batched [[2,1],[1,2]] and [[3,1],[1,3]]: eigenvalues {1, 3} and {2, 4}
    xb = np.array([[[2.0, 1.0], [1.0, 2.0]], [[3.0, 1.0], [1.0, 3.0]]], np.float32)
    a, v = oracle.jacobi_eigh(xb, 8, 1e-6)
    np.testing.assert_allclose(np.sort(np.diagonal(a, axis1=1, axis2=2)), [[1, 3], [2, 4]], rtol=1e-5)


def test_oracle_fft_reference_vectors_and_numpy():
    # test/numpy-fft.test.ts:91-96 and :170-174
    r, i = oracle.fft(np.array([6, -2, -2, -2], np.float32), np.array([0, 2, 0, -2], np.float32), factor_fft_size(4), inverse=True)
    np.testing.assert_allclose(r, [0, 1, 2, 3], atol=1e-6)
    np.testing.assert_allclose(i, [0, 0, 0, 0], atol=1e-6)
    r, i = oracle.fft(np.array([0, 1, 2, 3], np.float32), np.zeros(4, np.float32), factor_fft_size(4))
    np.testing.assert_allclose(r, [6, -2, -2, -2], atol=1e-5)
    np.testing.assert_allclose(i, [0, 2, 0, -2], atol=1e-5)
    rng = np.random.default_rng(2)
    for n in (1, 2, 3, 8, 12, 30, 49, 97, 128, 360, 1001):
        z = rng.standard_normal((3, n)) + 1j * rng.standard_normal((3, n))
        for inverse in (False, True):
            r, i = oracle.fft(z.real.astype(np.float32), z.imag.astype(np.float32), factor_fft_size(n), inverse)
            want = np.fft.ifft(z) if inverse else np.fft.fft(z)
            np.testing.assert_allclose(r + 1j * i, want, atol=2e-6 * np.abs(want).max() * max(1, np.log2(n)))


@pytest.mark.gpu
@pytest.mark.parametrize("batch,n", [(1, 1), (2, 2), (3, 3), (4, 17), (2, 64), (1, 150), (1, 200)])
def test_cuda_jacobi_eigh(backend, batch, n):
    x = _sym(np.random.default_rng(n), batch, n)
    x[:, np.triu_indices(n, 1)[0], np.triu_indices(n, 1)[1]] = 99.0      # only the lower triangle is read
    p = _eigh_params(n)
    a, v = _run(backend, Routines.JacobiEigh, [x], [x.shape, x.shape], [F32, F32], p)
    wa, wv = oracle.jacobi_eigh(x, p["maxSweeps"], p["tolerance"])
    # the same rotations in the same order with the same arithmetic: bit-identical
    assert np.array_equal(a, wa) and np.array_equal(v, wv)
    xs = np.tril(x) + np.tril(x, -1).transpose(0, 2, 1)
    vals = np.diagonal(a, axis1=1, axis2=2).astype(np.float64)
    vd = v.astype(np.float64)
    np.testing.assert_allclose(np.einsum("bij,bj,bkj->bik", vd, vals, vd), xs, rtol=1e-3, atol=1e-3 * max(1, np.sqrt(n) / 4))
    np.testing.assert_allclose(np.sort(vals), np.linalg.eigvalsh(xs.astype(np.float64)), rtol=1e-4, atol=1e-4 * np.sqrt(n))


@pytest.mark.gpu
def test_cuda_jacobi_eigh_float64_and_diagonal_input(backend):
    x = _sym(np.random.default_rng(4), 2, 12, np.float64)
    p = _eigh_params(12, np.float64)
    a, v = _run(backend, Routines.JacobiEigh, [x], [x.shape, x.shape], [F64, F64], p)
    wa, wv = oracle.jacobi_eigh(x, p["maxSweeps"], p["tolerance"])
    assert np.array_equal(a, wa) and np.array_equal(v, wv)
    d = np.diag([3.0, 1.0, 2.0]).astype(np.float32)[None]              # test/lax-linalg.test.ts:153-165
    a, v = _run(backend, Routines.JacobiEigh, [d], [d.shape, d.shape], [F32, F32], _eigh_params(3))
    assert np.array_equal(np.diag(a[0]), [3, 1, 2]) and np.array_equal(v[0], np.eye(3))


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1, 2, 3, 4, 8, 12, 30, 49, 97, 128, 360, 1001, 4096, 8192, 30030, 65536])   # from 8192 on a row exceeds shared memory
@pytest.mark.parametrize("inverse", [False, True])
def test_cuda_fft(backend, n, inverse):
    rng = np.random.default_rng(n)
    batch = 5 if n < 1000 else 2
    re, im = rng.standard_normal((batch, n)).astype(np.float32), rng.standard_normal((batch, n)).astype(np.float32)
    if n == 4:
        re[0], im[0] = ([6, -2, -2, -2], [0, 2, 0, -2]) if inverse else ([0, 1, 2, 3], [0, 0, 0, 0])
    f = factor_fft_size(n)
    r, i = _run(backend, Routines.Fft, [re, im], [re.shape, im.shape], [F32, F32], {"factors": f, "inverse": inverse})
    wr, wi = oracle.fft(re, im, f, inverse)
    scale = max(np.abs(wr).max(), np.abs(wi).max())
    # same arithmetic and stage rounding; the twiddles come from a table (one rounding apart from the reference's)
    assert np.abs(r - wr).max() <= 2e-6 * scale and np.abs(i - wi).max() <= 2e-6 * scale
    want = (np.fft.ifft if inverse else np.fft.fft)(re.astype(np.float64) + 1j * im.astype(np.float64))
    np.testing.assert_allclose(r + 1j * i, want, atol=3e-6 * np.abs(want).max() * max(1, np.log2(n)))
    if n == 4:      # test/numpy-fft.test.ts:91-96, :170-174
        np.testing.assert_allclose(r[0], [0, 1, 2, 3] if inverse else [6, -2, -2, -2], atol=1e-5)
        np.testing.assert_allclose(i[0], [0, 0, 0, 0] if inverse else [0, 2, 0, -2], atol=1e-5)


@pytest.mark.gpu
def test_cuda_fft_float64_and_bad_factors(backend):
    rng = np.random.default_rng(11)
    re, im = rng.standard_normal((3, 60)), rng.standard_normal((3, 60))
    r, i = _run(backend, Routines.Fft, [re, im], [re.shape, im.shape], [F64, F64], {"factors": factor_fft_size(60), "inverse": False})
    np.testing.assert_allclose(r + 1j * i, np.fft.fft(re + 1j * im), atol=1e-12)
    re, im = rng.standard_normal((2, 6000)), rng.standard_normal((2, 6000))      # float64 rows beyond shared memory
    r, i = _run(backend, Routines.Fft, [re, im], [re.shape, im.shape], [F64, F64], {"factors": factor_fft_size(6000), "inverse": True})
    np.testing.assert_allclose(r + 1j * i, np.fft.ifft(re + 1j * im), atol=1e-13)
    t = RoutineType([[8], [8]], [F32, F32], [[8], [8]], [F32, F32])
    with pytest.raises(ValueError, match="fft: factors do not multiply"):
        backend.prepare_routine(Routine(Routines.Fft, t, {"factors": [2, 2], "inverse": False}))


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


@pytest.mark.gpu
def test_cuda_routine_size_limits_are_reported_at_prepare(backend):
    """Sizes beyond what the routine kernels hold fail when the routine is prepared, with the limit
    in the message, not at the first dispatch."""
    from jax_js_b200.backend import UnsupportedOpError
    n = 30000
    t = RoutineType([[n, n], [1, n]], [F32, F32], [[1, n]], [F32])
    with pytest.raises(UnsupportedOpError, match="TriangularSolve: n = 30000 exceeds 25600"):
        backend.prepare_routine(Routine(Routines.TriangularSolve, t, {"unitDiagonal": False}))
    n = 40000
    t = RoutineType([[n, n]], [F32], [[n, n], [n, n]], [F32, F32])
    with pytest.raises(UnsupportedOpError, match="JacobiEigh: n = 40000 exceeds 32768"):
        backend.prepare_routine(Routine(Routines.JacobiEigh, t, {"maxSweeps": 10, "tolerance": 1e-6}))
    t = RoutineType([[70000, 256, 256]], [F32], [[70000, 256, 256]], [F32])
    with pytest.raises(UnsupportedOpError, match="batches of at most 65535"):
        backend.prepare_routine(Routine(Routines.Cholesky, t))
