"""Sort / Argsort routines against the reference's vectors (test/numpy.test.ts:4631-4801) and
against the oracle's restatement of src/routine.ts:185-214.  Compare-only: bit-exact."""
import numpy as np
import pytest

import oracle
from jax_js_b200 import DType, np_dtype
from jax_js_b200.routine import Routine, Routines, RoutineType

from util import assert_same_bits

pytestmark = pytest.mark.gpu
F32, I32, U32, BOOL, F16, F64 = DType.Float32, DType.Int32, DType.Uint32, DType.Bool, DType.Float16, DType.Float64


def cuda_sort(backend, x, dtype, arg=False):
    x = np.ascontiguousarray(x)
    shp = list(x.shape)
    t = RoutineType([shp], [dtype], [shp, shp] if arg else [shp], [dtype, I32] if arg else [dtype])
    exe = backend.prepare_routine(Routine(Routines.Argsort if arg else Routines.Sort, t))
    sx = backend.put(x)
    outs = [backend.malloc(x.nbytes)] + ([backend.malloc(x.size * 4)] if arg else [])
    try:
        backend.dispatch(exe, [sx], outs)
        res = [backend.read_sync(outs[0]).view(x.dtype).reshape(x.shape)]
        if arg:
            res.append(backend.read_sync(outs[1]).view(np.int32).reshape(x.shape))
    finally:
        for s in [sx] + outs:
            backend.dec_ref(s)
    return res if arg else res[0]


def test_reference_sort_vectors(backend):
    f = lambda *v: np.array(v, np.float32)
    assert cuda_sort(backend, f(3, 1, 4, 1, 5, 9, 2, 6), F32).tolist() == [1, 1, 2, 3, 4, 5, 6, 9]
    assert cuda_sort(backend, np.array([[3, 1, 2], [6, 4, 5]], np.float32), F32).tolist() == [[1, 2, 3], [4, 5, 6]]
    out = cuda_sort(backend, f(3, np.nan, 1, np.nan, 2), F32)
    assert out[:3].tolist() == [1, 2, 3] and np.isnan(out[3:]).all()
    assert cuda_sort(backend, np.array([3, 1, 4, 1, 5], np.int32), I32).tolist() == [1, 1, 3, 4, 5]
    assert cuda_sort(backend, np.array([3, 1, 4, 1, 5], np.uint32), U32).tolist() == [1, 1, 3, 4, 5]
    assert cuda_sort(backend, np.array([1, 0, 1, 0, 1], np.int32), BOOL).tolist() == [0, 0, 1, 1, 1]
    x = np.linspace(0, 1, 8192, dtype=np.float32)
    np.testing.assert_array_equal(cuda_sort(backend, x[::-1].copy(), F32), x)
    assert cuda_sort(backend, np.zeros((3, 0), np.float32), F32).shape == (3, 0)


def test_reference_argsort_vectors(backend):
    f = lambda *v: np.array(v, np.float32)
    assert cuda_sort(backend, f(3, 1, 4, 2, 5), F32, arg=True)[1].tolist() == [1, 3, 0, 2, 4]
    x = f(3, 1, 1, np.nan, np.inf, 2, np.nan, 1, 0, -0.0, np.inf)
    vals, idx = cuda_sort(backend, x, F32, arg=True)
    assert idx.tolist() == [8, 9, 1, 2, 7, 5, 0, 4, 10, 3, 6]
    assert_same_bits(vals, x[idx])
    big = np.linspace(0, 1, 8191, dtype=np.float32)[::-1].copy()
    assert cuda_sort(backend, big, F32, arg=True)[1].tolist() == list(range(8190, -1, -1))


@pytest.mark.parametrize("shape", [(1, 1), (7, 2), (5, 1000), (128, 1024), (3, 16384), (2, 40000), (1, 300001)])
@pytest.mark.parametrize("dtype", [F32, I32, U32, F16, F64])
def test_sort_and_argsort_match_oracle(backend, shape, dtype):
    rng = np.random.default_rng(shape[1] + int(dtype))
    if dtype in (F32, F16, F64):   # float64 sorts on 64-bit keys (rows beyond 16384 / 8192 items take the multi-pass path)
        x = rng.standard_normal(shape).astype(np_dtype(dtype))
        x.flat[::97] = np.nan
        x.flat[1::89] = 0.0
        x.flat[2::83] = -0.0
        x.flat[3::79] = np.inf
        x.flat[4::71] = 0.5   # duplicates
    else:
        x = rng.integers(-2**31 if dtype == I32 else 0, 2**31, shape).astype(np.int64).astype(np_dtype(dtype))
        x.flat[::3] = x.flat[0]
    assert_same_bits(cuda_sort(backend, x, dtype), oracle.sort(x, dtype), "sort")
    vals, idx = cuda_sort(backend, x, dtype, arg=True)
    wv, wi = oracle.argsort(x, dtype)
    assert (idx == wi).all(), "argsort indices"
    assert_same_bits(vals, wv, "argsort values")


def test_sort_bench_shape_is_sorted_permutation(backend):
    # bench/sort.bench.ts:15-40 sorts [32768, 1024]; checked through properties, not the oracle
    x = np.random.default_rng(0).standard_normal((32768, 1024)).astype(np.float32)
    y = cuda_sort(backend, x, F32)
    assert (np.diff(y, axis=1) >= 0).all()
    assert np.array_equal(np.sort(x, axis=1), y)
