"""The sort entry point that allocates nothing (`jaxcuda_sort_no_alloc`), called through the C ABI.

Collected last on purpose.  It must give the same bits as the Sort routine dispatched the usual
way, on two calls in a row that share its built-in work buffer (the second with other data and
another row length, so that what the first call left behind is seen not to matter), and it must
refuse inputs larger than that buffer instead of allocating."""
import numpy as np
import pytest

from jax_js_b200 import DType
from jax_js_b200.routine import Routine, Routines, RoutineType

from util import assert_same_bits

pytestmark = pytest.mark.gpu


def _sort_by_dispatch(backend, x):
    t = RoutineType([list(x.shape)], [DType.Float32], [list(x.shape)], [DType.Float32])
    exe = backend.prepare_routine(Routine(Routines.Sort, t))
    sx, so = backend.put(x), backend.malloc(x.nbytes)
    backend.dispatch(exe, [sx], [so])
    out = backend.read_sync(so).view(np.float32).reshape(x.shape)
    backend.dec_ref(sx)
    backend.dec_ref(so)
    return out


def test_no_alloc_sort_matches_dispatched_sort_twice_in_a_row(backend):
    rng = np.random.default_rng(7)
    cases = [rng.standard_normal((3, 100000)).astype(np.float32),     # pads to 3 x 131072 keys: uses the static buffer
             rng.standard_normal((5, 40001)).astype(np.float32) * 1e3]  # other shape, other data, same buffer
    for x in cases:
        x.flat[::101] = np.nan
        x.flat[1::103] = -0.0
        x.flat[2::107] = 0.0
        x.flat[3::109] = np.inf
    for x in cases:   # two calls in a row on the shared buffer
        sx, sy = backend.put(x), backend.malloc(x.nbytes)
        backend.sort_no_alloc(DType.Float32, sx, sy, x.shape[0], x.shape[1])
        got = backend.read_sync(sy).view(np.float32).reshape(x.shape)
        backend.dec_ref(sx)
        backend.dec_ref(sy)
        assert_same_bits(got, _sort_by_dispatch(backend, x), "sort_no_alloc vs dispatch")   # compare-only: bit-exact
    small = rng.standard_normal((64, 1000)).astype(np.float32)         # rows that fit shared memory skip the buffer
    sx, sy = backend.put(small), backend.malloc(small.nbytes)
    backend.sort_no_alloc(DType.Float32, sx, sy, 64, 1000)
    assert_same_bits(backend.read_sync(sy).view(np.float32).reshape(small.shape), np.sort(small, axis=1))
    backend.dec_ref(sx)
    backend.dec_ref(sy)


def test_no_alloc_sort_rejects_what_does_not_fit(backend):
    s = backend.malloc(16)
    with pytest.raises(ValueError, match="static work buffer holds"):
        backend.sort_no_alloc(DType.Float32, s, s, 64, 100000)          # 64 x 131072 keys > 4 Mi
    with pytest.raises(Exception, match="float64"):
        backend.sort_no_alloc(DType.Float64, s, s, 1, 100000)
    backend.dec_ref(s)
