"""Helpers shared by the parity tests: run one Kernel through the cuda backend and through the
oracle on the same arrays."""
import numpy as np

import oracle
from jax_js_b200 import DType, np_dtype


def run_cuda(backend, kernel, args, keep=False):
    slots = [backend.put(np.ascontiguousarray(a)) for a in args]
    out = backend.malloc(kernel.bytes)
    try:
        exe = backend.prepare_kernel_sync(kernel)
        backend.dispatch(exe, slots, [out])
        res = backend.read_sync(out).view(np_dtype(kernel.dtype)).copy()
    finally:
        for s in slots:
            backend.dec_ref(s)
        backend.dec_ref(out)
    return (res, exe) if keep else res


def assert_same_bits(got, want, what=""):
    """Bit-exact, except that any NaN matches any NaN."""
    got, want = np.asarray(got), np.asarray(want)
    assert got.shape == want.shape, what
    if got.dtype.kind == "f":
        nan = np.isnan(want)
        assert (np.isnan(got) == nan).all(), f"{what}: NaN pattern differs"
        ib = {2: np.uint16, 4: np.uint32, 8: np.uint64}[got.dtype.itemsize]
        assert (got.view(ib)[~nan] == want.view(ib)[~nan]).all(), f"{what}: bits differ"
    else:
        assert (got == want).all(), f"{what}: values differ"


def assert_close(got, want, rtol, scale=None, what=""):
    """|got - want| <= rtol * max(|want|, scale) elementwise; NaN/Inf patterns must agree.

    `scale` is the magnitude the tolerance is relative to where the result itself can be
    arbitrarily small through cancellation (for a sum: the sum of absolute terms).
    """
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, what
    assert (np.isnan(got) == np.isnan(want)).all(), f"{what}: NaN pattern differs"
    inf = np.isinf(want)
    assert (got[inf] == want[inf]).all(), f"{what}: infinities differ"
    ok = ~(np.isnan(want) | inf)
    ref = np.abs(want)
    if scale is not None:
        ref = np.maximum(ref, np.broadcast_to(np.asarray(scale, dtype=np.float64), want.shape))
    err = np.abs(got - want)[ok]
    bound = rtol * ref[ok]
    bad = err > bound + 1e-38
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} beyond rtol={rtol}; worst ratio {np.max(err / np.maximum(bound, 1e-300)):.3g}"
