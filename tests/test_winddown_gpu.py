"""The tensor-core GEMM's bounded waits: a pipeline stage that never arrives makes the waiting role give
up after its poll limit, the kernel winds down (copies landed, tensor memory freed) and the next
read reports which role gave up; the context stays usable.  The missing stage is arranged on the host
side (an option of a second context makes one CTA's producer announce a stage and not load it) and
every wait is bounded, so nothing hangs or traps."""
import os

import numpy as np
import pytest

import oracle
from jax_js_b200 import DType
from jax_js_b200 import programs as P
from jax_js_b200.backend import CudaBackend, CudaError

from util import assert_close, run_cuda

pytestmark = pytest.mark.gpu


def test_a_stage_that_never_arrives_is_reported_and_the_context_survives(backend):
    n = 256
    rng = np.random.default_rng(0)
    a = (rng.standard_normal((n, 512)) * 0.1).astype(np.float16)
    b = (rng.standard_normal((512, n)) * 0.1).astype(np.float16)
    k = P.dot_kernel(n, n, 512, DType.Float16)
    env = {"JAXCUDA_TC_FAULT": "1", "JAXCUDA_TC_SPIN_LIMIT": "4096", "JAXCUDA_TC_STREAMK": "0"}
    old = {key: os.environ.get(key) for key in env}
    os.environ.update(env)
    try:
        faulty = CudaBackend(backend.device)
    finally:
        for key, v in old.items():
            if v is None:
                os.environ.pop(key, None)
            else:
                os.environ[key] = v
    try:
        assert faulty.prepare_kernel(k).describe.startswith("gemm-tcgen05")
        sa, sb, sc = faulty.put(a), faulty.put(b), faulty.malloc(k.bytes)
        faulty.dispatch(faulty.prepare_kernel(k), [sa, sb], [sc])
        with pytest.raises(CudaError, match=r"pipeline wait timed out \(role [1-4]"):
            faulty.read_sync(sc)
        # the status word is cleared by the report: the same context goes on working (elementwise here,
        # since every GEMM this context compiles carries the injected fault)
        x = rng.standard_normal(4096).astype(np.float32)
        sx = faulty.put(x)
        assert np.array_equal(faulty.read_sync(sx).view(np.float32), x)
        for s in (sa, sb, sc, sx):
            faulty.dec_ref(s)
    finally:
        faulty.close()
    # and the session's own context, on the same GPU, runs the same GEMM correctly afterwards
    got = run_cuda(backend, k, [a, b]).astype(np.float64)
    want = oracle.run_kernel(k, [a, b], fma=True).astype(np.float64)
    assert_close(got / 512, want / 512, 2e-3, 0.1 * 0.1 * 9, "gemm after the wind-down")


def test_a_missing_stage_winds_down_a_cta_pair_too(backend):
    """The same on the paired kernel (two CTAs of a cluster on one tile): the even CTA's MMA role gives
    up on the stage that was announced and never loaded, both CTAs of every pair leave their loops,
    meet at the cluster barrier and free their tensor memory; the error names the role and the next
    GEMM on the ordinary context is correct."""
    m = n = 2304
    kk = 192
    rng = np.random.default_rng(1)
    a = (rng.standard_normal((m, kk)) * 0.1).astype(np.float16)
    b = (rng.standard_normal((kk, n)) * 0.1).astype(np.float16)
    k = P.dot_kernel(m, n, kk, DType.Float16)
    env = {"JAXCUDA_TC_FAULT": "1", "JAXCUDA_TC_SPIN_LIMIT": "4096", "JAXCUDA_TC_PAIR": "2"}
    old = {key: os.environ.get(key) for key in env}
    os.environ.update(env)
    try:
        faulty = CudaBackend(backend.device)
    finally:
        for key, v in old.items():
            if v is None:
                os.environ.pop(key, None)
            else:
                os.environ[key] = v
    try:
        assert "cta-pairs" in faulty.prepare_kernel(k).describe
        sa, sb, sc = faulty.put(a), faulty.put(b), faulty.malloc(k.bytes)
        faulty.dispatch(faulty.prepare_kernel(k), [sa, sb], [sc])
        with pytest.raises(CudaError, match=r"pipeline wait timed out \(role [1-4]"):
            faulty.read_sync(sc)
        x = rng.standard_normal(4096).astype(np.float32)
        sx = faulty.put(x)
        assert np.array_equal(faulty.read_sync(sx).view(np.float32), x)
        for s_ in (sa, sb, sc, sx):
            faulty.dec_ref(s_)
    finally:
        faulty.close()
    got = run_cuda(backend, k, [a, b]).astype(np.float64).reshape(m, n)
    want = a.astype(np.float64) @ b.astype(np.float64)
    assert_close(got / kk, want / kk, 2e-3, 0.01, "gemm after the wind-down of a pair")
