import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; runs through the C ABI of libjaxcuda.so")


@pytest.fixture(scope="session")
def lib():
    """The built C-ABI library (compiled on first use; no GPU needed to load it)."""
    from jax_js_b200 import build
    build.build()
    from jax_js_b200.backend import load_library
    return load_library()


@pytest.fixture(scope="session")
def backend(lib):
    """One cuda backend for the whole GPU session.  Fails loudly without a GPU."""
    from jax_js_b200.backend import CudaBackend
    be = CudaBackend(int(os.environ.get("JAXCUDA_DEVICE", "0")))
    yield be
    # A session run with JAXCUDA_CHECKED=1 is the memory check of the whole suite: no load whose range
    # the planner had proven may have fallen outside its buffer in any test.
    if os.environ.get("JAXCUDA_CHECKED", "0") not in ("", "0"):
        allowed, proven = be.checked_counts()
        print(f"\nchecked build: {allowed} loads outside their buffers by the Kernels' own indices, {proven} outside a proven range")
        assert proven == 0
    be.close()
