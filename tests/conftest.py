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
    be.close()
