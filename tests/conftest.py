import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with -m gpu on the GPU box")


@pytest.fixture(scope="session")
def backend():
    """The CUDA backend loaded through the C-ABI.  No skip and no fallback: a gpu-marked test
    fails loudly when the library or the device is missing."""
    from sptorch_b200.backend import FfiBackend
    b = FfiBackend.load()
    yield b
    b.synchronize()
    b.close()


@pytest.fixture(scope="session")
def oracle():
    from oracle import binding
    binding.build()
    return binding


def relerr(a, ref):
    """max |a - ref| / max |ref|  (per tensor)."""
    import numpy as np
    a = np.asarray(a, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(a - ref).max() / max(np.abs(ref).max(), 1e-30))
