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
    """max |a - ref| / max |ref|  (per tensor): the error measure the tolerances 2e-3 (TF32) / 2e-2 (bf16) are stated in."""
    import numpy as np
    a = np.asarray(a, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(a - ref).max() / max(np.abs(ref).max(), 1e-30))


def elementwise_excess(a, ref, tol):
    """The elementwise criterion beside relerr: |a - ref| <= atol + rtol * |ref| with rtol = tol and atol = 2 * tol * rms(ref),
    so that one large entry of ref cannot hide a relative error on the rest of the tensor (the absolute part is tied to the
    root mean square of the reference, which a single outlier does not move, not to its maximum; for these tensors the RMS is
    four to five times smaller than the maximum that relerr divides by).  Returns (fraction of elements outside the bound,
    largest |a - ref| / (atol + rtol |ref|)); a tensor passes when the second number is <= 1."""
    import numpy as np
    a = np.asarray(a, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    rms = float(np.sqrt(np.mean(ref * ref)))
    bound = tol * (2.0 * rms + np.abs(ref))
    ratio = np.abs(a - ref) / np.maximum(bound, 1e-300)
    return float((ratio > 1.0).mean()), float(ratio.max())


_PARITY_LINES = []


def parity_record(name, **figures):
    """Keeps a parity figure (max relative error, raw argmax agreement, ...) for the summary printed after the test run."""
    _PARITY_LINES.append((name, figures))


def pytest_terminal_summary(terminalreporter):
    if not _PARITY_LINES:
        return
    terminalreporter.write_sep("-", "parity figures (CUDA path against the CPU oracle)")
    for name, figures in _PARITY_LINES:
        terminalreporter.write_line(name + ": " + ", ".join(f"{k}={v:.4g}" if isinstance(v, float) else f"{k}={v}" for k, v in figures.items()))
