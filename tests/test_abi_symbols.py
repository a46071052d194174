"""CPU-side checks of the drop-in boundary: the library exists, exports every symbol that include/*.h
declares, and refuses to run without a B200 instead of falling back to the CPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sptorch_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from sptorch_b200 import _lib
    assert os.path.exists(_lib.LIB_PATH), "build the library first: python -m sptorch_b200.build"
    lib = ctypes.CDLL(_lib.LIB_PATH)
    hal = _declared("sptorch_b200_hal.h")
    ext = [s for s in _declared("sptorch_b200_ext.h") if s != "sptorch_allreduce_fn"]
    assert len(hal) == 20, hal      # the reference's contract: crates/hal-ffi/include/sptorch_hal.h:21-85
    for name in hal + ext:
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"
    # and the Python binding table covers exactly the declared set
    assert sorted(_lib.HAL_SYMBOLS) == hal
    assert sorted(_lib.EXT_SYMBOLS) == sorted(ext)


def test_reference_loader_symbol_names():
    # the 19 required + 1 optional names FfiBackend::load resolves (crates/hal-ffi/src/lib.rs:180-208)
    from sptorch_b200 import _lib
    required = ["sptorch_backend_init", "sptorch_backend_shutdown", "sptorch_backend_name", "sptorch_alloc", "sptorch_free",
                "sptorch_copy_h2d", "sptorch_copy_d2h", "sptorch_sync", "sptorch_add_f32", "sptorch_mul_f32", "sptorch_neg_f32",
                "sptorch_exp_f32", "sptorch_log_f32", "sptorch_relu_f32", "sptorch_gelu_f32", "sptorch_scale_f32",
                "sptorch_matmul_f32", "sptorch_batch_matmul_f32", "sptorch_softmax_f32"]
    for name in required + ["sptorch_query_runtime"]:
        assert name in _lib.HAL_SYMBOLS


def test_no_cpu_fallback_without_a_gpu():
    """On a host without a usable B200 every entry point must fail loudly; nothing may compute on the CPU."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present: covered by the gpu tests")
    from sptorch_b200 import _lib
    from sptorch_b200.backend import FfiBackend, HalError
    lib = _lib.load()
    assert lib.sptorch_backend_name() == b"sptorch_b200"
    with pytest.raises(HalError):
        FfiBackend.load()
    assert lib.sptorch_alloc(16) is None
    assert lib.sptorch_sync() != 0
    assert lib.sptorch_add_f32(None, None, None, 4) != 0
    assert b"not initialised" in lib.sptorch_ext_last_error()


def test_product_never_imports_the_oracle():
    """Nothing under sptorch_b200/ may import, link, load or include the CPU oracle."""
    pkg = os.path.join(ROOT, "sptorch_b200")
    pat = re.compile(r"from\s+oracle|import\s+oracle|liboracle|oracle/|oracle\.h|orc_\w+\(")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".hpp", ".cpp")):
                text = open(os.path.join(dirpath, f), errors="replace").read()
                m = pat.search(text)
                assert m is None, f"{f} references the oracle: {m.group(0)!r}"
