"""The C++ mirror of the trait surface (sptorch_b200/csrc/hal.hpp) driven by a C++ port of the reference's FFI test
(tests/ffi_port.cpp <- crates/hal-ffi/tests/test_ffi_mock.rs).  On CPU it must pass against the reference's own C
backend and must report a clean load failure for libsptorch_b200.so; on a B200 it must pass against our library."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "_build", "ffi_port")
LIB = os.path.join(ROOT, "sptorch_b200", "lib", "libsptorch_b200.so")
MOCK = os.path.join(ROOT, "oracle", "_ref", "libmock_npu.so")


def _build():
    src = os.path.join(ROOT, "tests", "ffi_port.cpp")
    hdr = os.path.join(ROOT, "sptorch_b200", "csrc", "hal.hpp")
    if not os.path.exists(EXE) or os.path.getmtime(EXE) < max(os.path.getmtime(src), os.path.getmtime(hdr)):
        os.makedirs(os.path.dirname(EXE), exist_ok=True)
        gxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
        subprocess.run([gxx, "-std=c++17", "-O1", "-o", EXE, src, "-ldl"], check=True)
    return EXE


def test_cpp_kv_cache_metadata():
    """KvCacheBufferSpec / KvCacheWindowState of the C++ mirror against the reference's tests (crates/hal/src/lib.rs:674-721)."""
    r = subprocess.run([_build(), "--metadata"], capture_output=True, text=True)
    assert r.returncode == 0 and "OK" in r.stdout, r.stdout + r.stderr


@pytest.mark.skipif(not os.path.exists(MOCK), reason="reference C backend not built")
def test_cpp_port_passes_on_reference_backend():
    r = subprocess.run([_build(), MOCK, "mock_npu"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr


def test_cpp_port_fails_loudly_without_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    r = subprocess.run([_build(), LIB], capture_output=True, text=True)
    assert r.returncode == 3 and "LOAD_FAILED" in r.stdout and "init failed" in r.stdout


@pytest.mark.gpu
def test_cpp_port_passes_on_b200():
    exe = EXE if os.path.exists(EXE) else _build()
    r = subprocess.run([exe, LIB, "sptorch_b200"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
