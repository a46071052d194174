"""sptorch_ext_matmul_f32_static -- the matmul entry point for callers that cannot let the library allocate
(fixed memory budgets, allocator-free inner loops, an exhausted pool).  Its scratch is a static array inside the
library, so it must give exactly what sptorch_matmul_f32 gives, call after call, while the pool is closed."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run(backend, fn, a, b, m, k, n):
    da, db, do = backend.upload(a), backend.upload(b), backend.alloc(m * n)
    try:
        backend._check(fn(da.handle, db.handle, do.handle, m, k, n), fn.__name__)
        out = do.to_host().reshape(m, n)
        backend.synchronize()
        return out
    finally:
        da.free(); db.free(); do.free()


def test_static_scratch_matmul_matches_pool_matmul_twice_in_a_row(backend):
    lib = backend.lib
    rng = np.random.default_rng(11)
    # two calls in a row with different shapes and data: the second must not see the first one's scratch contents
    for (m, k, n) in [(256, 192, 320), (130, 512, 264)]:
        a = rng.standard_normal((m, k)).astype(np.float32)
        b = rng.standard_normal((k, n)).astype(np.float32)
        ref = _run(backend, lib.sptorch_matmul_f32, a, b, m, k, n)
        da, db, do = backend.upload(a), backend.upload(b), backend.alloc(m * n)
        try:
            # close the pool completely: any allocation inside the call would now fail
            lib.sptorch_ext_set_alloc_budget(1)
            rc = lib.sptorch_ext_matmul_f32_static(da.handle, db.handle, do.handle, m, k, n)
            lib.sptorch_ext_set_alloc_budget(0)
            backend._check(rc, "matmul_f32_static")
            got = do.to_host().reshape(m, n)
            backend.synchronize()
        finally:
            lib.sptorch_ext_set_alloc_budget(0)
            da.free(); db.free(); do.free()
        assert np.array_equal(got, ref)                      # same kernels, same arithmetic: bit-identical
        assert np.abs(got - a.astype(np.float64) @ b.astype(np.float64)).max() <= 2e-3 * np.abs(ref).max()   # TF32 tolerance of the other tests


def test_static_scratch_at_its_size_limit(backend):
    """k * n exactly at the limit of 2,097,152 elements (the whole 8 MiB array in use) on the tensor-core path with the pool
    closed, and four elements past it, which must be refused before anything runs."""
    lib = backend.lib
    rng = np.random.default_rng(12)
    m, k, n = 128, 1024, 2048
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    ref = _run(backend, lib.sptorch_matmul_f32, a, b, m, k, n)
    da, db, do = backend.upload(a), backend.upload(b), backend.alloc(m * n)
    try:
        lib.sptorch_ext_set_alloc_budget(1)
        rc = lib.sptorch_ext_matmul_f32_static(da.handle, db.handle, do.handle, m, k, n)
        lib.sptorch_ext_set_alloc_budget(0)
        backend._check(rc, "matmul_f32_static")
        got = do.to_host().reshape(m, n)
        backend.synchronize()
        assert np.array_equal(got, ref)
        assert np.abs(got - a.astype(np.float64) @ b.astype(np.float64)).max() <= 2e-3 * np.abs(ref).max()
        # four elements past the limit: k * n = 4 * (2^19 + 1) = 2^21 + 4
        assert lib.sptorch_ext_matmul_f32_static(da.handle, db.handle, do.handle, 8, 4, (1 << 19) + 1) != 0
        assert b"static scratch" in lib.sptorch_ext_last_error()
        assert lib.sptorch_sync() != 0 and lib.sptorch_sync() == 0
    finally:
        lib.sptorch_ext_set_alloc_budget(0)
        da.free(); db.free(); do.free()


def test_static_scratch_rejects_oversize_and_handles_small(backend):
    lib = backend.lib
    d = backend.alloc(16)
    try:
        assert lib.sptorch_ext_matmul_f32_static(d.handle, d.handle, d.handle, 4, 2048, 2048) != 0    # k*n = 4 Mi > 2 Mi
        assert b"static scratch" in lib.sptorch_ext_last_error()
        assert lib.sptorch_sync() != 0 and lib.sptorch_sync() == 0
    finally:
        d.free()
    # a shape the tensor-core path does not take (tiny, unaligned) goes through the CUDA-core kernel, still without allocating
    a = np.array([1, 2, 3, 4, 5, 6], dtype=np.float32)
    b = np.array([7, 8, 9, 10, 11, 12], dtype=np.float32)
    out = _run(backend, lib.sptorch_ext_matmul_f32_static, a, b, 2, 3, 2)
    assert out.ravel().tolist() == [58, 64, 139, 154]
