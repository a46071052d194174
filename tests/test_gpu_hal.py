"""GPU parity tests of the 20-symbol C-ABI: a port of the reference's own FFI tests
(crates/hal-ffi/tests/test_ffi_mock.rs:48-157) run against libsptorch_b200.so, then each op against the
CPU oracle and the golden vectors produced by the reference's C implementation."""
import ctypes as C
import os

import numpy as np
import pytest

from conftest import relerr

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


# ---- port of test_ffi_mock.rs ----
def test_ffi_backend_name(backend):
    assert backend.name() == "sptorch_b200"


def test_ffi_add(backend):
    assert backend.add_f32([1, 2, 3], [4, 5, 6]).tolist() == [5, 7, 9]


def test_ffi_mul(backend):
    assert backend.mul_f32([2, 3], [4, 5]).tolist() == [8, 15]


def test_ffi_neg(backend):
    assert backend.neg_f32([1, -2, 3]).tolist() == [-1, 2, -3]


def test_ffi_scale(backend):
    assert backend.scale_f32([1, 2, 3], 0.5).tolist() == [0.5, 1.0, 1.5]


def test_ffi_relu(backend):
    assert backend.relu_f32([-1, 0, 2, -0.5]).tolist() == [0, 0, 2, 0]


def test_ffi_matmul(backend):
    out = backend.matmul_f32([1, 2, 3, 4, 5, 6], [7, 8, 9, 10, 11, 12], 2, 3, 2)
    assert out.ravel().tolist() == [58, 64, 139, 154]


def test_ffi_softmax(backend):
    out = backend.softmax_f32([1, 2, 3], 1, 3).ravel()
    assert abs(out.sum() - 1) < 1e-6 and out[2] > out[1] > out[0]


def test_ffi_upload_download(backend):
    data = np.array([1, 2, 3, 4], dtype=np.float32)
    buf = backend.upload(data)
    assert np.array_equal(buf.to_host(), data)
    buf.free()


def test_ffi_exp_log_roundtrip(backend):
    a = np.array([0, 1, 2], dtype=np.float32)
    assert np.abs(backend.log_f32(backend.exp_f32(a)) - a).max() < 1e-5


def test_ffi_query_runtime_optional_hook(backend):
    backend.synchronize()
    depth, online = backend.query_runtime()
    assert depth == 0 and online


# ---- KernelProvider KATs (crates/hal/src/lib.rs:724-891) ----
def test_batch_matmul_kat(backend):
    x = np.arange(1, 9, dtype=np.float32)
    ident = np.array([1, 0, 0, 1, 1, 0, 0, 1], dtype=np.float32)
    assert np.array_equal(backend.batch_matmul_f32(x, ident, 2, 2, 2, 2).ravel(), x)


def test_gelu_kat(backend):
    out = backend.gelu_f32([0.0, 1.0, -1.0])
    assert abs(out[0]) < 1e-6 and abs(out[1] - 0.8413) < 1e-3 and abs(out[2] + 0.1587) < 1e-3


def test_embedding_masked_fill_broadcast_sgd_kat(backend):
    assert np.array_equal(backend.embedding_lookup_f32([0.1, 0.2, 0.3, 0.4, 0.5, 0.6], [2, 0, 1], 3, 2).ravel(),
                          np.array([0.5, 0.6, 0.1, 0.2, 0.3, 0.4], dtype=np.float32))
    assert backend.masked_fill_f32([1, 2, 3, 4], [False, True, False, True], -999.0).tolist() == [1, -999, 3, -999]
    assert backend.broadcast_add_f32([1, 2, 3, 4, 5, 6], [10, 20, 30]).tolist() == [11, 22, 33, 14, 25, 36]
    p = backend.sgd_update_f32([1.0, 2.0], [0.1, 0.2], 0.1)
    assert abs(p[0] - 0.99) < 1e-6 and abs(p[1] - 1.98) < 1e-6


# ---- against the oracle: exact for +,*,neg,relu,scale; f32 libm-level tolerance for exp/log/gelu ----
@pytest.mark.parametrize("n", [1, 3, 4, 1023, 100003, (1 << 22) + 5])
def test_elementwise_vs_oracle(backend, oracle, n):
    rng = np.random.default_rng(n)
    x = rng.standard_normal(n).astype(np.float32)
    y = rng.standard_normal(n).astype(np.float32)
    assert np.array_equal(backend.add_f32(x, y), oracle.binary("add", x, y))
    assert np.array_equal(backend.mul_f32(x, y), oracle.binary("mul", x, y))
    assert np.array_equal(backend.neg_f32(x), oracle.unary("neg", x))
    assert np.array_equal(backend.relu_f32(x), oracle.unary("relu", x))
    assert np.array_equal(backend.scale_f32(x, 0.37), oracle.scale(x, 0.37))
    assert relerr(backend.exp_f32(x), oracle.unary("exp", x)) <= 2.5e-7       # 2 ulp of the device expf
    xl = np.abs(x) + 0.1
    assert np.abs(backend.log_f32(xl) - oracle.unary("log", xl)).max() <= 5e-7
    assert np.abs(backend.gelu_f32(x) - oracle.unary("gelu", x)).max() <= 1e-6


def test_empty_inputs(backend):
    e = np.zeros(0, dtype=np.float32)
    assert backend.add_f32(e, e).size == 0
    assert backend.gelu_f32(e).size == 0
    assert backend.softmax_f32(e, 0, 5).size == 0
    assert backend.matmul_f32(e, np.zeros((3, 2), np.float32), 0, 3, 2).size == 0
    assert np.array_equal(backend.matmul_f32(np.zeros((2, 0), np.float32), e, 2, 0, 3), np.zeros((2, 3), np.float32))   # k = 0
    assert backend.sum_f32(e) == 0.0


def test_golden_abi_ops_from_reference_c(backend):
    """Vectors written by the reference's own mock_npu.c (tests/golden/make_golden.py)."""
    g = np.load(os.path.join(GOLDEN, "abi_ops.npz"))
    x, y = g["x"], g["y"]
    assert np.array_equal(backend.add_f32(x, y), g["add"])
    assert np.array_equal(backend.mul_f32(x, y), g["mul"])
    assert np.array_equal(backend.neg_f32(x), g["neg"])
    assert np.array_equal(backend.relu_f32(x), g["relu"])
    assert np.array_equal(backend.scale_f32(x, 0.37), g["scale_0p37"])
    assert relerr(backend.exp_f32(x), g["exp"]) <= 2.5e-7
    assert np.abs(backend.log_f32(np.abs(x) + 0.1) - g["log"]).max() <= 5e-7
    assert np.abs(backend.gelu_f32(x) - g["gelu"]).max() <= 1e-6
    backend.lib.sptorch_ext_set_matmul_mode(2)     # f32 FMA on the CUDA cores: the reference's k order
    try:
        assert relerr(backend.matmul_f32(g["mm_a"], g["mm_b"], 24, 40, 16), g["matmul"]) <= 1e-6
        assert relerr(backend.batch_matmul_f32(g["bmm_a"], g["bmm_b"], 3, 8, 12, 8), g["batch_matmul"]) <= 1e-6
    finally:
        backend.lib.sptorch_ext_set_matmul_mode(0)
    assert relerr(backend.softmax_f32(g["sm_x"], 10, 50), g["softmax"]) <= 1e-6


@pytest.mark.parametrize("m,k,n", [(2, 3, 2), (70, 33, 45), (64, 64, 64), (256, 128, 192), (130, 260, 100)])
def test_matmul_vs_oracle_both_modes(backend, oracle, m, k, n):
    rng = np.random.default_rng(m * 1000 + n)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    ref = oracle.matmul(a, b, f64=True)
    assert relerr(backend.matmul_f32(a, b, m, k, n), ref) <= 2e-3           # TF32 tensor cores (north star tolerance)
    backend.lib.sptorch_ext_set_matmul_mode(2)
    try:
        assert relerr(backend.matmul_f32(a, b, m, k, n), ref) <= 2e-6       # f32 FMA
    finally:
        backend.lib.sptorch_ext_set_matmul_mode(0)


def test_batch_matmul_vs_oracle(backend, oracle):
    rng = np.random.default_rng(5)
    a = rng.standard_normal((5, 128, 64)).astype(np.float32)
    b = rng.standard_normal((5, 64, 136)).astype(np.float32)
    assert relerr(backend.batch_matmul_f32(a, b, 5, 128, 64, 136), oracle.batch_matmul(a, b)) <= 2e-3


def test_integer_valued_matmul_is_exact_on_tensor_cores(backend):
    # the reference pins matmul with small-integer KATs (e.g. hal-ffi/tests/test_serial_backend.rs:56-81, 32x32 / 64x64);
    # integers below 2^11 are exact in TF32, so the tensor-core path must reproduce them bit for bit
    rng = np.random.default_rng(6)
    for s in (32, 64, 128):
        a = rng.integers(-8, 9, (s, s)).astype(np.float32)
        b = rng.integers(-8, 9, (s, s)).astype(np.float32)
        assert np.array_equal(backend.matmul_f32(a, b, s, s, s), (a.astype(np.int64) @ b.astype(np.int64)).astype(np.float32))


def test_sum_softmax_misc_vs_oracle(backend, oracle):
    rng = np.random.default_rng(7)
    x = rng.standard_normal(300001).astype(np.float32)
    assert abs(backend.sum_f32(x) - float(x.astype(np.float64).sum())) <= 1e-3     # f64 tree vs the reference's sequential f32
    a = rng.standard_normal((37, 96)).astype(np.float32); b = rng.standard_normal(96).astype(np.float32)
    assert np.array_equal(backend.broadcast_add_f32(a, b), oracle.broadcast_add(a, b))
    a2 = rng.standard_normal((37, 97)).astype(np.float32); b2 = rng.standard_normal(97).astype(np.float32)
    assert np.array_equal(backend.broadcast_add_f32(a2, b2), oracle.broadcast_add(a2, b2))
    m = rng.random(a.size) < 0.3
    assert np.array_equal(backend.masked_fill_f32(a, m, -np.inf), oracle.masked_fill(a, m, -np.inf))
    w = rng.standard_normal((50, 24)).astype(np.float32); idx = rng.integers(0, 50, 77)
    assert np.array_equal(backend.embedding_lookup_f32(w, idx, 50, 24), oracle.embedding(w, idx))
    assert np.array_equal(backend.transpose(a), oracle.transpose(a))


def test_embedding_out_of_range_is_an_error_not_a_fault(backend):
    from sptorch_b200.backend import HalError
    w = np.ones((4, 8), dtype=np.float32)
    with pytest.raises(HalError):        # the reference asserts idx < num_embeddings (core-ops/src/lib.rs:1229)
        backend.embedding_lookup_f32(w, [1, 9], 4, 8)
    backend.synchronize()                # the error is consumed; the context stays usable
    assert backend.add_f32([1], [2]).tolist() == [3]


def test_adam_vs_oracle(backend, oracle):
    rng = np.random.default_rng(8)
    n = 1000
    p, g, m, v = (rng.standard_normal(n).astype(np.float32) for _ in range(4))
    v = np.abs(v)
    po, mo, vo = p.copy(), m.copy(), v.copy()
    fp = C.POINTER(C.c_float)
    oracle.lib().orc_adam_update(po.ctypes.data_as(fp), g.ctypes.data_as(fp), mo.ctypes.data_as(fp), vo.ctypes.data_as(fp), C.c_size_t(n),
                                 *(C.c_float(x) for x in (1e-3, 0.9, 0.999, 1e-8, 0.01, 0.1, 0.001)))
    pd, md, vd = backend.adam_update_f32(p, g, m, v, 1e-3, 0.9, 0.999, 1e-8, 0.01, 0.1, 0.001)
    assert np.abs(pd - po).max() <= 1e-6 and np.array_equal(md, mo) and np.array_equal(vd, vo)


def test_alloc_failure_and_lifecycle(backend):
    lib = backend.lib
    # injected OOM: NULL, not a poisoned stream
    lib.sptorch_ext_set_alloc_budget(1 << 20)
    try:
        assert lib.sptorch_alloc(1 << 30) is None
        assert b"budget" in lib.sptorch_ext_last_error()
    finally:
        lib.sptorch_ext_set_alloc_budget(0)
    assert lib.sptorch_sync() == 0
    lib.sptorch_free(None)               # tolerated
    # init / shutdown are reference counted: a second load + close leaves the first usable
    assert lib.sptorch_backend_init() == 0
    lib.sptorch_backend_shutdown()
    assert backend.add_f32([1, 2], [3, 4]).tolist() == [4, 6]
    # null handles are an error code, never a fault
    assert lib.sptorch_add_f32(None, None, None, 4) != 0
    assert lib.sptorch_sync() != 0       # sticky: reported again by sync, then cleared
    assert lib.sptorch_sync() == 0


def test_thread_safety_of_entry_points(backend):
    import threading
    errs = []

    def work(seed):
        try:
            rng = np.random.default_rng(seed)
            for _ in range(20):
                x = rng.standard_normal(5000).astype(np.float32)
                y = rng.standard_normal(5000).astype(np.float32)
                if not np.array_equal(backend.add_f32(x, y), x + y):
                    errs.append("mismatch")
        except Exception as e:  # noqa: BLE001
            errs.append(repr(e))

    ts = [threading.Thread(target=work, args=(i,)) for i in range(4)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert not errs, errs
