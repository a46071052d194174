"""Host-side mirror of sptorch's backend surface over the C-ABI.

``FfiBackend`` follows crates/hal-ffi/src/lib.rs:176-502 method for method: ``load`` resolves the 19
required symbols (+1 optional), calls ``sptorch_backend_init`` and fails on a non-zero return; every
kernel method takes host arrays and does alloc -> h2d -> op -> d2h -> free exactly as the Rust wrapper
does (hal-ffi/src/lib.rs:238-272), so the parity tests read like the reference's own
(crates/hal-ffi/tests/test_ffi_mock.rs).  It also carries the KernelProvider methods that the reference's
FFI bridge computes on the host (hal-ffi/src/lib.rs:448-502) -- here they run on the device through the
extension entry points -- and ``BackendDispatch``'s nine methods (crates/core-tensor/src/lib.rs:81-100).

Unlike the Rust wrapper, which ignores the return codes of op calls (hal-ffi/src/lib.rs:242-248), every
non-zero return raises ``HalError``.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib

F32, BF16 = 0, 1
MM_TF32, MM_BF16, MM_F32 = 0, 1, 2
EPI_NONE, EPI_GELU, EPI_SWIGLU = 0, 1, 2


class HalError(RuntimeError):
    """Mirror of hal::HalError (crates/hal/src/lib.rs:88-120)."""


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Host-side round-to-nearest-even f32 -> bf16 bit patterns (uint16)."""
    u = _f32(a).view(np.uint32)
    rounded = u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))
    return (rounded >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


class DeviceBuffer:
    """crates/core-tensor/src/lib.rs:271-290 (device, len, to_host) + FfiDeviceBuffer (hal-ffi/src/lib.rs:61-118):
    frees its handle when dropped."""

    def __init__(self, backend: "FfiBackend", handle: int, n: int, itemsize: int = 4):
        self._b, self.handle, self.n, self.itemsize = backend, handle, n, itemsize

    def __len__(self):
        return self.n

    @property
    def ptr(self) -> int:
        return self.handle

    def to_host(self) -> np.ndarray:
        if self.itemsize == 4:
            out = np.empty(self.n, dtype=np.float32)
            self._b._check(self._b.lib.sptorch_copy_d2h(self.handle, out.ctypes.data, self.n), "copy_d2h")
            return out
        out = np.empty(self.n, dtype=np.uint16)
        self._b._check(self._b.lib.sptorch_ext_copy_d2h_bytes(self.handle, out.ctypes.data, self.n * 2), "copy_d2h")
        return out

    def free(self):
        if self.handle:
            self._b.lib.sptorch_free(self.handle)
            self.handle = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class FfiBackend:
    """A loaded backend library.  ``FfiBackend.load()`` with no argument loads libsptorch_b200.so."""

    def __init__(self, lib):
        self.lib = lib
        self._open = True

    # -- lifecycle (hal-ffi/src/lib.rs:176-214, Drop at :146-153) --
    @classmethod
    def load(cls, path: str | None = None) -> "FfiBackend":
        lib = _lib.load(path)
        if lib.sptorch_backend_init() != 0:
            raise HalError("backend init failed: " + lib.sptorch_ext_last_error().decode(errors="replace"))
        return cls(lib)

    def close(self):
        if self._open:
            self._open = False
            self.lib.sptorch_backend_shutdown()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def _check(self, rc: int, what: str):
        if rc != 0:
            msg = self.lib.sptorch_ext_last_error().decode(errors="replace")
            # The library keeps a failure sticky until the next sync for callers that ignore return codes (the Rust
            # wrapper does: hal-ffi/src/lib.rs:242-248).  This wrapper has seen it, so it consumes the flag.
            self.lib.sptorch_sync()
            raise HalError(f"{what} failed: " + msg)

    # -- Backend trait (crates/hal/src/lib.rs:337-367) --
    def name(self) -> str:
        return self.lib.sptorch_backend_name().decode()

    def device_id(self):
        return ("cuda", self.lib.sptorch_ext_device())

    def allocate(self, nbytes: int) -> DeviceBuffer:
        h = self.lib.sptorch_ext_alloc_bytes(nbytes)
        if not h:
            raise HalError("allocate failed: " + self.lib.sptorch_ext_last_error().decode(errors="replace"))
        return DeviceBuffer(self, h, nbytes // 4)

    def alloc(self, n: int, itemsize: int = 4) -> DeviceBuffer:
        h = self.lib.sptorch_alloc(n) if itemsize == 4 else self.lib.sptorch_ext_alloc_bytes(n * itemsize)
        if not h:
            raise HalError("sptorch_alloc failed: " + self.lib.sptorch_ext_last_error().decode(errors="replace"))
        return DeviceBuffer(self, h, n, itemsize)

    def upload(self, data) -> DeviceBuffer:
        """hal-ffi/src/lib.rs:218-235: alloc + copy_h2d, handle freed if the copy fails."""
        a = _f32(data).reshape(-1)
        buf = self.alloc(a.size)
        rc = self.lib.sptorch_copy_h2d(a.ctypes.data, buf.handle, a.size)
        if rc != 0:
            buf.free()
            self._check(rc, "copy_h2d")
        return buf

    def upload_bytes(self, arr: np.ndarray) -> DeviceBuffer:
        a = np.ascontiguousarray(arr)
        buf = self.alloc(a.size, a.itemsize) if a.itemsize != 4 else self.alloc(a.size)
        buf.itemsize = a.itemsize
        self._check(self.lib.sptorch_ext_copy_h2d_bytes(a.ctypes.data, buf.handle, a.nbytes), "copy_h2d_bytes")
        return buf

    def upload_bf16(self, data) -> DeviceBuffer:
        return self.upload_bytes(f32_to_bf16_bits(np.asarray(data).reshape(-1)))

    def download(self, buf: DeviceBuffer, dtype=np.float32) -> np.ndarray:
        out = np.empty(buf.n, dtype=dtype)
        self._check(self.lib.sptorch_ext_copy_d2h_bytes(buf.handle, out.ctypes.data, out.nbytes), "copy_d2h_bytes")
        return out

    def synchronize(self):
        self._check(self.lib.sptorch_sync(), "sync")

    def query_runtime(self):
        """hal-ffi/src/lib.rs:276-285 -> (queue_depth, online) or None."""
        q, o = C.c_uint32(0), C.c_uint32(0)
        if self.lib.sptorch_query_runtime(C.byref(q), C.byref(o)) != 0:
            return None
        return q.value, bool(o.value)

    # -- helpers: the alloc -> h2d -> op -> d2h -> free round trip of hal-ffi/src/lib.rs:238-272 --
    def _unary(self, fn, a, *extra):
        a = _f32(a)
        da, do = self.upload(a), self.alloc(a.size)
        try:
            self._check(fn(da.handle, *extra, do.handle, a.size), fn.__name__)
            return do.to_host().reshape(a.shape)
        finally:
            da.free(); do.free()

    def _binary(self, fn, a, b):
        a, b = _f32(a), _f32(b)
        if a.size != b.size:
            raise HalError("binary op: length mismatch")
        da, db, do = self.upload(a), self.upload(b), self.alloc(a.size)
        try:
            self._check(fn(da.handle, db.handle, do.handle, a.size), fn.__name__)
            return do.to_host().reshape(a.shape)
        finally:
            da.free(); db.free(); do.free()

    # -- KernelProvider (crates/hal/src/lib.rs:374-458) and BackendDispatch (core-tensor/src/lib.rs:81-100) --
    def add_f32(self, a, b): return self._binary(self.lib.sptorch_add_f32, a, b)
    def mul_f32(self, a, b): return self._binary(self.lib.sptorch_mul_f32, a, b)
    def neg_f32(self, a): return self._unary(self.lib.sptorch_neg_f32, a)
    def exp_f32(self, a): return self._unary(self.lib.sptorch_exp_f32, a)
    def log_f32(self, a): return self._unary(self.lib.sptorch_log_f32, a)
    def relu_f32(self, a): return self._unary(self.lib.sptorch_relu_f32, a)
    def gelu_f32(self, a): return self._unary(self.lib.sptorch_gelu_f32, a)

    def scale_f32(self, a, scalar: float):
        return self._unary(self.lib.sptorch_scale_f32, a, C.c_float(scalar))

    def matmul_f32(self, a, b, m: int, k: int, n: int):
        a, b = _f32(a), _f32(b)
        da, db, do = self.upload(a), self.upload(b), self.alloc(m * n)
        try:
            self._check(self.lib.sptorch_matmul_f32(da.handle, db.handle, do.handle, m, k, n), "matmul_f32")
            return do.to_host().reshape(m, n)
        finally:
            da.free(); db.free(); do.free()

    def batch_matmul_f32(self, a, b, batch: int, m: int, k: int, n: int):
        a, b = _f32(a), _f32(b)
        da, db, do = self.upload(a), self.upload(b), self.alloc(batch * m * n)
        try:
            self._check(self.lib.sptorch_batch_matmul_f32(da.handle, db.handle, do.handle, batch, m, k, n), "batch_matmul_f32")
            return do.to_host().reshape(batch, m, n)
        finally:
            da.free(); db.free(); do.free()

    def sum_f32(self, a) -> float:
        a = _f32(a)
        da = self.upload(a)
        try:
            r = C.c_float(0)
            self._check(self.lib.sptorch_ext_sum_f32(da.handle, a.size, C.byref(r)), "sum_f32")
            return r.value
        finally:
            da.free()

    def softmax_f32(self, a, rows: int, cols: int):
        a = _f32(a)
        da, do = self.upload(a), self.alloc(rows * cols)
        try:
            self._check(self.lib.sptorch_softmax_f32(da.handle, do.handle, rows, cols), "softmax_f32")
            return do.to_host().reshape(rows, cols)
        finally:
            da.free(); do.free()

    def masked_fill_f32(self, a, mask, fill_value: float):
        a = _f32(a)
        m = np.ascontiguousarray(mask, dtype=np.uint8).reshape(-1)
        if m.size != a.size:
            raise HalError("masked_fill: mask length mismatch")
        da, dm, do = self.upload(a), self.upload_bytes(m), self.alloc(a.size)
        try:
            self._check(self.lib.sptorch_ext_masked_fill_f32(da.handle, dm.handle, C.c_float(fill_value), do.handle, a.size), "masked_fill")
            return do.to_host().reshape(a.shape)
        finally:
            da.free(); dm.free(); do.free()

    def broadcast_add_f32(self, a, b):
        a, b = _f32(a), _f32(b)
        da, db, do = self.upload(a), self.upload(b), self.alloc(a.size)
        try:
            self._check(self.lib.sptorch_ext_broadcast_add_f32(da.handle, db.handle, do.handle, a.size, b.size), "broadcast_add")
            return do.to_host().reshape(a.shape)
        finally:
            da.free(); db.free(); do.free()

    def embedding_lookup_f32(self, weight, indices, vocab: int, dim: int):
        w = _f32(weight)
        idx = np.ascontiguousarray(indices, dtype=np.int64).reshape(-1)
        dw, di, do = self.upload(w), self.upload_bytes(idx), self.alloc(idx.size * dim)
        try:
            self._check(self.lib.sptorch_ext_embedding_lookup_f32(dw.handle, di.handle, do.handle, idx.size, vocab, dim), "embedding_lookup")
            out = do.to_host().reshape(idx.size, dim)
            self.synchronize()   # an out-of-range id surfaces here (the reference panics: core-ops/src/lib.rs:1229)
            return out
        finally:
            dw.free(); di.free(); do.free()

    def sgd_update_f32(self, params, grad, lr: float):
        p, g = _f32(params), _f32(grad)
        dp, dg = self.upload(p), self.upload(g)
        try:
            self._check(self.lib.sptorch_ext_sgd_update_f32(dp.handle, dg.handle, C.c_float(lr), p.size), "sgd_update")
            return dp.to_host().reshape(p.shape)
        finally:
            dp.free(); dg.free()

    def adam_update_f32(self, params, grad, m, v, lr, beta1, beta2, eps, weight_decay, bc1, bc2):
        p, g, m_, v_ = _f32(params), _f32(grad), _f32(m), _f32(v)
        bufs = [self.upload(x) for x in (p, g, m_, v_)]
        try:
            self._check(self.lib.sptorch_ext_adam_update_f32(bufs[0].handle, bufs[1].handle, bufs[2].handle, bufs[3].handle, p.size,
                                                             *(C.c_float(x) for x in (lr, beta1, beta2, eps, weight_decay, bc1, bc2))), "adam_update")
            return bufs[0].to_host(), bufs[2].to_host(), bufs[3].to_host()
        finally:
            for b in bufs:
                b.free()

    # -- nn-level ops the reference computes inline on the host --
    def layernorm(self, x, gamma, beta, eps=1e-5, dtype=F32):
        x = _f32(x)
        rows, dim = int(np.prod(x.shape[:-1])), x.shape[-1]
        dg, db = self.upload(gamma), self.upload(beta)
        dx = self.upload(x) if dtype == F32 else self.upload_bf16(x)
        do = self.alloc(x.size, 4 if dtype == F32 else 2)
        try:
            self._check(self.lib.sptorch_ext_layernorm(dx.handle, dg.handle, db.handle, do.handle, rows, dim, C.c_float(eps), dtype), "layernorm")
            out = do.to_host()
            return (out if dtype == F32 else bf16_bits_to_f32(out)).reshape(x.shape)
        finally:
            for b in (dg, db, dx, do):
                b.free()

    def causal_softmax(self, scores, scale: float, dtype=F32):
        s = _f32(scores)
        bh, t, _ = s.shape
        dx = self.upload(s) if dtype == F32 else self.upload_bf16(s)
        do = self.alloc(s.size, 4 if dtype == F32 else 2)
        try:
            self._check(self.lib.sptorch_ext_causal_softmax(dx.handle, do.handle, bh, t, C.c_float(scale), dtype), "causal_softmax")
            out = do.to_host()
            return (out if dtype == F32 else bf16_bits_to_f32(out)).reshape(s.shape)
        finally:
            dx.free(); do.free()

    def masked_softmax(self, a, keep):
        a = _f32(a)
        rank1 = a.ndim == 1
        rows, cols = (1, a.size) if rank1 else (int(np.prod(a.shape[:-1])), a.shape[-1])
        k = np.ascontiguousarray(keep, dtype=np.uint8).reshape(-1)
        da, dk, do = self.upload(a), self.upload_bytes(k), self.alloc(a.size)
        try:
            self._check(self.lib.sptorch_ext_masked_softmax_f32(da.handle, dk.handle, do.handle, rows, cols, int(rank1)), "masked_softmax")
            return do.to_host().reshape(a.shape)
        finally:
            da.free(); dk.free(); do.free()

    def gelu(self, a, dtype=F32):
        a = _f32(a)
        dx = self.upload(a) if dtype == F32 else self.upload_bf16(a)
        do = self.alloc(a.size, 4 if dtype == F32 else 2)
        try:
            self._check(self.lib.sptorch_ext_gelu(dx.handle, do.handle, a.size, dtype), "gelu")
            out = do.to_host()
            return (out if dtype == F32 else bf16_bits_to_f32(out)).reshape(a.shape)
        finally:
            dx.free(); do.free()

    def rms_norm(self, x, weight, eps=1e-6, dtype=F32):
        """core-ops rms_norm (crates/core-ops/src/lib.rs:1453-1491)."""
        x = _f32(x)
        rows, dim = int(np.prod(x.shape[:-1])), x.shape[-1]
        dw = self.upload(weight)
        dx = self.upload(x) if dtype == F32 else self.upload_bf16(x)
        do = self.alloc(x.size, 4 if dtype == F32 else 2)
        try:
            self._check(self.lib.sptorch_ext_rms_norm(dx.handle, dw.handle, do.handle, rows, dim, C.c_float(eps), dtype), "rms_norm")
            out = do.to_host()
            return (out if dtype == F32 else bf16_bits_to_f32(out)).reshape(x.shape)
        finally:
            for b in (dw, dx, do):
                b.free()

    def swiglu(self, x, gate, dtype=F32):
        """core-ops swiglu (crates/core-ops/src/lib.rs:1529-1556)."""
        x, g = _f32(x), _f32(gate)
        up = self.upload if dtype == F32 else self.upload_bf16
        dx, dg = up(x), up(g)
        do = self.alloc(x.size, 4 if dtype == F32 else 2)
        try:
            self._check(self.lib.sptorch_ext_swiglu(dx.handle, dg.handle, do.handle, x.size, dtype), "swiglu")
            out = do.to_host()
            return (out if dtype == F32 else bf16_bits_to_f32(out)).reshape(x.shape)
        finally:
            for b in (dx, dg, do):
                b.free()

    def cross_entropy_loss(self, logits, targets, ignore_index=None, dtype=F32):
        """core-ops cross_entropy_loss / cross_entropy_loss_ignore_index (crates/core-ops/src/lib.rs:1079-1194)."""
        x = _f32(logits)
        if x.ndim == 1:
            x = x.reshape(1, -1)
        rows, classes = x.shape
        t = np.ascontiguousarray(targets, dtype=np.int64).reshape(-1)
        dx = self.upload(x) if dtype == F32 else self.upload_bf16(x)
        dt, dl = self.upload_bytes(t), self.alloc(rows + 1)
        try:
            mean = C.c_float(0)
            self._check(self.lib.sptorch_ext_cross_entropy(dx.handle, classes, dt.handle, rows, classes, int(ignore_index is not None),
                                                           int(ignore_index) if ignore_index is not None else 0, dl.handle, C.byref(mean), dtype), "cross_entropy")
            self.synchronize()        # an out-of-range target surfaces here (the reference asserts)
            return mean.value
        finally:
            for b in (dx, dt, dl):
                b.free()

    def transpose(self, a):
        a = _f32(a)
        da, do = self.upload(a), self.alloc(a.size)
        try:
            self._check(self.lib.sptorch_ext_transpose_f32(da.handle, do.handle, a.shape[0], a.shape[1]), "transpose")
            return do.to_host().reshape(a.shape[1], a.shape[0])
        finally:
            da.free(); do.free()

    def embedding_sum(self, tok_w, pos_w, ids, T: int, dtype=F32):
        tok_w, pos_w = _f32(tok_w), _f32(pos_w)
        ids = np.ascontiguousarray(ids, dtype=np.int32).reshape(-1)
        up = self.upload if dtype == F32 else self.upload_bf16
        dt, dp, di = up(tok_w), up(pos_w), self.upload_bytes(ids)
        dim = tok_w.shape[1]
        do = self.alloc(ids.size * dim, 4 if dtype == F32 else 2)
        try:
            self._check(self.lib.sptorch_ext_embedding_sum(dt.handle, dp.handle, di.handle, do.handle, ids.size, T, tok_w.shape[0], dim, dtype), "embedding_sum")
            out = do.to_host()
            self.synchronize()
            return (out if dtype == F32 else bf16_bits_to_f32(out)).reshape(ids.size, dim)
        finally:
            for b in (dt, dp, di, do):
                b.free()

    def sampling_candidates(self, logits, vocab_size=None, temperature=1.0, top_k=0, top_p=1.0, repetition_penalty=1.0, history=(),
                            dtype=F32, allowed=None):
        """sampling_candidates (crates/nn/src/lib.rs:2381-2418): one row of logits -> (token ids, scaled logits, probabilities)
        in the reference's candidate order.  ``logits`` may be a host array (uploaded here) or a DeviceBuffer."""
        own = not isinstance(logits, DeviceBuffer)
        d = (self.upload_bf16(_f32(logits).ravel()) if dtype == BF16 else self.upload(_f32(logits).ravel())) if own else logits
        V = d.n if vocab_size is None else vocab_size
        h = np.ascontiguousarray(history, dtype=np.int64)
        cap = max(V, 1)
        ids, lg, pr = np.empty(cap, np.int32), np.empty(cap, np.float32), np.empty(cap, np.float32)
        n = C.c_size_t(0)
        try:
            if allowed is None:
                rc = self.lib.sptorch_ext_sampling_candidates(d.handle, d.n, dtype, V, C.c_float(temperature), top_k, C.c_float(top_p),
                                                              C.c_float(repetition_penalty), h.ctypes.data, h.size,
                                                              ids.ctypes.data, lg.ctypes.data, pr.ctypes.data, cap, C.byref(n))
            else:       # a TokenConstraint's allowed_next set (nn/src/lib.rs:2465-2480)
                a = np.ascontiguousarray(sorted(allowed), dtype=np.int64)
                rc = self.lib.sptorch_ext_sampling_candidates_constrained(d.handle, d.n, dtype, V, C.c_float(temperature), top_k, C.c_float(top_p),
                                                                          C.c_float(repetition_penalty), h.ctypes.data, h.size, a.ctypes.data, a.size,
                                                                          ids.ctypes.data, lg.ctypes.data, pr.ctypes.data, cap, C.byref(n))
            self._check(rc, "sampling_candidates")
        finally:
            if own:
                d.free()
        return ids[:n.value].copy(), lg[:n.value].copy(), pr[:n.value].copy()

    def sample_from_candidates(self, ids, probs, threshold: float) -> int:
        """sample_from_candidates (nn/src/lib.rs:2420-2429) for a uniform draw ``threshold`` in [0, 1)."""
        ids = np.ascontiguousarray(ids, np.int32); probs = np.ascontiguousarray(probs, np.float32)
        return int(self.lib.sptorch_ext_sample_from_candidates(ids.ctypes.data, probs.ctypes.data, ids.size, C.c_float(threshold)))

    def rope(self, x, rope_base=10000.0, position_offset=0, dtype=F32):
        """rotary_position_embedding_with_offset (crates/nn/src/lib.rs:975-983): x [n_head, seq_len, head_dim] as in the reference;
        the device kernel works on the token-major layout, so the permutes happen here on the host."""
        x = _f32(x)
        H, T, hd = x.shape
        tm = np.ascontiguousarray(x.transpose(1, 0, 2)).reshape(T, H * hd)
        d = self.upload_bf16(tm) if dtype == BF16 else self.upload(tm)
        try:
            self._check(self.lib.sptorch_ext_rope(d.handle, T, T, H, hd, H * hd, C.c_float(rope_base), position_offset, dtype), "rope")
            out = d.to_host()
            self.synchronize()
            out = bf16_bits_to_f32(out) if dtype == BF16 else out
            return np.ascontiguousarray(out.reshape(T, H, hd).transpose(1, 0, 2))
        finally:
            d.free()

    def linear(self, x, w, bias=None, residual=None, alpha=1.0, epilogue=EPI_NONE, mode=MM_TF32, out_dtype=None):
        """nn::Linear::forward (crates/nn/src/lib.rs:121-133) with optional fused epilogue."""
        x, w = _f32(x), _f32(w)
        M, K = x.shape
        N = w.shape[0]
        bf = mode == MM_BF16
        if out_dtype is None:
            out_dtype = BF16 if bf else F32
        up = self.upload_bf16 if bf else self.upload
        dx, dw = up(x), up(w)
        db = self.upload(bias) if bias is not None else None
        dr = None
        if residual is not None:
            dr = self.upload_bf16(residual) if out_dtype == BF16 else self.upload(residual)
        do = self.alloc(M * N, 2 if out_dtype == BF16 else 4)
        try:
            self._check(self.lib.sptorch_ext_linear(dx.handle, dw.handle, db.handle if db else None, dr.handle if dr else None, do.handle,
                                                    M, K, N, 0, C.c_float(alpha), epilogue, mode, out_dtype), "linear")
            out = do.to_host()
            self.synchronize()
            return (bf16_bits_to_f32(out) if out_dtype == BF16 else out).reshape(M, N)
        finally:
            for b in (dx, dw, db, dr, do):
                if b is not None:
                    b.free()

    def attention_causal(self, q, k, v, n_head: int, dtype=F32):
        """q,k,v: [B,T,d] host arrays -> [B,T,d] (crates/nn/src/lib.rs:600-637)."""
        q, k, v = _f32(q), _f32(k), _f32(v)
        B, T, d = q.shape
        hd = d // n_head
        up = self.upload if dtype == F32 else self.upload_bf16
        dq, dk, dv = up(q), up(k), up(v)
        es = 4 if dtype == F32 else 2
        do = self.alloc(q.size, es)
        ws = self.lib.sptorch_ext_attention_workspace(B, T, n_head, hd, dtype)
        dws = self.alloc(ws, 1)
        try:
            self._check(self.lib.sptorch_ext_attention_causal(dq.handle, dk.handle, dv.handle, do.handle, dws.handle, B, T, n_head, hd, d, dtype), "attention_causal")
            out = do.to_host()
            self.synchronize()
            return (out if dtype == F32 else bf16_bits_to_f32(out)).reshape(B, T, d)
        finally:
            for b in (dq, dk, dv, do, dws):
                b.free()

    def attention_last_token(self, q, k_cache, v_cache, n_head: int, n: int, dtype=F32):
        """q [B, d]; k_cache, v_cache [B, positions, d] with the first n valid -> [B, d] (crates/nn/src/lib.rs:727-755)."""
        q, k, v = _f32(q), _f32(k_cache), _f32(v_cache)
        B, P, d = k.shape
        up = self.upload if dtype == F32 else self.upload_bf16
        dq, dk, dv = up(q), up(k), up(v)
        do = self.alloc(B * d, 4 if dtype == F32 else 2)
        try:
            self._check(self.lib.sptorch_ext_attention_last_token(dq.handle, dk.handle, dv.handle, do.handle, B, n_head, d // n_head, n, P, dtype), "attention_last_token")
            out = do.to_host()
            self.synchronize()
            return (out if dtype == F32 else bf16_bits_to_f32(out)).reshape(B, d)
        finally:
            for x in (dq, dk, dv, do):
                x.free()

    # -- timing on the library's stream --
    def timer_begin(self):
        self._check(self.lib.sptorch_ext_timer_begin(), "timer_begin")

    def timer_end(self) -> float:
        ms = C.c_float(0)
        self._check(self.lib.sptorch_ext_timer_end(C.byref(ms)), "timer_end")
        return ms.value

    def flush_l2(self):
        self._check(self.lib.sptorch_ext_flush_l2(), "flush_l2")
