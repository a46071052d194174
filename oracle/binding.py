"""ctypes binding of oracle/liboracle.so and oracle/_ref/libmock_npu.so.

TEST INFRASTRUCTURE ONLY: the shipped package never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_f = C.POINTER(C.c_float)
_u8 = C.POINTER(C.c_uint8)
_i64 = C.POINTER(C.c_int64)
_sz = C.c_size_t


class GptConfig(C.Structure):
    _fields_ = [("vocab", C.c_int), ("d_model", C.c_int), ("n_layer", C.c_int), ("n_head", C.c_int),
                ("d_ff", C.c_int), ("seq_len", C.c_int), ("eps", C.c_float)]


def build(force: bool = False) -> None:
    so = os.path.join(_HERE, "liboracle.so")
    src_newer = (not os.path.exists(so)) or any(
        os.path.getmtime(os.path.join(_HERE, f)) > os.path.getmtime(so) for f in ("oracle.c", "oracle.h"))
    # the reference checkout: SPTORCH_REFERENCE in the environment, else a directory named reference beside this repository
    ref_dir = os.environ.get("SPTORCH_REFERENCE") or os.path.abspath(os.path.join(_HERE, "..", "..", "reference"))
    ref_missing = os.path.isdir(ref_dir) and not os.path.exists(os.path.join(_HERE, "_ref", "libmock_npu.so"))
    if force or src_newer or ref_missing:
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)


_lib = None


def lib():
    global _lib
    if _lib is None:
        so = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(so):
            build()
        _lib = C.CDLL(so)
        L = _lib
        L.orc_sum.restype = C.c_float
        L.orc_cross_entropy.restype = C.c_float
        L.orc_gpt_param_count.restype = _sz
        L.orc_gpt_param_count.argtypes = [C.POINTER(GptConfig)]
        L.orc_sampling_candidates.restype = C.c_long
        L.orc_qwen_param_count.restype = _sz
        L.orc_qwen_param_count.argtypes = [C.POINTER(GptConfig)]
    return _lib


def ref_lib():
    """The reference's own C implementation of the C-ABI (mock_npu.c compiled in place), or None."""
    so = os.path.join(_HERE, "_ref", "libmock_npu.so")
    if not os.path.exists(so):
        return None
    L = C.CDLL(so)
    L.sptorch_alloc.restype = C.c_void_p
    L.sptorch_backend_name.restype = C.c_char_p
    return L


def _p(a):
    return a.ctypes.data_as(_f)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def unary(name, a):
    a = _f32(a); out = np.empty_like(a)
    getattr(lib(), "orc_" + name)(_p(a), _p(out), _sz(a.size))
    return out


def binary(name, a, b):
    a = _f32(a); b = _f32(b); out = np.empty_like(a)
    getattr(lib(), "orc_" + name)(_p(a), _p(b), _p(out), _sz(a.size))
    return out


def scale(a, s):
    a = _f32(a); out = np.empty_like(a)
    lib().orc_scale(_p(a), C.c_float(s), _p(out), _sz(a.size))
    return out


def sum_(a):
    a = _f32(a)
    return float(lib().orc_sum(_p(a), _sz(a.size)))


def broadcast_add(a, b):
    a = _f32(a); b = _f32(b); out = np.empty_like(a)
    lib().orc_broadcast_add(_p(a), _p(b), _p(out), _sz(a.size), _sz(b.size))
    return out


def masked_fill(a, mask, fill):
    a = _f32(a); m = np.ascontiguousarray(mask, dtype=np.uint8); out = np.empty_like(a)
    lib().orc_masked_fill(_p(a), m.ctypes.data_as(_u8), C.c_float(fill), _p(out), _sz(a.size))
    return out


def embedding(w, idx):
    w = _f32(w); idx = np.ascontiguousarray(idx, dtype=np.int64)
    out = np.empty((idx.size, w.shape[1]), dtype=np.float32)
    rc = lib().orc_embedding(_p(w), idx.ctypes.data_as(_i64), _p(out), _sz(idx.size), _sz(w.shape[0]), _sz(w.shape[1]))
    if rc != 0:
        raise IndexError("embedding index out of range")
    return out


def transpose(a):
    a = _f32(a); out = np.empty((a.shape[1], a.shape[0]), dtype=np.float32)
    lib().orc_transpose(_p(a), _p(out), _sz(a.shape[0]), _sz(a.shape[1]))
    return out


def matmul(a, b, f64=False):
    a = _f32(a); b = _f32(b)
    m, k = a.shape; n = b.shape[1]
    out = np.empty((m, n), dtype=np.float32)
    (lib().orc_matmul_f64 if f64 else lib().orc_matmul)(_p(a), _p(b), _p(out), _sz(m), _sz(k), _sz(n))
    return out


def batch_matmul(a, b):
    a = _f32(a); b = _f32(b)
    z, m, k = a.shape; n = b.shape[2]
    out = np.empty((z, m, n), dtype=np.float32)
    lib().orc_batch_matmul(_p(a), _p(b), _p(out), _sz(z), _sz(m), _sz(k), _sz(n))
    return out


def softmax(a, hal=False):
    a = _f32(a); rows, cols = a.shape; out = np.empty_like(a)
    (lib().orc_softmax_hal if hal else lib().orc_softmax)(_p(a), _p(out), _sz(rows), _sz(cols))
    return out


def masked_softmax(a, keep):
    a = _f32(a); rank1 = a.ndim == 1
    a2 = a.reshape(1, -1) if rank1 else a.reshape(-1, a.shape[-1])
    k = np.ascontiguousarray(keep, dtype=np.uint8).reshape(a2.shape)
    out = np.empty_like(a2)
    lib().orc_masked_softmax(_p(a2), k.ctypes.data_as(_u8), _p(out), _sz(a2.shape[0]), _sz(a2.shape[1]), C.c_int(int(rank1)))
    return out.reshape(a.shape)


def causal_softmax(scores, scale_):
    """scale -> masked_fill(j>i, -inf) -> 2-D softmax, as crates/nn/src/lib.rs:612-632 composes them.
    scores: [BH, T, T]."""
    s = _f32(scores)
    bh, t, _ = s.shape
    x = scale(s, scale_).reshape(bh, t, t)
    mask = np.triu(np.ones((t, t), dtype=np.uint8), k=1)
    x = masked_fill(x, np.broadcast_to(mask, x.shape), -np.inf).reshape(bh * t, t)
    return softmax(x).reshape(bh, t, t)


def layernorm(x, gamma, beta, eps=1e-5):
    x = _f32(x); g = _f32(gamma); b = _f32(beta)
    x2 = x.reshape(-1, x.shape[-1]); out = np.empty_like(x2)
    lib().orc_layernorm(_p(x2), _p(g), _p(b), _p(out), _sz(x2.shape[0]), _sz(x2.shape[1]), C.c_float(eps))
    return out.reshape(x.shape)


def rms_norm(x, w, eps=1e-6):
    x = _f32(x); w = _f32(w)
    x2 = x.reshape(-1, x.shape[-1]); out = np.empty_like(x2)
    lib().orc_rms_norm(_p(x2), _p(w), _p(out), _sz(x2.shape[0]), _sz(x2.shape[1]), C.c_float(eps))
    return out.reshape(x.shape)


def swiglu(x, gate):
    x = _f32(x); g = _f32(gate); out = np.empty_like(x)
    lib().orc_swiglu(_p(x), _p(g), _p(out), _sz(x.size))
    return out


def cross_entropy(logits, targets, ignore_index=None):
    x = _f32(logits); t = np.ascontiguousarray(targets, dtype=np.int64)
    bad = C.c_int(0)
    r = lib().orc_cross_entropy(_p(x), t.ctypes.data_as(_i64), _sz(x.shape[0]), _sz(x.shape[1]), C.c_int(ignore_index is not None),
                                C.c_int64(ignore_index if ignore_index is not None else 0), C.byref(bad))
    if bad.value:
        raise IndexError("cross_entropy target out of range")
    return float(r)


def linear(x, w, bias=None, fast=0):
    x = _f32(x); w = _f32(w)
    M, K = x.shape; N = w.shape[0]
    y = np.empty((M, N), dtype=np.float32)
    b = _f32(bias) if bias is not None else None
    lib().orc_linear(_p(x), _p(w), _p(b) if b is not None else None, _p(y), _sz(M), _sz(K), _sz(N), C.c_int(fast))
    return y


def mha_causal(x, wq, wk, wv, wo, n_head, fast=0):
    x = _f32(x); T, d = x.shape
    out = np.empty_like(x)
    lib().orc_mha_causal(_p(x), _p(_f32(wq)), _p(_f32(wk)), _p(_f32(wv)), _p(_f32(wo)), _p(out),
                         _sz(T), _sz(d), _sz(n_head), C.c_int(fast))
    return out


def rope(x, rope_base=10000.0, position_offset=0, inverse=False):
    """x [n_head, seq_len, head_dim] (crates/nn/src/lib.rs:930-961)."""
    x = _f32(x); H, T, hd = x.shape
    out = np.empty_like(x)
    if lib().orc_rope(_p(x), _p(out), _sz(H), _sz(T), _sz(hd), C.c_float(rope_base), _sz(position_offset), C.c_int(int(inverse))) != 0:
        raise ValueError("rope requires an even head dimension")
    return out


def mha_causal_rope(x, wq, wk, wv, wo, n_head, rope_base=10000.0, position_offset=0, fast=0):
    x = _f32(x); T, d = x.shape
    out = np.empty_like(x)
    lib().orc_mha_causal_rope(_p(x), _p(_f32(wq)), _p(_f32(wk)), _p(_f32(wv)), _p(_f32(wo)), _p(out),
                              _sz(T), _sz(d), _sz(n_head), C.c_int(fast), C.c_float(rope_base), _sz(position_offset))
    return out


def attention_last_token(q, k, v):
    """q [H*hd]; k, v [H, n, hd] -> [H*hd]  (crates/nn/src/lib.rs:727-755)."""
    k = _f32(k); v = _f32(v); q = _f32(q)
    H, n, hd = k.shape
    out = np.empty(H * hd, dtype=np.float32)
    lib().orc_attention_last_token(_p(q), _p(k), _p(v), _p(out), _sz(H), _sz(n), _sz(hd))
    return out


def _cfg(cfg: dict) -> GptConfig:
    return GptConfig(cfg["vocab"], cfg["d_model"], cfg["n_layer"], cfg["n_head"], cfg["d_ff"], cfg["seq_len"],
                     float(cfg.get("eps", 1e-5)))


def max_threads() -> int:
    return int(lib().orc_max_threads())


def gpt_forward(cfg: dict, params: np.ndarray, ids: np.ndarray, fast=0, threads=1, want_taps=False):
    """ids [B,T] int64 -> logits [B,T,V] (and taps [B, L+2, T, d])."""
    c = _cfg(cfg)
    params = _f32(params)
    assert params.size == lib().orc_gpt_param_count(C.byref(c)), "parameter block size mismatch"
    ids = np.ascontiguousarray(ids, dtype=np.int64)
    B, T = ids.shape
    logits = np.empty((B, T, cfg["vocab"]), dtype=np.float32)
    taps = np.empty((B, cfg["n_layer"] + 2, T, cfg["d_model"]), dtype=np.float32) if want_taps else None
    rc = lib().orc_gpt_forward_batch(C.byref(c), _p(params), ids.ctypes.data_as(_i64), _sz(B), _sz(T), _p(logits),
                                     _p(taps) if taps is not None else None, C.c_int(fast), C.c_int(threads))
    if rc != 0:
        raise IndexError(f"oracle gpt forward failed rc={rc}")
    return (logits, taps) if want_taps else logits


def qwen_forward(cfg: dict, params: np.ndarray, ids: np.ndarray, fast=0, threads=1, want_taps=False, rope_base=10000.0):
    """QwenLikeGPT: ids [B,T] int64 -> logits [B,T,V] (and taps [B, L+2, T, d]); cfg["eps"] is the RMSNorm epsilon (1e-6)."""
    cfg = dict(cfg); cfg.setdefault("eps", 1e-6)
    c = _cfg(cfg)
    params = _f32(params)
    assert params.size == lib().orc_qwen_param_count(C.byref(c)), "parameter block size mismatch"
    ids = np.ascontiguousarray(ids, dtype=np.int64)
    B, T = ids.shape
    logits = np.empty((B, T, cfg["vocab"]), dtype=np.float32)
    taps = np.empty((B, cfg["n_layer"] + 2, T, cfg["d_model"]), dtype=np.float32) if want_taps else None
    rc = lib().orc_qwen_forward_batch(C.byref(c), C.c_float(rope_base), _p(params), ids.ctypes.data_as(_i64), _sz(B), _sz(T), _p(logits),
                                      _p(taps) if taps is not None else None, C.c_int(fast), C.c_int(threads))
    if rc != 0:
        raise IndexError(f"oracle qwen forward failed rc={rc}")
    return (logits, taps) if want_taps else logits


def sampling_candidates(logits, vocab_size=None, temperature=1.0, top_k=0, top_p=1.0, repetition_penalty=1.0, history=(), allowed=None):
    """sampling_candidates (crates/nn/src/lib.rs:2381-2418) -> (ids int64, scaled logits, probabilities); ``allowed`` applies
    filtered_step_logits (:2465-2480) first."""
    x = _f32(logits).ravel()
    if allowed is not None:
        a = np.ascontiguousarray(sorted(allowed), dtype=np.int64)
        y = np.empty_like(x)
        lib().orc_filter_step_logits(_p(x), _sz(x.size), a.ctypes.data_as(_i64), _sz(a.size), _p(y))
        x = y
    V = x.size if vocab_size is None else vocab_size
    h = np.ascontiguousarray(history, dtype=np.int64)
    ids = np.empty(max(V, 1), np.int64); lg = np.empty(max(V, 1), np.float32); pr = np.empty(max(V, 1), np.float32)
    n = lib().orc_sampling_candidates(_p(x), _sz(x.size), _sz(V), C.c_float(temperature), _sz(top_k), C.c_float(top_p),
                                      C.c_float(repetition_penalty), h.ctypes.data_as(_i64), _sz(h.size),
                                      ids.ctypes.data_as(_i64), _p(lg), _p(pr))
    if n < 0:
        raise ValueError("vocab_size must not exceed logits length")
    return ids[:n].copy(), lg[:n].copy(), pr[:n].copy()
