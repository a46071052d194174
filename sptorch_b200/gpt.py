"""nn::GPT on the device (crates/nn/src/lib.rs:1263-1437): same constructor arguments, same parameter
names, ``forward_ids`` with the reference's meaning (token ids in, logits [T, V] out), plus a batched
device-resident ``forward`` that the benchmark uses."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from .backend import BF16, F32, FfiBackend, HalError, bf16_bits_to_f32
from .synth import gpt_param_layout, qwen_param_layout

ARCH_GPT, ARCH_QWEN_LIKE = 0, 1


def _lib_view(backend, buf, offset_elems: int, n: int, itemsize: int):
    """A DeviceBuffer over part of another one (not owning: freeing it is a no-op)."""
    from .backend import DeviceBuffer
    v = DeviceBuffer(backend, buf.handle + offset_elems * itemsize, n, itemsize)
    v.free = lambda: None
    return v


class GPT:
    def __init__(self, backend: FfiBackend, vocab_size: int, d_model: int, n_head: int, n_layer: int, d_ff: int,
                 seq_len: int, dtype: int = F32, max_batch: int = 1, eps: float = 1e-5, tp_rank: int = 0, tp_size: int = 1,
                 arch: int = ARCH_GPT, rope_base: float = 10000.0):
        # argument order of GPT::new (nn/src/lib.rs:1332)
        self.b = backend
        self.cfg = dict(vocab=vocab_size, d_model=d_model, n_layer=n_layer, n_head=n_head, d_ff=d_ff, seq_len=seq_len)
        self.dtype, self.max_batch, self.arch = dtype, max_batch, arch
        c = _lib.GptConfig(vocab_size, d_model, n_layer, n_head, d_ff, seq_len, dtype, max_batch, eps, tp_rank, tp_size, arch, rope_base)
        self.h = backend.lib.sptorch_ext_gpt_create(C.byref(c))
        if not self.h:
            raise HalError("gpt_create failed: " + _lib.last_error())
        self.ldl = backend.lib.sptorch_ext_gpt_logits_ld(self.h)
        self.es = 2 if dtype == BF16 else 4
        self._logits = None
        self._ids = None
        self._gen_ctx = None
        self._prompt_len = 0
        self.kv_cache_enabled = False

    def close(self):
        if self.h:
            for buf in (self._logits, self._ids):
                if buf is not None:
                    buf.free()
            self.b.lib.sptorch_ext_gpt_destroy(self.h)
            self.h = None

    def named_parameters(self):
        return (qwen_param_layout if self.arch == ARCH_QWEN_LIKE else gpt_param_layout)(**self.cfg)

    def load_flat(self, flat: np.ndarray, index: dict):
        """flat f32 block + {name: (offset, shape)} as produced by synth.gpt_params."""
        for name, (off, shape) in index.items():
            self.set_param(name, flat[off:off + int(np.prod(shape))])

    def set_param(self, name: str, values):
        a = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
        self.b._check(self.b.lib.sptorch_ext_gpt_set_param(self.h, name.encode(), a.ctypes.data, a.size), f"set_param({name})")

    def enable_ln_fold(self, on=True):
        """LayerNorm applied inside the epilogues of the consuming GEMMs (bf16 GPT only; off by default)."""
        self.b._check(self.b.lib.sptorch_ext_gpt_enable_ln_fold(self.h, int(on)), "enable_ln_fold")

    def enable_taps(self, on=True):
        self.b._check(self.b.lib.sptorch_ext_gpt_enable_taps(self.h, int(on)), "enable_taps")

    def tap(self, i: int, n_tokens: int) -> np.ndarray:
        p = self.b.lib.sptorch_ext_gpt_tap(self.h, i)
        if not p:
            raise HalError("taps are not enabled")
        d = self.cfg["d_model"]
        raw = np.empty(n_tokens * d, dtype=np.uint16 if self.dtype == BF16 else np.float32)
        self.b._check(self.b.lib.sptorch_ext_copy_d2h_bytes(p, raw.ctypes.data, raw.nbytes), "tap d2h")
        return (bf16_bits_to_f32(raw) if self.dtype == BF16 else raw).reshape(n_tokens, d)

    # -- device-resident batched forward --
    def stage_ids(self, ids: np.ndarray):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        if self._ids is None or self._ids.n < ids.size:
            if self._ids is not None:
                self._ids.free()
            self._ids = self.b.alloc(ids.size)
        self.b._check(self.b.lib.sptorch_ext_copy_h2d_bytes(ids.ctypes.data, self._ids.handle, ids.nbytes), "ids h2d")
        return self._ids

    def logits_buffer(self, n_tokens: int):
        need = n_tokens * self.ldl
        if self._logits is None or self._logits.n < need:
            if self._logits is not None:
                self._logits.free()
            self._logits = self.b.alloc(need, self.es)
        return self._logits

    def forward_device(self, ids_dev, batch: int, T: int, logits_dev):
        self.b._check(self.b.lib.sptorch_ext_gpt_forward(self.h, ids_dev.handle, batch, T, logits_dev.handle), "gpt_forward")

    def forward(self, ids: np.ndarray) -> np.ndarray:
        """ids [B, T] -> logits [B, T, V] float32 on the host."""
        ids = np.asarray(ids)
        B, T0 = ids.shape
        V = self.cfg["vocab"]
        if T0 > self.cfg["seq_len"]:
            raise HalError("sequence longer than seq_len")   # the reference asserts (nn/src/lib.rs:1351)
        # The kernels want T to be a multiple of one 16-byte vector.  A ragged length is padded at the END with token 0:
        # under the causal mask no earlier position can see the padding, so rows 0..T0-1 are unchanged; the padded
        # rows are dropped here.
        vec = 8 if self.dtype == BF16 else 4
        T = -(-T0 // vec) * vec
        if T != T0:
            if T > self.cfg["seq_len"]:
                raise HalError(f"T={T0} cannot be padded to a multiple of {vec} within seq_len={self.cfg['seq_len']}")
            ids = np.concatenate([ids, np.zeros((B, T - T0), dtype=ids.dtype)], axis=1)
        d_ids = self.stage_ids(ids)
        d_log = self.logits_buffer(B * T)
        self.forward_device(d_ids, B, T, d_log)
        raw = np.empty(B * T * self.ldl, dtype=np.uint16 if self.dtype == BF16 else np.float32)
        self.b._check(self.b.lib.sptorch_ext_copy_d2h_bytes(d_log.handle, raw.ctypes.data, raw.nbytes), "logits d2h")
        self.b.synchronize()
        out = bf16_bits_to_f32(raw) if self.dtype == BF16 else raw
        return out.reshape(B, T, self.ldl)[:, :T0, :V].copy()

    def forward_loss(self, ids: np.ndarray, targets=None, ignore_index=None, want_argmax: bool = True):
        """Forward fused with the step after it: ids [B, T] (T a multiple of the vector width) and int targets [B, T] ->
        (mean cross-entropy loss or None, greedy tokens [B, T] or None) without the [B*T, vocab] logits ever being written
        (cross_entropy_loss / cross_entropy_loss_ignore_index: core-ops/src/lib.rs:1079-1194; greedy token: the first of
        sampling_candidates' sorted candidates, nn/src/lib.rs:2381-2418)."""
        ids = np.asarray(ids)
        B, T = ids.shape
        d_ids = self.stage_ids(ids)
        bufs = []
        d_tgt = d_rows = d_arg = None
        if targets is not None:
            tg = np.ascontiguousarray(targets, dtype=np.int64).reshape(-1)
            d_tgt = self.b.alloc(tg.size, 8); bufs.append(d_tgt)
            self.b._check(self.b.lib.sptorch_ext_copy_h2d_bytes(tg.ctypes.data, d_tgt.handle, tg.nbytes), "targets h2d")
            self.b.synchronize()
            d_rows = self.b.alloc(B * T + 1); bufs.append(d_rows)
        if want_argmax:
            d_arg = self.b.alloc(B * T); bufs.append(d_arg)
        mean = C.c_float(0.0)
        try:
            self.b._check(self.b.lib.sptorch_ext_gpt_forward_loss(self.h, d_ids.handle, d_tgt.handle if d_tgt else None, B, T,
                                                                  int(ignore_index is not None), int(ignore_index or 0),
                                                                  d_arg.handle if d_arg else None, d_rows.handle if d_rows else None, C.byref(mean)), "gpt_forward_loss")
            arg = None
            if d_arg is not None:
                arg = np.empty(B * T, dtype=np.int32)
                self.b._check(self.b.lib.sptorch_ext_copy_d2h_bytes(d_arg.handle, arg.ctypes.data, arg.nbytes), "argmax d2h")
                arg = arg.reshape(B, T)
            self.b.synchronize()
            return (float(mean.value) if targets is not None else None), arg
        finally:
            for buf in bufs:
                buf.free()

    def forward_loss_host(self, ids_host_ptr: int, targets_host_ptr, batch: int, T: int, argmax_host_ptr, chunk: int, ignore_index=None) -> float:
        """Host-buffer form of forward_loss: pinned ids (int32) and targets (int64) in, greedy tokens (int32) and the mean loss out."""
        mean = C.c_float(0.0)
        self.b._check(self.b.lib.sptorch_ext_gpt_forward_loss_host(self.h, ids_host_ptr, targets_host_ptr, batch, T, int(ignore_index is not None),
                                                                   int(ignore_index or 0), argmax_host_ptr, C.byref(mean), chunk), "gpt_forward_loss_host")
        return float(mean.value)

    def forward_ids(self, token_ids) -> np.ndarray:
        """GPT::forward_ids (nn/src/lib.rs:1349-1364): one sequence of ids -> logits [T, V]."""
        ids = np.asarray(token_ids).reshape(1, -1)
        return self.forward(ids)[0]

    # -- incremental decode (PrefillCache / IncrementalDecode of the reference: nn/src/lib.rs:1540-1573, 1619-1646) --
    def enable_kv_cache(self, max_context: int = 0):
        self.b._check(self.b.lib.sptorch_ext_gpt_enable_kv_cache(self.h, max_context), "enable_kv_cache")
        self.kv_cache_enabled = True

    def cached_len(self) -> int:
        return self.b.lib.sptorch_ext_gpt_cached_len(self.h)

    def _read_logits(self, d_log, rows: int) -> np.ndarray:
        raw = np.empty(rows * self.ldl, dtype=np.uint16 if self.dtype == BF16 else np.float32)
        self.b._check(self.b.lib.sptorch_ext_copy_d2h_bytes(d_log.handle, raw.ctypes.data, raw.nbytes), "logits d2h")
        self.b.synchronize()
        out = bf16_bits_to_f32(raw) if self.dtype == BF16 else raw
        return out.reshape(rows, self.ldl)[:, :self.cfg["vocab"]].copy()

    def prefill_kv_cache(self, ids: np.ndarray) -> np.ndarray:
        """ids [B, T] (T a multiple of the vector width): fills the cache, returns the logits [B, T, V] of the prefix."""
        ids = np.asarray(ids)
        B, T = ids.shape
        d_ids, d_log = self.stage_ids(ids), self.logits_buffer(B * T)
        self.b._check(self.b.lib.sptorch_ext_gpt_prefill(self.h, d_ids.handle, B, T, d_log.handle), "gpt_prefill")
        return self._read_logits(d_log, B * T).reshape(B, T, -1)

    def decode_logits_from_cache(self, last_ids) -> np.ndarray:
        """Logits [B, V] of the last cached token, recomputed from the cache (no append)."""
        return self._decode(last_ids, 0)

    def append_and_decode(self, new_ids) -> np.ndarray:
        """Appends one new token per sequence to the cache and returns its logits [B, V]."""
        return self._decode(new_ids, 1)

    def _decode(self, ids, append: int) -> np.ndarray:
        ids = np.asarray(ids).reshape(-1)
        d_ids, d_log = self.stage_ids(ids), self.logits_buffer(ids.size)
        self.b._check(self.b.lib.sptorch_ext_gpt_decode(self.h, d_ids.handle, ids.size, append, d_log.handle), "gpt_decode")
        return self._read_logits(d_log, ids.size)

    # -- generation (generate_with_config_inner / decode_next_token_inner, nn/src/lib.rs:2431-2464, 2526-2553) --
    def _last_logits_device(self, context):
        """Logits of the last token of ``context`` as a device row: from the key/value cache while the context only grew by
        one token since the last call, otherwise by a fresh prefill (vector-aligned prefix) plus single-token appends."""
        n = len(context)
        vec = 8 if self.dtype == BF16 else 4
        d_log = self.logits_buffer(max(n, 1))
        grew_by_one = self._gen_ctx is not None and n == len(self._gen_ctx) + 1 and list(context[:-1]) == self._gen_ctx
        if grew_by_one and self.cached_len() == n - 1:
            d_ids = self.stage_ids(np.asarray(context[-1:]))
            self.b._check(self.b.lib.sptorch_ext_gpt_decode(self.h, d_ids.handle, 1, 1, d_log.handle), "gpt_decode")
        else:
            t0 = (n // vec) * vec
            if t0:
                d_ids = self.stage_ids(np.asarray(context[:t0]).reshape(1, t0))
                self.b._check(self.b.lib.sptorch_ext_gpt_prefill(self.h, d_ids.handle, 1, t0, d_log.handle), "gpt_prefill")
                rest = context[t0:]
                if not len(rest):      # the last row of the prefill is the row wanted: recompute it from the cache as a single row
                    d_ids = self.stage_ids(np.asarray(context[-1:]))
                    self.b._check(self.b.lib.sptorch_ext_gpt_decode(self.h, d_ids.handle, 1, 0, d_log.handle), "gpt_decode")
            else:                      # shorter than one vector: a padded forward, nothing cached
                self._gen_ctx = None
                ids = np.zeros((1, vec), dtype=np.int64); ids[0, :n] = context
                d_ids = self.stage_ids(ids)
                self.forward_device(d_ids, 1, vec, d_log)
                return _lib_view(self.b, d_log, (n - 1) * self.ldl, self.ldl, self.es)
            for tok in context[t0:]:
                d_ids = self.stage_ids(np.asarray([tok]))
                self.b._check(self.b.lib.sptorch_ext_gpt_decode(self.h, d_ids.handle, 1, 1, d_log.handle), "gpt_decode")
        self._gen_ctx = list(context)
        return _lib_view(self.b, d_log, 0, self.ldl, self.es)

    def decode_next_token(self, tokens: list, vocab_size=None, temperature=1.0, top_k=0, top_p=1.0, repetition_penalty=1.0,
                          eos_token_id=None, draw=None, constraint=None):
        """One step of decode_next_token_inner (nn/src/lib.rs:2431-2464) on ``tokens`` (prompt + generated so far, extended in
        place).  Returns (token or None, candidates (ids, logits, probs), stop_reason) with the reference's stop reasons.
        ``draw`` supplies the uniform numbers in [0, 1) of sample_from_candidates; default: numpy's global generator.
        ``constraint``: the reference's TokenConstraint as a callable generated_tokens -> set of allowed ids, or None for no limit."""
        V = self.cfg["vocab"] if vocab_size is None else vocab_size
        if V <= 0:
            raise HalError("vocab_size must be positive")                        # the reference asserts
        if eos_token_id is not None and tokens and tokens[-1] == eos_token_id:
            return None, (np.zeros(0, np.int32),) * 3, "AlreadyEnded"
        context = tokens[-self.cfg["seq_len"]:]                                  # InferenceState::context (nn/src/lib.rs:2242-2248)
        row = self._last_logits_device(context)
        allowed = constraint(tokens[self._prompt_len:]) if constraint is not None else None
        cand = self.b.sampling_candidates(row, vocab_size=V, temperature=temperature, top_k=top_k, top_p=top_p,
                                          repetition_penalty=repetition_penalty, history=tokens, dtype=self.dtype, allowed=allowed)
        if not len(cand[0]):
            return None, cand, "NoCandidates"
        u = float(np.random.random() if draw is None else draw())
        nxt = self.b.sample_from_candidates(cand[0], cand[2], u)
        tokens.append(nxt)
        return nxt, cand, ("EosToken" if nxt == eos_token_id else "NotStopped")

    def generate(self, prompt, max_new_tokens: int, vocab_size=None, temperature=1.0, top_k=0, top_p=1.0, repetition_penalty=1.0,
                 eos_token_id=None, draw=None, constraint=None) -> list:
        """generate_with_config (nn/src/lib.rs:2526-2553, 2584-2593): prompt + up to max_new_tokens sampled tokens; stops after an
        end-of-sequence token or when no candidate is left; a prompt that already ends with it is returned unchanged.
        ``top_k=1`` is the reference's greedy configuration."""
        if not self.kv_cache_enabled:
            self.enable_kv_cache()
            self.kv_cache_enabled = True
        self._gen_ctx = None
        tokens = [int(t) for t in prompt]
        self._prompt_len = len(tokens)
        if eos_token_id is not None and tokens and tokens[-1] == eos_token_id:
            return tokens
        for _ in range(max_new_tokens):
            nxt, _, reason = self.decode_next_token(tokens, vocab_size, temperature, top_k, top_p, repetition_penalty, eos_token_id, draw,
                                                    constraint)
            if nxt is None or reason != "NotStopped":
                break
        return tokens

    def forward_host(self, ids_host_ptr: int, batch: int, T: int, logits_host_ptr: int, chunk: int):
        """Host-buffer call through the C-ABI: pinned ids in, dense logits out, copies included."""
        self.b._check(self.b.lib.sptorch_ext_gpt_forward_host(self.h, ids_host_ptr, batch, T, logits_host_ptr, chunk), "gpt_forward_host")

    def launches(self, batch: int, T: int) -> int:
        return self.b.lib.sptorch_ext_gpt_launches(self.h, batch, T)


class QwenLikeGPT(GPT):
    """nn::QwenLikeGPT (crates/nn/src/lib.rs:1439-1467): same constructor arguments as the reference's ``new``; RMSNorm
    (eps 1e-6), RoPE on Q and K (base 10000), SwiGLU MLP.  ``forward_ids`` / ``forward`` and the key/value cache calls as for GPT
    (the cache holds the rotated keys, as project_kv_cache_with_offset stores them)."""

    def __init__(self, backend: FfiBackend, vocab_size: int, d_model: int, n_head: int, n_layer: int, d_ff: int, seq_len: int,
                 dtype: int = F32, max_batch: int = 1, eps: float = 1e-6, rope_base: float = 10000.0, tp_rank: int = 0, tp_size: int = 1):
        super().__init__(backend, vocab_size, d_model, n_head, n_layer, d_ff, seq_len, dtype=dtype, max_batch=max_batch, eps=eps,
                         tp_rank=tp_rank, tp_size=tp_size, arch=ARCH_QWEN_LIKE, rope_base=rope_base)
