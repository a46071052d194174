"""Seeded synthetic inputs shared by the CPU oracle and the device path.

The reference has no reproducible random fixture (all of its initialisers call
``rand::thread_rng()``: crates/nn/src/lib.rs:60,70,337), so this module defines
one: a counter-based SplitMix64 stream turned into uniforms and Box-Muller
normals.  Element ``i`` of stream ``seed`` depends only on ``(seed, i)``, so any
slice can be generated independently and identically on any host.
"""
from __future__ import annotations

import numpy as np

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = x + _GOLDEN
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def _bits(seed: int, start: int, n: int, lane: int) -> np.ndarray:
    """64 random bits for counters start..start+n-1 of (seed, lane)."""
    with np.errstate(over="ignore"):
        base = _splitmix64(np.array([seed * 4 + lane], dtype=np.uint64))[0]
        ctr = np.arange(start, start + n, dtype=np.uint64)
        return _splitmix64(ctr * _GOLDEN + base)


def uniform01(seed: int, n: int, start: int = 0, lane: int = 0) -> np.ndarray:
    """n doubles in (0, 1): top 53 bits, offset by half an ulp so 0 never occurs."""
    b = _bits(seed, start, n, lane)
    return ((b >> np.uint64(11)).astype(np.float64) + 0.5) * (1.0 / 9007199254740992.0)


def _normal_chunk(seed: int, start: int, m: int) -> np.ndarray:
    b = _bits(seed, start, m, lane=0)
    # one 64-bit draw per element: top 32 bits -> u1 in (0,1), low 32 bits -> u2 in (0,1)
    u1 = ((b >> np.uint64(32)).astype(np.float64) + 0.5) * (1.0 / 4294967296.0)
    u2 = ((b & np.uint64(0xFFFFFFFF)).astype(np.float64) + 0.5) * (1.0 / 4294967296.0)
    np.log(u1, out=u1)
    u1 *= -2.0
    np.sqrt(u1, out=u1)
    u2 *= 2.0 * np.pi
    np.cos(u2, out=u2)
    u1 *= u2
    return u1


def normal(seed: int, n: int, mean: float = 0.0, std: float = 1.0, start: int = 0,
           chunk: int = 1 << 21) -> np.ndarray:
    """n float32 normals: element i = mean + std * sqrt(-2 ln u1_i) * cos(2 pi u2_i), with
    (u1_i, u2_i) the two 32-bit halves of draw ``start + i``.  Chunks run on a thread pool
    (numpy releases the GIL); the result does not depend on the chunking."""
    out = np.empty(n, dtype=np.float32)

    def work(s):
        m = min(chunk, n - s)
        out[s:s + m] = (mean + std * _normal_chunk(seed, start + s, m)).astype(np.float32)

    starts = range(0, n, chunk)
    if n > chunk:
        from concurrent.futures import ThreadPoolExecutor
        import os
        with ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 1)) as ex:
            list(ex.map(work, starts))
    else:
        for s in starts:
            work(s)
    return out


def randint(seed: int, n: int, high: int, start: int = 0) -> np.ndarray:
    """n int64 ids uniform in [0, high) (multiply-shift on the top 32 bits)."""
    b = _bits(seed, start, n, lane=2) >> np.uint64(32)
    return ((b * np.uint64(high)) >> np.uint64(32)).astype(np.int64)


# ---- GPT parameter block in GPT::named_parameters order (crates/nn/src/lib.rs:1382-1392) ----

def gpt_param_layout(vocab, d_model, n_layer, n_head, d_ff, seq_len):
    """[(name, shape)] in the reference's named_parameters order."""
    d, F = d_model, d_ff
    names = [("token_emb.weight", (vocab, d)), ("pos_emb.weight", (seq_len, d))]
    for i in range(n_layer):
        p = f"blocks.{i}."
        names += [
            (p + "ln1.gamma", (d,)), (p + "ln1.beta", (d,)),
            (p + "attn.wq.weight", (d, d)), (p + "attn.wk.weight", (d, d)),
            (p + "attn.wv.weight", (d, d)), (p + "attn.wo.weight", (d, d)),
            (p + "ln2.gamma", (d,)), (p + "ln2.beta", (d,)),
            (p + "ffn_up.weight", (F, d)), (p + "ffn_up.bias", (F,)),
            (p + "ffn_down.weight", (d, F)), (p + "ffn_down.bias", (d,)),
        ]
    names += [("ln_f.gamma", (d,)), ("ln_f.beta", (d,)), ("lm_head.weight", (vocab, d))]
    return names


def qwen_param_layout(vocab, d_model, n_layer, n_head, d_ff, seq_len):
    """[(name, shape)] of QwenLikeGPT::named_parameters (crates/nn/src/lib.rs:1483-1492, block :1157-1166)."""
    d, F = d_model, d_ff
    names = [("token_emb.weight", (vocab, d))]
    for i in range(n_layer):
        p = f"blocks.{i}."
        names += [
            (p + "norm1.weight", (d,)),
            (p + "attn.wq.weight", (d, d)), (p + "attn.wk.weight", (d, d)),
            (p + "attn.wv.weight", (d, d)), (p + "attn.wo.weight", (d, d)),
            (p + "norm2.weight", (d,)),
            (p + "ffn_up.weight", (F, d)), (p + "ffn_up.bias", (F,)),
            (p + "ffn_gate.weight", (F, d)), (p + "ffn_gate.bias", (F,)),
            (p + "ffn_down.weight", (d, F)), (p + "ffn_down.bias", (d,)),
        ]
    names += [("norm_f.weight", (d,)), ("lm_head.weight", (vocab, d))]
    return names


def gpt_params(cfg: dict, seed: int = 0, residual_scale: bool = False, randomize_affine: bool = False, arch: str = "gpt"):
    """Flat float32 parameter block + {name: (offset, shape)}.

    Every ``*.weight`` ~ N(0, 0.02) drawn from one stream in layout order, biases 0,
    gamma (and RMSNorm weights) 1, beta 0.  ``arch="qwen"`` gives the QwenLikeGPT block instead.  ``residual_scale`` multiplies attn.wo and ffn_down weights by
    1/sqrt(2*n_layer).  ``randomize_affine`` (tests only) draws gamma/beta/biases too so
    that a wrong bias or affine path cannot hide behind zeros.
    """
    layout = (qwen_param_layout if arch == "qwen" else gpt_param_layout)(cfg["vocab"], cfg["d_model"], cfg["n_layer"], cfg["n_head"],
                                                                         cfg["d_ff"], cfg["seq_len"])
    total = sum(int(np.prod(s)) for _, s in layout)
    flat = np.empty(total, dtype=np.float32)
    index = {}
    off = 0
    rs = 1.0 / np.sqrt(2.0 * cfg["n_layer"])
    for name, shape in layout:
        n = int(np.prod(shape))
        is_norm_scale = name.endswith(".gamma") or ".norm" in name or name.startswith("norm")     # LayerNorm gamma / RMSNorm weight: 1
        if name.endswith(".weight") and not is_norm_scale:
            w = normal(seed, n, 0.0, 0.02, start=off)
            if residual_scale and (name.endswith("attn.wo.weight") or name.endswith("ffn_down.weight")):
                w = (w * np.float32(rs)).astype(np.float32)
            flat[off:off + n] = w
        elif is_norm_scale:
            flat[off:off + n] = 1.0 + (normal(seed + 101, n, 0.0, 0.1, start=off) if randomize_affine else 0.0)
        else:  # beta / bias
            flat[off:off + n] = normal(seed + 202, n, 0.0, 0.05, start=off) if randomize_affine else 0.0
        index[name] = (off, shape)
        off += n
    return flat, index


CONFIGS = {
    # the tiny character model c1_tiny: tiny char-level GPT (f32)
    "c1_tiny": dict(vocab=256, d_model=128, n_layer=4, n_head=4, d_ff=512, seq_len=64, batch=8, ctx=64),
    # the GPT-2-small shape c4_gpt2s: GPT-2-small shape (bf16)
    "c4_gpt2s": dict(vocab=50257, d_model=768, n_layer=12, n_head=12, d_ff=3072, seq_len=1024, batch=64, ctx=1024),
    # the 1.3B shape c5_1p3b: 1.3B shape (bf16, tensor parallel)
    "c5_1p3b": dict(vocab=50257, d_model=2048, n_layer=24, n_head=16, d_ff=8192, seq_len=2048, batch=16, ctx=2048),
}
