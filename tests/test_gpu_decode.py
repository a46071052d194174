"""GPU tests of incremental decode with a key/value cache: the last-token attention kernel against the oracle's
restatement of causal_attention_last_token, and the reference's own self-consistency checks (crates/nn/src/lib.rs:3749-3830):
logits decoded from the cache equal the last row of the full forward; appending token by token equals prefilling."""
import numpy as np
import pytest

from conftest import relerr
from sptorch_b200 import synth
from sptorch_b200.backend import BF16, F32, HalError
from sptorch_b200.gpt import GPT

pytestmark = pytest.mark.gpu


# the later cases spread one (sequence, head) pair over a cluster of CTAs (few pairs, long caches): parts of unequal length, parts
# that are empty (n far below the capacity is a property of the graph-replayed step, here n == what the launch sees)
@pytest.mark.parametrize("B,H,hd,P,n", [(1, 2, 4, 6, 3), (3, 4, 32, 64, 64), (2, 12, 64, 256, 200), (2, 2, 128, 40, 1),
                                        (1, 12, 64, 1024, 531), (8, 12, 64, 1024, 700), (1, 2, 64, 2048, 2048), (1, 1, 128, 300, 257),
                                        (1, 3, 64, 1024, 5), (2, 1, 32, 4096, 4001)])
def test_attention_last_token_vs_oracle(backend, oracle, B, H, hd, P, n):
    rng = np.random.default_rng(P + n)
    d = H * hd
    q = rng.standard_normal((B, d)).astype(np.float32)
    k = rng.standard_normal((B, P, d)).astype(np.float32)
    v = rng.standard_normal((B, P, d)).astype(np.float32)
    out = backend.attention_last_token(q, k, v, H, n)
    for b in range(B):
        kh = k[b, :n].reshape(n, H, hd).transpose(1, 0, 2)      # the reference caches [H, n, hd]
        vh = v[b, :n].reshape(n, H, hd).transpose(1, 0, 2)
        ref = oracle.attention_last_token(q[b], kh, vh)
        assert np.abs(out[b] - ref).max() <= 1e-5 * max(1.0, np.abs(ref).max())
    assert relerr(backend.attention_last_token(q, k, v, H, n, dtype=BF16), out) <= 2e-2


def _model(backend, cfg, dtype, max_batch, params, index):
    m = GPT(backend, cfg["vocab"], cfg["d_model"], cfg["n_head"], cfg["n_layer"], cfg["d_ff"], cfg["seq_len"], dtype=dtype, max_batch=max_batch)
    m.load_flat(params, index)
    return m


@pytest.mark.parametrize("dtype,tol", [(F32, 2e-3), (BF16, 3e-2)])
def test_decode_over_a_long_cache_matches_full_forward(backend, dtype, tol):
    """A 512-position cache with two heads: the graph-replayed step launches the last-token attention as clusters of CTAs sized
    for the capacity while the number of valid positions (304, then growing) is read on the device, so some parts are empty.
    Every appended token's logits equal the row of the full forward at its position."""
    cfg = dict(vocab=96, d_model=128, n_layer=2, n_head=2, d_ff=256, seq_len=512)
    params, index = synth.gpt_params(cfg, 11, randomize_affine=True)
    m = _model(backend, cfg, dtype, 2, params, index)
    m.enable_kv_cache(512)
    ids = synth.randint(17, 2 * 312, 96).reshape(2, 312)
    full = m.forward(ids)                                          # causal: row t is the last row of the forward over ids[:, :t + 1]
    m.prefill_kv_cache(ids[:, :304])
    for t in range(304, 312):
        step = m.append_and_decode(ids[:, t])
        assert np.abs(step - full[:, t]).max() <= tol * np.abs(full).max(), t


@pytest.mark.parametrize("nseq", [20, 40, 64])
def test_decode_with_many_sequences_matches_full_forward(backend, nseq):
    """17 .. 64 sequences in bf16: the projections run the weight-streaming kernel with two or four 16-row groups behind a
    normalisation launch of its own, the attention one CTA of four warps per (sequence, head).  Every appended token's logits
    equal the row of the full forward at its position."""
    cfg = dict(vocab=96, d_model=128, n_layer=2, n_head=2, d_ff=256, seq_len=48)
    params, index = synth.gpt_params(cfg, 13, randomize_affine=True)
    m = _model(backend, cfg, BF16, nseq, params, index)
    m.enable_kv_cache(48)
    ids = synth.randint(19, nseq * 40, 96).reshape(nseq, 40)
    full = m.forward(ids)
    m.prefill_kv_cache(ids[:, :32])
    for t in range(32, 40):
        step = m.append_and_decode(ids[:, t])
        assert np.abs(step - full[:, t]).max() <= 3e-2 * np.abs(full).max(), t
    m.close()


# The reference asserts 1e-4 between its two exact-f32 paths.  Here the full forward contracts Q K^T and P V on the tensor
# cores (TF32 / bf16) while the decode kernel works in f32, so the two differ by the contraction tolerance of the mode.
@pytest.mark.parametrize("dtype,tol", [(F32, 2e-3), (BF16, 3e-2)])
def test_incremental_decode_logits_match_full_forward_last_token(backend, dtype, tol):
    # crates/nn/src/lib.rs:3749-3766
    cfg = dict(vocab=64, d_model=64, n_layer=2, n_head=2, d_ff=128, seq_len=32)
    params, index = synth.gpt_params(cfg, 5, randomize_affine=True)
    m = _model(backend, cfg, dtype, 3, params, index)
    m.enable_kv_cache()
    ids = synth.randint(3, 3 * 16, 64).reshape(3, 16)
    full = m.forward(ids)
    pre = m.prefill_kv_cache(ids)
    assert np.array_equal(pre, full)                               # prefill is the ordinary forward
    assert m.cached_len() == 16
    inc = m.decode_logits_from_cache(ids[:, -1])
    scale = np.abs(full).max()
    assert np.abs(inc - full[:, -1]).max() <= tol * scale
    assert m.cached_len() == 16                                    # nothing was appended
    m.close()


@pytest.mark.parametrize("dtype,tol", [(F32, 2e-3), (BF16, 3e-2)])
def test_append_token_by_token_equals_full_forward(backend, oracle, dtype, tol):
    # crates/nn/src/lib.rs:3768-3830: append == prefill; every appended step gives the full forward's row
    cfg = dict(vocab=64, d_model=64, n_layer=2, n_head=2, d_ff=128, seq_len=32)
    params, index = synth.gpt_params(cfg, 6, randomize_affine=True)
    m = _model(backend, cfg, dtype, 2, params, index)
    m.enable_kv_cache()
    ids = synth.randint(4, 2 * 24, 64).reshape(2, 24)
    full = m.forward(ids)
    scale = np.abs(full).max()
    m.prefill_kv_cache(ids[:, :8])
    for t in range(8, 24):
        step = m.append_and_decode(ids[:, t])
        assert m.cached_len() == t + 1
        assert np.abs(step - full[:, t]).max() <= tol * scale, f"position {t}"
    if dtype == F32:
        assert relerr(full, oracle.gpt_forward(cfg, params, ids)) <= 2e-3
    m.close()


def test_decode_error_paths(backend):
    cfg = dict(vocab=32, d_model=32, n_layer=1, n_head=2, d_ff=64, seq_len=16)
    params, index = synth.gpt_params(cfg, 0)
    m = _model(backend, cfg, F32, 2, params, index)
    with pytest.raises(HalError):
        m.decode_logits_from_cache([1, 2])                         # no cache yet
    m.enable_kv_cache(8)
    with pytest.raises(HalError):
        m.decode_logits_from_cache([1, 2])                         # empty cache
    with pytest.raises(HalError):
        m.prefill_kv_cache(np.zeros((2, 12), dtype=np.int64))      # longer than the cache
    m.prefill_kv_cache(np.zeros((2, 8), dtype=np.int64))
    assert np.isfinite(m.append_and_decode([1, 2])).all()          # cache full: the window slides, no error
    assert m.cached_len() == 8 and backend.lib.sptorch_ext_gpt_window_start(m.h) == 1
    with pytest.raises(HalError):
        m.decode_logits_from_cache([1])                            # batch differs from the cached batch
    assert backend.lib.sptorch_sync() == 0                      # the wrapper consumed every reported failure
    assert np.isfinite(m.decode_logits_from_cache([0, 0])).all()
    m.close()


def _oracle_incremental(oracle, cfg, params, index, ids, ctx):
    """decode_logits_from_cache after append_last_token_kv_cache for every token of one sequence, restated with the oracle's
    ops (crates/nn/src/lib.rs:1619-1646, 1205-1214, 706-760, 2165-2203): per layer a first-in-first-out list of the last `ctx`
    keys and values; the position table is read at min(position, seq_len - 1)."""
    def P(name):
        o, shape = index[name]
        return params[o:o + int(np.prod(shape))].reshape(shape)
    d, H, L, S = cfg["d_model"], cfg["n_head"], cfg["n_layer"], cfg["seq_len"]
    hd = d // H
    K = [[] for _ in range(L)]
    V = [[] for _ in range(L)]
    out = []
    for t, tok in enumerate(ids):
        x = (P("token_emb.weight")[tok] + P("pos_emb.weight")[min(t, S - 1)])[None, :].astype(np.float32)
        for l in range(L):
            p = f"blocks.{l}."
            h = oracle.layernorm(x, P(p + "ln1.gamma"), P(p + "ln1.beta"))
            q, k, v = (oracle.linear(h, P(p + f"attn.{n}.weight")) for n in ("wq", "wk", "wv"))
            K[l].append(k[0]); V[l].append(v[0])
            K[l], V[l] = K[l][-ctx:], V[l][-ctx:]
            kh = np.stack(K[l]).reshape(-1, H, hd).transpose(1, 0, 2)
            vh = np.stack(V[l]).reshape(-1, H, hd).transpose(1, 0, 2)
            a = oracle.attention_last_token(q[0], np.ascontiguousarray(kh), np.ascontiguousarray(vh))[None, :]
            x = x + oracle.linear(a, P(p + "attn.wo.weight"))
            h2 = oracle.layernorm(x, P(p + "ln2.gamma"), P(p + "ln2.beta"))
            f = oracle.unary("gelu", oracle.linear(h2, P(p + "ffn_up.weight"), P(p + "ffn_up.bias")))
            x = x + oracle.linear(f, P(p + "ffn_down.weight"), P(p + "ffn_down.bias"))
        out.append(oracle.linear(oracle.layernorm(x, P("ln_f.gamma"), P("ln_f.beta")), P("lm_head.weight"))[0])
    return np.stack(out)


def test_cache_slides_on_the_device_like_append_kv_tensor(backend, oracle):
    """Appending past the capacity of the cache keeps the last max_context positions (append_kv_tensor drops the oldest,
    nn/src/lib.rs:2165-2203) and reads the position table at min(position, seq_len - 1): every step's logits against the
    oracle's restatement of the incremental path, far past the point where the 8-position cache is full."""
    cfg = dict(vocab=50, d_model=32, n_layer=2, n_head=2, d_ff=64, seq_len=12)
    params, index = synth.gpt_params(cfg, 8, randomize_affine=True)
    ids = synth.randint(5, 30, 50)
    ref = _oracle_incremental(oracle, cfg, params, index, ids, ctx=8)
    m = _model(backend, cfg, F32, 1, params, index)
    m.enable_kv_cache(8)
    m.prefill_kv_cache(ids[None, :4])
    scale = np.abs(ref).max()
    for t in range(4, 30):
        step = m.append_and_decode(ids[t:t + 1])
        assert m.cached_len() == min(t + 1, 8)
        assert backend.lib.sptorch_ext_gpt_window_start(m.h) == max(0, t + 1 - 8)
        assert np.abs(step[0] - ref[t]).max() <= 2e-3 * scale, f"position {t}"
    m.close()
