"""GPU parity tests of the Qwen-like variant of the forward path (crates/nn/src/lib.rs: RoPE :930-983, QwenLikeBlock :1062-1131,
QwenLikeGPT :1439-1467): the rotary kernel, the SwiGLU epilogue of the gate projection, and the whole forward per layer."""
import numpy as np
import pytest

from conftest import relerr
from sptorch_b200 import synth
from sptorch_b200.backend import BF16, EPI_SWIGLU, F32, MM_BF16, MM_F32, MM_TF32, HalError, bf16_bits_to_f32, f32_to_bf16_bits
from sptorch_b200.gpt import QwenLikeGPT

pytestmark = pytest.mark.gpu
TOL = {F32: 2e-3, BF16: 2e-2}


def _bf16(x):
    return bf16_bits_to_f32(f32_to_bf16_bits(x)).reshape(np.shape(x))


def test_rope_known_answers(backend):
    # test_rope_keeps_position_zero_and_rotates_later_positions (nn/src/lib.rs:3313-3329)
    out = backend.rope(np.array([[[1, 2, 3, 4], [1, 0, 0, 1]]], np.float32))
    assert np.array_equal(out[0, 0], [1, 2, 3, 4])
    assert abs(out[0, 1, 0] - 1.0) > 1e-3 or abs(out[0, 1, 1]) > 1e-3
    assert np.allclose(out[0, 1], [np.cos(1.0), np.sin(1.0), -np.sin(0.01), np.cos(0.01)], atol=1e-6)
    # test_rope_offset_matches_sliced_full_sequence_position (:3331-3347)
    full = np.arange(1, 13, dtype=np.float32).reshape(1, 3, 4)
    assert np.array_equal(backend.rope(full)[0, 2], backend.rope(full[:, 2:3], position_offset=2)[0, 0])
    with pytest.raises(HalError):
        backend.rope(np.zeros((1, 2, 3), np.float32))          # odd head_dim: the reference asserts


@pytest.mark.parametrize("H,T,hd", [(1, 1, 2), (2, 7, 6), (4, 64, 32), (12, 128, 64), (3, 1024, 128), (2, 33, 20)])
def test_rope_vs_oracle(backend, oracle, H, T, hd):
    rng = np.random.default_rng(H * T + hd)
    x = rng.standard_normal((H, T, hd)).astype(np.float32)
    for off in (0, 5):
        ref = oracle.rope(x, 10000.0, off)
        # sincosf on the device and sinf / cosf on the host agree to a few ulp of a value <= 1
        assert np.abs(backend.rope(x, 10000.0, off) - ref).max() <= 4e-6 * max(1.0, np.abs(x).max())
    ref = oracle.rope(_bf16(x), 500.0, 3)
    assert np.abs(backend.rope(_bf16(x), 500.0, 3, dtype=BF16) - ref).max() <= 2 ** -8 * np.abs(ref).max()


@pytest.mark.parametrize("M,K,N", [(64, 32, 48), (200, 128, 328), (512, 768, 3072)])
def test_swiglu_epilogue_vs_oracle(backend, oracle, M, K, N):
    """gate projection with the SwiGLU product in the epilogue == swiglu(up, linear(h, Wgate, bgate)) of the oracle."""
    rng = np.random.default_rng(M + N)
    h = rng.standard_normal((M, K)).astype(np.float32)
    wg = (0.05 * rng.standard_normal((N, K))).astype(np.float32)
    bg = (0.1 * rng.standard_normal(N)).astype(np.float32)
    up = rng.standard_normal((M, N)).astype(np.float32)
    ref = oracle.swiglu(up, oracle.linear(h, wg, bg, fast=2))
    assert relerr(backend.linear(h, wg, bg, residual=up, epilogue=EPI_SWIGLU, mode=MM_F32), ref) <= 5e-6
    assert relerr(backend.linear(h, wg, bg, residual=up, epilogue=EPI_SWIGLU, mode=MM_TF32), ref) <= 2e-3
    assert relerr(backend.linear(h, wg, bg, residual=up, epilogue=EPI_SWIGLU, mode=MM_BF16), ref) <= 2e-2
    with pytest.raises(HalError):
        backend.linear(h, wg, bg, epilogue=EPI_SWIGLU, mode=MM_TF32)     # the product needs its other factor


def _qwen(backend, cfg, dtype, max_batch, params, index):
    m = QwenLikeGPT(backend, cfg["vocab"], cfg["d_model"], cfg["n_head"], cfg["n_layer"], cfg["d_ff"], cfg["seq_len"], dtype=dtype, max_batch=max_batch)
    m.load_flat(params, index)
    return m


def test_qwen_like_reference_test_shape(backend, oracle):
    # test_qwen_like_gpt_forward_and_backward (nn/src/lib.rs:3367-3376): QwenLikeGPT::new(12, 8, 2, 1, 16, 6), ids [0,1,2,3] -> [4, 12]
    cfg = dict(vocab=12, d_model=8, n_layer=1, n_head=2, d_ff=16, seq_len=6)
    params, index = synth.gpt_params(cfg, 0, arch="qwen", randomize_affine=True)
    m = _qwen(backend, cfg, F32, 1, params, index)
    out = m.forward_ids([0, 1, 2, 3])
    assert out.shape == (4, 12)
    assert relerr(out, oracle.qwen_forward(cfg, params, np.array([[0, 1, 2, 3]]))[0]) <= 2e-3
    with pytest.raises(HalError):
        m.set_param("pos_emb.weight", np.zeros(6 * 8, np.float32))       # no position table in this model
    m.close()


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_qwen_like_forward_vs_oracle_per_layer(backend, oracle, dtype):
    cfg = dict(vocab=256, d_model=128, n_layer=4, n_head=4, d_ff=512, seq_len=64)     # the dimensions of c1_tiny
    params, index = synth.gpt_params(cfg, 3, arch="qwen", randomize_affine=True)
    ids = synth.randint(7, 8 * 64, 256).reshape(8, 64)
    ref, taps = oracle.qwen_forward(cfg, params, ids, fast=0, threads=oracle.max_threads(), want_taps=True)
    m = _qwen(backend, cfg, dtype, 8, params, index)
    m.enable_taps()
    out = m.forward(ids)
    assert relerr(out, ref) <= TOL[dtype]
    for i in range(cfg["n_layer"] + 2):
        assert relerr(m.tap(i, 8 * 64).reshape(8, 64, -1), taps[:, i]) <= TOL[dtype], f"layer tap {i}"
    # graph replay (third call onwards) gives the same bits as the eager first call
    m.enable_taps(False)
    d_ids, d_log = m.stage_ids(ids), m.logits_buffer(8 * 64)
    outs = []
    for _ in range(4):
        m.forward_device(d_ids, 8, 64, d_log)
        outs.append(d_log.to_host().copy())
    assert all(np.array_equal(outs[0], o) for o in outs[1:])
    m.close()


def test_qwen_like_gpt2_small_shape_layer_slice(backend, oracle):
    """Two layers at the c4_gpt2s widths (d 768, 12 heads x 64, d_ff 3072, T 256): the fused attention kernel and the
    wide GEMMs on the RoPE / SwiGLU path."""
    cfg = dict(vocab=1000, d_model=768, n_layer=2, n_head=12, d_ff=3072, seq_len=256)
    params, index = synth.gpt_params(cfg, 5, arch="qwen", residual_scale=True, randomize_affine=True)
    ids = synth.randint(11, 2 * 256, 1000).reshape(2, 256)
    ref = oracle.qwen_forward(cfg, params, ids, fast=1, threads=oracle.max_threads())
    m = _qwen(backend, cfg, BF16, 2, params, index)
    assert relerr(m.forward(ids), ref) <= 2e-2
    m.close()


# 2 sequences: the projections normalise their rows themselves; 20: a normalisation launch of its own in front of them (17 .. 64 rows)
@pytest.mark.parametrize("nseq", [2, 20])
@pytest.mark.parametrize("dtype,tol", [(F32, 2e-3), (BF16, 3e-2)])
def test_qwen_like_incremental_decode_equals_full_forward(backend, dtype, tol, nseq):
    """The reference's self-consistency checks for the cache path (crates/nn/src/lib.rs:3749-3830) on the RoPE model: decoding from
    the cache equals the last row of the full forward, appending token by token equals the full forward's rows.  The cache
    holds rotated keys (project_kv_cache_with_offset, :672-683); the query is rotated to its absolute position (:718-721)."""
    cfg = dict(vocab=64, d_model=64, n_layer=2, n_head=2, d_ff=128, seq_len=32)
    params, index = synth.gpt_params(cfg, 9, arch="qwen", randomize_affine=True)
    m = _qwen(backend, cfg, dtype, nseq, params, index)
    m.enable_kv_cache()
    ids = synth.randint(4, nseq * 24, 64).reshape(nseq, 24)
    full = m.forward(ids)
    scale = np.abs(full).max()
    pre = m.prefill_kv_cache(ids[:, :8])
    assert np.array_equal(pre, m.forward(ids[:, :8]))
    assert np.abs(m.decode_logits_from_cache(ids[:, 7]) - full[:, 7]).max() <= tol * scale
    for t in range(8, 24):
        step = m.append_and_decode(ids[:, t])
        assert m.cached_len() == t + 1
        assert np.abs(step - full[:, t]).max() <= tol * scale, f"position {t}"
    m.close()
