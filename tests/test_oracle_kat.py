"""Pins the CPU oracle: replays the known-answer vectors of the reference's own unit tests and
cross-checks the eleven C-ABI ops against the reference's C implementation compiled in place
(oracle/_ref/libmock_npu.so, built from crates/hal-ffi/mock_npu/mock_npu.c)."""
import ctypes as C
import json
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_add_mul_neg_scale_relu_kat(oracle):
    # crates/hal/src/lib.rs:724-742, 767-822; crates/hal-ffi/tests/test_ffi_mock.rs:58-103
    assert oracle.binary("add", [1, 2, 3], [4, 5, 6]).tolist() == [5, 7, 9]
    assert oracle.binary("mul", [2, 3], [4, 5]).tolist() == [8, 15]
    assert oracle.unary("neg", [1, -2, 3]).tolist() == [-1, 2, -3]
    assert oracle.scale([1, 2, 3], 0.5).tolist() == [0.5, 1.0, 1.5]
    assert oracle.unary("relu", [-1, 0, 2, -0.5]).tolist() == [0, 0, 2, 0]


def test_matmul_kat(oracle):
    # crates/core-ops/src/lib.rs:2006-2011; crates/hal/src/lib.rs:746-754; test_ffi_mock.rs:105-113
    a = np.array([[1, 2, 3], [4, 5, 6]], dtype=np.float32)
    b = np.array([[7, 8], [9, 10], [11, 12]], dtype=np.float32)
    assert oracle.matmul(a, b).ravel().tolist() == [58, 64, 139, 154]
    assert oracle.matmul(a, b, f64=True).ravel().tolist() == [58, 64, 139, 154]


def test_batch_matmul_kat(oracle):
    # crates/core-ops/src/lib.rs:2578-2605; crates/hal/src/lib.rs:838-846
    c = oracle.batch_matmul(np.array([1, 2, 3, 4], dtype=np.float32).reshape(1, 2, 2), np.array([5, 6, 7, 8], dtype=np.float32).reshape(1, 2, 2))
    assert c.ravel().tolist() == [19, 22, 43, 50]
    a = np.array([1, 0, 0, 1, 2, 0, 0, 2], dtype=np.float32).reshape(2, 2, 2)
    b = np.array([3, 4, 5, 6, 3, 4, 5, 6], dtype=np.float32).reshape(2, 2, 2)
    assert oracle.batch_matmul(a, b).ravel().tolist() == [3, 4, 5, 6, 6, 8, 10, 12]
    ident = np.array([1, 0, 0, 1, 1, 0, 0, 1], dtype=np.float32).reshape(2, 2, 2)
    x = np.arange(1, 9, dtype=np.float32).reshape(2, 2, 2)
    assert np.array_equal(oracle.batch_matmul(x, ident), x)


def test_softmax_kat(oracle):
    # crates/core-ops/src/lib.rs:2296-2314; crates/hal/src/lib.rs:826-834
    for hal in (False, True):
        s = oracle.softmax(np.array([[1, 2, 3], [1, 2, 3]], dtype=np.float32), hal=hal)
        assert abs(s[0].sum() - 1) < 1e-6 and abs(s[1].sum() - 1) < 1e-6
        assert s[0, 2] > s[0, 1] > s[0, 0]
    # the two statements of softmax in the reference agree to rounding
    x = np.random.default_rng(0).standard_normal((7, 33)).astype(np.float32)
    assert np.abs(oracle.softmax(x) - oracle.softmax(x, hal=True)).max() < 1e-7


def test_embedding_kat(oracle):
    # crates/core-ops/src/lib.rs:2418-2427; crates/hal/src/lib.rs:861-869
    w = np.array([0.1, 0.2, 0.3, 0.4, 0.5, 0.6, 0.7, 0.8, 0.9, 1.0, 1.1, 1.2], dtype=np.float32).reshape(4, 3)
    assert np.array_equal(oracle.embedding(w, [0, 2, 3]).ravel(), np.array([0.1, 0.2, 0.3, 0.7, 0.8, 0.9, 1.0, 1.1, 1.2], dtype=np.float32))
    w2 = np.array([0.1, 0.2, 0.3, 0.4, 0.5, 0.6], dtype=np.float32).reshape(3, 2)
    assert np.array_equal(oracle.embedding(w2, [2, 0, 1]).ravel(), np.array([0.5, 0.6, 0.1, 0.2, 0.3, 0.4], dtype=np.float32))
    with pytest.raises(IndexError):   # the reference asserts idx < num_embeddings (core-ops/src/lib.rs:1229)
        oracle.embedding(w2, [3])


def test_gelu_kat(oracle):
    # crates/core-ops/src/lib.rs:2467-2473; crates/hal/src/lib.rs:804-812
    d = oracle.unary("gelu", [-1.0, 0.0, 1.0, 2.0])
    assert abs(d[1]) < 1e-6 and d[0] < 0 and d[2] > 0.8
    assert abs(d[2] - 0.8413) < 1e-3 and abs(d[0] + 0.1587) < 1e-3


def test_masked_fill_kat(oracle):
    # crates/core-ops/src/lib.rs:2539-2548; crates/hal/src/lib.rs:873-880
    out = oracle.masked_fill([1, 2, 3, 4], [False, True, False, True], -np.inf)
    assert out[0] == 1 and out[2] == 3 and np.isneginf(out[1]) and np.isneginf(out[3])
    assert oracle.masked_fill([1, 2, 3, 4], [0, 1, 0, 1], -999.0).tolist() == [1, -999, 3, -999]


def test_masked_softmax_kat(oracle):
    # crates/core-ops/src/lib.rs:2561-2574: keep-polarity, masked entries exactly zero
    d = oracle.masked_softmax(np.array([[1, 2], [3, 4]], dtype=np.float32), [True, False, True, True]).ravel()
    assert d[0] == 1.0 and d[1] == 0.0 and abs(d[2] + d[3] - 1) < 1e-6
    # a row with nothing kept stays zero (2-D); rank-1 with everything underflowing -> uniform over kept
    z = oracle.masked_softmax(np.array([[1, 2], [3, 4]], dtype=np.float32), [False, False, True, True])
    assert z[0].tolist() == [0, 0]
    r1 = oracle.masked_softmax(np.array([-np.inf, -np.inf, 1.0], dtype=np.float32), [True, True, False])
    assert r1.tolist() == [0.5, 0.5, 0.0]


def test_rms_norm_swiglu_cross_entropy_kat(oracle):
    # crates/core-ops/src/lib.rs:2482-2490, 2505-2511, 2366-2380, 2394-2397
    d = oracle.rms_norm(np.array([[3, 4], [1, 2]], np.float32), [1, 2], 1e-6).ravel()
    assert abs(d[0] - 0.8485) < 1e-3 and abs(d[1] - 2.2627) < 1e-3
    s = oracle.swiglu([1.0, 2.0], [0.0, 1.0])
    assert abs(s[0]) < 1e-6 and abs(s[1] - 1.4621) < 1e-3
    assert abs(oracle.cross_entropy(np.zeros((1, 3), np.float32), [0]) - np.log(3)) < 1e-5
    assert abs(oracle.cross_entropy(np.zeros((2, 3), np.float32), [0, 1]) - np.log(3)) < 1e-5
    big = np.iinfo(np.int64).max
    assert abs(oracle.cross_entropy(np.zeros((2, 3), np.float32), [big, 1], ignore_index=big) - np.log(3)) < 1e-5
    assert oracle.cross_entropy(np.zeros((2, 3), np.float32), [big, big], ignore_index=big) == 0.0
    with pytest.raises(IndexError):
        oracle.cross_entropy(np.zeros((2, 3), np.float32), [0, 3])


def test_broadcast_add_kat(oracle):
    # crates/core-ops/src/lib.rs:2621-2626; crates/hal/src/lib.rs:884-891
    assert oracle.broadcast_add([1, 2, 3, 4, 5, 6], [10, 20, 30]).tolist() == [11, 22, 33, 14, 25, 36]


def test_transpose_and_heads(oracle):
    a = np.arange(6, dtype=np.float32).reshape(2, 3)
    assert np.array_equal(oracle.transpose(a), a.T)


def test_layernorm_properties(oracle):
    # crates/nn/src/lib.rs:3239-3262: gamma=1, beta=0 -> per-row mean ~ 0, variance ~ 1
    x = np.random.default_rng(1).standard_normal((5, 64)).astype(np.float32) * 3 + 0.5
    y = oracle.layernorm(x, np.ones(64), np.zeros(64))
    assert np.abs(y.mean(-1)).max() < 1e-5
    assert np.abs(y.var(-1) - 1).max() < 1e-3
    ref = (x - x.mean(-1, keepdims=True)) / np.sqrt(x.var(-1, keepdims=True) + 1e-5)
    assert np.abs(y - ref).max() < 1e-5


def test_sgd_kat(oracle):
    # crates/hal/src/lib.rs:850-857
    p = np.array([1.0, 2.0], dtype=np.float32); g = np.array([0.1, 0.2], dtype=np.float32)
    oracle.lib().orc_sgd_update(p.ctypes.data_as(C.POINTER(C.c_float)), g.ctypes.data_as(C.POINTER(C.c_float)), C.c_float(0.1), C.c_size_t(2))
    assert abs(p[0] - 0.99) < 1e-6 and abs(p[1] - 1.98) < 1e-6


def test_causal_attention_first_row_is_one_hot(oracle):
    # crates/nn/src/lib.rs:612-632: row 0 of the causal softmax is [1, 0, ..., 0] exactly
    s = np.random.default_rng(2).standard_normal((2, 8, 8)).astype(np.float32)
    p = oracle.causal_softmax(s, 0.5)
    assert np.array_equal(p[:, 0, :], np.eye(8, dtype=np.float32)[0][None].repeat(2, 0))
    assert (np.triu(p, 1) == 0).all() and np.abs(p.sum(-1) - 1).max() < 1e-6


def test_linear_variants_agree(oracle):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((17, 40)).astype(np.float32); w = rng.standard_normal((9, 40)).astype(np.float32); b = rng.standard_normal(9).astype(np.float32)
    y0, y1, y2 = (oracle.linear(x, w, b, fast=f) for f in (0, 1, 2))
    assert np.abs(y0 - y2).max() < 2e-5 and np.abs(y1 - y2).max() < 2e-5
    # strict variant == transpose + matmul + bias exactly (crates/nn/src/lib.rs:123-133)
    assert np.array_equal(y0, oracle.matmul(x, oracle.transpose(w)) + b)


def test_gpt_self_consistency(oracle):
    # the reference has no golden logits; its own self-consistency check is prefix stability of the causal model
    # (crates/nn/src/lib.rs:3749-3766): logits of a prefix do not depend on later tokens
    from sptorch_b200 import synth
    cfg = dict(vocab=50, d_model=32, n_layer=2, n_head=4, d_ff=64, seq_len=16)
    p, _ = synth.gpt_params(cfg, 0, randomize_affine=True)
    ids = synth.randint(1, 16, 50).reshape(1, 16)
    full = oracle.gpt_forward(cfg, p, ids)
    pre = oracle.gpt_forward(cfg, p, ids[:, :9])
    assert np.abs(full[0, :9] - pre[0]).max() < 1e-5


ABI_UNARY = ["neg", "exp", "log", "relu", "gelu"]


@pytest.mark.skipif(not os.path.exists(os.path.join(os.path.dirname(__file__), "..", "oracle", "_ref", "libmock_npu.so")),
                    reason="reference C implementation not built (no reference checkout)")
def test_oracle_vs_reference_c_implementation(oracle):
    """The reference's own C file implements 11 ops of the path; the restatement must agree with it."""
    ref = oracle.ref_lib()
    assert ref.sptorch_backend_init() == 0
    assert ref.sptorch_backend_name() == b"mock_npu"
    rng = np.random.default_rng(4)
    fp = C.POINTER(C.c_float)
    n = 4099
    x = rng.standard_normal(n).astype(np.float32); y = rng.standard_normal(n).astype(np.float32)
    out = np.empty(n, dtype=np.float32)
    p = lambda a: a.ctypes.data_as(fp)
    for name in ("add", "mul"):
        getattr(ref, f"sptorch_{name}_f32")(p(x), p(y), p(out), C.c_size_t(n))
        assert np.array_equal(out, oracle.binary(name, x, y)), name
    for name in ABI_UNARY:
        xin = np.abs(x) + 0.1 if name == "log" else x
        getattr(ref, f"sptorch_{name}_f32")(p(xin), p(out), C.c_size_t(n))
        got = oracle.unary(name, xin)
        if name == "gelu":   # mock_npu.c uses sqrtf(2/3.14159265f) and x*x*x: <= 2 ulp apart from core-ops' form
            assert np.abs(out - got).max() <= 4e-7 * max(1.0, np.abs(got).max()), name
        else:
            assert np.array_equal(out, got), name
    ref.sptorch_scale_f32(p(x), C.c_float(0.37), p(out), C.c_size_t(n))
    assert np.array_equal(out, oracle.scale(x, 0.37))
    a = rng.standard_normal((13, 29)).astype(np.float32); b = rng.standard_normal((29, 7)).astype(np.float32)
    o = np.empty((13, 7), dtype=np.float32)
    ref.sptorch_matmul_f32(p(a), p(b), p(o), C.c_size_t(13), C.c_size_t(29), C.c_size_t(7))
    assert np.array_equal(o, oracle.matmul(a, b))
    a3 = rng.standard_normal((3, 5, 6)).astype(np.float32); b3 = rng.standard_normal((3, 6, 4)).astype(np.float32)
    o3 = np.empty((3, 5, 4), dtype=np.float32)
    ref.sptorch_batch_matmul_f32(p(a3), p(b3), p(o3), C.c_size_t(3), C.c_size_t(5), C.c_size_t(6), C.c_size_t(4))
    assert np.array_equal(o3, oracle.batch_matmul(a3, b3))
    s = rng.standard_normal((11, 37)).astype(np.float32); so = np.empty_like(s)
    ref.sptorch_softmax_f32(p(s), p(so), C.c_size_t(11), C.c_size_t(37))
    assert np.array_equal(so, oracle.softmax(s, hal=True))
    assert np.abs(so - oracle.softmax(s)).max() < 1e-7


def test_golden_fixture_matches_oracle(oracle):
    """tests/golden/c1_tiny.npz was written by tests/golden/make_golden.py from the oracle (strict order) and,
    for the C-ABI ops, from the reference's C implementation; the oracle must still reproduce it."""
    from sptorch_b200 import synth
    path = os.path.join(GOLDEN, "c1_tiny.npz")
    g = np.load(path)
    cfg = synth.CONFIGS["c1_tiny"]
    p, _ = synth.gpt_params(cfg, 0)
    ids = synth.randint(1, 8 * 64, 256).reshape(8, 64)
    assert np.array_equal(ids[:2], g["ids"])
    logits = oracle.gpt_forward(cfg, p, ids[:2], fast=0)
    assert np.abs(logits[:, :, :64] - g["logits_first64"]).max() < 1e-5
    assert np.array_equal(logits.argmax(-1), g["argmax"])


def test_rope_known_answers_and_numpy_restatement(oracle):
    # test_rope_keeps_position_zero_and_rotates_later_positions (nn/src/lib.rs:3313-3329)
    out = oracle.rope(np.array([[[1, 2, 3, 4], [1, 0, 0, 1]]], np.float32))
    assert np.array_equal(out[0, 0], [1, 2, 3, 4])
    assert abs(out[0, 1, 0] - 1.0) > 1e-3 or abs(out[0, 1, 1]) > 1e-3
    # test_rope_offset_matches_sliced_full_sequence_position (:3331-3347)
    full = np.arange(1, 13, dtype=np.float32).reshape(1, 3, 4)
    assert np.array_equal(oracle.rope(full)[0, 2], oracle.rope(full[:, 2:3], position_offset=2)[0, 0])
    # the inverse rotation (the backward of the reference, :1010-1023) undoes the forward one
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 17, 8)).astype(np.float32)
    assert np.allclose(oracle.rope(oracle.rope(x, 10000.0, 4), 10000.0, 4, inverse=True), x, atol=1e-5)
    # independent float64 statement of the same rotation
    pos = np.arange(17)[None, :, None] + 4
    theta = pos / (10000.0 ** (2 * np.arange(4)[None, None, :] / 8))
    ev, od = x[..., 0::2].astype(np.float64), x[..., 1::2].astype(np.float64)
    ref = np.empty_like(x, dtype=np.float64)
    ref[..., 0::2] = ev * np.cos(theta) - od * np.sin(theta)
    ref[..., 1::2] = ev * np.sin(theta) + od * np.cos(theta)
    assert np.allclose(oracle.rope(x, 10000.0, 4), ref, atol=2e-6)
    with pytest.raises(ValueError):
        oracle.rope(np.zeros((1, 2, 3), np.float32))


def test_qwen_like_forward_against_numpy_restatement(oracle):
    """QwenLikeGPT::forward_ids (nn/src/lib.rs:1454-1467) at the size of the reference's own test (:3367-3376), against a float64
    numpy statement of the same graph written independently of oracle.c."""
    from sptorch_b200 import synth
    cfg = dict(vocab=12, d_model=8, n_layer=2, n_head=2, d_ff=16, seq_len=6)
    params, index = synth.gpt_params(cfg, 0, arch="qwen", randomize_affine=True)
    P = {k: params[o:o + int(np.prod(s))].reshape(s).astype(np.float64) for k, (o, s) in index.items()}
    ids = np.array([[0, 1, 2, 3], [11, 5, 5, 7]])
    out, taps = oracle.qwen_forward(cfg, params, ids, want_taps=True)
    assert out.shape == (2, 4, 12)
    d, H, hd, T = 8, 2, 4, 4

    def rms(v, w):
        return v / np.sqrt((v * v).mean(-1, keepdims=True) + 1e-6) * w

    def rope(v):                      # [T, d] token-major, head h at columns h*hd
        v = v.reshape(T, H, hd).copy()
        theta = np.arange(T)[:, None, None] / (10000.0 ** (2 * np.arange(hd // 2)[None, None, :] / hd))
        ev, od = v[..., 0::2].copy(), v[..., 1::2].copy()
        v[..., 0::2] = ev * np.cos(theta) - od * np.sin(theta)
        v[..., 1::2] = ev * np.sin(theta) + od * np.cos(theta)
        return v

    for b in range(2):
        x = P["token_emb.weight"][ids[b]]
        for l in range(2):
            p = f"blocks.{l}."
            h = rms(x, P[p + "norm1.weight"])
            q, k = rope(h @ P[p + "attn.wq.weight"].T), rope(h @ P[p + "attn.wk.weight"].T)
            v = (h @ P[p + "attn.wv.weight"].T).reshape(T, H, hd)
            sc = np.einsum("ihe,jhe->hij", q, k) / np.sqrt(hd)
            sc = np.where(np.triu(np.ones((T, T), bool), 1)[None], -np.inf, sc)
            pr = np.exp(sc - sc.max(-1, keepdims=True)); pr /= pr.sum(-1, keepdims=True)
            x = x + np.einsum("hij,jhe->ihe", pr, v).reshape(T, d) @ P[p + "attn.wo.weight"].T
            h = rms(x, P[p + "norm2.weight"])
            up = h @ P[p + "ffn_up.weight"].T + P[p + "ffn_up.bias"]
            g = h @ P[p + "ffn_gate.weight"].T + P[p + "ffn_gate.bias"]
            x = x + (up * g / (1 + np.exp(-g))) @ P[p + "ffn_down.weight"].T + P[p + "ffn_down.bias"]
            assert np.allclose(taps[b, l + 1], x, atol=1e-5)
        logits = rms(x, P["norm_f.weight"]) @ P["lm_head.weight"].T
        assert np.allclose(out[b], logits, atol=1e-5)


def test_sampling_candidates_known_answers(oracle):
    # test_sampling_candidates_apply_top_p_after_probability_sort (nn/src/lib.rs:3833-3845)
    ids, lg, pr = oracle.sampling_candidates([3.0, 2.0, 1.0, 0.0], top_p=0.75)
    assert list(ids) == [0, 1] and abs(pr.sum() - 1.0) < 1e-6
    # test_sampling_candidates_repetition_penalty_can_suppress_seen_token (:3847-3858)
    ids, lg, pr = oracle.sampling_candidates([3.0, 2.5, 1.0], repetition_penalty=3.0, top_k=1, history=[0])
    assert len(ids) == 1 and ids[0] == 1
    # edge cases the function defines: ties keep token order, non-finite logits drop out, a negative logit is multiplied,
    # temperature is floored, top_p 0 still keeps one candidate, an empty candidate set is possible
    ids, lg, pr = oracle.sampling_candidates([1.0, 2.0, 2.0, -np.inf, np.nan, 2.0])
    assert list(ids) == [1, 2, 5, 0]
    ids, lg, pr = oracle.sampling_candidates([-1.0, -1.5], repetition_penalty=2.0, history=[0])
    assert list(ids) == [1, 0] and list(lg) == [-1.5, -2.0]
    ids, lg, pr = oracle.sampling_candidates([1.0, 0.0], temperature=0.0)
    assert lg[0] == np.float32(1.0) / np.float32(1e-8) and pr[0] == 1.0
    assert len(oracle.sampling_candidates([0.3, 0.2, 0.1], top_p=0.0)[0]) == 1
    assert len(oracle.sampling_candidates([np.inf, np.nan])[0]) == 0
    with pytest.raises(ValueError):
        oracle.sampling_candidates([1.0, 2.0], vocab_size=3)
    # independent numpy statement on random rows
    rng = np.random.default_rng(4)
    for V, k, p, t, rp in [(50, 0, 1.0, 1.0, 1.0), (300, 40, 0.9, 0.7, 1.3), (1000, 0, 0.5, 1.5, 2.0), (257, 5, 0.3, 0.2, 1.0)]:
        x = (rng.standard_normal(V) * 3).astype(np.float32)
        hist = rng.integers(0, V, 20)
        ids, lg, pr = oracle.sampling_candidates(x, temperature=t, top_k=k, top_p=p, repetition_penalty=rp, history=hist)
        y = x.copy()
        seen = np.zeros(V, bool); seen[hist] = True
        if rp != 1.0:
            y = np.where(seen, np.where(np.signbit(y), y * np.float32(rp), y / np.float32(rp)), y).astype(np.float32)
        y = (y / np.float32(t)).astype(np.float32)
        order = np.argsort(-y, kind="stable")
        if k:
            order = order[:k]
        e = np.exp((y[order] - y[order].max()).astype(np.float64)); q = e / e.sum()
        if p < 1.0:
            n = int(np.searchsorted(np.cumsum(q), p - 1e-9) + 1)
            order = order[:n]; e = e[:n]; q = e / e.sum()
        assert list(ids) == list(order) and np.array_equal(lg, y[order]) and np.allclose(pr, q, atol=1e-6)
