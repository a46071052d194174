"""GPU parity tests of the ops next to the forward path (the reference's Qwen-like blocks and the loss that consumes
the logits): rms_norm, swiglu, cross_entropy_loss(_ignore_index) -- known answers of the reference's tests, then the
CPU oracle on random inputs including the LM-head width."""
import numpy as np
import pytest

from conftest import relerr
from sptorch_b200.backend import BF16, F32, HalError, bf16_bits_to_f32, f32_to_bf16_bits

pytestmark = pytest.mark.gpu


def _bf16(x):
    return bf16_bits_to_f32(f32_to_bf16_bits(x)).reshape(np.shape(x))


def test_kats(backend):
    # crates/core-ops/src/lib.rs:2482-2490, 2505-2511, 2366-2380, 2394-2397
    d = backend.rms_norm(np.array([[3, 4], [1, 2]], np.float32), [1, 2], 1e-6).ravel()
    assert abs(d[0] - 0.8485) < 1e-3 and abs(d[1] - 2.2627) < 1e-3
    s = backend.swiglu([1.0, 2.0], [0.0, 1.0])
    assert abs(s[0]) < 1e-6 and abs(s[1] - 1.4621) < 1e-3
    assert abs(backend.cross_entropy_loss(np.zeros(3, np.float32), [0]) - np.log(3)) < 1e-5
    assert abs(backend.cross_entropy_loss(np.zeros((2, 3), np.float32), [0, 1]) - np.log(3)) < 1e-5
    big = np.iinfo(np.int64).max
    assert abs(backend.cross_entropy_loss(np.zeros((2, 3), np.float32), [big, 1], ignore_index=big) - np.log(3)) < 1e-5
    assert backend.cross_entropy_loss(np.zeros((2, 3), np.float32), [big, big], ignore_index=big) == 0.0


@pytest.mark.parametrize("rows,dim", [(1, 1), (7, 3), (64, 128), (33, 768), (5, 2048), (3, 4096), (2, 5000)])
def test_rms_norm_vs_oracle(backend, oracle, rows, dim):
    rng = np.random.default_rng(dim)
    x = (rng.standard_normal((rows, dim)) * 2).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    assert relerr(backend.rms_norm(x, w, 1e-5), oracle.rms_norm(x, w, 1e-5)) <= 2e-6
    if dim % 8 == 0:
        xb = _bf16(x)
        ref = oracle.rms_norm(xb, w, 1e-5)
        assert np.abs(backend.rms_norm(xb, w, 1e-5, dtype=BF16) - ref).max() <= 2 ** -8 * np.abs(ref).max()


@pytest.mark.parametrize("n", [1, 5, 4096, 100003])
def test_swiglu_vs_oracle(backend, oracle, n):
    rng = np.random.default_rng(n)
    x, g = rng.standard_normal(n).astype(np.float32), (rng.standard_normal(n) * 3).astype(np.float32)
    assert np.abs(backend.swiglu(x, g) - oracle.swiglu(x, g)).max() <= 1e-6 * max(1.0, np.abs(x * g).max())
    if n % 8 == 0:
        xb, gb = _bf16(x), _bf16(g)
        ref = oracle.swiglu(xb, gb)
        assert np.abs(backend.swiglu(xb, gb, dtype=BF16) - ref).max() <= 2 ** -8 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("rows,classes", [(1, 2), (9, 256), (64, 1000), (16, 50257)])
def test_cross_entropy_vs_oracle(backend, oracle, rows, classes):
    rng = np.random.default_rng(classes)
    x = (rng.standard_normal((rows, classes)) * 3).astype(np.float32)
    t = rng.integers(0, classes, rows)
    # the reference sums `classes` exponentials sequentially in f32; the device merges per-thread running sums: allow the
    # rounding of a 50k-term f32 sum
    tol = 2e-6 if classes <= 1000 else 3e-5
    ref = oracle.cross_entropy(x, t)
    assert abs(backend.cross_entropy_loss(x, t) - ref) <= tol * max(1.0, abs(ref))
    t2 = t.copy(); t2[::3] = -100
    ref2 = oracle.cross_entropy(x, t2, ignore_index=-100)
    assert abs(backend.cross_entropy_loss(x, t2, ignore_index=-100) - ref2) <= tol * max(1.0, abs(ref2))
    xb = _bf16(x)
    refb = oracle.cross_entropy(xb, t)
    assert abs(backend.cross_entropy_loss(xb, t, dtype=BF16) - refb) <= tol * max(1.0, abs(refb))


def test_cross_entropy_bad_target_is_an_error_not_a_fault(backend):
    with pytest.raises(HalError):        # the reference asserts target < num_classes (core-ops/src/lib.rs:1148-1153)
        backend.cross_entropy_loss(np.zeros((2, 3), np.float32), [0, 3])
    backend.synchronize()
    assert abs(backend.cross_entropy_loss(np.zeros((2, 3), np.float32), [0, 1]) - np.log(3)) < 1e-5


def test_sampling_candidates_known_answers(backend):
    # test_sampling_candidates_apply_top_p_after_probability_sort (crates/nn/src/lib.rs:3833-3845)
    ids, lg, pr = backend.sampling_candidates([3.0, 2.0, 1.0, 0.0], top_p=0.75)
    assert list(ids) == [0, 1] and abs(pr.sum() - 1.0) < 1e-6
    # test_sampling_candidates_repetition_penalty_can_suppress_seen_token (:3847-3858)
    ids, lg, pr = backend.sampling_candidates([3.0, 2.5, 1.0], repetition_penalty=3.0, top_k=1, history=[0])
    assert len(ids) == 1 and ids[0] == 1
    ids, lg, pr = backend.sampling_candidates([1.0, 2.0, 2.0, -np.inf, np.nan, 2.0])
    assert list(ids) == [1, 2, 5, 0]                                  # ties in token order, non-finite values dropped
    ids, lg, pr = backend.sampling_candidates([-1.0, -1.5], repetition_penalty=2.0, history=[0])
    assert list(ids) == [1, 0] and list(lg) == [-1.5, -2.0]           # a negative logit is multiplied by the penalty
    assert len(backend.sampling_candidates([0.3, 0.2, 0.1], top_p=0.0)[0]) == 1
    assert len(backend.sampling_candidates([np.inf, np.nan])[0]) == 0
    with pytest.raises(HalError):
        backend.sampling_candidates([1.0, 2.0], vocab_size=3)         # the reference asserts vocab_size <= logits length
    # sample_from_candidates (:2420-2429)
    assert backend.sample_from_candidates([7, 8, 9], [0.5, 0.3, 0.2], 0.49) == 7
    assert backend.sample_from_candidates([7, 8, 9], [0.5, 0.3, 0.2], 0.51) == 8
    assert backend.sample_from_candidates([7, 8, 9], [0.5, 0.3, 0.1], 0.99) == 9     # falls off the end: the last candidate
    assert backend.sample_from_candidates([], [], 0.5) == -1


@pytest.mark.parametrize("V,k,p,t,rp", [(50, 0, 1.0, 1.0, 1.0), (300, 40, 0.9, 0.7, 1.3), (1000, 0, 0.5, 1.5, 2.0), (257, 5, 0.3, 0.2, 1.0),
                                        (50257, 50, 0.95, 0.8, 1.2), (50257, 0, 0.9, 1.0, 1.1), (50257, 0, 1.0, 1.0, 1.0), (50304, 1, 1.0, 1e-9, 1.0)])
def test_sampling_candidates_vs_oracle(backend, oracle, V, k, p, t, rp):
    rng = np.random.default_rng(V + k)
    x = (rng.standard_normal(V) * 3).astype(np.float32)
    x[rng.integers(0, V, 3)] = -np.inf                               # constraint-masked tokens (filtered_step_logits, :2465-2480)
    hist = rng.integers(0, V, 64)
    want = oracle.sampling_candidates(x, temperature=t, top_k=k, top_p=p, repetition_penalty=rp, history=hist)
    got = backend.sampling_candidates(x, temperature=t, top_k=k, top_p=p, repetition_penalty=rp, history=hist)
    assert np.array_equal(got[0], want[0])                            # same candidates in the same order
    assert np.array_equal(got[1], want[1])                            # scaled logits: the same f32 operations
    assert np.allclose(got[2], want[2], rtol=2e-6, atol=1e-9)         # expf differs by an ulp between host and device
    # bf16 logits of the LM head: same candidates as the oracle on the widened row
    xb = _bf16(np.where(np.isfinite(x), x, 0.0)).ravel()
    want = oracle.sampling_candidates(xb, temperature=t, top_k=k, top_p=1.0, repetition_penalty=rp, history=hist)
    got = backend.sampling_candidates(xb, temperature=t, top_k=k, top_p=1.0, repetition_penalty=rp, history=hist, dtype=BF16)
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])


def test_constrained_sampling_vs_oracle(backend, oracle):
    """A TokenConstraint's allowed set (filtered_step_logits, crates/nn/src/lib.rs:2465-2480) applied before the candidates are built."""
    rng = np.random.default_rng(9)
    V = 5000
    x = (rng.standard_normal(V) * 3).astype(np.float32)
    allowed = set(int(t) for t in rng.integers(0, V, 40))
    for k, p in ((0, 1.0), (5, 1.0), (0, 0.6)):
        want = oracle.sampling_candidates(x, top_k=k, top_p=p, temperature=0.9, repetition_penalty=1.2, history=[1, 2, 3], allowed=allowed)
        got = backend.sampling_candidates(x, top_k=k, top_p=p, temperature=0.9, repetition_penalty=1.2, history=[1, 2, 3], allowed=allowed)
        assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1]) and np.allclose(got[2], want[2], rtol=2e-6)
        assert set(got[0]) <= allowed
    assert len(backend.sampling_candidates(x, allowed=set())[0]) == 0            # an empty set leaves no candidate (NoCandidates)
    assert len(backend.sampling_candidates(x, allowed=None)[0]) == V


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_lm_head_fused_with_loss_and_greedy_token(backend, oracle, dtype):
    """The forward whose LM-head epilogue reduces the logits instead of storing them: the greedy tokens equal the argmax of the
    logits the ordinary forward stores, bit for bit (first maximum on ties), and the mean loss equals the reference's
    cross_entropy_loss / cross_entropy_loss_ignore_index of those logits (core-ops/src/lib.rs:1079-1194) to 1e-5 relative.
    Vocabulary 777: the last 256-column tile is ragged and its second half empty."""
    from sptorch_b200 import synth
    from sptorch_b200.gpt import GPT
    cfg = dict(vocab=777, d_model=128, n_layer=2, n_head=2, d_ff=256, seq_len=64)
    params, index = synth.gpt_params(cfg, 5, randomize_affine=True)
    m = GPT(backend, cfg["vocab"], cfg["d_model"], cfg["n_head"], cfg["n_layer"], cfg["d_ff"], cfg["seq_len"], dtype=dtype, max_batch=4)
    m.load_flat(params, index)
    ids = synth.randint(3, 4 * 64, 777).reshape(4, 64)
    targets = synth.randint(4, 4 * 64, 777).reshape(4, 64).astype(np.int64)
    logits = m.forward(ids)                                   # the stored logits (bf16 values widened, or f32)
    for _ in range(3):                                        # eager, captured, replayed
        loss, greedy = m.forward_loss(ids, targets)
        assert np.array_equal(greedy, logits.argmax(-1))
        ref = oracle.cross_entropy(logits.reshape(-1, 777), targets.reshape(-1))
        assert abs(loss - ref) <= 1e-5 * abs(ref)
    # rows to ignore
    t2 = targets.copy(); t2[1, :] = -100; t2[3, 5:40] = -100
    loss2, _ = m.forward_loss(ids, t2, ignore_index=-100)
    ref2 = oracle.cross_entropy(logits.reshape(-1, 777), t2.reshape(-1), ignore_index=-100)
    assert abs(loss2 - ref2) <= 1e-5 * abs(ref2)
    # greedy tokens alone; loss alone
    none_loss, g3 = m.forward_loss(ids)
    assert none_loss is None and np.array_equal(g3, greedy)
    loss4, none_arg = m.forward_loss(ids, targets, want_argmax=False)
    assert none_arg is None and loss4 == loss
    # a target outside the vocabulary is reported at the next sync (the reference panics)
    t5 = targets.copy(); t5[0, 0] = 777
    from sptorch_b200.backend import HalError
    with pytest.raises(HalError):
        m.forward_loss(ids, t5)
        backend.synchronize()
    m.close()
    # ties: every logit of a row equal -> the first column wins, as a stable descending sort has it
    cfg0 = dict(vocab=300, d_model=64, n_layer=0, n_head=2, d_ff=128, seq_len=8)
    p0, i0 = synth.gpt_params(cfg0, 1)
    o, shp = i0["lm_head.weight"]
    p0[o:o + 300 * 64] = 0.0
    m0 = GPT(backend, 300, 64, 2, 0, 128, 8, dtype=dtype, max_batch=1)
    m0.load_flat(p0, i0)
    _, g0 = m0.forward_loss(np.zeros((1, 8), dtype=np.int64))
    assert (g0 == 0).all()
    m0.close()


def test_lm_head_fused_host_call_matches_device_call(backend, oracle):
    import ctypes as C
    from sptorch_b200 import synth
    from sptorch_b200.gpt import GPT
    cfg = dict(vocab=1000, d_model=64, n_layer=2, n_head=1, d_ff=128, seq_len=32)
    params, index = synth.gpt_params(cfg, 1)
    m = GPT(backend, 1000, 64, 1, 2, 128, 32, dtype=BF16, max_batch=6)
    m.load_flat(params, index)
    ids = synth.randint(2, 6 * 32, 1000).reshape(6, 32).astype(np.int32)
    targets = synth.randint(9, 6 * 32, 1000).reshape(6, 32).astype(np.int64)
    loss, greedy = m.forward_loss(ids, targets)
    lib = backend.lib
    pin_ids, pin_t, pin_a = lib.sptorch_ext_alloc_pinned(ids.nbytes), lib.sptorch_ext_alloc_pinned(targets.nbytes), lib.sptorch_ext_alloc_pinned(ids.nbytes)
    C.memmove(pin_ids, ids.ctypes.data, ids.nbytes)
    C.memmove(pin_t, targets.ctypes.data, targets.nbytes)
    for chunk in (6, 4, 1):
        C.memset(pin_a, 0xff, ids.nbytes)
        l2 = m.forward_loss_host(pin_ids, pin_t, 6, 32, pin_a, chunk)
        got = np.ctypeslib.as_array(C.cast(pin_a, C.POINTER(C.c_int32)), shape=(6 * 32,)).copy().reshape(6, 32)
        assert np.array_equal(got, greedy), f"chunk {chunk}"
        assert abs(l2 - loss) <= 1e-6 * abs(loss), f"chunk {chunk}"
    for ptr in (pin_ids, pin_t, pin_a):
        lib.sptorch_ext_free_pinned(ptr)
    m.close()
