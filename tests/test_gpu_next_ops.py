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
