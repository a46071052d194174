"""The generation loop over the device model (generate_with_config / decode_next_token, crates/nn/src/lib.rs:2431-2464, 2526-2593):
the reference's own tests (nn/src/lib.rs:3860-3930) restated on models the kernels can hold, and greedy decoding with the
key/value cache against greedy decoding by full forwards."""
import numpy as np
import pytest

from sptorch_b200 import synth
from sptorch_b200.backend import BF16, F32
from sptorch_b200.gpt import GPT, QwenLikeGPT

pytestmark = pytest.mark.gpu


def _counting_model(backend, cls, vocab=6, d=8, seq_len=5, gain=5.0):
    """A layer-free model whose next token is (token + 1) % vocab with a wide margin: token t embeds to the unit vector e_t and
    the head row t+1 reads it back.  The reference's eos test builds the same kind of model by hand (nn/src/lib.rs:3878-3898)."""
    m = cls(backend, vocab, d, 2, 0, 16, seq_len, dtype=F32, max_batch=1)
    emb = np.zeros((vocab, d), np.float32); head = np.zeros((vocab, d), np.float32)
    for t in range(vocab):
        emb[t, t] = 1.0
        head[(t + 1) % vocab, t] = gain
    m.set_param("token_emb.weight", emb)
    m.set_param("lm_head.weight", head)
    if cls is GPT:
        m.set_param("pos_emb.weight", np.zeros((seq_len, d), np.float32))
        m.set_param("ln_f.gamma", np.ones(d, np.float32)); m.set_param("ln_f.beta", np.zeros(d, np.float32))
    else:
        m.set_param("norm_f.weight", np.ones(d, np.float32))
    return m


@pytest.mark.parametrize("cls", [GPT, QwenLikeGPT])
def test_generation_length_eos_and_window(backend, cls):
    m = _counting_model(backend, cls)
    # test_qwen_like_generation_uses_shared_config (:3860-3866): prompt of 2, greedy(2, 6) -> 4 tokens
    assert m.generate([0, 1], 2, vocab_size=6, top_k=1) == [0, 1, 2, 3]
    # test_generation_stops_immediately_when_prompt_already_has_eos (:3868-3882)
    assert m.generate([1, 2], 3, vocab_size=6, top_k=1, eos_token_id=2) == [1, 2]
    # test_generation_stops_after_sampling_eos_token (:3884-3906): the eos token is written, then generation stops
    assert m.generate([1], 4, vocab_size=6, top_k=1, eos_token_id=3) == [1, 2, 3]
    # more tokens than the context holds: the window slides (InferenceState::context) and the count goes on
    assert m.generate([4], 9, vocab_size=6, top_k=1) == [4, 5, 0, 1, 2, 3, 4, 5, 0, 1]
    # test_decode_next_token_appends_to_state_and_returns_candidates (:3908-3922)
    tokens = [1]
    tok, cand, reason = m.decode_next_token(tokens, vocab_size=6, top_k=1)
    assert tok == 2 and reason == "NotStopped" and len(cand[0]) == 1 and tokens == [1, 2]
    # a vocabulary cut that leaves nothing finite: every logit masked by the penalty-free -inf is impossible here, so cut to the
    # sampled distribution instead: with all mass on one candidate any draw returns it
    assert m.generate([0], 3, vocab_size=6, top_p=0.0, draw=lambda: 0.999) == [0, 1, 2, 3]
    # a constraint (TokenConstraint::allowed_next on the generated tokens, nn/src/lib.rs:2465-2480): only even tokens allowed, then nothing
    assert m.generate([0], 3, vocab_size=6, top_k=1, constraint=lambda gen: {0, 2, 4}) [1:] != [1, 2, 3]
    out = m.generate([0], 5, vocab_size=6, top_k=1, constraint=lambda gen: {2, 4} if len(gen) < 2 else set())
    assert len(out) == 3 and set(out[1:]) <= {2, 4}                   # stops with NoCandidates when the set is empty
    m.close()


@pytest.mark.parametrize("cls,arch", [(GPT, "gpt"), (QwenLikeGPT, "qwen")])
def test_greedy_generation_with_cache_equals_full_forwards(backend, cls, arch):
    """Greedy decoding through the key/value cache against greedy decoding where every step is a full forward of the context,
    as the reference's generate does it.  The two paths contract differently (f32 last-token attention vs tensor cores), so a
    step is only required to agree when the full forward's top-1 margin is above that difference."""
    cfg = dict(vocab=96, d_model=64, n_layer=2, n_head=2, d_ff=128, seq_len=48)
    params, index = synth.gpt_params(cfg, 11, arch=arch, randomize_affine=True)
    params = params.copy()
    off, shape = index["lm_head.weight"]
    params[off:off + int(np.prod(shape))] *= 20.0                    # sharper logits: clear winners
    m = cls(backend, cfg["vocab"], cfg["d_model"], cfg["n_head"], cfg["n_layer"], cfg["d_ff"], cfg["seq_len"], dtype=F32, max_batch=1)
    m.load_flat(params, index)
    prompt = [int(t) for t in synth.randint(2, 5, 96)]
    out = m.generate(prompt, 30, top_k=1)
    assert len(out) == 35 and out[:5] == prompt
    tokens = list(prompt)
    for step in range(30):
        logits = m.forward_ids(tokens)[-1]
        top2 = np.sort(logits)[-2:]
        if top2[1] - top2[0] <= 4e-3 * np.abs(logits).max():
            break                                                    # a near tie: the two paths may legitimately differ from here
        assert out[len(tokens)] == int(logits.argmax()), f"step {step}"
        tokens.append(int(logits.argmax()))
    assert len(tokens) - len(prompt) >= 5                            # the comparison covered a real stretch
    m.close()
