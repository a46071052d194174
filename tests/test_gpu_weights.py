"""Loading the reference's weight files into the device model: each format must give the same logits as feeding the same
arrays through set_param, and a rejected file must leave the model untouched (crates/serialize/src/lib.rs:65-131, 237-313,
366-441; safetensors.rs:85-116; the load -> forward check of crates/nn/tests/test_gpt_training_loop.rs:111-207)."""
import numpy as np
import pytest

import weight_files as wf
from sptorch_b200 import synth
from sptorch_b200 import weights as W
from sptorch_b200.backend import BF16, F32
from sptorch_b200.gpt import GPT, QwenLikeGPT

pytestmark = pytest.mark.gpu
CFG = dict(vocab=64, d_model=32, n_layer=2, n_head=4, d_ff=64, seq_len=16)


def _make(backend, arch, dtype=F32):
    cls = QwenLikeGPT if arch == "qwen" else GPT
    return cls(backend, CFG["vocab"], CFG["d_model"], CFG["n_head"], CFG["n_layer"], CFG["d_ff"], CFG["seq_len"], dtype=dtype, max_batch=2)


def _named(params, index):
    return [(n, params[o:o + int(np.prod(s))].reshape(s)) for n, (o, s) in index.items()]


@pytest.mark.parametrize("arch", ["gpt", "qwen"])
def test_every_format_loads_the_same_model(backend, tmp_path, arch):
    params, index = synth.gpt_params(CFG, 2, arch=arch, randomize_affine=True)
    named = _named(params, index)
    ids = synth.randint(3, 2 * 16, 64).reshape(2, 16)
    ref_model = _make(backend, arch)
    assert W.model_parameters(ref_model) == [(n, tuple(a.shape)) for n, a in named]       # the reference's names, order and shapes
    ref_model.load_flat(params, index)
    want = ref_model.forward(ids)
    ref_model.close()

    wf.write_sptc(tmp_path / "m.sptc", [a for _, a in named])
    wf.write_state_dict(tmp_path / "m.json", named[::-1])                                 # by name: file order is free
    wf.write_state_dict(tmp_path / "b.json", named)
    wf.write_manifest(tmp_path / "b.json", [n for n, _ in named])
    wf.write_safetensors(tmp_path / "m.safetensors", named, metadata={"format": "pt"})
    for load in (lambda m: W.load_into(m, tmp_path / "m.sptc"), lambda m: W.load_into(m, tmp_path / "m.json"),
                 lambda m: W.load_bundle(m, tmp_path / "b.json"), lambda m: W.load_into(m, tmp_path / "m.safetensors")):
        m = _make(backend, arch)
        load(m)
        assert np.array_equal(m.forward(ids), want)
        m.close()
    # half-precision safetensors: the loader widens exactly, so the result equals set_param of the widened values
    for dt, narrow in (("F16", lambda a: a.astype(np.float16).astype(np.float32)),
                       ("BF16", lambda a: (a.view(np.uint32) & 0xFFFF0000).view(np.float32))):
        wf.write_safetensors(tmp_path / "h.safetensors", named, dtype=dt)
        a, b = _make(backend, arch, BF16), _make(backend, arch, BF16)
        W.load_into(a, tmp_path / "h.safetensors")
        for n, arr in named:
            b.set_param(n, narrow(np.ascontiguousarray(arr)))
        assert np.array_equal(a.forward(ids), b.forward(ids))
        a.close(); b.close()


def test_rejected_files_leave_the_model_untouched(backend, tmp_path):
    params, index = synth.gpt_params(CFG, 2, randomize_affine=True)
    named = _named(params, index)
    ids = synth.randint(3, 2 * 16, 64).reshape(2, 16)
    m = _make(backend, "gpt")
    m.load_flat(params, index)
    want = m.forward(ids)
    other = [(n, a + 1.0) for n, a in named]

    def rejected(match, load):
        with pytest.raises(W.WeightsError, match=match):
            load()
        assert np.array_equal(m.forward(ids), want)

    wf.write_sptc(tmp_path / "x.sptc", [a for _, a in other][:-1])
    rejected("param count mismatch: checkpoint has 28, model has 29", lambda: W.load_into(m, tmp_path / "x.sptc"))
    arrs = [a for _, a in other]
    arrs[5] = arrs[5].T.copy().reshape(16, 64)
    wf.write_sptc(tmp_path / "x.sptc", arrs)
    rejected(r"shape mismatch at param\[5\]", lambda: W.load_into(m, tmp_path / "x.sptc"))
    wf.write_state_dict(tmp_path / "x.json", other[:-1] + [other[0]])
    rejected("duplicate parameter 'token_emb.weight'", lambda: W.load_into(m, tmp_path / "x.json"))
    wf.write_state_dict(tmp_path / "x.json", other[:-1] + [("extra.weight", other[-1][1])])
    rejected("missing parameter 'lm_head.weight'", lambda: W.load_into(m, tmp_path / "x.json"))
    wf.write_state_dict(tmp_path / "x.json", other[:-1])
    rejected("parameter count mismatch: state has 28, model has 29", lambda: W.load_into(m, tmp_path / "x.json"))
    wf.write_state_dict(tmp_path / "x.json", other, dtype="BF16")
    rejected("dtype mismatch for 'token_emb.weight': state BF16, model F32", lambda: W.load_into(m, tmp_path / "x.json"))
    wf.write_state_dict(tmp_path / "x.json", other)
    wf.write_manifest(tmp_path / "x.json", [n for n, _ in other], weights_file="elsewhere.json")
    rejected("manifest weights file elsewhere.json does not match", lambda: W.load_bundle(m, tmp_path / "x.json"))
    wf.write_manifest(tmp_path / "x.json", [n for n, _ in other][::-1])
    rejected("manifest parameter names do not match", lambda: W.load_bundle(m, tmp_path / "x.json"))
    wf.write_manifest(tmp_path / "x.json", [n for n, _ in other], schema="v0")
    rejected("unsupported checkpoint manifest schema v0", lambda: W.load_bundle(m, tmp_path / "x.json"))
    wf.write_safetensors(tmp_path / "x.safetensors", other[:-1])
    rejected("tensor 'lm_head.weight' not found in safetensors", lambda: W.load_into(m, tmp_path / "x.safetensors"))
    # a mapping writes only the listed parameters, under foreign names, with the shape check of load_into
    wf.write_safetensors(tmp_path / "hf.safetensors", [("transformer.wte.weight", other[0][1]), ("wrong", np.zeros((3, 3), np.float32))])
    rejected("shape mismatch for 'wrong'", lambda: W.load_into(m, tmp_path / "hf.safetensors", mapping={"lm_head.weight": "wrong"}))
    rejected("'nope' is not a parameter of the model", lambda: W.load_into(m, tmp_path / "hf.safetensors", mapping={"nope": "wrong"}))
    W.load_into(m, tmp_path / "hf.safetensors", mapping={"token_emb.weight": "transformer.wte.weight"})
    m2 = _make(backend, "gpt")
    m2.load_flat(params, index)
    m2.set_param("token_emb.weight", other[0][1])
    assert np.array_equal(m.forward(ids), m2.forward(ids))
    m.close(); m2.close()
