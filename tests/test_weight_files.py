"""Host-side readers of the reference's weight formats (no GPU needed): the reference's own small cases
(crates/serialize/src/safetensors.rs:190-301, src/lib.rs tests) and the error paths its loaders define."""
import json
import struct

import numpy as np
import pytest

import weight_files as wf
from sptorch_b200 import weights as W


def test_binary_checkpoint_round_trip(tmp_path):
    rng = np.random.default_rng(0)
    arrays = [rng.standard_normal((3, 4)).astype(np.float32), rng.standard_normal(5).astype(np.float32), np.zeros((2, 0, 3), np.float32),
              np.float32(7.5).reshape(())]
    p = tmp_path / "m.sptc"
    wf.write_sptc(p, arrays)
    with W.WeightFile(p) as f:
        assert f.format == W.SPTC and len(f) == 4 and f.names() == ["", "", "", ""]
        for i, a in enumerate(arrays):
            name, shape, dtype, data = f.entry(i)
            assert shape == a.shape and dtype == "F32" and np.array_equal(data, a.ravel())


def test_binary_checkpoint_errors(tmp_path):
    p = tmp_path / "bad.sptc"
    wf.write_sptc(p, [np.ones(3, np.float32)], version=2)
    with pytest.raises(W.WeightsError, match="unsupported checkpoint version 2"):
        W.WeightFile(p)
    wf.write_sptc(p, [np.ones(3, np.float32)], magic=0x12345678)
    with pytest.raises(W.WeightsError, match="invalid checkpoint magic"):
        W.WeightFile(p, W.SPTC)
    wf.write_sptc(p, [np.ones(300, np.float32)])
    raw = p.read_bytes()
    p.write_bytes(raw[:200])                                  # truncated data
    with pytest.raises(W.WeightsError, match="past the end"):
        W.WeightFile(p)
    with pytest.raises(W.WeightsError, match="cannot open"):
        W.WeightFile(tmp_path / "missing.sptc")


def test_state_dict_by_name(tmp_path):
    # test_state_dict_roundtrip_by_name (serialize/src/lib.rs:508-528): linear.weight [2,2] = 1..4, linear.bias [2] = 5, 6
    p = tmp_path / "sd.json"
    wf.write_state_dict(p, [("linear.weight", np.array([[1, 2], [3, 4]], np.float32)), ("linear.bias", np.array([5, 6], np.float32))])
    with W.WeightFile(p) as f:
        assert f.format == W.STATE_DICT and f.names() == ["linear.weight", "linear.bias"]
        assert f.get("linear.weight")[1] == (2, 2) and np.array_equal(f.get("linear.weight")[3], [1, 2, 3, 4])
        assert np.array_equal(f.get("linear.bias")[3], [5, 6])
    # values survive the decimal round trip bit for bit
    rng = np.random.default_rng(1)
    a = np.concatenate([rng.standard_normal(500) * 10.0 ** rng.integers(-30, 30, 500), [0.0, -0.0, 1e-45, 3.4028235e38]]).astype(np.float32)
    for shortest in (True, False):
        wf.write_state_dict(p, [("x", a)], shortest=shortest)
        json.loads(p.read_text())                            # the writer emits valid JSON
        with W.WeightFile(p) as f:
            assert np.array_equal(f.entry(0)[3].view(np.uint32), a.view(np.uint32))
    wf.write_state_dict(p, [("x", a)], schema="other.schema")
    with pytest.raises(W.WeightsError, match="unsupported state_dict schema other.schema"):
        W.WeightFile(p)
    wf.write_state_dict(p, [("x", a)], version=3)
    with pytest.raises(W.WeightsError, match="unsupported state_dict version 3"):
        W.WeightFile(p)
    wf.write_state_dict(p, [("x", a)], dtype="I8")
    with pytest.raises(W.WeightsError, match="unsupported dtype 'I8'"):
        W.WeightFile(p)
    p.write_text('{"schema": "sptorch.state_dict.v1", "format_version": 1, "entries": [')
    with pytest.raises(W.WeightsError, match="invalid JSON"):
        W.WeightFile(p)
    # escapes and non-ASCII names
    p.write_text(json.dumps({"schema": "sptorch.state_dict.v1", "format_version": 1,
                             "entries": [{"name": "a\"b\\cé\U0001F600", "shape": [1], "dtype": "F32", "data": [1.5e0]}]}))
    with W.WeightFile(p) as f:
        assert f.names() == ["a\"b\\cé\U0001F600"]


def test_safetensors_reference_cases(tmp_path):
    # test_load_safetensors_synthetic (serialize/src/safetensors.rs:230-265)
    p = tmp_path / "s.safetensors"
    wf.write_safetensors(p, [("weight", np.arange(1, 7, dtype=np.float32).reshape(2, 3))])
    with W.WeightFile(p) as f:
        assert f.format == W.SAFETENSORS and "weight" in f.names()
        name, shape, dtype, data = f.get("weight")
        assert shape == (2, 3) and np.array_equal(data, [1, 2, 3, 4, 5, 6])
    # test_f16_to_f32_basic / test_bf16_to_f32_basic (:194-219): 0x3C00 -> 1, 0xBC00 -> -1, 0 -> 0; bf16 0x3F80 -> 1
    hdr = json.dumps({"h": {"dtype": "F16", "shape": [6], "data_offsets": [0, 12]}, "b": {"dtype": "BF16", "shape": [2], "data_offsets": [12, 16]},
                      "__metadata__": {"format": "pt"}}).encode()
    body = struct.pack("<6H", 0x3C00, 0xBC00, 0x0000, 0x0001, 0x7C00, 0x8000) + struct.pack("<2H", 0x3F80, 0x0000)
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + body)
    with W.WeightFile(p) as f:
        h = f.get("h")[3]
        assert list(h[:3]) == [1.0, -1.0, 0.0] and h[3] == np.float32(2.0 ** -24) and np.isinf(h[4]) and h[5] == 0 and np.signbit(h[5])
        assert list(f.get("b")[3]) == [1.0, 0.0] and f.get("b")[2] == "BF16"
    # every f16 bit pattern widens like numpy's conversion
    bits = np.arange(65536, dtype=np.uint16)
    hdr = json.dumps({"all": {"dtype": "F16", "shape": [65536], "data_offsets": [0, 131072]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + bits.astype("<u2").tobytes())
    with W.WeightFile(p) as f:
        got, want = f.entry(0)[3], bits.view(np.float16).astype(np.float32)
        nan = np.isnan(want)
        assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32)) and np.isnan(got[nan]).all()
    # malformed files
    p.write_bytes(b"\x01\x02")
    with pytest.raises(W.WeightsError, match="file too small"):
        W.WeightFile(p, W.SAFETENSORS)
    p.write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(W.WeightsError, match="header size exceeds file"):
        W.WeightFile(p, W.SAFETENSORS)
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(W.WeightsError, match="outside the file"):
        W.WeightFile(p)
    hdr = json.dumps({"w": {"dtype": "I64", "shape": [1], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(W.WeightsError, match="unsupported dtype: I64"):
        W.WeightFile(p)
