"""Writers of the reference's weight-file formats, for tests only: each follows the reference's writer line by line
(crates/serialize/src/lib.rs:34-58 save_checkpoint, :315-328 save_state_dict, :340-364 save_state_dict_bundle;
the safetensors layout of serialize/src/safetensors.rs:25-73).  Independent of the C++ readers under test."""
import json
import os
import struct

import numpy as np


def write_sptc(path, arrays, magic=0x53505443, version=1):
    with open(path, "wb") as f:
        f.write(struct.pack("<III", magic, version, len(arrays)))
        for a in arrays:
            a = np.asarray(a, dtype="<f4")
            f.write(struct.pack("<I", a.ndim))
            f.write(struct.pack(f"<{a.ndim}I", *a.shape))
            f.write(a.tobytes())


def _num(x, shortest):
    """One f32 as JSON text: the shortest digits that round-trip (what serde_json prints for an f32), or the exact value
    written with float64 digits."""
    x = np.float32(x)
    if shortest:
        t = np.format_float_scientific(x, unique=True, trim="0")
        return t.replace("e+", "e").replace("e0", "e") if not t.endswith("e+00") else t[:-4]
    return repr(float(x))


def write_state_dict(path, named, schema="sptorch.state_dict.v1", version=1, dtype="F32", shortest=True):
    entries = []
    for n, a in named:
        a = np.asarray(a, np.float32)
        data = ",\n        ".join(_num(x, shortest) for x in a.ravel())
        entries.append("    {\n      \"name\": %s,\n      \"shape\": %s,\n      \"dtype\": %s,\n      \"data\": [\n        %s\n      ]\n    }"
                       % (json.dumps(n), json.dumps(list(a.shape)), json.dumps(dtype), data))
    with open(path, "w") as f:
        f.write("{\n  \"schema\": %s,\n  \"format_version\": %d,\n  \"entries\": [\n%s\n  ]\n}" % (json.dumps(schema), version, ",\n".join(entries)))


def write_manifest(weights_path, names, **over):
    m = {"schema": "sptorch.checkpoint_manifest.v1", "format_version": 1, "model_name": "test-model", "save_kind": "state_dict",
         "weights_file": os.path.basename(weights_path), "parameter_count": len(names), "parameter_names": list(names),
         "state_dict_schema": "sptorch.state_dict.v1", "created_at_ms": 1234, "note": "written by the tests"}
    m.update(over)
    with open(str(weights_path) + ".manifest.json", "w") as f:
        json.dump(m, f, indent=2)


def f32_to_f16_bits(a):
    return np.asarray(a, np.float32).astype(np.float16).view(np.uint16)


def f32_to_bf16_bits_trunc(a):
    return (np.asarray(a, np.float32).view(np.uint32) >> 16).astype(np.uint16)


def write_safetensors(path, named, dtype="F32", metadata=None):
    header, blobs, off = {}, [], 0
    if metadata is not None:
        header["__metadata__"] = metadata
    for n, a in named:
        a = np.asarray(a, np.float32)
        raw = (a.astype("<f4").tobytes() if dtype == "F32" else
               f32_to_f16_bits(a).astype("<u2").tobytes() if dtype == "F16" else f32_to_bf16_bits_trunc(a).astype("<u2").tobytes())
        header[n] = {"dtype": dtype, "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hb = json.dumps(header, separators=(",", ":")).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for b in blobs:
            f.write(b)
