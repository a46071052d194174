"""Writes the committed golden fixtures.  Run from the repo root in a checkout that has the reference
beside it:  python tests/golden/make_golden.py

c1_tiny.npz   the tiny character model c1_tiny (tiny char GPT, f32), first two sequences: ids, logits[:, :, :64], argmax,
              per-layer taps of sequence 0 -- from the CPU oracle in strict order (fast=0).
abi_ops.npz   inputs + outputs of the eleven C-ABI ops produced by the REFERENCE's own C implementation
              (crates/hal-ffi/mock_npu/mock_npu.c compiled in place as oracle/_ref/libmock_npu.so).
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import binding as O  # noqa: E402
from sptorch_b200 import synth  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    O.build()
    cfg = synth.CONFIGS["c1_tiny"]
    p, _ = synth.gpt_params(cfg, 0)
    ids = synth.randint(1, 8 * 64, 256).reshape(8, 64)
    logits, taps = O.gpt_forward(cfg, p, ids[:2], fast=0, want_taps=True)
    np.savez_compressed(os.path.join(HERE, "c1_tiny.npz"), ids=ids[:2], logits_first64=logits[:, :, :64].astype(np.float32),
                        argmax=logits.argmax(-1).astype(np.int64), taps_seq0=taps[0].astype(np.float32))

    ref = O.ref_lib()
    if ref is None:
        raise SystemExit("oracle/_ref/libmock_npu.so missing: build it with `make -C oracle` next to the reference checkout")
    fp = C.POINTER(C.c_float)
    p_ = lambda a: a.ctypes.data_as(fp)
    n = 1000
    x = synth.normal(11, n); y = synth.normal(12, n)
    out = {"x": x, "y": y}
    for name in ("add", "mul"):
        o = np.empty(n, dtype=np.float32); getattr(ref, f"sptorch_{name}_f32")(p_(x), p_(y), p_(o), C.c_size_t(n)); out[name] = o
    for name in ("neg", "exp", "relu", "gelu"):
        o = np.empty(n, dtype=np.float32); getattr(ref, f"sptorch_{name}_f32")(p_(x), p_(o), C.c_size_t(n)); out[name] = o
    xl = (np.abs(x) + 0.1).astype(np.float32)
    o = np.empty(n, dtype=np.float32); ref.sptorch_log_f32(p_(xl), p_(o), C.c_size_t(n)); out["log"] = o
    o = np.empty(n, dtype=np.float32); ref.sptorch_scale_f32(p_(x), C.c_float(0.37), p_(o), C.c_size_t(n)); out["scale_0p37"] = o
    a = synth.normal(13, 24 * 40).reshape(24, 40); b = synth.normal(14, 40 * 16).reshape(40, 16)
    o = np.empty((24, 16), dtype=np.float32); ref.sptorch_matmul_f32(p_(a), p_(b), p_(o), C.c_size_t(24), C.c_size_t(40), C.c_size_t(16))
    out.update(mm_a=a, mm_b=b, matmul=o)
    a3 = synth.normal(15, 3 * 8 * 12).reshape(3, 8, 12); b3 = synth.normal(16, 3 * 12 * 8).reshape(3, 12, 8)
    o3 = np.empty((3, 8, 8), dtype=np.float32)
    ref.sptorch_batch_matmul_f32(p_(a3), p_(b3), p_(o3), C.c_size_t(3), C.c_size_t(8), C.c_size_t(12), C.c_size_t(8))
    out.update(bmm_a=a3, bmm_b=b3, batch_matmul=o3)
    s = (synth.normal(17, 10 * 50) * 2).astype(np.float32).reshape(10, 50); so = np.empty_like(s)
    ref.sptorch_softmax_f32(p_(s), p_(so), C.c_size_t(10), C.c_size_t(50))
    out.update(sm_x=s, softmax=so)
    np.savez_compressed(os.path.join(HERE, "abi_ops.npz"), **out)
    print("wrote", os.listdir(HERE))


if __name__ == "__main__":
    main()
