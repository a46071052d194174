#!/usr/bin/env python
"""Benchmark of the GPT forward hot path (workload c4_gpt2s: GPT-2-small shape, global batch 64 x 1024
tokens, bf16 weights/activations, f32 accumulate), batch-sharded over N GPUs of one node.

    python bench.py --gpus N --steps K --warmup W              # this repository's CUDA path
    python bench.py --impl reference --gpus N --steps K ...    # the reference's CPU arithmetic (oracle port)

One JSON line on stdout (rank 0).  `value` = tokens/s of the whole job with ids and weights resident in
HBM; `e2e` = the same through the host-buffer C-ABI call (pinned ids in, dense logits out, copies inside
the timed region).  A "step" is one forward over the global batch.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from sptorch_b200 import synth  # noqa: E402

WORKLOAD = "c4_gpt2s"


def flops_per_forward(cfg, n_seq, T):
    """Algorithmic FLOP: linear layers 2*M*K*N; attention counted on the causal-necessary half."""
    d, L, F, V = cfg["d_model"], cfg["n_layer"], cfg["d_ff"], cfg["vocab"]
    M = n_seq * T
    linear = M * (L * (8 * d * d + 4 * d * F) + 2 * d * V)
    attn = n_seq * L * 2 * T * (T + 1) * d
    return linear, attn


def read_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return dict(hbm=p["hbm_gbs"], tf=p["bf16_tflops"], tf_sustained=p["bf16_tflops_sustained"], source="measured")
    except Exception:
        return dict(hbm=6650.0, tf=1590.0, tf_sustained=1400.0, source="fallback")


class ClockSampler:
    """SM clock and throttle reasons read through NVML every 20 ms on a thread while the timed region runs
    (read-only queries; nothing is set)."""

    def __init__(self, index):
        self.index, self.samples, self._stop, self._t = index, [], None, None

    def start(self):
        import threading
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self._max = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
        except Exception as e:  # noqa: BLE001
            self._err = repr(e)
            return
        self._stop = threading.Event()

        def loop():
            while not self._stop.is_set():
                try:
                    sm = pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
                    rs = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h) if hasattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons") \
                        else pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                    pw = pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0
                    self.samples.append((sm, rs, pw))
                except Exception:  # noqa: BLE001
                    pass
                self._stop.wait(0.02)

        self._t = threading.Thread(target=loop, daemon=True)
        self._t.start()

    def stop(self):
        if self._t is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable: " + getattr(self, "_err", "?")]}
        self._stop.set()
        self._t.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": float(self._max), "reasons": ["no samples"]}
        bits = {"hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40, "sw_power_cap": 0x4}
        reasons = sorted(name for name, bit in bits.items() if any(r & bit for _, r, _ in self.samples))
        return {"sm_mhz": statistics.median(sm for sm, _, _ in self.samples), "sm_max_mhz": float(self._max), "reasons": reasons,
                "samples": len(self.samples), "power_w_max": max(p for _, _, p in self.samples)}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def shard(n_items, world, rank):
    """DataParallel::scatter's rule (crates/distributed/src/data_parallel.rs:21-37): remainder to the first ranks."""
    base, rem = divmod(n_items, world)
    start = rank * base + min(rank, rem)
    return start, base + (1 if rank < rem else 0)


def host_threads():
    """Cores this process may run on (torchrun exports OMP_NUM_THREADS=1, which must not shrink the CPU arm)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_baseline(cfg, T, seconds_hint=20.0):
    """The reference's CPU arithmetic (oracle port) on a bounded sample of the same workload."""
    from oracle import binding as O
    O.build()
    threads = host_threads()
    params, _ = synth.gpt_params(cfg, 0, residual_scale=True)
    ids = synth.randint(1, T, cfg["vocab"]).reshape(1, T)
    t0 = time.perf_counter()
    O.gpt_forward(cfg, params, ids, fast=1, threads=threads)
    dt = time.perf_counter() - t0
    # the reference itself is single-threaded (matrixmultiply without its threading feature, no rayon): the same port on
    # one thread, on a shorter sequence so that the leg stays bounded
    T1 = min(T, 128)
    t1 = time.perf_counter()
    O.gpt_forward(cfg, params, ids[:, :T1], fast=1, threads=1)
    dt1 = time.perf_counter() - t1
    return {"value": T / dt, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"1 sequence of {T} tokens of the same model, rows/heads split over {threads} OpenMP threads, {dt:.1f} s",
            "single_thread": {"value": T1 / dt1, "unit": "tokens/s", "cores": 1,
                              "sample": f"1 sequence of {T1} tokens on one thread (how the reference itself runs), {dt1:.1f} s"}}


def run_reference(args):
    rank, _, world = dist_env()
    if rank != 0:
        return 0
    from oracle import binding as O
    O.build()
    cfg = dict(synth.CONFIGS[WORKLOAD])
    T = cfg["ctx"]
    threads = host_threads()
    params, _ = synth.gpt_params(cfg, 0, residual_scale=True)
    # one step = a bounded sample of the global batch: n_seq sequences of the full context length
    n_seq = 1
    ids_all = synth.randint(1, cfg["batch"] * T, cfg["vocab"]).reshape(cfg["batch"], T)
    for w in range(args.warmup):
        O.gpt_forward(cfg, params, ids_all[:1, :128], fast=1, threads=threads)   # page in weights / spin up the pool
    t0 = time.perf_counter()
    for s in range(args.steps):
        O.gpt_forward(cfg, params, ids_all[s % cfg["batch"]:s % cfg["batch"] + n_seq], fast=1, threads=threads)
    dt = time.perf_counter() - t0
    tok_s = args.steps * n_seq * T / dt
    sample = f"{n_seq} sequence of {T} tokens per step ({args.steps} steps), all {threads} host threads; warm-up on 128-token prefixes"
    line = {
        "impl": "reference", "metric": "gpt_forward_tokens_per_s", "value": tok_s, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_batch": cfg["batch"], "seq_len": T, "sequences_per_step": n_seq,
                   "note": "CPU port of the reference arithmetic; the Rust reference cannot be built here; a step is ONE sequence of the "
                           "global batch (the reference has no batch dimension), tokens/s is comparable"},
        "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# DRAM bytes (read + write) of ONE launch of the dominant GEMM per algorithmic byte, from a small ncu capture of a single
# Linear launch (the W_up shape at 8192 rows, two launches captured); the bench scales it by the algorithmic bytes of the
# launches it times (203.5 MB of DRAM traffic for 256.4 MB of operands and output: part of the output is still in L2 at the end).
GEMM_DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE = 0.794


def gemm_bytes(cfg, nseq, T):
    """Operand, residual and output bytes of the Linear launches (QKV, Wo, up, down per layer; LM head) of one bf16 forward over
    nseq sequences."""
    d, F, V, L, M = cfg["d_model"], cfg["d_ff"], cfg["vocab"], cfg["n_layer"], nseq * T
    ldl = -(-V // 64) * 64
    per_layer = (M * d + 3 * d * d + 3 * M * d) + (M * d + d * d + 2 * M * d) + (M * d + F * d + M * F) + (M * F + d * F + 2 * M * d)
    return 2.0 * (L * per_layer + M * d + V * d + M * ldl)


def run_ours(args):
    rank, local_rank, world = dist_env()
    if world != args.gpus and world > 1:
        print(f"warning: WORLD_SIZE={world} differs from --gpus {args.gpus}", file=sys.stderr)
    import torch
    os.environ.setdefault("SPTORCH_B200_DEVICE", str(local_rank))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from sptorch_b200.backend import BF16, FfiBackend
    from sptorch_b200.gpt import GPT

    b = FfiBackend.load()
    lib = b.lib
    cfg = dict(synth.CONFIGS[WORKLOAD])
    T, GB = cfg["ctx"], cfg["batch"]
    if args.batch:
        GB = args.batch
    start, nseq = shard(GB, world, rank)
    model = GPT(b, cfg["vocab"], cfg["d_model"], cfg["n_head"], cfg["n_layer"], cfg["d_ff"], cfg["seq_len"], dtype=BF16, max_batch=max(nseq, 1))
    params, index = synth.gpt_params(cfg, 0, residual_scale=True)
    model.load_flat(params, index)
    b._check(lib.sptorch_ext_gpt_enable_ln_fold(model.h, int(args.ln_fold)), "ln_fold")
    del params
    ids_all = synth.randint(1, GB * T, cfg["vocab"]).reshape(GB, T).astype(np.int32)
    ids = np.ascontiguousarray(ids_all[start:start + nseq])
    d_ids = model.stage_ids(ids)
    d_logits = model.logits_buffer(nseq * T)
    b.synchronize()

    def barrier():
        b.synchronize()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(x):
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident timing: K forwards, replayed as a CUDA graph after the first two ----
    for _ in range(max(args.warmup, 3)):
        model.forward_device(d_ids, nseq, T, d_logits)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    b.timer_begin()
    for _ in range(args.steps):
        model.forward_device(d_ids, nseq, T, d_logits)
    ms_local = b.timer_end()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = max_over_ranks(ms_local)
    # ---- per-kernel pass: the same K forwards launched eagerly with CUDA events around every launch ----
    lib.sptorch_ext_prof_enable(1)
    lib.sptorch_ext_prof_read(None, None, 0)
    barrier()
    b.timer_begin()
    for _ in range(args.steps):
        model.forward_device(d_ids, nseq, T, d_logits)
    ms_eager = max_over_ranks(b.timer_end())
    prof_ms = (C.c_float * 7)()
    prof_n = (C.c_uint32 * 7)()
    lib.sptorch_ext_prof_read(prof_ms, prof_n, 7)
    lib.sptorch_ext_prof_enable(0)
    barrier()
    tokens_per_step = GB * T
    value = tokens_per_step * args.steps / (ms * 1e-3)

    # ---- end to end through the host-buffer call ----
    V = cfg["vocab"]
    chunk = min(args.chunk, nseq)
    ids_pinned = lib.sptorch_ext_alloc_pinned(ids.nbytes)
    out_bytes = nseq * T * V * 2
    out_pinned = lib.sptorch_ext_alloc_pinned(out_bytes)
    e2e = None
    if ids_pinned and out_pinned and args.e2e_steps > 0:
        C.memmove(ids_pinned, ids.ctypes.data, ids.nbytes)
        e2e_steps = max(1, min(args.steps, args.e2e_steps))
        model.forward_host(ids_pinned, nseq, T, out_pinned, chunk)   # warm-up (allocates the staging buffers)
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            model.forward_host(ids_pinned, nseq, T, out_pinned, chunk)
        b.synchronize()
        dt = time.perf_counter() - t0
        dt = max_over_ranks(dt)
        # the roof of this call: the same bytes as one plain contiguous device-to-host copy into the same pinned buffer, all ranks at once
        barrier()
        t0 = time.perf_counter()
        b._check(lib.sptorch_ext_copy_d2h_bytes(d_logits.handle, out_pinned, out_bytes), "d2h roof")
        dt_copy = max_over_ranks(time.perf_counter() - t0)
        e2e = {"value": tokens_per_step * e2e_steps / dt, "unit": "tokens/s", "h2d_bytes_per_step": int(GB * T * 4),
               "d2h_bytes_per_step": int(GB * T * V * 2), "steps": e2e_steps, "chunk_sequences": chunk,
               "ms_per_step": 1e3 * dt / e2e_steps,
               "d2h_gbs": GB * T * V * 2 * e2e_steps / dt / 1e9,
               "d2h_peak_gbs": world * out_bytes / dt_copy / 1e9,
               "d2h_peak_note": "one contiguous cudaMemcpyAsync of this rank's logits bytes into the same pinned buffer, all ranks at the same time "
                                "(whole-job GB/s, max time over ranks): the end-to-end call cannot be faster than this copy",
               "api": "sptorch_ext_gpt_forward_host (pinned ids in, dense bf16 logits [B*T,V] out; the padded logits are compacted on the device "
                      "and leave as one contiguous copy per micro-batch, overlapped with the next micro-batch's compute)"}
        lib.sptorch_ext_free_pinned(out_pinned)
        out_pinned = None
    # ---- the same step when the caller wants the loss and the greedy tokens, not the logits: LM head fused with both ----
    e2e_loss = None
    tgt_pinned = lib.sptorch_ext_alloc_pinned(nseq * T * 8)
    arg_pinned = lib.sptorch_ext_alloc_pinned(nseq * T * 4)
    if ids_pinned and tgt_pinned and arg_pinned and args.e2e_steps > 0:
        targets = np.ascontiguousarray(np.roll(ids_all, -1, axis=1)[start:start + nseq], dtype=np.int64)      # next-token targets
        C.memmove(ids_pinned, ids.ctypes.data, ids.nbytes)
        C.memmove(tgt_pinned, targets.ctypes.data, targets.nbytes)
        steps_l = max(1, min(args.steps, max(args.e2e_steps, 5)))
        loss_chunk = nseq      # nothing large leaves the device, so there is no copy to hide behind micro-batches: one forward over the rank's batch
        for _ in range(3):                                   # eager, captured, replayed
            loss = model.forward_loss_host(ids_pinned, tgt_pinned, nseq, T, arg_pinned, loss_chunk)
        barrier()
        t0 = time.perf_counter()
        for _ in range(steps_l):
            loss = model.forward_loss_host(ids_pinned, tgt_pinned, nseq, T, arg_pinned, loss_chunk)
        b.synchronize()
        dt = max_over_ranks(time.perf_counter() - t0)
        e2e_loss = {"value": tokens_per_step * steps_l / dt, "unit": "tokens/s", "h2d_bytes_per_step": int(GB * T * 12),
                    "d2h_bytes_per_step": int(GB * T * 4 + 4 * world), "steps": steps_l, "chunk_sequences": loss_chunk, "ms_per_step": 1e3 * dt / steps_l,
                    "mean_loss_rank0": loss,
                    "api": "sptorch_ext_gpt_forward_loss_host (pinned ids and next-token targets in; greedy tokens and the mean cross-entropy "
                           "loss out; the LM head's epilogue reduces the logits tile by tile, the [B*T, V] matrix is never written)"}
    for ptr in (ids_pinned, out_pinned, tgt_pinned, arg_pinned):
        if ptr:
            lib.sptorch_ext_free_pinned(ptr)
    barrier()

    if rank == 0:
        peaks = read_peaks()
        lin_flop, attn_flop = flops_per_forward(cfg, nseq, T)
        lin_ms = float(prof_ms[0]) / args.steps
        lin_launches = int(prof_n[0]) // args.steps
        achieved = lin_flop / (lin_ms * 1e-3) / 1e12 if lin_ms > 0 else 0.0
        cats = ["linear_gemm", "attention_gemm", "causal_softmax", "layernorm", "embedding", "other", "attention_fused"]
        breakdown = {c: {"ms_per_step": float(prof_ms[i]) / args.steps, "launches_per_step": int(prof_n[i]) // args.steps} for i, c in enumerate(cats) if prof_n[i]}
        line = {
            "metric": "gpt_forward_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "global_batch": GB, "seq_len": T, "parallelism": f"batch-shard x{world}",
                       "l2": "inputs larger than L2 (326 MB of weights + >1 GB of activations per step); no explicit flush",
                       "model": "vocab 50257, d 768, 12 layers, 12 heads, d_ff 3072, pre-LN, untied head; N(0,0.02) seed 0, residual projections / sqrt(24)"},
            "clocks": clocks,
            "e2e": e2e,
            "e2e_loss": e2e_loss,
            "gpu_launches": int(sum(prof_n)) if sum(prof_n) else model.launches(nseq, T) * args.steps,
            "roofline": {"bound": "tensor", "kernel": "gemm_tcgen05_kernel<bf16> (Linear: [Wq;Wk;Wv], Wo, up, down, LM head)",
                         "achieved": achieved, "peak": peaks["tf_sustained"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["tf_sustained"] if peaks["tf_sustained"] else None,
                         "peak_source": f"{peaks['source']} (sustained cuBLAS bf16, kernel timed inside a long step)",
                         "launches_per_step": lin_launches, "avg_launch_ms": lin_ms / max(lin_launches, 1),
                         "timing": "CUDA events around each launch on the library stream, in a second pass of the same K steps launched eagerly "
                                   "(the first pass, which gives `value`, replays a CUDA graph and cannot be instrumented per kernel)",
                         "eager_pass_ms_per_step": ms_eager / args.steps,
                         "algorithmic_flop_per_step_this_rank": lin_flop,
                         "traffic": (GEMM_DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE * gemm_bytes(cfg, nseq, T) / max(lin_launches, 1)
                                     if GEMM_DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE else None),
                         "traffic_unit": "bytes per launch (ncu dram__bytes_read.sum + dram__bytes_write.sum)",
                         "traffic_source": "ratio of DRAM bytes to algorithmic bytes measured by ncu on one small Linear launch of the same kernel, "
                                           "times the algorithmic bytes per launch of this run (DRAM traffic of this kernel grows with the bytes it streams)",
                         "algorithmic_bytes_per_launch": gemm_bytes(cfg, nseq, T) / max(lin_launches, 1)},
            "breakdown": breakdown,
            "whole_forward": {"algorithmic_tflop_per_step": (lin_flop + attn_flop) * world / 1e12,
                              "achieved_tflops_per_gpu": (lin_flop + attn_flop) / (ms / args.steps * 1e-3) / 1e12},
        }
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(cfg, T)
    model.close()
    # ---- the rest of the record: op sweeps on one GPU, the tensor-parallel split on several ----
    if world == 1 and args.sweeps:
        line["sweeps"] = compact_sweeps(b, read_peaks(), args.sweep_iters)
    if world > 1 and args.tp:
        rec = tp_measure(b, rank, world, dist, max(2, min(args.steps, 5)), args.warmup, layers=args.layers)
        if rank == 0:
            line["c5_tp"] = rec
    if rank == 0:
        print(json.dumps(line), flush=True)
    b.close()
    if dist is not None:
        dist.destroy_process_group()
    return 0


def _fill(b, buf, n_elems, es, seed, mean=0.0, std=1.0):
    """Fill a device buffer with seeded normals: a 4 Mi-element host block generated once and tiled."""
    from sptorch_b200.backend import f32_to_bf16_bits
    block = synth.normal(seed, min(n_elems, 1 << 22), mean, std)
    host = block if es == 4 else f32_to_bf16_bits(block)
    off = 0
    while off < n_elems:
        m = min(host.size, n_elems - off)
        b._check(b.lib.sptorch_ext_copy_h2d_bytes(host.ctypes.data, buf.handle + off * es, m * es), "fill")
        off += m
    b.synchronize()


def _time_op(b, fn, iters, warmup=3):
    """Median device time of fn() over iters launches, L2 flushed (256 MiB overwrite) before each."""
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        b.flush_l2()
        b.timer_begin()
        fn()
        ts.append(b.timer_end())
    return statistics.median(ts), min(ts)


def _time_stream(b, fns, launches=8):
    """Device time per launch of `launches` launches issued back to back between one pair of events, alternating between the given
    closures (each works on its own buffers; together they exceed L2, so no launch finds its input there).  What a kernel costs
    inside a stream of launches, as in the forward; _time_op times one launch alone, launch latency included."""
    for f in fns:
        f()
    b.flush_l2()
    b.timer_begin()
    for i in range(launches):
        fns[i % len(fns)]()
    return b.timer_end() / launches


def sweep_abi(args, b):
    """The eleven ops of the reference's C-ABI through sptorch_*_f32 with HOST slices (upload, kernel, download: what the
    reference's FfiBackend wrapper does per op, crates/hal-ffi/src/lib.rs:337-446), device-resident, and the reference's own C
    implementation (crates/hal-ffi/mock_npu/mock_npu.c compiled in place) on one host thread."""
    import ctypes as C
    from oracle import binding as O
    ref = O.ref_lib()
    lib = b.lib
    rng = np.random.default_rng(0)
    sz = C.c_size_t
    n = 1 << 24
    x = rng.standard_normal(n).astype(np.float32); y = rng.standard_normal(n).astype(np.float32); pos = (np.abs(x) + 0.1).astype(np.float32)
    m_, k_, n_ = 512, 512, 512
    A = rng.standard_normal((m_, k_)).astype(np.float32); Bm = rng.standard_normal((k_, n_)).astype(np.float32)
    bt, bm, bk, bn = 12, 256, 64, 256
    BA = rng.standard_normal((bt, bm, bk)).astype(np.float32); BB = rng.standard_normal((bt, bk, bn)).astype(np.float32)
    rows, cols = 8192, 1024
    S = rng.standard_normal((rows, cols)).astype(np.float32)
    # (symbol, inputs, output elements, argument builder from handles/pointers, algorithmic bytes or flop, unit)
    cases = [("sptorch_add_f32", [x, y], n, lambda i, o: (i[0], i[1], o, sz(n)), 12 * n, "B"),
             ("sptorch_mul_f32", [x, y], n, lambda i, o: (i[0], i[1], o, sz(n)), 12 * n, "B")]
    for op, arr in (("neg", x), ("exp", x), ("log", pos), ("relu", x), ("gelu", x)):
        cases.append((f"sptorch_{op}_f32", [arr], n, lambda i, o: (i[0], o, sz(n)), 8 * n, "B"))
    cases += [("sptorch_scale_f32", [x], n, lambda i, o: (i[0], C.c_float(0.5), o, sz(n)), 8 * n, "B"),
              ("sptorch_softmax_f32", [S], rows * cols, lambda i, o: (i[0], o, sz(rows), sz(cols)), 8 * rows * cols, "B"),
              ("sptorch_matmul_f32", [A, Bm], m_ * n_, lambda i, o: (i[0], i[1], o, sz(m_), sz(k_), sz(n_)), 2 * m_ * k_ * n_, "FLOP"),
              ("sptorch_batch_matmul_f32", [BA, BB], bt * bm * bn, lambda i, o: (i[0], i[1], o, sz(bt), sz(bm), sz(bk), sz(bn)), 2 * bt * bm * bk * bn, "FLOP")]
    out = []
    for name, ins, out_n, build, work, unit in cases:
        fn = getattr(lib, name)
        # host slices in, host slice out
        ts = []
        for _ in range(5):
            t0 = time.perf_counter()
            bufs = [b.upload(a_) for a_ in ins]
            o = b.alloc(out_n)
            b._check(fn(*build([u.handle for u in bufs], o.handle)), name)
            got = o.to_host()
            b.synchronize()
            ts.append(time.perf_counter() - t0)
            for u in bufs + [o]:
                u.free()
        host_ms = statistics.median(ts) * 1e3
        # device-resident
        bufs = [b.upload(a_) for a_ in ins]
        o = b.alloc(out_n)
        dev_ms, _ = _time_op(b, lambda: b._check(fn(*build([u.handle for u in bufs], o.handle)), name), args.iters)
        for u in bufs + [o]:
            u.free()
        line = {"op": name, "elements_out": out_n, "host_slices_ms": host_ms, "device_resident_ms": dev_ms,
                "device_rate": work / (dev_ms * 1e-3) / 1e9, "device_rate_unit": "GB/s" if unit == "B" else "GFLOP/s"}
        if ref is not None:
            ro = np.empty(out_n, np.float32)
            rf = getattr(ref, name)
            t0 = time.perf_counter()
            rf(*build([a_.ctypes.data_as(C.c_void_p) for a_ in ins], ro.ctypes.data_as(C.c_void_p)))
            line["reference_c_ms"] = (time.perf_counter() - t0) * 1e3
            line["reference_c"] = "crates/hal-ffi/mock_npu/mock_npu.c, one host thread"
            scale = max(1.0, float(np.abs(ro).max()))
            line["max_abs_diff_vs_reference_c"] = float(np.abs(got - ro.ravel()).max() / scale)
        out.append(line)
        print(json.dumps(line), flush=True)
    return out


LINEAR_SWEEP_SHAPES = [(M, K, N) for M in (512, 4096, 16384) for (K, N) in ((768, 768), (768, 3072), (3072, 768), (4096, 4096))]
ATTENTION_SWEEP_SHAPES = [(64, 1024, 12, 64), (16, 2048, 16, 128)]       # one layer of c4_gpt2s and of c5_1p3b


def sweep_linear(b, peaks, iters, shapes=None, emit=None):
    """Standalone Linear y = x W^T + b at the sweep's shapes, bf16 and TF32: TFLOP/s and the fraction of the measured burst peak."""
    from sptorch_b200.backend import BF16, F32, MM_BF16, MM_TF32
    lib, out = b.lib, []
    for (M, K, N) in (shapes or LINEAR_SWEEP_SHAPES):
        for mode, name, es in ((MM_BF16, "bf16", 2), (MM_TF32, "tf32", 4)):
            x, w, y = b.alloc(M * K, es), b.alloc(N * K, es), b.alloc(M * N, es)
            bias = b.alloc(N)
            _fill(b, x, M * K, es, 1); _fill(b, w, N * K, es, 2, std=0.02); _fill(b, bias, N, 4, 3, std=0.01)
            fn = lambda: b._check(lib.sptorch_ext_linear(x.handle, w.handle, bias.handle, None, y.handle, M, K, N, 0, C.c_float(1.0), 0, mode,
                                                         BF16 if mode == MM_BF16 else F32), "linear")
            med, best = _time_op(b, fn, iters)
            tf = 2.0 * M * K * N / (med * 1e-3) / 1e12
            peak = peaks["tf"] if mode == MM_BF16 else peaks["tf"] / 2
            out.append({"op": "linear", "M": M, "K": K, "N": N, "mode": name, "ms": med, "ms_best": best, "tflops": tf,
                        "frac": tf / peak, "peak": peak, "peak_note": f"{peaks['source']} burst cuBLAS bf16" + ("" if mode == MM_BF16 else " / 2 (TF32 runs at half the bf16 rate)"),
                        "frac_nominal": tf / (2250.0 if mode == MM_BF16 else 1125.0)})
            if emit:
                emit(out[-1])
            for buf in (x, w, y, bias):
                buf.free()
    return out


def sweep_attention(b, peaks, iters, shapes=None, emit=None):
    """Causal attention core of one layer (bf16, fused kernel): TFLOP/s on the causal-necessary FLOP."""
    from sptorch_b200.backend import BF16
    lib, out = b.lib, []
    for (B_, T_, H_, hd_) in (shapes or ATTENTION_SWEEP_SHAPES):
        d_ = H_ * hd_
        q, k, v, o = (b.alloc(B_ * T_ * d_, 2) for _ in range(4))
        for i, buf in enumerate((q, k, v)):
            _fill(b, buf, B_ * T_ * d_, 2, 20 + i)
        ws = b.alloc(lib.sptorch_ext_attention_workspace(B_, T_, H_, hd_, BF16), 1)
        fn = lambda: b._check(lib.sptorch_ext_attention_causal(q.handle, k.handle, v.handle, o.handle, ws.handle, B_, T_, H_, hd_, d_, BF16), "attention")
        med, best = _time_op(b, fn, iters)
        flop = 2.0 * B_ * H_ * T_ * (T_ + 1) * hd_
        out.append({"op": "attention_causal", "B": B_, "T": T_, "H": H_, "hd": hd_, "dtype": "bf16", "ms": med, "ms_best": best,
                    "tflops": flop / (med * 1e-3) / 1e12, "frac": flop / (med * 1e-3) / 1e12 / peaks["tf"], "peak": peaks["tf"],
                    "note": "FLOP counted on the causal-necessary half (2 T (T+1) hd per sequence and head)"})
        if emit:
            emit(out[-1])
        for buf in (q, k, v, o, ws):
            buf.free()
    return out


def sweep_rowops(b, peaks, iters, emit=None):
    """LayerNorm (65536 rows of 768 / 2048 / 4096), causal softmax [16, 12, 1024, 1024] and GELU over 64 Mi elements, f32 and bf16:
    achieved GB/s on the minimal necessary traffic and the fraction of the measured copy bandwidth."""
    from sptorch_b200.backend import BF16, F32
    lib, out = b.lib, []

    def rec(entry):
        out.append(entry)
        if emit:
            emit(entry)

    for dim in (768, 2048, 4096):
        for dt, name, es in ((F32, "f32", 4), (BF16, "bf16", 2)):
            rows = 65536
            x, y = b.alloc(rows * dim, es), b.alloc(rows * dim, es)
            g, be = b.upload(np.ones(dim, np.float32)), b.upload(np.zeros(dim, np.float32))
            _fill(b, x, rows * dim, es, 4, mean=0.5, std=3.0)
            fn = lambda: b._check(lib.sptorch_ext_layernorm(x.handle, g.handle, be.handle, y.handle, rows, dim, C.c_float(1e-5), dt), "layernorm")
            med, best = _time_op(b, fn, iters)
            x2, y2 = b.alloc(rows * dim, es), b.alloc(rows * dim, es)
            _fill(b, x2, rows * dim, es, 7, mean=0.5, std=3.0)
            fn2 = lambda: b._check(lib.sptorch_ext_layernorm(x2.handle, g.handle, be.handle, y2.handle, rows, dim, C.c_float(1e-5), dt), "layernorm")
            ms_s = _time_stream(b, [fn, fn2])
            nbytes = 2 * rows * dim * es + 2 * dim * 4
            rec({"op": "layernorm", "rows": rows, "dim": dim, "dtype": name, "ms": med, "ms_best": best, "gbs": nbytes / (med * 1e-3) / 1e9,
                 "frac": nbytes / (med * 1e-3) / 1e9 / peaks["hbm"], "peak": peaks["hbm"], "algorithmic_bytes": nbytes,
                 "ms_back_to_back": ms_s, "frac_back_to_back": nbytes / (ms_s * 1e-3) / 1e9 / peaks["hbm"]})
            for buf in (x, y, g, be, x2, y2):
                buf.free()
    for dt, name, es in ((F32, "f32", 4), (BF16, "bf16", 2)):
        B_, H_, T_ = 16, 12, 1024
        n = B_ * H_ * T_ * T_
        x, y = b.alloc(n, es), b.alloc(n, es)
        _fill(b, x, n, es, 5, std=2.0)
        fn = lambda: b._check(lib.sptorch_ext_causal_softmax(x.handle, y.handle, B_ * H_, T_, C.c_float(1.0), dt), "causal_softmax")
        med, best = _time_op(b, fn, iters)
        x2, y2 = b.alloc(n, es), b.alloc(n, es)
        _fill(b, x2, n, es, 8, std=2.0)
        fn2 = lambda: b._check(lib.sptorch_ext_causal_softmax(x2.handle, y2.handle, B_ * H_, T_, C.c_float(1.0), dt), "causal_softmax")
        ms_s = _time_stream(b, [fn, fn2])
        nbytes = (T_ * (T_ + 1) // 2 + T_ * T_) * B_ * H_ * es
        rec({"op": "causal_softmax", "shape": [B_, H_, T_, T_], "dtype": name, "ms": med, "ms_best": best, "gbs": nbytes / (med * 1e-3) / 1e9,
             "frac": nbytes / (med * 1e-3) / 1e9 / peaks["hbm"], "peak": peaks["hbm"], "algorithmic_bytes": nbytes, "full_read_bytes": 2 * n * es,
             "ms_back_to_back": ms_s, "frac_back_to_back": nbytes / (ms_s * 1e-3) / 1e9 / peaks["hbm"]})
        for buf in (x, y, x2, y2):
            buf.free()
    for dt, name, es in ((F32, "f32", 4), (BF16, "bf16", 2)):
        n = 64 << 20
        x, y = b.alloc(n, es), b.alloc(n, es)
        _fill(b, x, n, es, 6)
        fn = lambda: b._check(lib.sptorch_ext_gelu(x.handle, y.handle, n, dt), "gelu")
        med, best = _time_op(b, fn, iters)
        x2, y2 = b.alloc(n, es), b.alloc(n, es)
        _fill(b, x2, n, es, 9)
        fn2 = lambda: b._check(lib.sptorch_ext_gelu(x2.handle, y2.handle, n, dt), "gelu")
        ms_s = _time_stream(b, [fn, fn2])
        nbytes = 2 * n * es
        rec({"op": "gelu", "n": n, "dtype": name, "ms": med, "ms_best": best, "gbs": nbytes / (med * 1e-3) / 1e9,
             "frac": nbytes / (med * 1e-3) / 1e9 / peaks["hbm"], "peak": peaks["hbm"], "algorithmic_bytes": nbytes,
             "ms_back_to_back": ms_s, "frac_back_to_back": nbytes / (ms_s * 1e-3) / 1e9 / peaks["hbm"]})
        for buf in (x, y, x2, y2):
            buf.free()
    return out


def sweep_decode(b, peaks, steps=32, emit=None, batches=(1, 8, 64)):
    """Incremental decode of the GPT-2-small shape through the key/value cache: `batch` sequences with 512 cached positions, one
    new token each per step.  HBM-bound: a step reads every weight once (325 MB in bf16) plus the cached keys and values."""
    from sptorch_b200.backend import BF16
    from sptorch_b200.gpt import GPT
    cfg = dict(synth.CONFIGS[WORKLOAD])
    d, F, V, L = cfg["d_model"], cfg["d_ff"], cfg["vocab"], cfg["n_layer"]
    out = []
    for batch in batches:
        model = GPT(b, V, d, cfg["n_head"], L, F, cfg["seq_len"], dtype=BF16, max_batch=batch)
        _load_timing_weights(model, cfg)
        model.enable_kv_cache(1024)
        ctx0 = 512
        ids = synth.randint(1, batch * ctx0, V).reshape(batch, ctx0)
        model.prefill_kv_cache(ids)
        nxt = synth.randint(2, batch, V).astype(np.int32)
        d_ids, d_log = model.stage_ids(nxt), model.logits_buffer(batch)
        for _ in range(3):
            b._check(b.lib.sptorch_ext_gpt_decode(model.h, d_ids.handle, batch, 1, d_log.handle), "gpt_decode")
        b.synchronize()
        b.timer_begin()
        for _ in range(steps):
            b._check(b.lib.sptorch_ext_gpt_decode(model.h, d_ids.handle, batch, 1, d_log.handle), "gpt_decode")
        ms = b.timer_end() / steps
        n_ctx = ctx0 + 3 + steps // 2
        nbytes = 2 * (L * (4 * d * d + 2 * d * F) + V * d) + 2 * 2 * L * batch * n_ctx * d
        out.append({"op": "decode_step", "batch": batch, "cached_positions": n_ctx, "ms_per_step": ms, "tokens_per_s": batch / (ms * 1e-3),
                    "gbs": nbytes / (ms * 1e-3) / 1e9, "frac": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm"], "peak": peaks["hbm"],
                    "algorithmic_bytes": nbytes})
        if batch == 1:
            # the reference's generation loop (decode_next_token: decode step, sampling candidates on the device, the draw on the
            # host) in its greedy configuration, host-driven, wall clock: the first call prefills the prompt and is not timed
            import time
            toks = [int(t) for t in ids[0]]
            model._gen_ctx, model._prompt_len = None, len(toks)
            model.decode_next_token(toks, top_k=1)
            b.synchronize()
            t0 = time.perf_counter()
            for _ in range(32):
                model.decode_next_token(toks, top_k=1)
            b.synchronize()
            out[-1]["generate_greedy_tokens_per_s"] = 32 / (time.perf_counter() - t0)
        if emit:
            emit(out[-1])
        model.close()
    return out


def compact_sweeps(b, peaks, iters):
    """The three sweeps in the short form the bench line carries: one entry per case with its time and fraction of the roof
    (Linear and attention: measured burst bf16 tensor peak, TF32 against half of it; row ops: measured copy bandwidth)."""
    lin = sweep_linear(b, peaks, iters)
    att = sweep_attention(b, peaks, iters)
    row = sweep_rowops(b, peaks, iters)
    dec = sweep_decode(b, peaks)
    r3 = lambda v: float(f"{v:.4g}")
    return {
        "timing": f"median of {iters} launches, CUDA events on the library stream, 256 MiB L2 flush before each launch, 3 warm-up launches",
        "linear": [{"M": e["M"], "K": e["K"], "N": e["N"], "mode": e["mode"], "ms": r3(e["ms"]), "tflops": r3(e["tflops"]), "frac": r3(e["frac"])} for e in lin],
        "linear_roof": f"{peaks['tf']} TFLOP/s bf16 ({peaks['source']} burst), TF32 against half of it",
        "attention": [{"B": e["B"], "T": e["T"], "H": e["H"], "hd": e["hd"], "ms": r3(e["ms"]), "tflops": r3(e["tflops"]), "frac": r3(e["frac"])} for e in att],
        "rowops": [{"op": e["op"], "dtype": e["dtype"], **({"dim": e["dim"]} if "dim" in e else {}), "ms": r3(e["ms"]), "gbs": r3(e["gbs"]), "frac": r3(e["frac"]),
                    "ms_back_to_back": r3(e["ms_back_to_back"]), "frac_back_to_back": r3(e["frac_back_to_back"])} for e in row],
        "rowops_roof": f"{peaks['hbm']} GB/s ({peaks['source']} copy bandwidth); frac: one launch timed alone (its launch latency included); "
                       "frac_back_to_back: eight launches between one pair of events, alternating between two sets of buffers (together larger than L2)",
        "decode": [{"batch": e["batch"], "cached_positions": e["cached_positions"], "ms_per_step": r3(e["ms_per_step"]), "tokens_per_s": r3(e["tokens_per_s"]),
                    "frac": r3(e["frac"]), **({"generate_greedy_tokens_per_s": r3(e["generate_greedy_tokens_per_s"])} if "generate_greedy_tokens_per_s" in e else {})}
                   for e in dec],
        "decode_note": "one new token per sequence through the key/value cache of the GPT-2-small shape; frac = (weights + cached K/V bytes) per step over the copy bandwidth; generate_greedy_tokens_per_s: the host-driven generation loop (decode step + device sampling candidates + host draw), wall clock",
    }


def run_sweep(args):
    """The standalone Linear sweep, the row-op sweep and the attention core: one JSON line per case."""
    os.environ.setdefault("SPTORCH_B200_DEVICE", "0")
    from sptorch_b200.backend import FfiBackend
    b = FfiBackend.load()
    peaks = read_peaks()
    emit = lambda e: print(json.dumps(e), flush=True)
    one = [tuple(int(v) for v in args.shape.split(","))] if args.shape else None
    if args.sweep in ("linear", "all"):
        sweep_linear(b, peaks, args.iters, one if args.sweep == "linear" else None, emit)
    if args.sweep == "abi":
        sweep_abi(args, b)
    if args.sweep in ("attention", "all"):
        sweep_attention(b, peaks, args.iters, one if args.sweep == "attention" else None, emit)
    if args.sweep in ("rowops", "all"):
        sweep_rowops(b, peaks, args.iters, emit)
    if args.sweep in ("decode", "all"):
        if args.sweep == "decode" and args.shape:       # a single batch size and step count: "batch,steps"
            bt, st = (int(v) for v in args.shape.split(","))
            sweep_decode(b, peaks, steps=st, emit=emit, batches=(bt,))
        else:
            sweep_decode(b, peaks, emit=emit)
    b.close()
    return 0


def _load_timing_weights(model, cfg, seed=0):
    """Weights for a timing run of a model too large to draw element by element on every rank: each matrix is a seeded
    4 Mi-element N(0, 0.02) block repeated to size (residual projections scaled by 1/sqrt(2 L), biases 0, gamma 1, beta 0),
    uploaded one parameter at a time.  Parity runs use synth.gpt_params instead."""
    block = synth.normal(seed, 1 << 22, 0.0, 0.02)
    rs = np.float32(1.0 / np.sqrt(2.0 * cfg["n_layer"]))
    for i, (name, shape) in enumerate(model.named_parameters()):
        n = int(np.prod(shape))
        if name.endswith(".gamma"):
            w = np.ones(n, np.float32)
        elif name.endswith(".beta") or name.endswith(".bias"):
            w = np.zeros(n, np.float32)
        else:
            w = np.resize(np.roll(block, 7919 * i), n)
            if name.endswith("attn.wo.weight") or name.endswith("ffn_down.weight"):
                w = w * rs
        model.set_param(name, w)


def _nccl_for_model(b, lib, dist, rank, world, model):
    uid = C.create_string_buffer(128)
    if rank == 0:
        b._check(lib.sptorch_ext_nccl_unique_id(None, uid), "nccl_unique_id")
    box = [uid.raw]
    dist.broadcast_object_list(box, src=0)
    uid = C.create_string_buffer(box[0], 128)
    b._check(lib.sptorch_ext_nccl_init(None, uid, rank, world), "nccl_init")


def tp_measure(b, rank, world, dist, steps, warmup, layers=0, batch=0, tp_overlap=-1, sm_reserve=0, check_only=False):
    """Tensor-parallel forward over the launched ranks (wq/wk/wv/ffn_up split by rows, wo/ffn_down along K, one NCCL all-reduce per
    attention and per MLP block).  Two parts: a small model (4 or 8 heads of 64, 2 layers) whose logits are compared with the CPU
    oracle on rank 0 -- once with the all-reduces in line and once with them overlapped with the other half of the batch -- and -- unless check_only -- the 1.3B shape c5_1p3b (vocab 50257, d 2048, 24 layers, 16 heads of 128,
    d_ff 8192, batch 16 x 2048 tokens, bf16) timed on the device, max over ranks.  Returns the record rank 0 prints."""
    import torch
    from sptorch_b200.backend import BF16
    from sptorch_b200.gpt import GPT
    lib = b.lib
    if world > 1:
        _nccl_for_model(b, lib, dist, rank, world, None)
    rec = {}
    # ---- parity of the partition on a small model ----
    heads = 4 if world <= 4 else 8                      # heads of 64: the fused attention, which the overlapped forward needs
    cfg = dict(vocab=1000, d_model=64 * heads, n_layer=2, n_head=heads, d_ff=256 * heads, seq_len=256, batch=2, ctx=256)
    model = GPT(b, cfg["vocab"], cfg["d_model"], cfg["n_head"], cfg["n_layer"], cfg["d_ff"], cfg["seq_len"], dtype=BF16,
                max_batch=2, tp_rank=rank, tp_size=world)
    params, index = synth.gpt_params(cfg, 0, residual_scale=True, randomize_affine=True)
    model.load_flat(params, index)
    if world > 1:
        b._check(lib.sptorch_ext_gpt_use_nccl(model.h), "gpt_use_nccl")
    ids = synth.randint(1, 2 * 256, cfg["vocab"]).reshape(2, 256).astype(np.int32)
    outs = []
    for mode in (0, 1):
        b._check(lib.sptorch_ext_gpt_enable_tp_overlap(model.h, mode), "tp_overlap")
        outs.append(model.forward(ids))
    out, out_ov = outs
    model.close()
    if rank == 0:
        from oracle import binding as O
        O.build()
        ref = O.gpt_forward(cfg, params, ids, fast=1, threads=host_threads())
        err = float(np.abs(out - ref).max() / np.abs(ref).max())
        err_ov = float(np.abs(out_ov - ref).max() / np.abs(ref).max())
        rec.update({"tp_size": world, "check_model": "vocab 1000, d %d, 2 layers, %d heads, d_ff %d, 2 x 256 tokens, bf16" % (cfg["d_model"], heads, cfg["d_ff"]),
                    "max_rel_err_vs_oracle": err, "max_rel_err_vs_oracle_overlapped": err_ov, "overlapped_equals_serial": bool(np.array_equal(out, out_ov)),
                    "tolerance": 2e-2, "check_ok": bool(err <= 2e-2 and err_ov <= 2e-2)})
    if check_only:
        if world > 1:
            lib.sptorch_ext_nccl_shutdown()
        return rec
    # ---- the 1.3B shape, timed ----
    cfg = dict(synth.CONFIGS["c5_1p3b"])
    if layers:
        cfg["n_layer"] = layers
    T, B = cfg["ctx"], batch or cfg["batch"]
    model = GPT(b, cfg["vocab"], cfg["d_model"], cfg["n_head"], cfg["n_layer"], cfg["d_ff"], cfg["seq_len"], dtype=BF16,
                max_batch=B, tp_rank=rank, tp_size=world)
    _load_timing_weights(model, cfg)
    if world > 1:
        b._check(lib.sptorch_ext_gpt_use_nccl(model.h), "gpt_use_nccl")
        if tp_overlap >= 0:                              # otherwise the library's rule: overlapped from four ranks up
            b._check(lib.sptorch_ext_gpt_enable_tp_overlap(model.h, int(tp_overlap)), "tp_overlap")
        if sm_reserve > 0:                               # otherwise the library leaves 32 SMs free while an overlapped forward runs
            b._check(lib.sptorch_ext_set_sm_reserve(sm_reserve), "sm_reserve")
    overlapped = world > 1 and (tp_overlap == 1 or (tp_overlap < 0 and world >= 4))
    ids = synth.randint(1, B * T, cfg["vocab"]).reshape(B, T).astype(np.int32)
    d_ids, d_logits = model.stage_ids(ids), model.logits_buffer(B * T)

    def sync():
        b.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(warmup, 3)):
        model.forward_device(d_ids, B, T, d_logits)
    sync()
    lib.sptorch_ext_prof_enable(1); lib.sptorch_ext_prof_read(None, None, 0)
    b.timer_begin()
    for _ in range(steps):
        model.forward_device(d_ids, B, T, d_logits)
    ms = b.timer_end()
    sync()
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX); ms = float(t.item())
    pm, pn = (C.c_float * 7)(), (C.c_uint32 * 7)()
    lib.sptorch_ext_prof_read(pm, pn, 7); lib.sptorch_ext_prof_enable(0)
    if sm_reserve > 0:
        b._check(lib.sptorch_ext_set_sm_reserve(0), "sm_reserve")
    model.close()
    if world > 1:
        lib.sptorch_ext_nccl_shutdown()
    if rank == 0:
        cats = ["linear_gemm", "attention_gemm", "causal_softmax", "layernorm", "embedding", "allreduce_and_other", "attention_fused"]
        lin, attn = flops_per_forward(cfg, B, T)
        rec.update({"workload": "c5_1p3b", "n_layer": cfg["n_layer"], "batch": B, "seq_len": T, "parallelism": f"tensor-parallel x{world}",
                    "tp_overlap": bool(overlapped), "steps": steps, "ms_per_step": ms / steps, "tokens_per_s": B * T * steps / (ms * 1e-3),
                    "achieved_tflops_whole_job": (lin + attn) / (ms / steps * 1e-3) / 1e12,
                    "allreduce_ms_per_step_rank0": None if overlapped else float(pm[5]) / steps, "allreduces_per_step": 2 * cfg["n_layer"],
                    "allreduce_bytes_each": B * T * cfg["d_model"] * 2,
                    "breakdown_rank0_ms": {c: float(pm[i]) / steps for i, c in enumerate(cats) if pn[i]},
                    "weights": "seeded N(0,0.02) block repeated per matrix (timing only; parity is the small check model above)"})
    return rec


def run_tp(args):
    """Stand-alone tensor-parallel run (--workload c5_1p3b, or tp_check for the parity part alone)."""
    rank, local_rank, world = dist_env()
    import torch
    import torch.distributed as dist
    os.environ.setdefault("SPTORCH_B200_DEVICE", str(local_rank))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    from sptorch_b200.backend import FfiBackend
    b = FfiBackend.load()
    rec = tp_measure(b, rank, world, dist, args.steps, args.warmup, layers=args.layers, batch=args.batch, tp_overlap=args.tp_overlap,
                     sm_reserve=args.sm_reserve, check_only=args.workload == "tp_check")
    if rank == 0:
        print(json.dumps(rec), flush=True)
    b.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=0, help="override the global batch (sequences); 0 = the workload's 64")
    ap.add_argument("--chunk", type=int, default=8, help="sequences per micro-batch of the host-buffer call")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--sweep", default="", choices=["", "linear", "rowops", "attention", "decode", "abi", "all"], help="standalone op sweeps (the standalone Linear and row-op sweeps) instead of the GPT step")
    ap.add_argument("--shape", default="", help="with --sweep linear: a single M,K,N; with --sweep decode: batch,steps")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--workload", default=WORKLOAD, choices=[WORKLOAD, "c5_1p3b", "tp_check"],
                    help="c4_gpt2s: the bench line (batch sharding); c5_1p3b / tp_check: tensor parallel over the launched ranks")
    ap.add_argument("--ln-fold", type=int, default=0, help="1: LayerNorm folded into the GEMM epilogues instead of separate kernels")
    ap.add_argument("--tp-overlap", type=int, default=-1, help="tensor parallel: overlap the all-reduces with the other half of the batch (0 / 1; -1: the library's rule, on from four ranks up)")
    ap.add_argument("--sm-reserve", type=int, default=0, help="SMs left free for NCCL by every persistent kernel (0: the library leaves 32 free during an overlapped forward)")
    ap.add_argument("--layers", type=int, default=0, help="tensor-parallel model: run fewer than its 24 layers")
    ap.add_argument("--sweeps", type=int, default=1, help="1 GPU: append the compact Linear / row-op / attention sweeps to the line (0 = skip)")
    ap.add_argument("--sweep-iters", type=int, default=7, help="timed launches per case of the compact sweeps")
    ap.add_argument("--tp", type=int, default=1, help="several GPUs: append the tensor-parallel record c5_tp to the line (0 = skip)")
    args = ap.parse_args()
    if args.sweep:
        return run_sweep(args)
    if args.impl == "reference":
        return run_reference(args)
    if args.workload != WORKLOAD:
        return run_tp(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
