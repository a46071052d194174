"""Host-side logic that needs no GPU: seeded inputs, bf16 conversion, parameter layout, batch sharding
(single process and two gloo ranks)."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_synth_is_counter_based_and_deterministic():
    from sptorch_b200 import synth
    a = synth.normal(0, 10000, 0.0, 0.02)
    b = synth.normal(0, 10000, 0.0, 0.02)
    assert np.array_equal(a, b)
    assert np.array_equal(synth.normal(0, 100, start=500), synth.normal(0, 1000)[500:600])
    assert abs(float(a.std()) - 0.02) < 1e-3 and abs(float(a.mean())) < 1e-3
    ids = synth.randint(1, 100000, 50257)
    assert ids.min() >= 0 and ids.max() < 50257 and len(np.unique(ids)) > 40000
    assert not np.array_equal(synth.normal(0, 100), synth.normal(1, 100))


def test_param_layout_matches_named_parameters_order():
    # crates/nn/src/lib.rs:1382-1392
    from sptorch_b200 import synth
    names = [n for n, _ in synth.gpt_param_layout(256, 128, 2, 4, 512, 64)]
    assert names[:2] == ["token_emb.weight", "pos_emb.weight"]
    assert names[2:14] == ["blocks.0." + s for s in ("ln1.gamma", "ln1.beta", "attn.wq.weight", "attn.wk.weight", "attn.wv.weight",
                                                     "attn.wo.weight", "ln2.gamma", "ln2.beta", "ffn_up.weight", "ffn_up.bias",
                                                     "ffn_down.weight", "ffn_down.bias")]
    assert names[-3:] == ["ln_f.gamma", "ln_f.beta", "lm_head.weight"]
    cfg = synth.CONFIGS["c4_gpt2s"]
    total = sum(int(np.prod(s)) for _, s in synth.gpt_param_layout(cfg["vocab"], cfg["d_model"], cfg["n_layer"], cfg["n_head"], cfg["d_ff"], cfg["seq_len"]))
    assert total == 163_000_320      # untied head


def test_bf16_round_to_nearest_even():
    from sptorch_b200.backend import bf16_bits_to_f32, f32_to_bf16_bits
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e38, 1e-40], dtype=np.float32)
    back = bf16_bits_to_f32(f32_to_bf16_bits(x))
    assert back[0] == 1.0
    assert back[1] == 1.0            # exactly half way between 1.0 and 1.0078125: ties to even
    assert back[2] == np.float32(1.015625)
    assert back[3] == -2.5
    import torch
    t = torch.from_numpy(np.random.default_rng(0).standard_normal(10000).astype(np.float32))
    assert np.array_equal(bf16_bits_to_f32(f32_to_bf16_bits(t.numpy())), t.to(torch.bfloat16).to(torch.float32).numpy())


def test_shard_rule_remainder_to_first_ranks():
    # DataParallel::scatter, crates/distributed/src/data_parallel.rs:21-37
    sys.path.insert(0, ROOT)
    import bench
    assert [bench.shard(64, 8, r) for r in range(8)] == [(8 * r, 8) for r in range(8)]
    parts = [bench.shard(10, 4, r) for r in range(4)]
    assert parts == [(0, 3), (3, 3), (6, 2), (8, 2)]
    assert sum(n for _, n in parts) == 10
    assert [bench.shard(2, 4, r)[1] for r in range(4)] == [1, 1, 0, 0]


def _gloo_worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import torch
    sys.path.insert(0, ROOT)
    import bench
    from oracle import binding as O
    from sptorch_b200 import synth
    cfg = dict(vocab=64, d_model=32, n_layer=1, n_head=2, d_ff=64, seq_len=16)
    p, _ = synth.gpt_params(cfg, 0)
    ids = synth.randint(1, 6 * 16, 64).reshape(6, 16)
    s, n = bench.shard(6, world, rank)
    mine = O.gpt_forward(cfg, p, ids[s:s + n])           # this rank's sequences only: no collective in the forward
    # checksum exchange: sum of all ranks' logits equals the unsharded run's
    t = torch.tensor([float(mine.astype(np.float64).sum()), float(n)], dtype=torch.float64)
    dist.all_reduce(t)
    # timing convention of the bench: max over ranks
    tm = torch.tensor([0.1 * (rank + 1)], dtype=torch.float64)
    dist.all_reduce(tm, op=dist.ReduceOp.MAX)
    if rank == 0:
        full = O.gpt_forward(cfg, p, ids)
        q.put((float(t[0]), float(full.astype(np.float64).sum()), float(t[1]), float(tm[0])))
    dist.destroy_process_group()


def test_batch_sharding_two_gloo_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 1000
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    sharded_sum, full_sum, n, tmax = got
    assert n == 6
    assert abs(sharded_sum - full_sum) < 1e-6 * max(1.0, abs(full_sum))
    assert abs(tmax - 0.2) < 1e-12


def _tp_worker(rank, world, port, q):
    """Tensor-parallel MLP + attention-output partition on CPU ranks: the slicing rule of sptorch_b200/csrc/gpt.cu
    (ffn_up / wq,wk,wv split by output rows, ffn_down / wo split along K, residual and ffn_down bias folded into rank
    0's partial) followed by a sum all-reduce must reproduce the unsharded block."""
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    from oracle import binding as O
    from sptorch_b200 import synth
    d, F, M = 32, 64, 10
    x = synth.normal(1, M * d).reshape(M, d)
    h = synth.normal(2, M * d).reshape(M, d)                 # LayerNorm output feeding the MLP
    w1 = synth.normal(3, F * d, std=0.1).reshape(F, d); b1 = synth.normal(4, F, std=0.1)
    w2 = synth.normal(5, d * F, std=0.1).reshape(d, F); b2 = synth.normal(6, d, std=0.1)
    Fl = F // world
    rows = slice(rank * Fl, (rank + 1) * Fl)
    f = O.unary("gelu", O.linear(h, w1[rows], b1[rows]))     # column-parallel up projection + GELU
    part = O.linear(f, np.ascontiguousarray(w2[:, rows]), b2 if rank == 0 else None)   # row-parallel down projection
    if rank == 0:
        part = part + x                                      # residual folded into rank 0's partial
    t = torch.from_numpy(part.copy())
    dist.all_reduce(t)                                       # the one collective of the MLP block
    if rank == 0:
        full = x + O.linear(O.unary("gelu", O.linear(h, w1, b1)), w2, b2)
        q.put(float(np.abs(t.numpy() - full).max()))
    dist.destroy_process_group()


def test_tensor_parallel_partition_two_gloo_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + os.getpid() % 1000
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    err = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert err < 1e-5


def test_kv_cache_metadata_mirrors_the_reference():
    # crates/hal/src/lib.rs:674-721
    from sptorch_b200.kv_cache import KvCacheBufferSpec, KvCacheWindowState
    spec = KvCacheBufferSpec(("cuda", 0), "BF16", 2, 4, 3, 8)
    assert spec.elements_per_kind() == 2 * 4 * 3 * 8
    assert spec.total_elements() == 2 * 2 * 4 * 3 * 8
    assert spec.total_bytes() == 2 * 2 * 4 * 3 * 8 * 2
    assert spec.element_offset(1, 2, 1, 3) == (((4 + 2) * 3 + 1) * 8) + 3
    with pytest.raises(IndexError):
        spec.element_offset(0, 4, 0, 0)
    with pytest.raises(ValueError):
        KvCacheBufferSpec(("cpu", 0), "F32", 1, 0, 2, 4)
    w = KvCacheWindowState(3)
    assert w.next_position() == 0 and w.last_position() is None
    w.prefill(5, 2)
    assert (w.window_start, w.cached_len, w.last_position(), w.next_position()) == (5, 2, 6, 7)
    w.append(2)
    assert (w.window_start, w.cached_len, w.last_position(), w.next_position()) == (6, 3, 8, 9)
    v = KvCacheWindowState(3)
    v.prefill(10, 3); v.append(1)
    assert v == KvCacheWindowState(3, 11, 3)
    assert KvCacheBufferSpec(("cpu", 0), "F32", 1, 3, 2, 4).total_bytes() == 2 * 1 * 3 * 2 * 4 * 4
