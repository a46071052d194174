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


def _tp_shard(lib, name, full, rank, world):
    """This rank's shard of a full parameter, cut by the library's own rule (the functions gpt_set_param uses on upload)."""
    import ctypes as C
    full = np.ascontiguousarray(full, dtype=np.float32)
    rows, cols = (full.shape[0], 1) if full.ndim == 1 else full.shape
    kind, begin, count = C.c_int(), C.c_size_t(), C.c_size_t()
    assert lib.sptorch_ext_tp_param_shard(name.encode(), rank, world, rows, cols, C.byref(kind), C.byref(begin), C.byref(count)) == 0
    shape = {0: (rows, cols), 1: (count.value, cols), 2: (rows, count.value)}[kind.value]
    out = np.empty(shape, dtype=np.float32)
    assert lib.sptorch_ext_tp_slice_host(full.ctypes.data, rows, cols, kind.value, begin.value, count.value, out.ctypes.data) == 0
    return (out.reshape(-1) if full.ndim == 1 else out), kind.value, begin.value, count.value


def _tp_worker(rank, world, port, q):
    """One transformer block (attention + MLP) cut over CPU ranks with the LIBRARY's shard rule -- sptorch_ext_tp_param_shard /
    sptorch_ext_tp_slice_host / sptorch_ext_tp_rank_folds_residual, the host functions sptorch_ext_gpt_set_param itself applies
    when it uploads a rank's weights -- followed by one sum all-reduce per attention and per MLP block, must reproduce the
    unsharded block.  (The arithmetic around the slices is the oracle's; what is under test is which slice each rank owns.)"""
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    from oracle import binding as O
    from sptorch_b200 import _lib, synth
    lib = _lib.load()                                         # host functions only: no device is needed
    d, F, T, H = 32, 64, 10, 4
    hd = d // H
    x = synth.normal(1, T * d).reshape(T, d)
    h1 = synth.normal(2, T * d).reshape(T, d)                 # LayerNorm outputs feeding attention / the MLP
    h2 = synth.normal(7, T * d).reshape(T, d)
    full = {"attn.wq.weight": synth.normal(10, d * d, std=0.2).reshape(d, d), "attn.wk.weight": synth.normal(11, d * d, std=0.2).reshape(d, d),
            "attn.wv.weight": synth.normal(12, d * d, std=0.2).reshape(d, d), "attn.wo.weight": synth.normal(13, d * d, std=0.2).reshape(d, d),
            "ffn_up.weight": synth.normal(3, F * d, std=0.1).reshape(F, d), "ffn_up.bias": synth.normal(4, F, std=0.1),
            "ffn_down.weight": synth.normal(5, d * F, std=0.1).reshape(d, F), "ffn_down.bias": synth.normal(6, d, std=0.1)}
    mine = {}
    kinds = {}
    for name, w in full.items():
        mine[name], kinds[name], begin, count = _tp_shard(lib, "blocks.0." + name, w, rank, world)
    lead = bool(lib.sptorch_ext_tp_rank_folds_residual(rank))
    Hl = H // world
    # attention: this rank's heads (rows of wq / wk / wv), then its K-slice of wo; partial [T, d]
    ql, kl, vl = (O.linear(h1, mine[n]) for n in ("attn.wq.weight", "attn.wk.weight", "attn.wv.weight"))
    # the attention core of the local heads: per head softmax(q k^T / sqrt(hd)) v under the causal mask
    ao = np.empty((T, Hl * hd), np.float32)
    for hh in range(Hl):
        sl = slice(hh * hd, (hh + 1) * hd)
        sc = O.matmul(ql[:, sl], O.transpose(kl[:, sl]))[None]
        p = O.causal_softmax(sc, 1.0 / np.sqrt(np.float32(hd)))[0]
        ao[:, sl] = O.matmul(p, vl[:, sl])
    part = O.linear(ao, mine["attn.wo.weight"])
    if lead:
        part = part + x
    t1 = torch.from_numpy(part.copy())
    dist.all_reduce(t1)                                       # the one collective of the attention block
    x1 = t1.numpy()
    # MLP: rows of ffn_up (+ its bias slice), GELU, K-slice of ffn_down; bias and residual on the folding rank only
    f = O.unary("gelu", O.linear(h2, mine["ffn_up.weight"], mine["ffn_up.bias"]))
    part = O.linear(f, mine["ffn_down.weight"], mine["ffn_down.bias"] if lead else None)
    if lead:
        part = part + x1
    t2 = torch.from_numpy(part.copy())
    dist.all_reduce(t2)                                       # the one collective of the MLP block
    if rank == 0:
        attn_full = O.mha_causal(h1, full["attn.wq.weight"], full["attn.wk.weight"], full["attn.wv.weight"], full["attn.wo.weight"], H)
        x1_full = x + attn_full
        x2_full = x1_full + O.linear(O.unary("gelu", O.linear(h2, full["ffn_up.weight"], full["ffn_up.bias"])), full["ffn_down.weight"], full["ffn_down.bias"])
        q.put((float(np.abs(x1 - x1_full).max()), float(np.abs(t2.numpy() - x2_full).max()), kinds, mine["ffn_down.bias"].shape[0]))
    dist.destroy_process_group()


def test_tensor_parallel_partition_two_gloo_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + os.getpid() % 1000
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    err_attn, err_mlp, kinds, bias_len = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert err_attn < 1e-5 and err_mlp < 1e-5
    assert kinds == {"attn.wq.weight": 1, "attn.wk.weight": 1, "attn.wv.weight": 1, "attn.wo.weight": 2, "ffn_up.weight": 1,
                     "ffn_up.bias": 1, "ffn_down.weight": 2, "ffn_down.bias": 0}
    assert bias_len == 32                                     # the row-parallel bias is replicated, added by one rank only


def test_tensor_parallel_shard_rule_edges():
    """Replicated parameters, a rank outside the group, an extent that does not divide."""
    import ctypes as C
    from sptorch_b200 import _lib
    lib = _lib.load()
    kind, begin, count = C.c_int(), C.c_size_t(), C.c_size_t()
    for name in (b"token_emb.weight", b"pos_emb.weight", b"lm_head.weight", b"ln_f.gamma", b"blocks.3.ln1.gamma", b"blocks.3.ffn_down.bias"):
        assert lib.sptorch_ext_tp_param_shard(name, 1, 4, 8, 8, C.byref(kind), C.byref(begin), C.byref(count)) == 0
        assert (kind.value, begin.value, count.value) == (0, 0, 8)
    assert lib.sptorch_ext_tp_param_shard(b"blocks.0.ffn_gate.weight", 3, 4, 16, 8, C.byref(kind), C.byref(begin), C.byref(count)) == 0
    assert (kind.value, begin.value, count.value) == (1, 12, 4)
    assert lib.sptorch_ext_tp_param_shard(b"blocks.0.attn.wo.weight", 4, 4, 8, 8, C.byref(kind), C.byref(begin), C.byref(count)) != 0
    assert lib.sptorch_ext_tp_param_shard(b"blocks.0.attn.wo.weight", 0, 3, 8, 8, C.byref(kind), C.byref(begin), C.byref(count)) != 0
    assert [lib.sptorch_ext_tp_rank_folds_residual(r) for r in range(4)] == [1, 0, 0, 0]
    full = np.arange(12, dtype=np.float32).reshape(3, 4)
    out = np.empty((3, 2), np.float32)
    assert lib.sptorch_ext_tp_slice_host(full.ctypes.data, 3, 4, 2, 2, 2, out.ctypes.data) == 0
    assert np.array_equal(out, full[:, 2:4])
    assert lib.sptorch_ext_tp_slice_host(full.ctypes.data, 3, 4, 2, 3, 2, out.ctypes.data) != 0


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
