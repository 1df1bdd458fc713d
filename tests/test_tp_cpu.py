"""Tensor-parallel sharding on CPU: two gloo ranks each hold their shard of a small model, compute their part of every
linear with the oracle, exchange through the collective the GPU path uses (all_reduce sum for the row-parallel
matrices, all_gather for the column-parallel ones), and must reproduce the unsharded products."""
import importlib
import os
import sys

import numpy as np
import pytest

from conftest import ROOT, oracle, pkg

torch = pytest.importorskip("torch")


def _worker(rank, world, port, seed, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    synth = importlib.import_module("3080lab_b200.synth")
    tp = importlib.import_module("3080lab_b200.tp")
    o = importlib.import_module("oracle.q4ref")
    cfg = synth.TINY
    model = synth.synth_model(cfg, seed)
    shard = tp.shard_model(model, rank, world)
    lc = shard["cfg"]
    rng = np.random.default_rng(seed)
    B = 3
    x = rng.standard_normal((B, cfg.hidden)).astype(np.float16)
    att = rng.standard_normal((B, cfg.q_rows)).astype(np.float16)
    act = rng.standard_normal((B, cfg.ffn)).astype(np.float16)
    L, Ls = model["layers"][0], shard["layers"][0]
    # column-parallel: local rows of qkv and gate/up, gathered
    qkv_loc = torch.from_numpy(x.astype(np.float64) @ o.dequant(*Ls["qkv"]).T + Ls["qkv_b"])
    parts = [torch.zeros_like(qkv_loc) for _ in range(world)]
    dist.all_gather(parts, qkv_loc)
    gu_loc = torch.from_numpy(x.astype(np.float64) @ o.dequant(*Ls["gu"]).T)
    gparts = [torch.zeros_like(gu_loc) for _ in range(world)]
    dist.all_gather(gparts, gu_loc)
    # row-parallel: K slices (zero-padded to a multiple of 256), partial sums all-reduced
    q0 = rank * lc.q_rows
    ko = Ls["o"][0].shape[1] * 8
    att_loc = np.zeros((B, ko), np.float16)
    att_loc[:, :lc.q_rows] = att[:, q0:q0 + lc.q_rows]
    xq, xd, _ = o.quant_q8_1(att_loc)
    o_part = torch.from_numpy(o.mmq(*Ls["o"], xq, xd))
    dist.all_reduce(o_part)
    f0 = rank * lc.ffn
    kd = Ls["down"][0].shape[1] * 8
    act_loc = np.zeros((B, kd), np.float16)
    act_loc[:, :lc.ffn] = act[:, f0:f0 + lc.ffn]
    xq, xd, _ = o.quant_q8_1(act_loc)
    d_part = torch.from_numpy(o.mmq(*Ls["down"], xq, xd))
    dist.all_reduce(d_part)
    if rank == 0:
        full_qkv = x.astype(np.float64) @ o.dequant(*L["qkv"]).T + L["qkv_b"]
        hd, nh, nkv = cfg.head_dim, cfg.n_heads // world, cfg.n_kv_heads // world
        got = np.concatenate([p.numpy()[:, :nh * hd] for p in parts] + [p.numpy()[:, nh * hd:(nh + nkv) * hd] for p in parts]
                             + [p.numpy()[:, (nh + nkv) * hd:] for p in parts], axis=1)
        assert np.allclose(got, full_qkv, rtol=0, atol=1e-12)
        full_gu = x.astype(np.float64) @ o.dequant(*L["gu"]).T
        assert np.allclose(np.concatenate([p.numpy() for p in gparts], axis=1), full_gu, rtol=0, atol=1e-12)
        xq, xd, _ = o.quant_q8_1(att)
        assert np.allclose(o_part.numpy(), o.mmq(*L["o"], xq, xd), rtol=1e-12, atol=1e-9)      # block-aligned K slices
        xq, xd, _ = o.quant_q8_1(act)
        assert np.allclose(d_part.numpy(), o.mmq(*L["down"], xq, xd), rtol=1e-12, atol=1e-9)
        assert ko % 256 == 0 and kd % 256 == 0
        open(os.path.join(out_dir, "ok"), "w").write("ok")
    dist.barrier()
    dist.destroy_process_group()


def test_tp2_sharding_reproduces_unsharded_linears(tmp_path):
    import torch.multiprocessing as mp
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, 7, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok").exists()


def test_shard_config_rejects_uneven_splits():
    s, tp = pkg("synth"), pkg("tp")
    with pytest.raises(ValueError):
        tp.shard_config(s.QWEN25_7B, 8)          # 28 query heads / 4 KV heads do not divide by 8
    c = tp.shard_config(s.QWEN25_7B, 4)
    assert (c.n_heads, c.n_kv_heads, c.ffn) == (7, 1, 4736)


def test_synth_shard_replicated_parts_and_shapes():
    """Shards drawn directly in the local shapes: replicated tensors identical on every rank, K slices padded to 256."""
    synth, tp = pkg("synth"), pkg("tp")
    cfg = synth.ModelConfig("tp-shape", 2, 512, 1536, 8, 4, 64, 2048, tied_fp16_head=False)
    shards = [tp.synth_shard(cfg, r, 4, seed=3) for r in range(4)]
    lc = shards[0]["cfg"]
    assert (lc.n_heads, lc.n_kv_heads, lc.ffn) == (2, 1, 384)
    for s in shards[1:]:
        assert np.array_equal(s["embed"], shards[0]["embed"]) and np.array_equal(s["norm"], shards[0]["norm"])
        assert np.array_equal(s["head"][0], shards[0]["head"][0])
        for a, b in zip(s["layers"], shards[0]["layers"]):
            assert np.array_equal(a["ln1"], b["ln1"]) and np.array_equal(a["ln2"], b["ln2"])
            assert not np.array_equal(a["qkv"][0], b["qkv"][0])
    L = shards[2]["layers"][1]
    assert L["qkv"][0].shape == (lc.qkv_rows, cfg.hidden // 8) and L["gu"][0].shape == (2 * lc.ffn, cfg.hidden // 8)
    assert L["o"][0].shape == (cfg.hidden, 256 // 8)             # 128 local q columns padded to one 256-wide group
    assert L["down"][0].shape == (cfg.hidden, 512 // 8)          # 384 -> 512
    assert np.all(L["o"][1][:, 128 // 32:] == 0)                 # padding blocks carry a zero scale
