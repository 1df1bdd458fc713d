"""Tensor-parallel batched decode on two GPUs (NCCL all-reduce after o_proj and down_proj) against the single-GPU
batched engine.  Needs two devices: skipped on a one-GPU box."""
import importlib
import os
import sys

import numpy as np
import pytest

from conftest import ROOT, pkg

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    synth = importlib.import_module("3080lab_b200.synth")
    tp = importlib.import_module("3080lab_b200.tp")
    E = importlib.import_module("3080lab_b200.engine")
    cfg = synth.ModelConfig("tp-small", 3, 512, 1536, 4, 2, 128, 4096)
    model = synth.synth_model(cfg, 11)
    B, steps = 8, 12
    eng = tp.TPBatched(tp.shard_model(model, rank, world), B, 64, f"cuda:{rank}", group=dist.group.WORLD)
    ref = E.Batched(E.FusedQwen(model, max_len=64, device=f"cuda:{rank}"), B) if rank == 0 else None
    toks = torch.from_numpy(np.stack([synth.synth_prompt(cfg, 1, 100 + b) for b in range(B)])[:, 0]).cuda(rank)
    errs = []
    for _ in range(steps):
        dist.broadcast(toks, 0)                                   # every rank feeds the same (reference) tokens
        eng.tok.copy_(toks)
        eng.step()
        if rank == 0:
            ref.tok.copy_(toks)
            ref.step()
            a, b = eng.logits.float().cpu().numpy(), ref.logits.float().cpu().numpy()
            errs.append(np.max(np.abs(a - b), axis=1) / np.max(np.abs(b), axis=1))
            for s in range(B):
                if int(eng.tok[s]) != int(ref.tok[s]):
                    gap = b[s].max() - b[s][int(eng.tok[s])]
                    assert gap <= 2 * np.max(np.abs(a[s] - b[s])) + 1e-6
            toks = ref.tok.clone()
    eng.status.check("tensor-parallel decode")
    # all ranks hold the same greedy tokens
    mine = eng.tok.clone()
    dist.broadcast(mine, 0)
    assert torch.equal(mine, eng.tok)
    if rank == 0:
        errs = np.concatenate(errs)
        assert np.median(errs) < 1e-5, np.median(errs)
        assert errs.max() < 5e-2, errs.max()
        open(os.path.join(out_dir, "ok"), "w").write(f"{np.median(errs):.2e} {errs.max():.2e}")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tp2_matches_single_gpu(tmp_path):
    import torch.multiprocessing as mp
    port = 29600 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok").exists()
    print("tp2 vs single GPU logits error (median, max):", (tmp_path / "ok").read_text())
