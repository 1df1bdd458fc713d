"""Paired benchmark protocol: rotated arms, an A/A control, central estimates with a bootstrap interval, and a
bit-level diff of the state two arms leave behind.

The reference compares decode implementations this way (scripts/decode_paired.py:1-13: every round runs every arm once,
in an order rotated by one position per round, so drift or background load hits each arm at every position; a duplicate
of one arm gives the A/A noise; per pair the statistic is the per-round throughput ratio: median over rounds, min-max,
bootstrap 95 % interval of the mean log ratio; scripts/decode_ab.py diffs K/V/h between configurations).  Here the arms
are configurations of this library in ONE process:

    python 3080lab_b200/paired.py                      # tensor-core GEMV vs CUDA-core GEMV, + A/A duplicate, 1.5B shape
    python 3080lab_b200/paired.py --arms tc,persistent --rounds 6 --steps 64
    python 3080lab_b200/paired.py --arms b_q8,b_f16 --batch 32   # batched decode: Q8_1 x Q4_0 MMQ vs fp16 MMA on dequantised weights

The statistics are plain functions (`rotated_rounds`, `ratio_stats`) and are tested without a GPU.
"""
from __future__ import annotations

import argparse
import importlib
import json
import math
import random
import statistics
import sys
from pathlib import Path
from typing import Callable, Dict, List, Sequence

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def rotated_rounds(arms: Dict[str, Callable[[], float]], rounds: int) -> Dict[str, List[float]]:
    """Run every arm once per round, the order rotated by one position per round.  -> arm -> [value per round]."""
    names = list(arms)
    out: Dict[str, List[float]] = {n: [] for n in names}
    for r in range(rounds):
        k = r % len(names)
        for n in names[k:] + names[:k]:
            out[n].append(float(arms[n]()))
    return out


def ratio_stats(a: Sequence[float], b: Sequence[float], boot: int = 2000, seed: int = 0) -> dict:
    """Per-round ratios a[i] / b[i]: median, min, max and a bootstrap 95 % interval of exp(mean log ratio)."""
    if len(a) != len(b) or not a:
        raise ValueError("paired samples must have equal, non-zero length")
    ratios = [x / y for x, y in zip(a, b)]
    logs = [math.log(r) for r in ratios]
    rng = random.Random(seed)
    means = sorted(sum(rng.choice(logs) for _ in logs) / len(logs) for _ in range(boot))
    lo, hi = means[int(0.025 * boot)], means[min(boot - 1, int(0.975 * boot))]
    return {"median": statistics.median(ratios), "min": min(ratios), "max": max(ratios),
            "geo_mean": math.exp(sum(logs) / len(logs)), "ci95": [math.exp(lo), math.exp(hi)], "rounds": len(ratios)}


def state_diff(a, b) -> dict:
    """Largest absolute difference of the residual stream and the K/V caches two engines hold (0.0 = bit-identical)."""
    import torch
    return {"h": float((a.h - b.h).abs().max()), "k": float((a.kc.float() - b.kc.float()).abs().max()),
            "v": float((a.vc.float() - b.vc.float()).abs().max()), "tok_equal": bool(torch.equal(a.tok, b.tok))}


ARMS = {
    "tc": dict(tensor_core=True),            # tcgen05 exact GEMV (the default path)
    "cuda": dict(tensor_core=False),         # CUDA-core GEMV with the reference's inner-loop arithmetic
    "persistent": dict(tensor_core=True, persistent=True),
    # batched decode of --batch sequences at a 1024-token context (engine.Batched): the two routes of the linears
    "b_q8": dict(batched="q8"),
    "b_f16": dict(batched="f16"),
}


def _batched_main(args, names, torch, synth, engine, model, cfg) -> None:
    """The paired protocol on `engine.Batched` arms: all arms share one set of weights; every arm holds its own
    activations and KV cache (filled with the same N(0, 1) context, as scripts/decode_ab.py:56-58 does)."""
    ctx = 1024
    m = engine.FusedQwen(model, max_len=ctx + args.steps + 64)
    gen = torch.Generator(device="cuda").manual_seed(0)
    kv = None
    engines, graphs = {}, {}
    toks = torch.from_numpy(synth.synth_prompt(cfg, args.batch, 5)).cuda()
    for n in names:
        bm = engine.Batched(m, args.batch, linears=ARMS[n.replace("_dup", "")]["batched"])
        if kv is None:
            kv = (torch.randn(bm.kc.shape, generator=gen, device="cuda", dtype=torch.float16),
                  torch.randn(bm.vc.shape, generator=gen, device="cuda", dtype=torch.float16))
        bm.kc.copy_(kv[0])
        bm.vc.copy_(kv[1])
        bm.pos.fill_(ctx)
        bm.tok.copy_(toks)
        engines[n] = bm
    for bm in engines.values():                                             # one step each from the same state: the diff
        bm.step()
    torch.cuda.synchronize()
    first = engines[names[0]]
    diffs = {}
    for n in names[1:]:
        e = engines[n]
        scale = float(first.logits.abs().max())
        diffs[n] = {"logits_rel": float((e.logits - first.logits).abs().max()) / scale,
                    "tokens_equal": int((e.tok == first.tok).sum()), "of": args.batch}
    for n, bm in engines.items():
        bm.pos.fill_(ctx)
        bm.tok.copy_(toks)
        graphs[n] = bm.capture()

    def arm(n):
        def run() -> float:
            bm, g = engines[n], graphs[n]
            bm.pos.fill_(ctx)
            bm.tok.copy_(toks)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            s.record()
            for _ in range(args.steps):
                g.replay()
            e.record()
            torch.cuda.synchronize()
            bm.status.check("batched decode")
            return args.batch * args.steps / s.elapsed_time(e) * 1e3        # tok/s over all sequences
        return run

    res = rotated_rounds({n: arm(n) for n in names}, args.rounds)
    base = names[0]
    out = {"batch": args.batch, "context": ctx, "rounds": args.rounds, "steps": args.steps,
           "tok_per_s_median": {n: statistics.median(v) for n, v in res.items()},
           "ratio_vs_" + base: {n: ratio_stats(res[n], res[base]) for n in names[1:]},
           "first_step_vs_" + base: diffs}
    print(json.dumps(out, indent=1))


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--arms", default="tc,cuda", help="comma list of: " + ", ".join(ARMS))
    ap.add_argument("--rounds", type=int, default=6)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--prompt", type=int, default=64)
    ap.add_argument("--layers", type=int, default=28)
    ap.add_argument("--batch", type=int, default=8, help="sequences of the batched arms (b_q8, b_f16)")
    args = ap.parse_args()
    import torch
    synth = importlib.import_module("3080lab_b200.synth")
    engine = importlib.import_module("3080lab_b200.engine")
    c0 = synth.QWEN25_1P5B
    cfg = synth.ModelConfig(c0.name, args.layers, c0.hidden, c0.ffn, c0.n_heads, c0.n_kv_heads, c0.head_dim, c0.vocab)
    model = synth.synth_model(cfg, 0)
    ids = synth.synth_prompt(cfg, args.prompt, 1)
    names = args.arms.split(",")
    names = names + [names[0] + "_dup"]                                   # the A/A control
    batched = ["batched" in ARMS[n.replace("_dup", "")] for n in names]
    if any(batched):
        if not all(batched):
            raise SystemExit("batched arms (b_q8, b_f16) cannot be mixed with batch-1 arms")
        args.steps = min(args.steps, 128)
        return _batched_main(args, names, torch, synth, engine, model, cfg)
    engines, graphs = {}, {}
    for n in names:
        m = engine.FusedQwen(model, max_len=args.prompt + args.steps + 64, **ARMS[n.replace("_dup", "")])
        m.reset()
        m.feed(ids)
        engines[n] = m
    # the state diff is taken here, where every arm has consumed exactly the same tokens (free-running greedy decode
    # lets arms that differ in the last bit drift onto different sequences)
    torch.cuda.synchronize()
    diffs = {n: state_diff(engines[n], engines[names[0]]) for n in names[1:]}
    for n in names:
        graphs[n] = engines[n].capture()
    start = {n: (engines[n].pos.clone(), engines[n].tok.clone()) for n in names}

    def arm(n):
        def run() -> float:
            m, g = engines[n], graphs[n]
            m.pos.copy_(start[n][0])
            m.tok.copy_(start[n][1])
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            s.record()
            for _ in range(args.steps):
                g.replay()
            e.record()
            torch.cuda.synchronize()
            return args.steps / s.elapsed_time(e) * 1e3                    # tok/s
        return run

    res = rotated_rounds({n: arm(n) for n in names}, args.rounds)
    base = names[0]
    out = {"rounds": args.rounds, "steps": args.steps, "tok_per_s_median": {n: statistics.median(v) for n, v in res.items()},
           "ratio_vs_" + base: {n: ratio_stats(res[n], res[base]) for n in names[1:]},
           "state_diff_after_prompt_vs_" + base: diffs}
    print(json.dumps(out, indent=1))


if __name__ == "__main__":
    main()
