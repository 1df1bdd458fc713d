"""In-kernel timelines (%globaltimer stamps written by thread 0 of every CTA) of the decode kernels.

The tensor-core kernels can stamp their phases into a caller-provided device buffer (`q4b_trace_buffer`,
`q4b_decode_persistent_trace`; off by default, a few predicated instructions when off).  This tool runs one isolated
launch of a kernel with stamping on and prints, per phase, the median and the maximum over the CTAs of the time since
the first CTA started.  The numbers explain where a kernel's microseconds go; they are not benchmark values (an isolated
launch has no programmatic overlap with its neighbours and its weights sit in L2 after the warm-up launches).

    python 3080lab_b200/timeline.py gemv              # the four linears of a layer at batch 1 (streaming mma.sync GEMV)
    python 3080lab_b200/timeline.py gemv --tcgen05    # the same four through the tcgen05 exact-digit GEMV
    python 3080lab_b200/timeline.py mmq --batch 32    # the same four as Q8_1 x Q4_0 MMQ for 32 sequences
    python 3080lab_b200/timeline.py attn --batch 32   # batched decode attention, 1024-token context
    python 3080lab_b200/timeline.py persistent        # one token through the persistent all-layers kernel (8 layers)
    python 3080lab_b200/timeline.py chain             # one captured batch-1 decode step of the full 1.5B shape, launch by launch
    python 3080lab_b200/timeline.py prefill           # pipeline roles of one CTA of the prefill GEMM (gate/up shape), per k-block

`chain` uses `q4b_trace_chain`: every GEMV / attention launch of the captured step keeps its own stamp region, so the
replayed graph shows when each launch's CTAs start (how far ahead of their dependency wait they move in), when the wait
returns, and when the launch ends, all on one clock.  Stamp order of `attn_cached_kernel`: start, cache rows requested,
predecessor complete, operands staged, chunk scored, cluster barrier passed, combined (first CTA of a cluster only).

Stamp order of `gemv_mma_kernel`: start, bulk copies issued, predecessor complete, activation operand staged, main loop
done, split-K reduced.  Of `mmq_stream_kernel`: start, TMEM allocated, barriers ready, bulk copies issued, predecessor complete,
activation operand staged, one stamp per batch of k-blocks (expanded and issued), all batches folded, split-K reduced,
end.  Of `attn_decode_mma_kernel`: start, predecessor complete, q / new row prepared, one per 64-position tile, warps
merged, cluster barrier passed, end.  The persistent kernel labels its stamps (see `decode_persistent.cu`).
"""
from __future__ import annotations

import argparse
import importlib
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def _mods():
    names = ("synth", "engine", "_ffi", "qwen_kernels")
    return [importlib.import_module("3080lab_b200." + n) for n in names]


def _report(name: str, buf) -> None:
    t = buf.cpu().numpy().reshape(-1, 16)
    t = t[t[:, 15] > 0]
    t0 = t[:, 0].min()
    for n in sorted({int(x) for x in t[:, 15]}):
        rows = t[t[:, 15] == n]
        rel = (rows[:, :n] - t0) / 1e3
        print(f"{name}: {len(rows)} CTAs with {n} stamps")
        print("   median us:", np.round(np.median(rel, axis=0), 2).tolist())
        print("   max    us:", np.round(rel.max(axis=0), 2).tolist())


def _traced(ffi, torch, fn, name: str) -> None:
    buf = torch.zeros(4096 * 16, dtype=torch.int64, device="cuda")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ffi.call("q4b_trace_buffer", buf.data_ptr(), buf.numel())
    fn()
    torch.cuda.synchronize()
    ffi.call("q4b_trace_buffer", None, 0)
    _report(name, buf)


def _chain(torch, synth, engine, ffi) -> None:
    import ctypes as C
    cfg = synth.QWEN25_1P5B
    m = engine.FusedQwen(synth.synth_model(cfg, 0), max_len=1024)
    m.kc.normal_()
    m.vc.normal_()
    m.pos.fill_(600)
    for _ in range(3):
        m.step()
    torch.cuda.synchronize()
    buf = torch.zeros(8 << 20, dtype=torch.int64, device="cuda")
    m.pos.fill_(600)
    ffi.call("q4b_trace_chain", buf.data_ptr(), buf.numel())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        m.step()
    ffi.call("q4b_trace_chain", None, 0)
    rec = (C.c_int64 * (3 * 4096))()
    n = ffi.lib().q4b_trace_chain_log(rec, 4096)
    recs = np.frombuffer(rec, dtype=np.int64)[:3 * n].reshape(n, 3)
    for _ in range(5):
        m.pos.fill_(600)
        g.replay()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(20):
        g.replay()
    e.record()
    torch.cuda.synchronize()
    print(f"step: {1e3 * s.elapsed_time(e) / 20:.1f} us per token while stamping (context 600..620)")
    m.pos.fill_(600)
    g.replay()
    torch.cuda.synchronize()
    m.check_status()
    raw = buf.cpu().numpy()
    names = {1: "gemv", 2: "attn"}
    t00 = None
    lo = 5 * (cfg.layers // 2)
    print("launches of one layer in the middle of the step; us since the first stamp of the step")
    print("kernel  CTAs   first start   last start   wait returns (median)   last stamp   all stamps (median over CTAs)")
    for i, (kid, ctas, off) in enumerate(recs):
        t = raw[off:off + ctas * 16].reshape(ctas, 16)
        t = t[t[:, 15] > 0]
        if t00 is None:
            t00 = t[:, 0].min()
        if not lo <= i < lo + 6:
            continue
        ns = int(np.median(t[:, 15]))
        rel = (t[:, :ns] - t00) / 1e3
        wi = 2 if kid == 1 else 2                       # both kernels stamp: start, requests issued, wait returned, ...
        last = max(t[j, int(t[j, 15]) - 1] for j in range(len(t)))
        print(f"{names[int(kid)]:6s} {int(ctas):5d} {rel[:, 0].min():12.2f} {rel[:, 0].max():12.2f} {np.median(rel[:, wi]):14.2f}"
              f" {(last - t00) / 1e3:20.2f}   {np.round(np.median(rel, axis=0), 2).tolist()}")


def _prefill_sweep(torch, QB, rng, st, P) -> None:
    """Whole-launch time of the gate/up shape against K (replayed graph): the slope is the cost of a k-block, the
    intercept the fixed cost of a tile (set-up, pipeline fill, epilogue, CTA turnover), both per round of CTAs."""
    n = 17920
    ks, ts = (256, 512, 1024, 1536, 3072), []
    for k in ks:
        W = torch.from_numpy(rng.integers(0, 2 ** 32, size=(n, k // 8), dtype=np.uint32).view(np.int32)).cuda()
        S = torch.from_numpy(rng.uniform(0.002, 0.02, size=(n, k // 32)).astype(np.float16)).cuda()
        Wt, St = QB.pack_q4(W, S)
        xt = QB.q8_tiled_buffer(P, k, "cuda")
        QB.quant_q8_tiled(torch.randn(P, k, device="cuda").half(), xt)
        y = torch.zeros(P, n // 2, dtype=torch.float16, device="cuda")
        fn = lambda: QB.gemm8_prefill(Wt, St, xt, y, None, n, k, P, "swiglu", n // 2, st)
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        for _ in range(3):
            g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(1e3 * e0.elapsed_time(e1) / 10)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    rounds = -(-(n // 128) * (P // 128) // sms)
    slope, icpt = np.polyfit(np.array(ks) / 32, np.array(ts), 1)
    print(f"gate/up launch time against K (us): {dict(zip(ks, [round(t, 1) for t in ts]))}; {rounds} rounds of CTAs: "
          f"{slope / rounds:.3f} us per k-block, {icpt / rounds:.2f} us fixed per tile")


def _prefill(torch, ffi) -> None:
    """SM-clock stamps of CTA (0, 0, 0) of one gate/up-shaped prefill GEMM (`q4b_mmq_prefill_trace`): per k-block, when each
    pipeline role got to it.  Printed as clocks since the first stamp, and the steady-state period of every role."""
    QB = importlib.import_module("3080lab_b200.qwen_batched")
    rng = np.random.default_rng(0)
    n, k, P = 17920, 1536, 2048
    W = torch.from_numpy(rng.integers(0, 2 ** 32, size=(n, k // 8), dtype=np.uint32).view(np.int32)).cuda()
    S = torch.from_numpy(rng.uniform(0.002, 0.02, size=(n, k // 32)).astype(np.float16)).cuda()
    Wt, St = QB.pack_q4(W, S)
    x = torch.randn(P, k, device="cuda").half()
    xt = QB.q8_tiled_buffer(P, k, "cuda")
    QB.quant_q8_tiled(x, xt)
    y = torch.zeros(P, n // 2, dtype=torch.float16, device="cuda")
    st = QB.Status("cuda")
    for _ in range(2):
        QB.gemm8_prefill(Wt, St, xt, y, None, n, k, P, "swiglu", n // 2, st)
    buf = torch.zeros(11 * 64, dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    ffi.call("q4b_mmq_prefill_trace", buf.data_ptr(), buf.numel())
    QB.gemm8_prefill(Wt, St, xt, y, None, n, k, P, "swiglu", n // 2, st)
    torch.cuda.synchronize()
    ffi.call("q4b_mmq_prefill_trace", None, 0)
    st.check()
    full = buf.cpu().numpy().reshape(11, 64).astype(np.int64)
    _prefill_sweep(torch, QB, rng, st, P)
    t = full[:, :k // 32]
    t0 = t[t > 0].min()
    names = ["stage requested", "A operand written", "MMA issued", "accumulator seen", "slot handed back", "folded"]
    print("clocks since the first stamp; k-blocks 0..47 of CTA (0,0,0), gate/up shape 2048 x 17920 x 1536")
    for r, nm in enumerate(names):
        row = t[r] - t0
        per = np.diff(row[16:44])
        print(f"{nm:20s} period median {np.median(per):7.0f} (min {per.min():.0f}, max {per.max():.0f})   first 12: {row[:12].tolist()}")
    w = lambda a, b: (float(np.median((t[b] - t[a])[16:44])), (t[b] - t[a])[:6].tolist())
    print("MMA issuer, clocks spent per k-block (median over k-blocks 16..43; first six k-blocks):")
    print(f"  waiting for the A operand {w(6, 7)}; for the activation stage {w(7, 8)}; for a free accumulator slot {w(8, 9)}; "
          f"issue + commits {w(9, 2)}")
    def phases(name, full, kb):
        ph = full[10, :7]
        mid = f"(of which: wait for the previous grid {ph[5] - ph[2]}, tile through shared memory {ph[6] - ph[5]}) " if ph[6] else f"(of which: wait for the previous grid {ph[5] - ph[2]}) "
        print(f"phases of the CTA [{name}], clocks: entry -> set-up done {ph[1] - ph[0]}; -> first activation stage requested {full[0, 0] - ph[1]}; "
              f"-> first MMA issued {full[2, 0] - full[0, 0]}; -> first k-block folded {full[5, 0] - full[2, 0]}; "
              f"k-block {min(kb, 64) - 1} folded at {full[5, min(kb, 64) - 1] - ph[0]}; main loop left at {ph[2] - ph[0]}; -> epilogue written {ph[3] - ph[2]} {mid}"
              f"-> tensor memory released {ph[4] - ph[3]}; whole CTA {ph[4] - ph[0]}")

    phases("gate/up, swiglu", full, k // 32)
    # the other launches of a prefill layer: phases only
    def traced(fn):
        for _ in range(2):
            fn()
        buf.zero_()
        torch.cuda.synchronize()
        ffi.call("q4b_mmq_prefill_trace", buf.data_ptr(), buf.numel())
        fn()
        torch.cuda.synchronize()
        ffi.call("q4b_mmq_prefill_trace", None, 0)
        return buf.cpu().numpy().reshape(11, 64).astype(np.int64)

    xt2 = QB.q8_tiled_buffer(P, n // 2, "cuda")
    phases("gate/up, swiglu_q8", traced(lambda: QB.gemm8_prefill(Wt, St, xt, xt2, None, n, k, P, "swiglu_q8", n // 2, st)), k // 32)
    Wo, So = QB.pack_q4(W[:1536].contiguous(), S[:1536].contiguous())
    h = torch.zeros(P, 1536, device="cuda")
    phases("o_proj, resid", traced(lambda: QB.gemm8_prefill(Wo, So, xt, h, None, 1536, k, P, "resid", 1536, st)), k // 32)
    Wq, Sq = QB.pack_q4(W[:2048].contiguous(), S[:2048].contiguous())
    qkv = torch.zeros(P, 2048, dtype=torch.float16, device="cuda")
    bias = torch.zeros(2048, device="cuda")
    phases("qkv, biasf", traced(lambda: QB.gemm8_prefill(Wq, Sq, xt, qkv, bias, 2048, k, P, "biasf", 2048, st)), k // 32)
    # fp16 mode of the same kernel (256 rows x 128 tokens per CTA, units of four k-blocks): phases and unit pace
    xt16 = QB.f16_tiled_buffer(P, k, "cuda")
    QB.f16_tile(x, xt16)
    xt16b = QB.f16_tiled_buffer(P, n // 2, "cuda")
    f16 = traced(lambda: QB.gemm16_prefill(Wt, St, xt16, xt16b, None, n, k, P, "swiglu_f16t", n // 2, st))
    nu = k // 32 // 4
    ph = f16[10, :6]
    print(f"fp16 mode [gate/up, swiglu_f16t], clocks from entry: set-up done {ph[1] - ph[0]}; units requested {(f16[0, :nu] - ph[0]).tolist()}; "
          f"expanded (first warp of each group) {(f16[1, :nu] - ph[0]).tolist()}; MMAs issued {(f16[2, :nu] - ph[0]).tolist()}; "
          f"main loop left {ph[2] - ph[0]}; both epilogue passes written {ph[3] - ph[0]}; tensor memory released {ph[4] - ph[0]}")
    st.check()
    print("lags per k-block (median over k-blocks 16..43), clocks:")
    lag = lambda a, b: float(np.median((t[b] - t[a])[16:44]))
    print(f"  A written -> MMA issued {lag(1, 2):.0f}; MMA issued -> accumulator seen {lag(2, 3):.0f}; seen -> slot handed back {lag(3, 4):.0f}; "
          f"handed back -> folded {lag(4, 5):.0f}; stage requested -> MMA issued {lag(0, 2):.0f}")


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["gemv", "mmq", "attn", "persistent", "chain", "prefill"])
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--tcgen05", action="store_true", help="gemv: the tcgen05 exact-digit kernel instead of the mma.sync one")
    args = ap.parse_args()
    import torch
    synth, engine, ffi, K = _mods()
    if args.what == "chain":
        _chain(torch, synth, engine, ffi)
        return
    if args.what == "prefill":
        K.init(0)
        _prefill(torch, ffi)
        return
    layers = 8 if args.what == "persistent" else 2
    cfg = synth.ModelConfig("qwen2.5-1.5b-cut", layers, 1536, 8960, 12, 2, 128, 8192)
    model = synth.synth_model(cfg, 0)
    c, H = cfg, cfg.hidden
    if args.what == "gemv":
        m = engine.FusedQwen(model, max_len=1024, mma=not args.tcgen05)
        m.pos.fill_(600)
        L = m.L[0]
        ops = {
            "qkv  (rmsnorm + 2048x1536 + bias)": lambda: m.norm_gemv(L["ln1"], L["qkv"], m.qkv, L["qkv_b"], c.qkv_rows, H, "biasf"),
            "o    (1536x1536 + residual)": lambda: m.gemv("o", L["o"], m.att, m.h, None, H, c.q_rows, "resid"),
            "gu   (rmsnorm + 17920x1536 + swiglu)": lambda: m.norm_gemv(L["ln2"], L["gu"], m.xm, None, 2 * c.ffn, H, "swiglu"),
            "down (1536x8960 + residual)": lambda: m.gemv("down", L["down"], m.xm, m.h, None, H, c.ffn, "resid"),
        }
        for name, f in ops.items():
            _traced(ffi, torch, f, name)
    elif args.what in ("mmq", "attn"):
        m = engine.FusedQwen(model, max_len=1280)
        bm = engine.Batched(m, args.batch)
        bm.kc.normal_()
        bm.vc.normal_()
        bm.qkv.normal_()
        bm.pos.fill_(1024)
        L = m.L[0]
        if args.what == "mmq":
            ops = {
                "qkv": lambda: bm.gemm8(L["qkv"], c.qkv_rows, H, bm.qkv, L["qkv_b"], "biasf", c.qkv_rows),
                "o": lambda: bm.gemm8(L["o"], H, c.q_rows, bm.h, None, "resid", H),
                "gu": lambda: bm.gemm8(L["gu"], 2 * c.ffn, H, bm.xm, None, "swiglu", c.ffn),
                "down": lambda: bm.gemm8(L["down"], H, c.ffn, bm.h, None, "resid", H),
            }
            for name, f in ops.items():
                _traced(ffi, torch, f, f"{name} ({args.batch} sequences)")
        else:
            _traced(ffi, torch, lambda: K.attn(bm.qkv, m.cos, m.sin, bm.pos, bm.kc[0], bm.vc[0], bm.att, c.n_heads,
                                               c.n_kv_heads, c.head_dim, m.max_len, m.scale, bm.attn_ws),
                    f"attention ({args.batch} sequences, context 1024)")
    else:
        m = engine.FusedQwen(model, max_len=1024, persistent=True)
        m.feed(synth.synth_prompt(cfg, 64, 1))
        torch.cuda.synchronize()
        m.check_status()
        cap = 48 * layers + 8
        nsm = torch.cuda.get_device_properties(0).multi_processor_count
        buf = torch.zeros(nsm * cap, dtype=torch.int64, device="cuda")
        ffi.call("q4b_decode_persistent_trace", buf.data_ptr(), -cap)      # negative: stages subdivided
        m.step()
        torch.cuda.synchronize()
        ffi.call("q4b_decode_persistent_trace", None, 0)
        raw = buf.cpu().numpy().view(np.uint64).reshape(nsm, cap)
        lab = (raw >> np.uint64(56)).astype(int)
        tm = (raw & np.uint64((1 << 56) - 1)).astype(np.float64)
        names = {0: "start", 1: "barrier left", 2: "end", 10: "operand staged", 11: "staging: loads + partial sums",
                 12: "staging: values", 13: "staging: digits", 14: "batches done", 20: "barrier entered",
                 21: "barrier: CTA arrived", 30: "attention: q/k/v rows", 31: "attention: RoPE", 32: "attention: chunks"}
        stages = ["qkv", "attention", "o", "gate_up", "down"]
        layer = layers // 2
        for si, sn in enumerate(stages):
            rows: dict = {}
            for cta in range(nsm):
                n = int((raw[cta] != 0).sum())
                outs = [i for i in range(n) if lab[cta, i] == 1]
                lo, hi = outs[5 * layer + si - 1], outs[5 * layer + si]
                for i in range(lo + 1, hi + 1):
                    rows.setdefault(names.get(lab[cta, i], str(lab[cta, i])), []).append((tm[cta, i] - tm[cta, i - 1]) / 1e3)
            print(f"layer {layer}, {sn}: us since the previous stamp (min / median / max over CTAs, count)")
            for k, v in rows.items():
                print(f"   {k:32s} {np.min(v):6.2f} {np.median(v):6.2f} {np.max(v):6.2f}  {len(v)}")
        ends = [tm[cta, int((raw[cta] != 0).sum()) - 1] for cta in range(nsm)]
        print(f"kernel: {(max(ends) - tm[:, 0].min()) / 1e3:.1f} us for {layers} layers")


if __name__ == "__main__":
    main()
