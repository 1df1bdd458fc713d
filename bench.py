"""Benchmark of the Qwen2.5-1.5B-shaped Q4_0 decode step (batch 1, 512-token prompt, greedy decode).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one greedy decode token of one sequence: the whole hot path (embed, 28 layers, LM head, argmax) replayed
as one CUDA graph.  With N > 1 (launched under torchrun) every rank decodes its own sequence on its own GPU with a full
weight copy and no collective on the data path (weak scaling); the value is total tokens per second, timed on the
device, maximum over ranks.  Prints ONE JSON line on rank 0.

The headline is batch 1; the same line carries, under "sub", the other configurations of the metric: at one GPU the
single ffn_up GEMV (34 distinct weight buffers rotated inside one graph), batched decode at 8 and 32 sequences and the
2048-token prefill; at N > 1 GPUs the tensor-parallel 7B configuration on the same ranks (TP = min(N, 4), replicas
beyond).  `--workload X` runs one of them alone and prints its object as the line.  The batched objects also carry, under
"other_routes", the same step with the linears through the tcgen05 MMQ and through the reference's fp16-weight arithmetic.

`--impl reference` times the reference's CPU implementation of the same step (its numpy dequantise-and-dot, restated
in oracle/q4ref.py) on the host cores; each of its steps is a bounded sample of the workload (see `cpu_baseline`).
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import sys as _sys

if "reference" in _sys.argv:
    # The CPU arm uses every host core: torchrun exports OMP_NUM_THREADS=1, which BLAS reads when numpy is imported.
    for _v in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[_v] = str(os.cpu_count() or 1)
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "decode_tok_per_s_batch1"
WORKLOAD = "qwen2.5-1.5b-shape Q4_0 decode, batch 1 per GPU, 512-token prompt then greedy decode"
PROMPT, MAX_LEN = 512, 1024
NOMINAL_HBM_GBS = 8000.0


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return json.loads(p.read_text()), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons every 200 ms while a timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.rows, self.proc, self.th = gpu_index, [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
        except OSError:
            self.proc = None
            return
        self.th = threading.Thread(target=self._read, daemon=True)
        self.th.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def blas_threads() -> int:
    """Threads numpy's BLAS actually uses (the `cores` of the CPU baseline)."""
    try:
        from threadpoolctl import threadpool_info
        n = [p.get("num_threads", 0) for p in threadpool_info() if p.get("user_api") == "blas"]
        if n:
            return int(max(n))
    except Exception:
        pass
    return int(os.environ.get("OMP_NUM_THREADS", os.cpu_count() or 1))


def algorithmic_bytes_per_token(cfg, ctx_mean: float) -> float:
    """Q4_0 layer weights + LM head + KV cache rows read, per decode token (activations < 0.1 %, left out)."""
    return cfg.q4_bytes_per_layer() * cfg.layers + cfg.head_bytes() + cfg.kv_bytes_per_position() * ctx_mean


# ------------------------------------------------------------------------------------------------------ CPU baseline
def cpu_baseline(model, cfg, budget_s: float = 20.0):
    """Reference numpy path on the host cores, bounded: a few layers + the LM head of one decode token at context 512,
    scaled to the full layer count."""
    ora = importlib.import_module("oracle.q4ref")
    synth = importlib.import_module("3080lab_b200.synth")
    cos, sin = synth.rope_tables(cfg, MAX_LEN)
    n_layers = min(cfg.layers, 4)
    dec = ora.CpuDecoder(model, MAX_LEN, cos, sin, layers=range(n_layers))
    rng = np.random.default_rng(0)
    dec.kc[:n_layers, :, :PROMPT] = rng.standard_normal((n_layers, cfg.n_kv_heads, PROMPT, cfg.head_dim)).astype(np.float16)
    dec.vc[:n_layers, :, :PROMPT] = rng.standard_normal((n_layers, cfg.n_kv_heads, PROMPT, cfg.head_dim)).astype(np.float16)
    h = model["embed"][17].astype(np.float32)
    h = dec.layer(0, h, PROMPT)                                     # warm-up (BLAS threads, page faults)
    t_layers, t0 = [], time.perf_counter()
    while True:
        for i in range(n_layers):
            t = time.perf_counter()
            h = dec.layer(i, h, PROMPT)
            t_layers.append(time.perf_counter() - t)
        if time.perf_counter() - t0 > budget_s * 0.6 or len(t_layers) >= 3 * n_layers:
            break
    t = time.perf_counter()
    dec.head(h)
    t_head = time.perf_counter() - t
    t_tok = statistics.mean(t_layers) * cfg.layers + t_head
    return {"value": 1.0 / t_tok, "unit": "tok/s", "cores": blas_threads(), "kind": "port",
            "sample": f"1 decode token at context {PROMPT}: {len(t_layers)} layer passes over {n_layers} of {cfg.layers} "
                      f"layers ({statistics.mean(t_layers):.3f} s each) + the full LM head ({t_head:.2f} s), layers scaled "
                      f"to {cfg.layers}; numpy fp32 dequantise-and-dot per linear, nothing cached",
            "s_per_token": t_tok}


def run_reference(args, rank: int) -> None:
    if rank != 0:
        return
    synth = importlib.import_module("3080lab_b200.synth")
    ora = importlib.import_module("oracle.q4ref")
    cfg = synth.QWEN25_1P5B
    model = synth.synth_model(cfg, 0)
    cos, sin = synth.rope_tables(cfg, MAX_LEN)
    # each step = `per` layers of one decode token; sized so K + W steps fit in ~2.5 minutes
    n_have = 4
    dec = ora.CpuDecoder(model, MAX_LEN, cos, sin, layers=range(n_have))
    rng = np.random.default_rng(0)
    dec.kc[:n_have, :, :PROMPT] = rng.standard_normal((n_have, cfg.n_kv_heads, PROMPT, cfg.head_dim)).astype(np.float16)
    dec.vc[:n_have, :, :PROMPT] = rng.standard_normal((n_have, cfg.n_kv_heads, PROMPT, cfg.head_dim)).astype(np.float16)
    h = model["embed"][17].astype(np.float32)
    t = time.perf_counter()
    h = dec.layer(0, h, PROMPT)
    t_est = time.perf_counter() - t
    t = time.perf_counter()
    dec.head(h)
    t_head = time.perf_counter() - t
    total = max(1, args.steps + args.warmup)
    per = int(max(1, min(n_have, (150.0 / total) / max(t_est, 1e-3))))
    for w in range(args.warmup):
        for i in range(per):
            h = dec.layer(i, h, PROMPT)
    t0 = time.perf_counter()
    for s in range(args.steps):
        for i in range(per):
            h = dec.layer(i, h, PROMPT)
    dt = time.perf_counter() - t0
    t_layer = dt / (args.steps * per)
    t_tok = t_layer * cfg.layers + t_head
    val = 1.0 / t_tok
    sample = (f"each step = {per} of {cfg.layers} layers of one decode token at context {PROMPT} (numpy fp32 dequantise-"
              f"and-dot per linear, {t_layer:.3f} s per layer); LM head timed once ({t_head:.2f} s); "
              f"tok/s = 1 / ({cfg.layers} x layer + head)")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * dt / max(1, args.steps), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "arm": "CPU numpy dequantise-and-dot at a 512-token context"},
        "cpu_baseline": {"value": val, "unit": "tok/s", "cores": blas_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


# ----------------------------------------------------------------------------------------------------------- GPU arm
def graph_of(fn, torch):
    """Capture `fn` (launches on the current stream) in a CUDA graph after an eager and a side-stream warm-up."""
    fn()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    torch.cuda.synchronize()
    return g


def time_kernel(fn, launches: int, reps: int, torch):
    """Average device time per launch, in microseconds: `fn` (which issues `launches` launches on the current stream) is
    captured in a CUDA graph so the host's launch rate does not limit it, replayed `reps` times between CUDA events."""
    g = graph_of(fn, torch)
    for _ in range(3):
        g.replay()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(reps):
        g.replay()
    e.record()
    torch.cuda.synchronize()
    return 1e3 * s.elapsed_time(e) / (reps * launches)


def ncu_traffic_table() -> dict:
    """dram__bytes_read.sum + dram__bytes_write.sum per launch as recorded by the committed ncu summary of the decode
    kernels (a markdown table with the columns: kernel key | traffic bytes).  Empty if the summary is missing."""
    out = {}
    f = ROOT / "profiles" / "decode_kernels_dram_traffic.md"
    if not f.exists():
        return out
    for line in f.read_text().splitlines():
        cells = [c.strip() for c in line.strip().strip("|").split("|")]
        if len(cells) >= 2 and cells[1].replace(" ", "").isdigit():
            out[cells[0].strip("`")] = int(cells[1].replace(" ", ""))
    return out


def measure_i8_peak(torch) -> dict:
    """tcgen05.mma.kind::i8 rate of this device (M 128, N 256, K 32 back to back on every SM), in TOP/s."""
    ffi = importlib.import_module("3080lab_b200._ffi")
    lib = ffi.lib()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    iters = 20000
    lib.q4b_peak_i8_launch(iters, status.data_ptr(), st)            # warm-up
    torch.cuda.synchronize()
    best = 0.0
    for _ in range(3):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        ops = lib.q4b_peak_i8_launch(iters, status.data_ptr(), st)
        e.record()
        torch.cuda.synchronize()
        if ops > 0:
            best = max(best, ops / (s.elapsed_time(e) * 1e-3) / 1e12)
    if int(status.item()) != 0 or best == 0.0:
        return {"tops": None, "how": "int8 peak micro-benchmark failed"}
    return {"tops": best, "how": f"{iters} back-to-back tcgen05.mma.kind::i8 M128 N256 K32 per SM on one accumulator tile, best of 3"}


def bench_gemv_config1(torch, peaks, peak_kind) -> dict:
    """BASELINE configuration 1: the 8960 x 1536 ffn_up GEMV with fp32 x (input recipe of lab/experiments/gemv5.py:40-46),
    rotated over 34 distinct weight buffers (263 MB, more than twice the L2) inside one CUDA graph."""
    QB = importlib.import_module("3080lab_b200.qwen_batched")
    gg = importlib.import_module("3080lab_b200.gguf")
    n, k, nbuf = 8960, 1536, 34
    rng = np.random.default_rng(n + k)
    q = rng.integers(0, 16, size=(n, k), dtype=np.uint32).astype(np.uint8)
    d = rng.uniform(0.002, 0.02, size=(n, k // 32)).astype(np.float16)
    x = torch.from_numpy(rng.standard_normal(k).astype(np.float32)).cuda()
    W0 = torch.from_numpy(gg.pack_nibbles(q)).cuda()
    S0 = torch.from_numpy(d).cuda()
    packs = []
    for i in range(nbuf):                                   # distinct buffers: the first holds the recipe's weights, the
        W = W0 if i == 0 else torch.roll(W0, i, 0)          # others the same rows rotated
        S = S0 if i == 0 else torch.roll(S0, i, 0)
        packs.append(QB.pack_q4(W.contiguous(), S.contiguous()))
    y = torch.empty(n, device="cuda")
    st = QB.Status("cuda")

    def all_bufs():
        for Wt, St in packs:
            QB.gemv_mma(Wt, St, x, y, None, n, k, "logits", st)
    us = time_kernel(all_bufs, nbuf, 20, torch)
    st.check("gemv")
    # end to end: x from pinned host memory in, y back out, one GEMV per step
    hx, hy = x.cpu().pin_memory(), torch.empty(n).pin_memory()
    g1 = graph_of(lambda: QB.gemv_mma(packs[0][0], packs[0][1], x, y, None, n, k, "logits", st), torch)
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 200
    s.record()
    for i in range(reps):
        x.copy_(hx, non_blocking=True)
        g1.replay()
        hy.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e.record()
    torch.cuda.synchronize()
    e2e_us = 1e3 * s.elapsed_time(e) / reps
    b = n * (k // 32) * 18 + k * 4 + n * 4
    ach = b / us / 1e3
    return {"metric": "gemv_ffn_up_hbm_gbs", "value": ach, "unit": "GB/s", "us_per_launch": us, "bytes_per_launch": b,
            "config": {"workload": "single Q4_0 GEMV 8960x1536, fp32 x, 34 distinct weight buffers rotated in one CUDA graph"},
            "roofline": {"bound": "hbm", "kernel": "gemv_mma_kernel (fp32 x)", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": ach / peaks["hbm_gbs"], "frac_of_nominal_8tbs": ach / NOMINAL_HBM_GBS, "peak_kind": f"of {peak_kind}",
                         "traffic": None},
            "e2e": {"value": b / e2e_us / 1e3, "unit": "GB/s", "us_per_call": e2e_us, "h2d_bytes_per_step": k * 4, "d2h_bytes_per_step": n * 4}}


def bench_batched(model, cfg, B: int, steps: int, warmup: int, local_rank: int, torch, peaks, peak_kind, routes: bool = True,
                  mmq: str = "auto") -> dict:
    """Batched decode at B concurrent sequences, each with a 1024-token KV context (Q8_1 activations, int8 MMQ)."""
    synth = importlib.import_module("3080lab_b200.synth")
    engine = importlib.import_module("3080lab_b200.engine")
    ctx, gen = 1024, min(steps, 128)
    m = engine.FusedQwen(model, max_len=ctx + 256, device=f"cuda:{local_rank}")
    bm = engine.Batched(m, B, mmq=mmq, attention="streaming" if mmq == "tc" else "auto")   # --mmq tc: the whole earlier route
    bm.kc.normal_()                                   # a 1024-token KV context per sequence (N(0,1) fp16, as the
    bm.vc.normal_()                                   # reference's decode A/B harness fills it, scripts/decode_ab.py:56-58)
    bm.pos.fill_(ctx)
    bm.tok.copy_(torch.from_numpy(synth.synth_prompt(cfg, B, 5)).cuda())
    g = bm.capture()
    for _ in range(max(warmup, 3)):
        g.replay()
    bm.pos.fill_(ctx)
    sampler = ClockSampler(local_rank)
    sampler.start()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    s.record()
    for _ in range(gen):
        g.replay()
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / gen
    clocks = sampler.stop()
    bm.status.check("batched decode")
    host_in = torch.zeros(B, dtype=torch.long).pin_memory()
    host_out = torch.zeros(B, dtype=torch.long).pin_memory()
    host_in.copy_(bm.tok)
    bm.pos.fill_(ctx)
    s.record()
    for _ in range(gen):
        bm.tok.copy_(host_in, non_blocking=True)
        g.replay()
        host_out.copy_(bm.tok, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        host_in.copy_(host_out)
    e.record()
    torch.cuda.synchronize()
    e2e_ms = s.elapsed_time(e) / gen
    step_bytes = cfg.q4_bytes_per_layer() * cfg.layers + cfg.head_bytes() + B * cfg.kv_bytes_per_position() * (ctx + gen / 2.0)
    ach = step_bytes / (ms * 1e-3) / 1e9
    # the other two routes of the linears, device-timed the same way: the tcgen05 MMQ (TMEM accumulators, one tile per
    # k-block) and the reference's own fp16-weight arithmetic; reported beside the default, not as the value
    others = {}
    for name, kw in ((("q8_tcgen05_mmq", dict(linears="q8", mmq="tc")), ("f16_weights_fp16_mma", dict(linears="f16"))) if routes else ()):
        b2 = engine.Batched(m, B, **kw)
        b2.kc.copy_(bm.kc)
        b2.vc.copy_(bm.vc)
        b2.pos.fill_(ctx)
        b2.tok.copy_(bm.tok)
        g2 = b2.capture()
        for _ in range(3):
            g2.replay()
        b2.pos.fill_(ctx)
        torch.cuda.synchronize()
        s.record()
        for _ in range(gen):
            g2.replay()
        e.record()
        torch.cuda.synchronize()
        b2.status.check("batched decode")
        others[name] = {"tok_per_s": B / (s.elapsed_time(e) / gen) * 1e3, "launches_per_step": b2.launches_per_step}
        del b2, g2
    out = {
        "metric": f"decode_tok_per_s_batch{B}", "value": B / ms * 1e3, "unit": "tok/s", "n_gpus": 1, "steps": gen,
        "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 x int4 -> int32, fp32 scaling", "data": "synthetic",
        "config": {"workload": f"qwen2.5-1.5b-shape batched decode, {B} sequences, 1024-token KV context, Q8_1 x Q4_0 MMQ",
                   "linears": "Q8_1 activations, exact int32 block dots by " + ("tcgen05.mma.kind::i8 with TMEM accumulators" if mmq == "tc"
                                                                                 else "mma.sync.m16n8k32.s8 with register accumulators"),
                   "l2": "1.2 GB of weights + KV streamed per step, larger than L2"},
        "other_routes": others,
        "roofline": {"bound": "hbm", "kernel": "whole step", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": ach / peaks["hbm_gbs"], "peak_kind": f"of {peak_kind}", "traffic": None},
        "e2e": {"value": B / e2e_ms * 1e3, "unit": "tok/s", "h2d_bytes_per_step": 8 * B, "d2h_bytes_per_step": 8 * B},
        "gpu_launches": bm.launches_per_step * gen, "clocks": clocks}
    del bm, m, g
    torch.cuda.empty_cache()
    return out


def bench_prefill(model, cfg, steps: int, warmup: int, local_rank: int, torch, i8_peak: dict, profile: bool = False,
                  profile_linears: str = "q8") -> dict:
    """One 2048-token prompt through the prefill path (tiled Q8_1 quantisers, tcgen05 int8 MMQ, causal flash attention)."""
    synth = importlib.import_module("3080lab_b200.synth")
    engine = importlib.import_module("3080lab_b200.engine")
    P = 2048
    m = engine.FusedQwen(model, max_len=P, device=f"cuda:{local_rank}")
    pf = engine.Prefill(m, P, linears=profile_linears if profile else "q8")   # a profiler run may look at the fp16 route alone
    ids = synth.synth_prompt(cfg, P, 0)
    host_ids = torch.from_numpy(ids).pin_memory()
    pf.tok.copy_(host_ids)
    g = graph_of(lambda: pf.chunk(0), torch)
    for _ in range(max(warmup, 3)):
        g.replay()
    steps = min(steps, 20)
    sampler = ClockSampler(local_rank)
    sampler.start()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    s.record()
    for _ in range(steps):
        g.replay()
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / steps
    clocks = sampler.stop()
    pf.status.check("prefill")
    if profile:                                           # a profiler run: the graph replays above are all it wants
        return {"profile_run": True, "ms_per_step": ms, "steps": steps}
    # end to end: token ids from pinned host memory in, first generated token back out
    host_out = torch.zeros(1, dtype=torch.long).pin_memory()
    s.record()
    for _ in range(steps):
        pf.tok.copy_(host_ids, non_blocking=True)
        g.replay()
        pf.finish(0)
        host_out.copy_(m.tok, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e.record()
    torch.cuda.synchronize()
    e2e_ms = s.elapsed_time(e) / steps
    # the dominant kernel alone: the gate/up MMQ of every layer in one graph
    L0 = m.L
    def gu_all():
        for L in L0:
            pf.gemm8(L["gu"], pf.xt, 2 * cfg.ffn, cfg.hidden, pf.xt2, None, "swiglu_q8", cfg.ffn)   # as the pass runs it
    us_gu = time_kernel(gu_all, cfg.layers, 3, torch)
    pf.status.check("prefill")
    ops_gu = 2.0 * P * 2 * cfg.ffn * cfg.hidden
    ops = 2.0 * P * 46792704 * cfg.layers
    nominal_int8 = 4500.0
    ach_gu = ops_gu / us_gu / 1e6
    # quality of int8 activations: mean next-token NLL of the first 512 prompt tokens under the prefill path and under
    # the fp16-activation decode path (the reference's perplexity check, scripts/qwen_prefill.py:315-333)
    nll = engine.perplexity(m, ids[:512], chunk=512)
    # the other route: fp16 activations, weights dequantised to fp16 inside the GEMM, fp32 tensor-core accumulation over
    # all of K (the arithmetic of the reference's `cublas` prefill mode, scripts/qwen_prefill.py:37-53, 156-160)
    pf16 = engine.Prefill(m, P, linears="f16")
    pf16.tok.copy_(host_ids)
    g16 = graph_of(lambda: pf16.chunk(0), torch)
    for _ in range(3):
        g16.replay()
    torch.cuda.synchronize()
    s.record()
    for _ in range(steps):
        g16.replay()
    e.record()
    torch.cuda.synchronize()
    ms16 = s.elapsed_time(e) / steps
    def gu16_all():
        for L in L0:
            Wt, St = m.packed[id(L["gu"][0])]
            QB_.gemm16_prefill(Wt, St, pf16.xt16, pf16.xt16b, None, 2 * cfg.ffn, cfg.hidden, P, "swiglu_f16t", cfg.ffn, pf16.status)   # as the pass runs it
    QB_ = importlib.import_module("3080lab_b200.qwen_batched")
    us_gu16 = time_kernel(gu16_all, cfg.layers, 3, torch)
    pf16.status.check("prefill, fp16 route")
    peaks, peak_kind = measured_peaks()
    f16_peak = peaks.get("bf16_tflops")
    other = {"f16": {"tok_per_s": P / ms16 * 1e3, "ms_per_step": ms16, "launches_per_step": pf16.launches_per_chunk,
                     "what": "Prefill(linears='f16'): fp16 activations x Q4_0 weights dequantised to fp16 in the GEMM, tcgen05.mma.kind::f16",
                     "gate_up_us": us_gu16, "gate_up_tflops": ops_gu / us_gu16 / 1e6,
                     "gate_up_frac_of_bf16_peak": (ops_gu / us_gu16 / 1e6 / f16_peak) if f16_peak else None,
                     "bf16_peak_tflops": f16_peak, "peak_kind": "of " + peak_kind + " (cuBLAS bf16 GEMM, burst)",
                     "whole_pass_tflops": ops / (ms16 * 1e-3) / 1e12}}
    del g16, pf16
    out = {
        "metric": "prefill_tok_per_s", "value": P / ms * 1e3, "unit": "tok/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 x int4 -> int32, fp32 scaling", "data": "synthetic",
        "config": {"workload": "qwen2.5-1.5b-shape prefill, one 2048-token prompt, Q8_1 x Q4_0 MMQ + causal flash attention",
                   "l2": "3.3 GB of activations and weights touched per pass, larger than L2"},
        "whole_pass": {"int8_tops": ops / (ms * 1e-3) / 1e12, "frac_of_nominal_4500": ops / (ms * 1e-3) / 1e12 / nominal_int8,
                       "frac_of_measured_i8_peak": (ops / (ms * 1e-3) / 1e12 / i8_peak["tops"]) if i8_peak.get("tops") else None},
        "roofline": {"bound": "tensor", "kernel": "mmq_prefill_kernel, gate/up 2048 x 17920 x 1536 with the swiglu_q8 epilogue (timed alone, all layers)",
                     "achieved": ach_gu, "peak": i8_peak.get("tops") or nominal_int8, "unit": "TOP/s (int8)",
                     "frac": ach_gu / (i8_peak.get("tops") or nominal_int8),
                     "peak_kind": "of measured (tcgen05.mma.kind::i8 micro-benchmark in this run)" if i8_peak.get("tops") else "of nominal dense int8",
                     "frac_of_nominal_4500": ach_gu / nominal_int8, "measured_i8_peak": i8_peak, "us_per_launch": us_gu,
                     "traffic": ncu_traffic_table().get("prefill_gate_up")},
        "e2e": {"value": P / e2e_ms * 1e3, "unit": "tok/s", "h2d_bytes_per_step": P * 8, "d2h_bytes_per_step": 8},
        "nll": {"int8_activations": nll["i8"], "fp16_prefill": nll["cublas"], "fp16_activations": nll["f16"], "tokens": nll["tokens"],
                "what": "mean next-token NLL over the first 512 prompt tokens (uniform random tokens): int8 prefill, fp16 prefill (the reference's cublas mode), token-by-token decode"},
        "other_routes": other,
        "gpu_launches": pf.launches_per_chunk * steps, "clocks": clocks}
    del pf, m, g
    torch.cuda.empty_cache()
    return out


def run_ours(args, rank: int, world: int, local_rank: int) -> None:
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
    synth = importlib.import_module("3080lab_b200.synth")
    engine = importlib.import_module("3080lab_b200.engine")
    K = importlib.import_module("3080lab_b200.qwen_kernels")
    QB = importlib.import_module("3080lab_b200.qwen_batched")
    cfg = synth.QWEN25_1P5B
    if args.layers:
        if not args.profile:
            raise SystemExit("--layers is for --profile runs; the benchmark always runs the full model")
        cfg = synth.ModelConfig(f"qwen2.5-1.5b-{args.layers}layers", args.layers, cfg.hidden, cfg.ffn, cfg.n_heads, cfg.n_kv_heads,
                                cfg.head_dim, cfg.vocab)
    model = synth.synth_model(cfg, 0)                       # same weights on every rank, a different prompt per rank
    m = engine.FusedQwen(model, max_len=MAX_LEN, device=f"cuda:{local_rank}", tensor_core=not args.cuda_core, mma=not args.tcgen05)
    prompt = synth.synth_prompt(cfg, args.prompt, seed=rank)
    if args.steps + max(args.warmup, 3) + args.prompt > MAX_LEN:
        raise SystemExit(f"prompt + steps + warmup must stay below {MAX_LEN}")
    m.reset()
    m.feed(prompt)
    g = m.capture()
    pos0, tok0 = m.pos.clone(), m.tok.clone()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing: W warm-up replays, then ROUNDS rounds of exactly K timed replays between CUDA events,
    # the position reset before each round so that every round decodes the same K tokens; the median round is reported
    for _ in range(max(args.warmup, 3)):
        g.replay()
    rounds = 1 if args.profile else 5
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    per_round = []
    for _ in range(rounds):
        m.pos.copy_(pos0 + args.warmup)
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(args.steps):
            g.replay()
        e.record()
        barrier()
        t = torch.tensor([s.elapsed_time(e)], device="cuda")
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        per_round.append(float(t.item()))
    m.check_status()
    clocks = sampler.stop() if rank == 0 else None
    ms_max = statistics.median(per_round)
    if args.profile:
        if rank == 0:
            print(json.dumps({"profile_run": True, "ms_per_step": ms_max / args.steps, "steps": args.steps}), flush=True)
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---- end to end through the public API: token id in from pinned host memory, generated token back, every step
    m.pos.copy_(pos0)
    m.tok.copy_(tok0)
    host_in = torch.zeros(1, dtype=torch.long).pin_memory()
    host_out = torch.zeros(1, dtype=torch.long).pin_memory()
    host_in[0] = int(tok0.item())
    for _ in range(3):
        m.tok.copy_(host_in, non_blocking=True)
        g.replay()
        host_out.copy_(m.tok, non_blocking=True)
        torch.cuda.synchronize()
    m.pos.copy_(pos0)
    host_in[0] = int(tok0.item())
    barrier()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    for _ in range(args.steps):
        m.tok.copy_(host_in, non_blocking=True)          # H2D: this step's input token
        g.replay()
        host_out.copy_(m.tok, non_blocking=True)         # D2H: this step's result
        torch.cuda.current_stream().synchronize()
        host_in[0] = host_out[0]                         # the host feeds the token it just read back
    e2.record()
    barrier()
    t2 = torch.tensor([s2.elapsed_time(e2)], device="cuda")
    if dist is not None:
        dist.all_reduce(t2, op=dist.ReduceOp.MAX)
    e2e_ms = float(t2.item())

    # ---- the tensor-parallel 7B configuration on the same ranks (N > 1 only); every rank takes part, rank 0 keeps the result
    sub = {}
    if world > 1:
        del g
        m_launches = m.launches_per_step
        del m
        torch.cuda.empty_cache()
        tp_res = bench_tp7b(args, rank, world, local_rank, torch, dist)
        if rank != 0:
            dist.destroy_process_group()
            return
        sub["tp7b"] = tp_res
        m = None
    else:
        m_launches = m.launches_per_step

    peaks, peak_kind = measured_peaks()
    c = cfg
    roofline = None
    if m is not None:
        # ---- roofline of the dominant kernels, timed alone on this stream (rank 0)
        rep = 10
        traffic = ncu_traffic_table()
        m.pos.copy_(pos0 + args.warmup)
        def gu_all():
            for L in m.L:
                m.norm_gemv(L["ln2"], L["gu"], m.xm, None, 2 * c.ffn, c.hidden, "swiglu")
        def down_all():
            for L in m.L:
                m.gemv("down", L["down"], m.xm, m.h, None, c.hidden, c.ffn, "resid")
        def head_once():
            K.head_argmax(m.embed, m.x, m.logits, None, None, m.head_ws)
        def attn_all():
            for i in range(c.layers):
                if m.mma:
                    QB.attn_cached(m.qkv, m.pos, m.kc[i], m.vc[i], m.att, c.n_heads, c.n_kv_heads, c.head_dim, m.max_len, m.scale)
                else:
                    K.attn(m.qkv, m.cos, m.sin, m.pos, m.kc[i], m.vc[i], m.att, c.n_heads, c.n_kv_heads, c.head_dim, m.max_len,
                           m.scale, m.attn_ws)
        # each graph walks all 28 layers' matrices (433 MB / 218 MB / 467 MB per replay: larger than the 126 MB L2)
        us_gu = time_kernel(gu_all, c.layers, rep, torch)
        us_down = time_kernel(down_all, c.layers, rep, torch)
        us_head = time_kernel(head_once, 1, rep, torch)
        us_attn = time_kernel(attn_all, c.layers, rep, torch)
        ctx_now = int(m.pos.item()) + 1
        b_gu = 2 * c.ffn * c.hidden // 32 * 18 + c.hidden * 4 + c.ffn * 2
        b_down = c.hidden * c.ffn // 32 * 18 + c.ffn * 2 + c.hidden * 8
        b_head = c.head_bytes() + c.hidden * 2 + c.vocab * 4
        b_attn = 2 * c.kv_rows * 2 * ctx_now + c.q_rows * 4
        gname = ("gemv_mma_kernel (mma.sync exact GEMV)" if m.mma else "mmq_stream (tcgen05 exact GEMV)") if m.tensor_core else "gemv_q4_0 (CUDA cores)"
        aname = "attn_cached_kernel" if m.mma else "attn_decode_cluster_kernel"
        kern = {
            f"{gname} rmsnorm + gate_up 17920x1536 (+swiglu)": (b_gu, us_gu, c.layers, traffic.get("gate_up")),
            f"{gname} down 1536x8960 (+resid)": (b_down, us_down, c.layers, traffic.get("down")),
            "head_f16_argmax 151936x1536": (b_head, us_head, 1, traffic.get("head")),
            f"{aname} (12/2 heads, context {ctx_now})": (b_attn, us_attn, c.layers, traffic.get("attention")),
        }
        # the dominant kernel of the step is the one with the most time per step among the weight-streaming ones
        dominant = max((k for k in kern if "attn" not in k), key=lambda k: kern[k][1] * kern[k][2])
        b, us, _, tr = kern[dominant]
        ach = b / us / 1e3
        roofline = {"bound": "hbm", "kernel": dominant, "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": ach / peaks["hbm_gbs"], "peak_kind": f"of {peak_kind}", "traffic": tr,
                    "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one captured launch, read from the "
                                      "committed ncu summary of the decode kernels" if tr else None,
                    "bytes_per_launch": b, "us_per_launch": us,
                    "others": {k: {"achieved": v[0] / v[1] / 1e3, "frac": v[0] / v[1] / 1e3 / peaks["hbm_gbs"],
                                   "us_per_launch": v[1], "launches_per_step": v[2], "us_per_step": v[1] * v[2]}
                               for k, v in kern.items() if k != dominant}}

    ctx_mean = args.prompt + args.warmup + (args.steps - 1) / 2.0
    step_bytes = algorithmic_bytes_per_token(cfg, ctx_mean)
    ms_step = ms_max / args.steps
    value = world * args.steps / (ms_max / 1e3)
    out = {
        "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "weights": "random-init Q4_0 from seed 0, tied fp16 LM head, fp16 KV cache", "context": f"{args.prompt}..{args.prompt + args.warmup + args.steps}",
                   "l2": "inputs larger than L2: 1.2 GB of weights streamed per step, no flush needed",
                   "parallelism": f"dp{world} (independent sequences, no collective)",
                   "timing": f"median of {rounds} rounds of {args.steps} steps (ms per round, max over ranks: "
                             f"{[round(x, 3) for x in per_round]})"},
        "step_hbm": {"algorithmic_bytes": step_bytes, "achieved_gbs": step_bytes / (ms_step * 1e-3) / 1e9,
                     "frac_of_measured_copy_peak": step_bytes / (ms_step * 1e-3) / 1e9 / peaks["hbm_gbs"],
                     "frac_of_nominal_8tbs": step_bytes / (ms_step * 1e-3) / 1e9 / NOMINAL_HBM_GBS},
        "roofline": roofline,
        "e2e": {"value": world * args.steps / (e2e_ms / 1e3), "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 8},
        "gpu_launches": m_launches * args.steps,
        "clocks": clocks,
    }
    if world == 1 and not args.no_sub:
        # ---- the other single-GPU configurations of the metric, each with its own roofline and end-to-end figure
        del g
        m = None
        torch.cuda.empty_cache()
        sub["gemv_ffn_up"] = bench_gemv_config1(torch, peaks, peak_kind)
        sub["batched8"] = bench_batched(model, cfg, 8, 128, args.warmup, local_rank, torch, peaks, peak_kind)
        sub["batched32"] = bench_batched(model, cfg, 32, 128, args.warmup, local_rank, torch, peaks, peak_kind)
        sub["prefill2048"] = bench_prefill(model, cfg, 10, args.warmup, local_rank, torch, measure_i8_peak(torch))
    if sub:
        out["sub"] = sub
    if world == 1 and not args.no_cpu:
        out["cpu_baseline"] = cpu_baseline(model, cfg)
    print(json.dumps(out), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_other_workload(args, local_rank: int) -> None:
    """One of the further single-GPU configurations alone (`--workload`); prints its object as the JSON line."""
    import torch
    torch.cuda.set_device(local_rank)
    synth = importlib.import_module("3080lab_b200.synth")
    importlib.import_module("3080lab_b200.qwen_kernels").init(local_rank)
    cfg = synth.QWEN25_1P5B
    peaks, peak_kind = measured_peaks()
    if args.workload == "gemv_ffn_up":
        print(json.dumps(bench_gemv_config1(torch, peaks, peak_kind)), flush=True)
        return
    model = synth.synth_model(cfg, 0)
    if args.workload == "prefill2048":
        print(json.dumps(bench_prefill(model, cfg, args.steps, args.warmup, local_rank, torch,
                                       {} if args.profile else measure_i8_peak(torch), args.profile, args.prefill_linears)), flush=True)
        return
    B = 8 if args.workload == "batched8" else 32
    print(json.dumps(bench_batched(model, cfg, B, args.steps, args.warmup, local_rank, torch, peaks, peak_kind,
                                   routes=not args.profile and args.mmq == "auto", mmq=args.mmq)), flush=True)


def bench_tp7b(args, rank: int, world: int, local_rank: int, torch, dist) -> dict:
    """Qwen2.5-7B shape, 64 sequences at a 2048-token context, tensor-parallel with an all-reduce after o_proj and
    down_proj.  The tensor-parallel degree is min(world, KV heads) = at most 4; further GPUs are data-parallel replicas
    of the whole batch (8 GPUs = 2 replicas x TP4, each replica its own group).  The process group must be initialised
    (world > 1).  Returns the result object on rank 0, None elsewhere."""
    synth = importlib.import_module("3080lab_b200.synth")
    tpm = importlib.import_module("3080lab_b200.tp")
    cfg = synth.QWEN25_7B
    tp = min(world, cfg.n_kv_heads)
    if world % tp:
        raise SystemExit(f"tp7b: {world} GPUs is not a multiple of the tensor-parallel degree {tp}")
    dp = world // tp
    group = None
    if world > 1:
        for r in range(dp):                                  # every rank creates every group, in the same order
            gr = dist.new_group(list(range(r * tp, (r + 1) * tp)))
            if rank // tp == r:
                group = gr
        if tp == 1:
            group = None
    B, ctx, gen = 64, 2048, min(args.steps, 64)
    if args.layers:
        cfg = synth.ModelConfig(cfg.name, args.layers, cfg.hidden, cfg.ffn, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.vocab,
                                cfg.eps, cfg.rope_theta, cfg.tied_fp16_head)
    shard = tpm.synth_shard(cfg, rank % tp, tp, seed=0)
    reduce = args.tp_reduce if tp > 1 else "nccl"
    eng, why = None, ""
    if reduce == "peer":
        # the peer-memory reduction needs symmetric memory across the group; if any rank cannot set it up, every rank
        # falls back to NCCL together (the choice is reported in config.collective)
        try:
            eng = tpm.TPBatched(shard, B, ctx + 128, f"cuda:{local_rank}", group, reduce="peer")
        except Exception as ex:                              # noqa: BLE001 - reported, then the NCCL form is used
            why = f"{type(ex).__name__}: {ex}"[:200]
        flag = torch.tensor([1 if eng is not None else 0], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            eng, reduce = None, "nccl"
            torch.cuda.empty_cache()
    if eng is None:
        eng = tpm.TPBatched(shard, B, ctx + 128, f"cuda:{local_rank}", group, reduce=reduce)
    eng.kc.normal_()
    eng.vc.normal_()
    eng.pos.fill_(ctx)
    eng.tok.copy_(torch.from_numpy(synth.synth_prompt(cfg, B, 5 + rank // tp)).cuda())
    sampler = ClockSampler(local_rank)
    # One GPU: the step is replayed as a CUDA graph.  With tensor parallelism the step is launched op by op (capturing a
    # graph that holds NCCL all-reduces is refused by TPBatched.capture, see there).
    run_step = eng.capture().replay if (tp == 1 or reduce == "peer") else eng.step

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        run_step()
    eng.pos.fill_(ctx)
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    if rank == 0:
        sampler.start()
    s.record()
    for _ in range(gen):
        run_step()
    e.record()
    barrier()
    ms = s.elapsed_time(e) / gen
    clocks = sampler.stop() if rank == 0 else None
    eng.status.check("tensor-parallel decode")
    host_in = torch.zeros(B, dtype=torch.long).pin_memory()
    host_out = torch.zeros(B, dtype=torch.long).pin_memory()
    host_in.copy_(eng.tok)
    eng.pos.fill_(ctx)
    barrier()
    s.record()
    for _ in range(gen):
        eng.tok.copy_(host_in, non_blocking=True)
        run_step()
        host_out.copy_(eng.tok, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        host_in.copy_(host_out)
    e.record()
    barrier()
    e2e_ms = s.elapsed_time(e) / gen
    if world > 1:
        tms = torch.tensor([ms, e2e_ms], device="cuda")
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(tms[0]), float(tms[1])
    launches = eng.launches_per_step
    lc = shard["cfg"]
    del eng
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    peaks, peak_kind = measured_peaks()
    # bytes one GPU streams per step: its weight shard, the replicated head, its share of the KV cache
    step_bytes = lc.q4_bytes_per_layer() * lc.layers + cfg.head_bytes() + B * lc.kv_bytes_per_position() * (ctx + gen / 2.0)
    ach = step_bytes / (ms * 1e-3) / 1e9
    return {
        "metric": "decode_tok_per_s_7b_batch64", "value": dp * B / ms * 1e3, "unit": "tok/s", "n_gpus": world, "steps": gen,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong" if dp == 1 else "strong within a replica (tp), weak across replicas (dp)", "vs_baseline": None,
        "dtype": "int8 x int4 -> int32, fp32 scaling", "data": "synthetic",
        "config": {"workload": f"qwen2.5-7b-shape batched decode, 64 sequences per replica, 2048-token KV context, "
                               f"{cfg.layers} layers", "parallelism": f"tp{tp} x dp{dp}",
                   "collective": "none" if tp == 1 else
                                 (f"own one-shot reduction of [64, {cfg.hidden}] fp32 over peer memory (plain NVLink loads), fused "
                                  f"with the residual add and the next RMSNorm + Q8_1" if reduce == "peer" else
                                  f"NCCL all-reduce of [64, {cfg.hidden}] fp32" + (f" (peer-memory reduction unavailable: {why})" if why else "")) +
                                 f" after o_proj and down_proj ({2 * cfg.layers} per step)",
                   "l2": "weights + KV streamed per step are larger than L2"},
        "roofline": {"bound": "hbm", "kernel": "whole step, per GPU", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": ach / peaks["hbm_gbs"], "peak_kind": f"of {peak_kind}", "traffic": None},
        "e2e": {"value": dp * B / e2e_ms * 1e3, "unit": "tok/s", "h2d_bytes_per_step": 8 * B, "d2h_bytes_per_step": 8 * B},
        "gpu_launches": gen * launches, "clocks": clocks}


def run_tp7b(args, rank: int, world: int, local_rank: int) -> None:
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
    res = bench_tp7b(args, rank, world, local_rank, torch, dist)
    if rank == 0:
        print(json.dumps(res), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--no-sub", action="store_true", help="skip the further configurations carried under \"sub\"")
    ap.add_argument("--workload", default="decode_b1",
                    choices=["decode_b1", "gemv_ffn_up", "batched8", "batched32", "prefill2048", "tp7b"],
                    help="decode_b1 is the benchmark (it carries the others under \"sub\"); the others run one configuration "
                         "alone; tp7b is the tensor-parallel 7B configuration (any --gpus, under torch.distributed.run)")
    ap.add_argument("--mmq", default="auto", choices=["auto", "tc"],
                    help="batched8 / batched32 alone: the int8 MMQ of the linears; tc = the tcgen05 kernel with TMEM accumulators "
                         "(and the streaming attention with the quantiser fused in) instead of the default register-accumulator one")
    ap.add_argument("--tp-reduce", default="peer", choices=["peer", "nccl"],
                    help="tp7b: the reduction after o_proj / down_proj: the library's fused peer-memory kernel or NCCL")
    ap.add_argument("--cuda-core", action="store_true", help="linears on the CUDA-core GEMV instead of the tensor-core kernels")
    ap.add_argument("--tcgen05", action="store_true", help="batch-1 linears on the tcgen05 exact-digit GEMV instead of the mma.sync one")
    ap.add_argument("--prompt", type=int, default=PROMPT, help="prompt length (512 = the benchmark configuration)")
    ap.add_argument("--layers", type=int, default=0, help="profile runs only: cut the model to this many layers")
    ap.add_argument("--prefill-linears", choices=["q8", "f16"], default="q8",
                    help="prefill2048 with --profile: which route's graph to replay (the benchmark itself times both)")
    ap.add_argument("--profile", action="store_true",
                    help="short run for a profiler: only the warm-up and timed graph replays, no e2e / roofline / CPU legs")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.workload == "tp7b":
        run_tp7b(args, rank, world, local_rank)
        return
    if args.workload != "decode_b1":
        if world > 1:
            raise SystemExit("--workload other than decode_b1 / tp7b runs on one GPU")
        run_other_workload(args, local_rank)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("bench.py --gpus N > 1 must be launched with torch.distributed.run --nproc-per-node N")
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
