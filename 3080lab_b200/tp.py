"""Tensor-parallel batched decode: one process per GPU, NCCL all-reduce over NVLink after o_proj and down_proj.

The reference is single-GPU (no NCCL anywhere); the target configuration adds this for the 7B shape.  Split:
  * QKV by heads (query heads and KV heads divided evenly; a rank keeps the K/V cache of its own KV heads),
  * gate/up by interleaved (gate, up) row pairs,
  * o_proj and down_proj along K (row-parallel): every rank produces a partial [B, hidden] that is summed across ranks
    (`all_reduce`, sum) before it is added to the residual stream.
K slices of the row-parallel matrices stay multiples of the 32-weight block, so no Q4_0 block or Q8_1 block straddles
a rank and the per-block int8 quantisation of a slice equals that of the full vector.  Where a slice is not a multiple
of the tensor-core kernels' 256-wide K group (7B: 3584/4 = 896, 18944/4 = 4736) it is padded with zero-weight blocks.
RMSNorm, residual stream, embedding and LM head are replicated (every rank computes the same greedy token).
"""
from __future__ import annotations

import numpy as np
import torch

from . import qwen_batched as QB
from . import qwen_kernels as K
from .engine import FusedQwen
from .synth import ModelConfig, synth_q4


def _pad_k(W: np.ndarray, S: np.ndarray, mult: int = 256):
    """Pad the K axis of a canonical Q4_0 matrix with zero-weight blocks (nibble 8, scale 0) up to a multiple of `mult`."""
    n, kw = W.shape
    k = kw * 8
    kp = -(-k // mult) * mult
    if kp == k:
        return W, S
    Wp = np.full((n, kp // 8), np.uint32(0x88888888).view(np.int32), np.int32)
    Sp = np.zeros((n, kp // 32), np.float16)
    Wp[:, :kw] = W
    Sp[:, :k // 32] = S
    return Wp, Sp


def shard_config(cfg: ModelConfig, tp: int) -> ModelConfig:
    if cfg.n_heads % tp or cfg.n_kv_heads % tp or cfg.ffn % tp or (cfg.ffn // tp) % 32:
        raise ValueError(f"tp={tp} does not divide {cfg.n_heads} query heads / {cfg.n_kv_heads} KV heads / ffn {cfg.ffn}")
    return ModelConfig(f"{cfg.name}-tp{tp}", cfg.layers, cfg.hidden, cfg.ffn // tp, cfg.n_heads // tp, cfg.n_kv_heads // tp,
                       cfg.head_dim, cfg.vocab, cfg.eps, cfg.rope_theta, cfg.tied_fp16_head)


def shard_model(model: dict, rank: int, tp: int) -> dict:
    """The weights rank `rank` of `tp` holds, as a model dict with the local head / ffn counts.  `o` and `down` are the
    K slices (padded to a multiple of 256); everything else is a row slice."""
    cfg: ModelConfig = model["cfg"]
    lc = shard_config(cfg, tp)
    hd = cfg.head_dim
    q0, q1 = rank * lc.n_heads * hd, (rank + 1) * lc.n_heads * hd
    k0, k1 = cfg.q_rows + rank * lc.n_kv_heads * hd, cfg.q_rows + (rank + 1) * lc.n_kv_heads * hd
    v0, v1 = k0 + cfg.kv_rows, k1 + cfg.kv_rows
    rows = np.r_[q0:q1, k0:k1, v0:v1]
    f0, f1 = rank * lc.ffn, (rank + 1) * lc.ffn
    layers = []
    for L in model["layers"]:
        Wq, Sq = L["qkv"]
        Wo, So = L["o"]
        Wg, Sg = L["gu"]
        Wd, Sd = L["down"]
        layers.append({
            "ln1": L["ln1"], "ln2": L["ln2"],
            "qkv": (np.ascontiguousarray(Wq[rows]), np.ascontiguousarray(Sq[rows])),
            "qkv_b": np.ascontiguousarray(L["qkv_b"][rows]),
            "o": _pad_k(np.ascontiguousarray(Wo[:, q0 // 8:q1 // 8]), np.ascontiguousarray(So[:, q0 // 32:q1 // 32])),
            "gu": (np.ascontiguousarray(Wg[2 * f0:2 * f1]), np.ascontiguousarray(Sg[2 * f0:2 * f1])),
            "down": _pad_k(np.ascontiguousarray(Wd[:, f0 // 8:f1 // 8]), np.ascontiguousarray(Sd[:, f0 // 32:f1 // 32])),
        })
    return {"cfg": lc, "full_cfg": cfg, "embed": model["embed"], "layers": layers, "norm": model["norm"], "head": model["head"],
            "rank": rank, "tp": tp}


def synth_shard(cfg: ModelConfig, rank: int, tp: int, seed: int = 0) -> dict:
    """Random-init weights of ONE rank, drawn directly in the local shapes (1/tp of the work of drawing the whole model
    and slicing it).  The global model these shards belong to is their concatenation: row slices for QKV and gate/up,
    K slices for o_proj and down_proj; embedding, norms, biases of the local rows and the LM head come from
    rank-independent streams, so every rank holds identical replicated parts."""
    from .synth import synth_model
    lc = shard_config(cfg, tp)
    rep = synth_model(ModelConfig(cfg.name, 0, cfg.hidden, cfg.ffn, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.vocab,
                                  cfg.eps, cfg.rope_theta, cfg.tied_fp16_head), seed)          # embed, norm, head only
    layers = []
    for i in range(cfg.layers):
        shared = np.random.default_rng([seed, i, 1 << 16])
        rng = np.random.default_rng([seed, i, rank])
        ln1 = (1.0 + 0.1 * shared.standard_normal(cfg.hidden)).astype(np.float32)
        ln2 = (1.0 + 0.1 * shared.standard_normal(cfg.hidden)).astype(np.float32)
        layers.append({
            "ln1": ln1, "ln2": ln2,
            "qkv": synth_q4(rng, lc.qkv_rows, cfg.hidden),
            "qkv_b": (0.1 * rng.standard_normal(lc.qkv_rows)).astype(np.float32),
            "o": _pad_k(*synth_q4(rng, cfg.hidden, lc.q_rows)),
            "gu": synth_q4(rng, 2 * lc.ffn, cfg.hidden),
            "down": _pad_k(*synth_q4(rng, cfg.hidden, lc.ffn)),
        })
    return {"cfg": lc, "full_cfg": cfg, "embed": rep["embed"], "layers": layers, "norm": rep["norm"], "head": rep["head"],
            "rank": rank, "tp": tp}


class PeerReduce:
    """The partial-sum buffers and arrival flags of the fused reduction kernel (`q4b_tp_allreduce_resid_rmsnorm_q8`):
    two partial buffers [rows, H] fp32 per rank, alternated from call to call, and one flag array per rank, all in
    symmetric memory so that every rank can address every peer's copy over NVLink.  torch's symmetric-memory allocator
    does the handle exchange; the data path is the library's own kernel (plain peer loads, no multicast).
    With group=None the "group" is this process alone (world 1): plain device memory, same kernel."""

    def __init__(self, rows: int, H: int, device, group=None):
        import ctypes as C
        self.rows, self.H, self.group = rows, H, group
        self.call = 0                                             # index of the next reduction inside the current step
        self.base = torch.zeros(1, dtype=torch.int32, device=device)   # reductions made by the steps before (device word)
        if group is None:
            self.rank, self.world = 0, 1
            self.parts = torch.zeros(2, rows, H, dtype=torch.float32, device=device)
            self.flags = torch.zeros(rows, dtype=torch.int32, device=device)
            part_ptrs, flag_ptrs = [self.parts.data_ptr()], [self.flags.data_ptr()]
        else:
            import os
            import torch.distributed as dist
            # plain peer mappings only: the kernel uses no multimem instruction, so no NVLink multicast object is bound
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm
            self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
            self.parts = symm.empty((2, rows, H), dtype=torch.float32, device=device)
            self.flags = symm.empty((self.world * rows,), dtype=torch.int32, device=device)
            self.parts.zero_()
            self.flags.zero_()
            hp = symm.rendezvous(self.parts, group)
            hf = symm.rendezvous(self.flags, group)
            part_ptrs, flag_ptrs = [int(p) for p in hp.buffer_ptrs], [int(p) for p in hf.buffer_ptrs]
            self._handles = (hp, hf)
            torch.cuda.synchronize(device)
            dist.barrier(group)                                   # every rank's flags are zero before anyone signals
        nbytes = rows * H * 4
        self._tables = []
        for k in range(2):                                        # pointer tables of the two alternating buffer sets
            pt = (C.c_void_p * self.world)(*[p + k * nbytes for p in part_ptrs])
            self._tables.append(pt)
        self._flag_table = (C.c_void_p * self.world)(*flag_ptrs)

    def part(self) -> torch.Tensor:
        """The buffer this rank's next partial goes into."""
        return self.parts[self.call & 1]

    def reduce_add(self, h, norm_w, eps: float, xq, xd, status) -> None:
        """h += sum of all ranks' current partials; optionally the RMSNorm + Q8_1 of the result into (xq, xd).  The epoch
        is (calls of the steps before, kept in a device word) + (index of this call in the step + 1)."""
        from . import _ffi
        from .qwen_kernels import _p, _stream
        k = self.call
        self.call += 1
        _ffi.call("q4b_tp_allreduce_resid_rmsnorm_q8", self._tables[k & 1], self._flag_table, self.rank, self.world, k + 1,
                  _p(self.base), _p(h), self.rows, self.H, _p(norm_w), float(eps), _p(xq), _p(xd), _p(status.word), _stream())

    def end_step(self) -> None:
        """Close a step: the device epoch word moves on by the number of reductions the step made (it must be even, so
        that the buffer alternation repeats), and the call index starts over.  Part of the step when it is captured."""
        from . import _ffi
        from .qwen_kernels import _p, _stream
        if self.call & 1:
            raise RuntimeError("PeerReduce: a step must make an even number of reductions")
        _ffi.call("q4b_tp_epoch_advance", _p(self.base), self.call, _stream())
        self.call = 0


class TPBatched:
    """B sequences, one decode token each per `step()`, on one rank of a tensor-parallel group.  Same op order as
    `engine.Batched`; the o_proj / down_proj partials are all-reduced (sum) before the residual add.  `group` is a
    torch.distributed process group (NCCL on GPUs); with group=None (tp = 1) it degenerates to the single-GPU path."""

    def __init__(self, shard: dict, B: int, max_len: int, device, group=None, reduce: str = "nccl"):
        """reduce: "nccl" = dist.all_reduce on the partial, then a residual add and the RMSNorm + Q8_1 launch;
        "peer" = the library's one-shot reduction over peer memory with the residual add and the next RMSNorm + Q8_1
        fused in (`PeerReduce`), one launch instead of three."""
        import torch.distributed as dist
        if reduce not in ("nccl", "peer"):
            raise ValueError("reduce: 'nccl' or 'peer'")
        self.dist, self.group, self.reduce = dist, group, reduce
        self.B = B
        self.full: ModelConfig = shard.get("full_cfg", shard["cfg"])
        self.m = FusedQwen(shard, max_len=max_len, device=device)        # local weights, RoPE tables, packing
        m, c = self.m, self.m.cfg
        self.ko = m.L[0]["o"][0].shape[1] * 8                             # padded K of the row-parallel slices
        self.kd = m.L[0]["down"][0].shape[1] * 8
        dv, f16, f32 = m.device, torch.float16, torch.float32
        self.h = torch.zeros(B, c.hidden, dtype=f32, device=dv)
        self.x = torch.zeros(B, c.hidden, dtype=f16, device=dv)
        self.qkv = torch.zeros(B, c.qkv_rows, dtype=f16, device=dv)
        self.att = torch.zeros(B, self.ko, dtype=f16, device=dv)         # zero beyond the local q rows (K padding)
        self.xm = torch.zeros(B, self.kd, dtype=f16, device=dv)
        self.peer = PeerReduce(B, c.hidden, dv, group) if reduce == "peer" else None
        self._part = None if self.peer else torch.zeros(B, c.hidden, dtype=f32, device=dv)
        kmax = max(c.hidden, self.ko, self.kd)
        self.xq = torch.zeros(B * kmax, dtype=torch.int8, device=dv)
        self.xd = torch.zeros(B * kmax // 32, dtype=f16, device=dv)
        self.logits = torch.zeros(B, c.vocab, dtype=f32, device=dv)
        self.tok = torch.zeros(B, dtype=torch.long, device=dv)
        self.pos = torch.zeros(B, dtype=torch.long, device=dv)
        self.kc = torch.zeros(c.layers, B, c.n_kv_heads, max_len, c.head_dim, dtype=f16, device=dv)
        self.vc = torch.zeros_like(self.kc)
        self.attn_ws = K.attn_workspace(B, c.n_heads, c.head_dim, max_len, dv)
        self.head_ws = K.head_workspace(c.vocab, B, dv)
        self.status = QB.Status(dv)
        self.att_view = self.att[:, :c.q_rows] if self.ko == c.q_rows else None
        # with K padding the attention output lands in a staging buffer first (allocated here, not inside step())
        self._att_tmp = None if self.att_view is not None else torch.zeros(B, c.q_rows, dtype=f16, device=dv)
        self.allreduces_per_step = 2 * c.layers
        groups = (B + 31) // 32                                          # column groups per linear (<= 32 rows per launch)
        self.launches_per_step = 1 + c.layers * (4 + 4 * groups + 2 + (0 if self.att_view is not None else 1)) + 2 + groups
        # (the peer path trades the two RMSNorm + Q8_1 launches of a layer for its two reduction launches: same count)

    def _gemm8(self, pair, N, Kdim, Y, aux, epi, ldy):
        """One linear over all B sequences; the MMQ (register accumulators, as engine.Batched uses it) takes up to 32
        activation rows per launch."""
        Wt, St = self.m.packed[id(pair[0])]
        Yf = Y.view(-1)
        for c0 in range(0, self.B, 32):
            n = min(32, self.B - c0)
            QB.gemm8_mma(Wt, St, self.xq[c0 * Kdim:], self.xd[c0 * (Kdim // 32):], Yf[c0 * ldy:], aux, N, Kdim, n, epi, ldy,
                         self.status)

    @property
    def part(self) -> torch.Tensor:
        """Where this rank's next partial [B, hidden] goes."""
        return self.peer.part() if self.peer else self._part

    def _next_norm(self, i: int, which: str):
        """The RMSNorm weights applied to h right after this reduction (None: the fp16-head path normalises separately)."""
        m = self.m
        if which == "o":
            return m.L[i]["ln2"]
        if i + 1 < len(m.L):
            return m.L[i + 1]["ln1"]
        return m.norm if m.head is not None else None

    def _reduce_add(self, i: int, which: str):
        """h += sum over ranks of the partial [B, hidden] (+ the next RMSNorm + Q8_1 on the peer path)."""
        if self.peer:
            nw = self._next_norm(i, which)
            self.peer.reduce_add(self.h, nw, self.m.cfg.eps, self.xq if nw is not None else None,
                                 self.xd if nw is not None else None, self.status)
            return
        if self.group is not None:
            self.dist.all_reduce(self._part, op=self.dist.ReduceOp.SUM, group=self.group)
        self.h.add_(self._part)

    def step(self) -> None:
        for i, which in self.phases():
            self._reduce_add(i, which)
        if self.peer:
            self.peer.end_step()

    def phases(self):
        """The step as a generator that stops wherever a partial [B, hidden] is ready in `self.part` (after o_proj and
        after down_proj of every layer): the caller reduces it over the ranks, adds it to `self.h` and resumes.  `step()`
        does that with the process group; `step_together` does it for several ranks living in one process."""
        m, c, H = self.m, self.m.cfg, self.m.cfg.hidden
        fused = self.peer is not None                                    # the reduction kernel leaves (xq, xd) behind
        K.embed(m.embed, self.tok, self.h)
        for i, L in enumerate(m.L):
            if not fused or i == 0:
                QB.rmsnorm_q8(self.h, L["ln1"], self.xq, self.xd, c.eps)
            self._gemm8(L["qkv"], c.qkv_rows, H, self.qkv, L["qkv_b"], "biasf", c.qkv_rows)
            if self.att_view is None:
                # the attention kernel writes rows of c.q_rows values; with K padding they land in a staging buffer first
                K.attn(self.qkv, m.cos, m.sin, self.pos, self.kc[i], self.vc[i], self._att_tmp, c.n_heads, c.n_kv_heads,
                       c.head_dim, m.max_len, m.scale, self.attn_ws)
                self.att[:, :c.q_rows].copy_(self._att_tmp)
            else:
                K.attn(self.qkv, m.cos, m.sin, self.pos, self.kc[i], self.vc[i], self.att, c.n_heads, c.n_kv_heads,
                       c.head_dim, m.max_len, m.scale, self.attn_ws)
            QB.quant_q8(self.att, self.xq, self.xd)
            self._gemm8(L["o"], H, self.ko, self.part, None, "logits", H)
            yield i, "o"
            if not fused:
                QB.rmsnorm_q8(self.h, L["ln2"], self.xq, self.xd, c.eps)
            if self.kd == c.ffn:
                self._gemm8(L["gu"], 2 * c.ffn, H, self.xm, None, "swiglu", c.ffn)
            else:
                self._gemm8(L["gu"], 2 * c.ffn, H, self.xm, None, "swiglu", self.kd)   # pitch = padded K, tail stays zero
            QB.quant_q8(self.xm, self.xq, self.xd)
            self._gemm8(L["down"], H, self.kd, self.part, None, "logits", H)
            yield i, "down"
        if m.head is None:
            K.rms(self.h, m.norm, self.x, c.eps)
            for c0 in range(0, self.B, 32):                               # the fp16 head kernel takes up to 32 rows
                QB.head_batched(m.head16, self.x[c0:c0 + 32], self.logits[c0:c0 + 32])
        else:
            if not fused:
                QB.rmsnorm_q8(self.h, m.norm, self.xq, self.xd, c.eps)
            self._gemm8(m.head, c.vocab, H, self.logits, None, "logits", c.vocab)
        K.finish(self.logits, self.tok, self.pos, self.head_ws)

    def capture(self) -> torch.cuda.CUDAGraph:
        """One `step()` as a CUDA graph (tok and pos are restored afterwards).  Only without a process group (tensor-parallel
        degree 1): a graph that held the NCCL all-reduces of a 2-rank step never completed its first replay on B200
        (driver 580, NCCL 2.28; no GPU fault, the run was ended by its time limit), and the cause has not been established.
        Candidates that reading the capture path leaves open: programmatic-dependent-launch edges on the kernels directly
        in front of and behind a captured NCCL kernel node; NCCL's internal stream joined into the capture through event
        waits after a warm-up that ran on a side stream; two communicators (the world group for barriers, the tensor-
        parallel group inside the graph) in flight on one GPU.  Until one of them is confirmed this method refuses to
        record that form.  With reduce="peer" the step holds only this library's kernels (the reduction included, its
        epochs taken from a device word) and is captured on any number of ranks; every rank must capture and replay in
        step with the others."""
        if self.group is not None and not self.peer:
            raise RuntimeError("TPBatched.capture: a CUDA graph holding the NCCL all-reduces did not complete on this "
                               "platform; run step() op by op, or build the engine with reduce='peer'")
        torch.cuda.synchronize()
        pos0, tok0 = self.pos.clone(), self.tok.clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.pos.copy_(pos0)
        self.tok.copy_(tok0)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.step()
        self.pos.copy_(pos0)
        self.tok.copy_(tok0)
        torch.cuda.synchronize()
        return g


def step_together(ranks) -> None:
    """One decode step of all tensor-parallel ranks held in ONE process (every `TPBatched` built with group=None, each on
    its own shard): the ranks advance in lock step and their partials are summed in rank order where a process group
    would all-reduce them.  This is the multi-rank data path without NCCL; it exists for tests on a single GPU."""
    gens = [r.phases() for r in ranks]
    while True:
        alive = [next(g, None) is not None for g in gens]
        if not any(alive):
            return
        if not all(alive):
            raise RuntimeError("tensor-parallel ranks fell out of step")
        total = ranks[0].part.clone()
        for r in ranks[1:]:
            total.add_(r.part.to(total.device))
        for r in ranks:
            r.h.add_(total.to(r.h.device))
