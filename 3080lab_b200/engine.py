"""Host engines: the batch-1 fused decode step and its greedy loop.

`FusedQwen` mirrors the reference class of that name (scripts/qwen_fused.py:55-145; GGUF variant
scripts/qwen_gguf.py:63-144): it owns the weights, the KV cache [L, NKV, max_len, HD], the fp32 residual stream and
the 16-bit activation buffers as torch CUDA tensors, keeps `tok` / `pos` on the device, and `step()` runs one decode
token.  `run_fused` mirrors the reference protocol (scripts/qwen_fused.py:148-180): the prompt goes through `step()`
token by token, one step is captured in a CUDA graph, the graph is replayed once per generated token."""
from __future__ import annotations

import ctypes as C
import math

import numpy as np
import torch

from . import _ffi
from . import qwen_batched as QB
from . import qwen_kernels as K
from .synth import ModelConfig, rope_tables


def _dev(a: np.ndarray, device):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


class FusedQwen:
    def __init__(self, model: dict, max_len: int = 1024, device="cuda:0", tensor_core: bool = True,
                 persistent: bool = False, mma: bool = True):
        """tensor_core: keep tile-packed weights and use the tensor-core kernels.  mma (needs tensor_core): the batch-1
        linears go through the mma.sync streaming GEMV with RoPE / K-V append fused into the QKV projection; False
        routes them through the tcgen05 exact-digit GEMV instead (kept as the second arm of A/B runs)."""
        if not torch.cuda.is_available():
            raise RuntimeError("FusedQwen needs a CUDA device; there is no CPU path")
        self.cfg: ModelConfig = model["cfg"]
        c = self.cfg
        self.device = torch.device(device)
        self.max_len = max_len
        torch.cuda.set_device(self.device)
        K.init(self.device.index or 0)
        self.embed = _dev(model["embed"], self.device)
        self.L = []
        for Lw in model["layers"]:
            d = {k: _dev(Lw[k], self.device) for k in ("ln1", "ln2", "qkv_b")}
            for k in ("qkv", "o", "gu", "down"):
                d[k] = (_dev(Lw[k][0], self.device), _dev(Lw[k][1], self.device))
            self.L.append(d)
        self.norm = _dev(model["norm"], self.device)
        self.head = None if model["head"] is None else tuple(_dev(a, self.device) for a in model["head"])
        # fp16 LM head table: the embedding (tied) unless the model brings its own (a GGUF `output.weight` kept in fp16)
        self.head16 = self.embed if model.get("head16") is None else _dev(model["head16"], self.device)
        # a Q6_K head kept at 6.5625 bits per weight (planes of gguf.q6_k_planes): used by the batch-1 step
        q6 = model.get("head_q6")
        self.head_q6 = None
        if q6 is not None and self.head is None and c.hidden % 512 == 0 and c.hidden <= 2048:
            self.head_q6 = tuple(_dev(a, self.device) for a in q6)
        # tile-packed copies for the tensor-core kernels (K a multiple of 256)
        self.tensor_core = tensor_core
        self.mma = bool(mma and tensor_core)
        self.packed = {}
        if tensor_core:
            for i, d in enumerate(self.L):
                for k in ("qkv", "o", "gu", "down"):
                    if self.mma or d[k][0].shape[1] * 8 % 256 == 0:
                        self.packed[id(d[k][0])] = QB.pack_q4(*d[k])
            if self.head is not None and (self.mma or c.hidden % 256 == 0):
                self.packed[id(self.head[0])] = QB.pack_q4(*self.head)
        cos, sin = rope_tables(c, max_len)
        self.cos, self.sin = _dev(cos, self.device), _dev(sin, self.device)
        f16, f32, dv = torch.float16, torch.float32, self.device
        self.kc = torch.zeros(c.layers, c.n_kv_heads, max_len, c.head_dim, dtype=f16, device=dv)
        self.vc = torch.zeros_like(self.kc)
        self.h = torch.zeros(c.hidden, dtype=f32, device=dv)
        self.x = torch.zeros(c.hidden, dtype=f16, device=dv)
        self.qkv = torch.zeros(c.qkv_rows, dtype=f16, device=dv)
        self.att = torch.zeros(c.q_rows, dtype=f16, device=dv)
        self.xm = torch.zeros(c.ffn, dtype=f16, device=dv)
        self.logits = torch.zeros(c.vocab, dtype=f32, device=dv)
        self.tok = torch.zeros(1, dtype=torch.long, device=dv)
        self.pos = torch.zeros(1, dtype=torch.long, device=dv)
        self.attn_ws = K.attn_workspace(1, c.n_heads, c.head_dim, max_len, dv)
        self.head_ws = K.head_workspace(c.vocab, 1, dv)
        self.scale = 1.0 / math.sqrt(c.head_dim)
        self.status = torch.zeros(1, dtype=torch.int32, device=dv)
        self._desc = self._make_desc()
        fused = tensor_core and (self.mma or c.hidden % 256 == 0)
        self.launches_per_step = 1 + (5 if fused else 7) * c.layers + 2
        self.persistent = False
        if persistent:
            self.enable_persistent()

    def enable_persistent(self) -> None:
        """Route `step()` through the one-kernel-for-all-layers path.  Raises if the model shape is not supported."""
        c = self.cfg
        need = _ffi.lib().q4b_decode_persistent_workspace(C.byref(self._desc))
        if need == 0 or not self.tensor_core:
            raise _ffi.Q4BError(_ffi.E_SHAPE, "persistent decode: model shape not supported (needs tile-packed weights, "
                                "hidden % 256 == 0, head_dim 64 or 128, at most 8 query heads per KV head)")
        self.persistent_ws = torch.zeros(need, dtype=torch.uint8, device=self.device)
        self._desc.persistent_ws = self.persistent_ws.data_ptr()
        self._desc.persistent_ws_bytes = need
        _ffi.call("q4b_decode_persistent_prepare", C.byref(self._desc), self.persistent_ws.data_ptr(), need)
        self._desc.flags |= _ffi.STEP_PERSISTENT
        self.persistent = True
        self.launches_per_step = 1 + 1 + 2

    # ---- descriptor for the one-call step -------------------------------------------------------------------------
    def _make_desc(self):
        c = self.cfg

        def lin(pair, n, k):
            pk = self.packed.get(id(pair[0]))
            return _ffi.Linear(pair[0].data_ptr(), pair[1].data_ptr(), n, k, pk[0].data_ptr() if pk else None,
                               pk[1].data_ptr() if pk else None)

        self._layers = (_ffi.Layer * c.layers)()
        for i, L in enumerate(self.L):
            self._layers[i] = _ffi.Layer(
                L["ln1"].data_ptr(), L["ln2"].data_ptr(), L["qkv_b"].data_ptr(),
                lin(L["qkv"], c.qkv_rows, c.hidden), lin(L["o"], c.hidden, c.q_rows),
                lin(L["gu"], 2 * c.ffn, c.hidden), lin(L["down"], c.hidden, c.ffn),
                self.kc[i].data_ptr(), self.vc[i].data_ptr())
        head = lin(self.head, c.vocab, c.hidden) if self.head is not None else _ffi.Linear(None, None, 0, 0, None, None)
        return _ffi.DecodeDesc(
            c.layers, c.hidden, c.ffn, c.n_heads, c.n_kv_heads, c.head_dim, c.vocab, self.max_len, c.eps, self.scale,
            self.embed.data_ptr(), C.cast(self._layers, C.POINTER(_ffi.Layer)), self.norm.data_ptr(), head,
            self.cos.data_ptr(), self.sin.data_ptr(), self.tok.data_ptr(), self.pos.data_ptr(), self.h.data_ptr(),
            self.x.data_ptr(), self.qkv.data_ptr(), self.att.data_ptr(), self.xm.data_ptr(), self.logits.data_ptr(),
            self.attn_ws.data_ptr(), self.attn_ws.numel(), self.head_ws.data_ptr(), self.head_ws.numel(),
            self.status.data_ptr(),
            (_ffi.STEP_TENSOR_CORE if self.tensor_core else 0) | (_ffi.STEP_MMA_GEMV if self.mma else 0), None, 0,
            None if self.head16 is self.embed else self.head16.data_ptr(),
            *(tuple(a.data_ptr() for a in self.head_q6) if self.head_q6 is not None else (None, None, None, None)))

    # ---- one decode token -------------------------------------------------------------------------------------------
    def step(self) -> None:
        """One decode token through q4b_decode_step (all launches issued from C, on the current stream)."""
        _ffi.call("q4b_decode_step", C.byref(self._desc), torch.cuda.current_stream().cuda_stream)

    def check_status(self) -> None:
        """Raise if a bounded device-side wait of the tensor-core kernels expired since the last check (synchronises)."""
        if int(self.status.item()) != 0:
            self.status.zero_()
            raise _ffi.Q4BError(_ffi.E_TIMEOUT, "decode step: a bounded wait on the tensor-core pipeline expired")

    def gemv(self, name, wsplit, X, Y, aux, N, Kdim, epi):
        pk = self.packed.get(id(wsplit[0]))
        if pk is not None and self.mma:
            _ffi.call("q4b_gemv_q4_0_mma", pk[0].data_ptr(), pk[1].data_ptr(), X.data_ptr(), Y.data_ptr(),
                      0 if aux is None else aux.data_ptr(), N, Kdim, _ffi.EPI[epi], _ffi.X_F16, self.status.data_ptr(),
                      torch.cuda.current_stream().cuda_stream)
        elif pk is not None and Kdim % 256 == 0:
            _ffi.call("q4b_gemv_q4_0_tc", pk[0].data_ptr(), pk[1].data_ptr(), X.data_ptr(), Y.data_ptr(),
                      0 if aux is None else aux.data_ptr(), N, Kdim, _ffi.EPI[epi], _ffi.X_F16, self.status.data_ptr(),
                      torch.cuda.current_stream().cuda_stream)
        else:
            K.gemv(wsplit[0], wsplit[1], X, Y, aux, N, Kdim, epi)

    def rms(self, w, out):
        K.rms(self.h, w, out, self.cfg.eps)

    def norm_gemv(self, nw, wsplit, Y, aux, N, Kdim, epi):
        """RMSNorm(h) * nw followed by a linear; one launch on the tensor-core path."""
        pk = self.packed.get(id(wsplit[0]))
        if pk is not None and self.mma:
            _ffi.call("q4b_rmsnorm_gemv_q4_0_mma", pk[0].data_ptr(), pk[1].data_ptr(), self.h.data_ptr(),
                      nw.data_ptr(), float(self.cfg.eps), Y.data_ptr(), 0 if aux is None else aux.data_ptr(), N, Kdim,
                      _ffi.EPI[epi], self.status.data_ptr(), torch.cuda.current_stream().cuda_stream)
        elif pk is not None and Kdim % 256 == 0:
            _ffi.call("q4b_rmsnorm_gemv_q4_0_tc", pk[0].data_ptr(), pk[1].data_ptr(), self.h.data_ptr(),
                      nw.data_ptr(), float(self.cfg.eps), Y.data_ptr(), 0 if aux is None else aux.data_ptr(), N, Kdim,
                      _ffi.EPI[epi], self.status.data_ptr(), torch.cuda.current_stream().cuda_stream)
        else:
            self.rms(nw, self.x)
            K.gemv(wsplit[0], wsplit[1], self.x, Y, aux, N, Kdim, epi)

    def step_ops(self) -> None:
        """The same token through the per-op entry points, in the reference's launch order
        (scripts/qwen_fused.py:113-145)."""
        c = self.cfg
        H = c.hidden
        K.embed(self.embed, self.tok, self.h)
        fused_kv = self.mma and 128 % c.head_dim == 0 and self.max_len <= 4096
        st = torch.cuda.current_stream().cuda_stream
        for i, L in enumerate(self.L):
            if fused_kv:
                pk = self.packed[id(L["qkv"][0])]
                _ffi.call("q4b_rmsnorm_qkv_rope_kv", pk[0].data_ptr(), pk[1].data_ptr(), self.h.data_ptr(),
                          L["ln1"].data_ptr(), float(c.eps), self.qkv.data_ptr(), L["qkv_b"].data_ptr(), H,
                          self.cos.data_ptr(), self.sin.data_ptr(), self.pos.data_ptr(), self.kc[i].data_ptr(),
                          self.vc[i].data_ptr(), c.n_heads, c.n_kv_heads, c.head_dim, self.max_len,
                          self.status.data_ptr(), st)
                _ffi.call("q4b_attn_decode_cached", self.qkv.data_ptr(), self.pos.data_ptr(), self.kc[i].data_ptr(),
                          self.vc[i].data_ptr(), self.att.data_ptr(), c.n_heads, c.n_kv_heads, c.head_dim, self.max_len,
                          float(self.scale), st)
                self.gemv("o", L["o"], self.att, self.h, None, H, c.q_rows, "resid")
                self.norm_gemv(L["ln2"], L["gu"], self.xm, None, 2 * c.ffn, H, "swiglu")
                self.gemv("down", L["down"], self.xm, self.h, None, H, c.ffn, "resid")
                continue
            self.norm_gemv(L["ln1"], L["qkv"], self.qkv, L["qkv_b"], c.qkv_rows, H, "biasf")
            K.attn(self.qkv, self.cos, self.sin, self.pos, self.kc[i], self.vc[i], self.att, c.n_heads, c.n_kv_heads,
                   c.head_dim, self.max_len, self.scale, self.attn_ws)
            self.gemv("o", L["o"], self.att, self.h, None, H, c.q_rows, "resid")
            self.norm_gemv(L["ln2"], L["gu"], self.xm, None, 2 * c.ffn, H, "swiglu")
            self.gemv("down", L["down"], self.xm, self.h, None, H, c.ffn, "resid")
        if self.head is None and self.head_q6 is not None:
            self.rms(self.norm, self.x)
            K.head_q6_argmax(self.head_q6, self.x, self.logits, self.tok, self.pos, self.head_ws)
        elif self.head is None:
            self.rms(self.norm, self.x)
            K.head_argmax(self.head16, self.x, self.logits, self.tok, self.pos, self.head_ws)
        else:
            self.norm_gemv(self.norm, self.head, self.logits, None, c.vocab, H, "logits")
            K.finish(self.logits, self.tok, self.pos, self.head_ws)

    # ---- graph + greedy loop ------------------------------------------------------------------------------------------
    def reset(self) -> None:
        self.kc.zero_()
        self.vc.zero_()
        self.pos.zero_()
        self.tok.zero_()

    def feed(self, ids) -> None:
        """Prompt through the decode path, token by token; leaves tok = first generated token, pos = len(ids)."""
        for t in ids:
            self.tok.fill_(int(t))
            self.step()

    def capture(self) -> torch.cuda.CUDAGraph:
        """Capture one `step()` in a CUDA graph (warm-up on a side stream first, state restored afterwards)."""
        torch.cuda.synchronize()
        pos0, tok0 = self.pos.clone(), self.tok.clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.step()
        torch.cuda.current_stream().wait_stream(side)
        self.pos.copy_(pos0)
        self.tok.copy_(tok0)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.step()
        self.pos.copy_(pos0)
        self.tok.copy_(tok0)
        torch.cuda.synchronize()
        return g


def run_fused(m: FusedQwen, ids, gen: int):
    """Greedy decode after a prompt, by graph replay.  -> (tokens [gen], ms per token of a second, timed pass)."""
    m.reset()
    m.feed(ids)
    g = m.capture()
    pos0, tok0 = m.pos.clone(), m.tok.clone()
    toks = [int(tok0.item())]
    for _ in range(gen - 1):
        g.replay()
        toks.append(int(m.tok.item()))
    m.check_status()
    m.pos.copy_(pos0)
    m.tok.copy_(tok0)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(gen):
        g.replay()
    e.record()
    torch.cuda.synchronize()
    return toks, s.elapsed_time(e) / gen


MMQ_MMA_MAX_ROWS = 32


class Batched:
    """B concurrent sequences, one decode token each per `step()` — the reference's `Batched(m, B)`
    (scripts/qwen_batched_decode.py:86-187) with the linears routed through Q8_1 activations and the int8
    tensor-core MMQ, as the target configuration asks (the reference's batched path uses fp16 `mma` on dequantised
    weights; its int8 MMQ serves prefill, scripts/qwen_prefill.py:176-246).  Shares the weights of a `FusedQwen`.
    KV cache [L, B, NKV, max_len, HD] (scripts/qwen_batched_decode.py:99).

    `linears="f16"` selects the reference's own batched-decode arithmetic instead: fp16 activations against weights
    dequantised to fp16 on fp16 tensor-core MMAs (gemv_v2_source, lab/qwen_batched.py:467-641), 7 launches per layer
    (rmsnorm, qkv, attention, o, rmsnorm, gate/up, down: scripts/qwen_batched_decode.py:156-187)."""

    def __init__(self, m: FusedQwen, B: int, linears: str = "q8", mmq: str = "auto", attention: str = "auto"):
        if not 1 <= B <= 32:
            raise ValueError("1 <= B <= 32 sequences")
        if linears not in ("q8", "f16"):
            raise ValueError("linears: 'q8' (Q8_1 x Q4_0 MMQ) or 'f16' (fp16 MMA on dequantised weights)")
        if not m.tensor_core or m.cfg.hidden % 256 or m.cfg.q_rows % 256 or m.cfg.ffn % 256:
            raise ValueError("the batched path needs tile-packed weights (K multiples of 256)")
        self.m, self.B, self.linears = m, B, linears
        c, dv = m.cfg, m.device
        f16, f32 = torch.float16, torch.float32
        self.h = torch.zeros(B, c.hidden, dtype=f32, device=dv)
        self.x = torch.zeros(B, c.hidden, dtype=f16, device=dv)
        self.qkv = torch.zeros(B, c.qkv_rows, dtype=f16, device=dv)
        self.att = torch.zeros(B, c.q_rows, dtype=f16, device=dv)
        self.xm = torch.zeros(B, c.ffn, dtype=f16, device=dv)
        kmax = max(c.hidden, c.q_rows, c.ffn)
        self.xq = torch.zeros(B * kmax, dtype=torch.int8, device=dv)
        self.xd = torch.zeros(B * kmax // 32, dtype=f16, device=dv)
        self.xq2 = torch.zeros(B * c.ffn, dtype=torch.int8, device=dv)       # Q8_1 SwiGLU product written by gate/up
        self.xd2 = torch.zeros(B * c.ffn // 32, dtype=f16, device=dv)
        # fused SwiGLU + quantiser epilogue: measured +0.7 % at 8 sequences and -5 % at 32 (16 columns per thread to reduce
        # and quantise), so it is tried only for up to 8 sequences; None = decided by the first step
        self._fuse_gu = None if B <= 8 else False
        self.logits = torch.zeros(B, c.vocab, dtype=f32, device=dv)
        self.tok = torch.zeros(B, dtype=torch.long, device=dv)
        self.pos = torch.zeros(B, dtype=torch.long, device=dv)
        self.kc = torch.zeros(c.layers, B, c.n_kv_heads, m.max_len, c.head_dim, dtype=f16, device=dv)
        self.vc = torch.zeros_like(self.kc)
        self.attn_ws = K.attn_workspace(B, c.n_heads, c.head_dim, m.max_len, dv)
        self.head_ws = K.head_workspace(c.vocab, B, dv)
        self.status = QB.Status(dv)
        # contexts up to 2048: attention through the shared-memory-resident kernel (K / V requested ahead of the dependency
        # wait) + the quantiser, instead of the streaming kernel with the quantiser fused in
        self.attn_cached = c.head_dim == 128 and c.n_heads // c.n_kv_heads <= 8 and m.max_len <= 2048
        # Q8_1 x Q4_0 with register accumulators (mma.sync) instead of tcgen05 tiles: the rescale costs three fp32
        # operations per output and k-block on the CUDA cores either way, but register accumulators have no per-tile
        # retirement latency; measured faster up to MMQ_MMA_MAX_ROWS sequences
        self.mmq_mma = mmq == "mma" or (mmq == "auto" and B <= MMQ_MMA_MAX_ROWS)
        if attention not in ("auto", "streaming"):
            raise ValueError("attention: 'auto' (shared-memory-resident kernel where the context fits) or 'streaming'")
        self.attention = attention
        if attention == "streaming":
            self.attn_cached = False
        if self.mmq_mma:
            # (the quantisers stay separate launches: run inside the o_proj / down_proj launches instead, through
            # QB.quant_gemm8_mma, every CTA requantises its K window after the dependency wait, and the step was slower:
            # 1230 against 1188 us at 8 sequences, 2346 against 2094 us at 32)
            self._fuse_gu = None                          # SwiGLU + quantiser in the gate/up epilogue where it is unsplit
        self._attn_fused = True                           # settled by the first step, like _fuse_gu

    @property
    def launches_per_step(self) -> int:
        """Kernel launches of one step: embed + per layer 7 (both quantisers of the int8 route fused into their producers;
        one more for each that is a launch of its own) + final norm, head, argmax."""
        per_layer = 7
        if self.linears == "q8":
            per_layer += (0 if self._fuse_gu else 1) + (0 if self._attn_fused else 1)
        return 1 + per_layer * self.m.cfg.layers + 3

    def gemm8(self, pair, N, Kdim, Y, aux, epi, ldy, xq=None, xd=None):
        Wt, St = self.m.packed[id(pair[0])]
        fn = QB.gemm8_mma if self.mmq_mma else QB.gemm8
        fn(Wt, St, self.xq if xq is None else xq, self.xd if xd is None else xd, Y, aux, N, Kdim, self.B, epi, ldy, self.status)

    def gemv16(self, pair, N, Kdim, X, Y, aux, epi, ldy):
        Wt, St = self.m.packed[id(pair[0])]
        QB.gemv_f16mma(Wt, St, X, Y, aux, N, Kdim, epi, ldy, self.status)

    def _step_f16(self) -> None:
        m, c = self.m, self.m.cfg
        H = c.hidden
        K.embed(m.embed, self.tok, self.h)
        for i, L in enumerate(m.L):
            K.rms(self.h, L["ln1"], self.x, c.eps)
            self.gemv16(L["qkv"], c.qkv_rows, H, self.x, self.qkv, L["qkv_b"], "biasf", c.qkv_rows)
            K.attn(self.qkv, m.cos, m.sin, self.pos, self.kc[i], self.vc[i], self.att, c.n_heads, c.n_kv_heads, c.head_dim,
                   m.max_len, m.scale, self.attn_ws)
            self.gemv16(L["o"], H, c.q_rows, self.att, self.h, None, "resid", H)
            K.rms(self.h, L["ln2"], self.x, c.eps)
            self.gemv16(L["gu"], 2 * c.ffn, H, self.x, self.xm, None, "swiglu", c.ffn)
            self.gemv16(L["down"], H, c.ffn, self.xm, self.h, None, "resid", H)
        K.rms(self.h, m.norm, self.x, c.eps)
        if m.head is None:
            QB.head_batched(m.head16, self.x, self.logits)
        else:
            self.gemv16(m.head, c.vocab, H, self.x, self.logits, None, "logits", c.vocab)
        K.finish(self.logits, self.tok, self.pos, self.head_ws)

    def step(self) -> None:
        if self.attention == "streaming":                 # process-wide selector: set for the launches of this step only
            _ffi.call("q4b_attn_batched_kernel", 1)
            try:
                self._step()
            finally:
                _ffi.call("q4b_attn_batched_kernel", 0)
        else:
            self._step()

    def _step(self) -> None:
        if self.linears == "f16":
            return self._step_f16()
        m, c, B = self.m, self.m.cfg, self.B
        H = c.hidden
        K.embed(m.embed, self.tok, self.h)
        for i, L in enumerate(m.L):
            QB.rmsnorm_q8(self.h, L["ln1"], self.xq, self.xd, c.eps)
            self.gemm8(L["qkv"], c.qkv_rows, H, self.qkv, L["qkv_b"], "biasf", c.qkv_rows)
            # attention with the Q8_1 quantiser of its output fused in (either kernel has one); False = no fused form here
            # With the shared-memory-resident kernel the fused quantiser pays only for few sequences (8: 1139 -> 1130 us
            # per step; 32, two waves of CTAs: 1849 -> 1920 us), so beyond 8 the quantiser stays a launch of its own there.
            self._attn_fused = (not self.attn_cached or B <= 8) and K.attn_q8(
                self.qkv, m.cos, m.sin, self.pos, self.kc[i], self.vc[i], self.att, self.xq, self.xd, c.n_heads, c.n_kv_heads,
                c.head_dim, m.max_len, m.scale)
            if not self._attn_fused:
                K.attn(self.qkv, m.cos, m.sin, self.pos, self.kc[i], self.vc[i], self.att, c.n_heads, c.n_kv_heads,
                       c.head_dim, m.max_len, m.scale, self.attn_ws)
                QB.quant_q8(self.att, self.xq, self.xd)
            self.gemm8(L["o"], H, c.q_rows, self.h, None, "resid", H)
            QB.rmsnorm_q8(self.h, L["ln2"], self.xq, self.xd, c.eps)
            if self._fuse_gu is not False:
                # SwiGLU product quantised in the gate/up epilogue (second buffer pair: xq / xd are this GEMM's input)
                try:
                    self.gemm8(L["gu"], 2 * c.ffn, H, self.xq2, self.xd2, "swiglu_q8", c.ffn)
                    self._fuse_gu = True
                except _ffi.Q4BError as e:
                    if e.code != _ffi.E_SHAPE or self._fuse_gu:
                        raise
                    self._fuse_gu = False                  # no fused form for this shape: separate quantiser from now on
            if self._fuse_gu:
                self.gemm8(L["down"], H, c.ffn, self.h, None, "resid", H, self.xq2, self.xd2)
            else:
                self.gemm8(L["gu"], 2 * c.ffn, H, self.xm, None, "swiglu", c.ffn)
                QB.quant_q8(self.xm, self.xq, self.xd)
                self.gemm8(L["down"], H, c.ffn, self.h, None, "resid", H)
        if m.head is None:
            K.rms(self.h, m.norm, self.x, c.eps)
            QB.head_batched(m.head16, self.x, self.logits)
        else:
            QB.rmsnorm_q8(self.h, m.norm, self.xq, self.xd, c.eps)
            self.gemm8(m.head, c.vocab, H, self.logits, None, "logits", c.vocab)
        K.finish(self.logits, self.tok, self.pos, self.head_ws)

    def reset(self) -> None:
        self.kc.zero_()
        self.vc.zero_()
        self.pos.zero_()
        self.tok.zero_()

    def feed(self, prompts) -> None:
        """prompts: int array [B, P]; every sequence advances one prompt token per step."""
        prompts = np.asarray(prompts)
        for j in range(prompts.shape[1]):
            self.tok.copy_(torch.from_numpy(np.ascontiguousarray(prompts[:, j])).to(self.tok.device))
            self.step()

    def capture(self) -> torch.cuda.CUDAGraph:
        torch.cuda.synchronize()
        pos0, tok0 = self.pos.clone(), self.tok.clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.step()
        torch.cuda.current_stream().wait_stream(side)
        self.pos.copy_(pos0)
        self.tok.copy_(tok0)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.step()
        self.pos.copy_(pos0)
        self.tok.copy_(tok0)
        torch.cuda.synchronize()
        return g


def run_batched(bm: Batched, prompts, gen: int):
    """Greedy decode of B sequences after their prompts, by graph replay (scripts/qwen_batched_decode.py:203-237).
    -> (tokens [B, gen], ms per step of a second, timed pass)."""
    bm.reset()
    bm.feed(prompts)
    g = bm.capture()
    pos0, tok0 = bm.pos.clone(), bm.tok.clone()
    seqs = [tok0.clone()]
    for _ in range(gen - 1):
        g.replay()
        seqs.append(bm.tok.clone())
    toks = torch.stack(seqs, 1).cpu().numpy()
    bm.status.check("batched decode")
    bm.pos.copy_(pos0)
    bm.tok.copy_(tok0)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(gen):
        g.replay()
    e.record()
    torch.cuda.synchronize()
    return toks, s.elapsed_time(e) / gen


class Prefill:
    """P prompt tokens of one sequence per `chunk()` — the reference's `Prefill(m, P, "i8")`
    (scripts/qwen_prefill.py:82-246): RMSNorm+Q8_1 -> int8 MMQ QKV (+bias) -> K/V append + causal flash attention ->
    Q8_1 -> MMQ o (+residual) -> RMSNorm+Q8_1 -> MMQ gate/up (+SwiGLU) -> Q8_1 -> MMQ down (+residual).  Writes the KV
    cache of the `FusedQwen` it wraps, so decode continues from the prefilled state."""

    def __init__(self, m: FusedQwen, P: int, fused: bool = True, split_k=None, linears: str = "q8"):
        """linears: "q8" = the reference's `i8` prefill mode (Q8_1 activations, int8 MMQ, described above); "f16" = the
        arithmetic of its `cublas` mode (scripts/qwen_prefill.py:37-53, 156-160: weights dequantised to fp16, fp16
        activations, fp32 accumulation), with the dequantisation inside the GEMM kernel - about three times
        faster per pass and without the int8 rounding of the activations, nine launches per layer (RMSNorm into the operand
        order, GEMM, attention, operand tiling, GEMM ...).
        fused: the reference's seven launches per layer (scripts/qwen_prefill.py:196-246): the QKV GEMM rotates and
        appends K/V (`biasf_kv`), the flash kernel emits the o-projection's Q8_1 input (`q8`), the gate/up GEMM emits the
        down GEMM's (`swiglu_q8`).  fused=False keeps those three steps as separate launches (ten per layer); both give
        the same bits.
        split_k: launch o_proj and down_proj as two to four CTAs per output tile, each over a part of K (the further parts
        land in `h2` and are added by the next RMSNorm + Q8_1 launch).  Default: on where their grid would otherwise fill the SMs in a ragged second
        round (12 row tiles x P / 128 token tiles between one and two times the SM count)."""
        c = m.cfg
        if not m.tensor_core or c.hidden % 256 or c.q_rows % 256 or c.ffn % 256 or c.head_dim != 128:
            raise ValueError("the prefill path needs tile-packed weights (K multiples of 256) and head_dim 128")
        if linears not in ("q8", "f16"):
            raise ValueError("linears is 'q8' or 'f16'")
        self.m, self.P, self.fused, self.linears = m, P, fused, linears
        dv, f16, f32 = m.device, torch.float16, torch.float32
        self.h = torch.zeros(P, c.hidden, dtype=f32, device=dv)
        self.qkv = torch.zeros(P, c.qkv_rows, dtype=f16, device=dv)
        self.att = torch.zeros(P, c.q_rows, dtype=f16, device=dv)
        self.xm = torch.zeros(P, c.ffn, dtype=f16, device=dv)
        self.tok = torch.zeros(P, dtype=torch.long, device=dv)
        self.xt = QB.q8_tiled_buffer(P, max(c.hidden, c.q_rows), dv)
        self.xt2 = QB.q8_tiled_buffer(P, c.ffn, dv)          # the down GEMM's input, written while gate/up reads xt
        self.status = QB.Status(dv)
        tiles = ((c.hidden + 127) // 128) * ((P + 127) // 128)
        sms = torch.cuda.get_device_properties(dv).multi_processor_count
        self.split_k = (sms < tiles < 2 * sms) if split_k is None else bool(split_k)

        def parts_for(Kdim: int) -> int:
            """Parts that leave the fewest rounds of CTAs per unit of work (ceil(tiles * n / SMs) / n), with at least 64
            k-blocks per part so that a CTA's fixed costs stay small."""
            best, cost = 1, -(-tiles // sms)
            for n in (2, 3, 4):
                if Kdim // 32 // n < 64 and n > 2:
                    break
                if Kdim < 512:
                    break
                cn = -(-tiles * n // sms) / n
                if cn < cost - 1e-9:
                    best, cost = n, cn
            return best
        self.parts = {Kd: (parts_for(Kd) if self.split_k else 1) for Kd in (c.q_rows, c.ffn)}
        nbuf = max(self.parts.values()) - 1
        self.h2 = torch.zeros(nbuf, P, c.hidden, dtype=f32, device=dv) if nbuf > 0 else None
        self.launches_per_chunk = 1 + (7 if fused else 10) * c.layers + (1 if self.split_k else 0)
        if linears == "f16":
            # 256 weight rows per CTA: half as many tiles; split along K where that leaves SMs idle (down_proj)
            tiles16 = ((c.hidden + 255) // 256) * ((P + 127) // 128)

            def parts16(Kdim: int) -> int:
                best, cost = 1, -(-tiles16 // sms)
                for n in (2, 3, 4):
                    if Kdim // 32 // n < 64:
                        break
                    cn = -(-tiles16 * n // sms) / n
                    if cn < cost - 1e-9:
                        best, cost = n, cn
                return best
            on = (tiles16 < sms) if split_k is None else bool(split_k)
            self.parts = {Kd: (parts16(Kd) if on else 1) for Kd in (c.q_rows, c.ffn)}
            nbuf = max(self.parts.values()) - 1
            self.h2 = torch.zeros(nbuf, P, c.hidden, dtype=f32, device=dv) if nbuf > 0 else None
            self.xt16 = QB.f16_tiled_buffer(P, max(c.hidden, c.q_rows), dv)
            self.xt16b = QB.f16_tiled_buffer(P, c.ffn, dv)
            self.launches_per_chunk = 1 + 9 * c.layers + (1 if nbuf > 0 else 0)

    def gemm8(self, pair, xt, N, Kdim, Y, aux, epi, ldy):
        Wt, St = self.m.packed[id(pair[0])]
        QB.gemm8_prefill(Wt, St, xt, Y, aux, N, Kdim, self.P, epi, ldy, self.status)

    def resid(self, pair, xt, Kdim):
        """h += linear(xt): one launch; with split_k the further K parts go to h2[0 ..] and `self._pending` records how many
        still have to be added (the next `norm_q8` does it)."""
        Wt, St = self.m.packed[id(pair[0])]
        H = self.m.cfg.hidden
        n = self.parts.get(Kdim, 1)
        if n > 1:
            QB.gemm8_prefill_resid_ksplit(Wt, St, xt, self.h, self.h2[:n - 1], H, Kdim, self.P, H, self.status)
            self._pending = n - 1
        else:
            QB.gemm8_prefill(Wt, St, xt, self.h, None, H, Kdim, self.P, "resid", H, self.status)

    def norm_q8(self, w):
        """RMSNorm + tiled Q8_1 of h into xt, completing h with a pending second K half first."""
        if self._pending:
            QB.rmsnorm_q8_tiled_add(self.h, self.h2[:self._pending], w, self.xt, self.m.cfg.eps)
            self._pending = 0
        else:
            QB.rmsnorm_q8_tiled(self.h, w, self.xt, self.m.cfg.eps)

    def gemm16(self, pair, xt, x, N, Kdim, Y, aux, epi, ldy):
        """fp16 route: x [P, Kdim] fp16 (None: already there) -> operand buffer xt -> the GEMM; a `resid` GEMM may be split
        along K like the int8 one (`self._pending` parts left for the next norm to add)."""
        Wt, St = self.m.packed[id(pair[0])]
        if x is not None:
            QB.f16_tile(x, xt)
        n = self.parts.get(Kdim, 1) if epi == "resid" else 1
        if n > 1:
            QB.gemm16_prefill_resid_ksplit(Wt, St, xt, Y, self.h2[:n - 1], N, Kdim, self.P, ldy, self.status)
            self._pending = n - 1
        else:
            QB.gemm16_prefill(Wt, St, xt, Y, aux, N, Kdim, self.P, epi, ldy, self.status)

    def norm16(self, w):
        """RMSNorm of h straight into the operand buffer, completing h with pending K parts first."""
        QB.rmsnorm_f16_tiled(self.h, w, self.xt16, self.m.cfg.eps, self.h2[:self._pending] if self._pending else None)
        self._pending = 0

    def _chunk_f16(self, pos0: int) -> None:
        m, c, H = self.m, self.m.cfg, self.m.cfg.hidden
        K.embed(m.embed, self.tok, self.h)
        self._pending = 0
        for i, L in enumerate(m.L):
            self.norm16(L["ln1"])
            self.gemm16(L["qkv"], self.xt16, None, c.qkv_rows, H, self.qkv, L["qkv_b"], "biasf", c.qkv_rows)
            QB.attn_prefill(self.qkv, m.cos, m.sin, m.kc[i], m.vc[i], self.att, c.n_heads, c.n_kv_heads, c.head_dim,
                            m.max_len, pos0, m.scale)
            self.gemm16(L["o"], self.xt16, self.att, H, c.q_rows, self.h, None, "resid", H)
            self.norm16(L["ln2"])
            self.gemm16(L["gu"], self.xt16, None, 2 * c.ffn, H, self.xt16b, None, "swiglu_f16t", c.ffn)   # products land in down's operand order
            self.gemm16(L["down"], self.xt16b, None, H, c.ffn, self.h, None, "resid", H)
        if self._pending:
            QB.add_rows(self.h, self.h2[:self._pending])
            self._pending = 0

    def chunk(self, pos0: int = 0) -> None:
        """One pass over the P tokens in self.tok at positions pos0 .. pos0 + P - 1."""
        if self.linears == "f16":
            return self._chunk_f16(pos0)
        m, c, H = self.m, self.m.cfg, self.m.cfg.hidden
        K.embed(m.embed, self.tok, self.h)
        self._pending = 0
        for i, L in enumerate(m.L):
            self.norm_q8(L["ln1"])
            if self.fused:
                Wt, St = m.packed[id(L["qkv"][0])]
                QB.gemm8_prefill_qkv_rope_kv(Wt, St, self.xt, self.qkv, L["qkv_b"], H, self.P, m.cos, m.sin, pos0, m.kc[i],
                                             m.vc[i], c.n_heads, c.n_kv_heads, c.head_dim, m.max_len, self.status)
                QB.attn_prefill_cached(self.qkv, m.kc[i], m.vc[i], None, self.xt, c.n_heads, c.n_kv_heads, c.head_dim,
                                       m.max_len, pos0, m.scale)
            else:
                self.gemm8(L["qkv"], self.xt, c.qkv_rows, H, self.qkv, L["qkv_b"], "biasf", c.qkv_rows)
                QB.attn_prefill(self.qkv, m.cos, m.sin, m.kc[i], m.vc[i], self.att, c.n_heads, c.n_kv_heads, c.head_dim,
                                m.max_len, pos0, m.scale)
                QB.quant_q8_tiled(self.att, self.xt)
            self.resid(L["o"], self.xt, c.q_rows)
            self.norm_q8(L["ln2"])
            if self.fused:
                self.gemm8(L["gu"], self.xt, 2 * c.ffn, H, self.xt2, None, "swiglu_q8", c.ffn)
            else:
                self.gemm8(L["gu"], self.xt, 2 * c.ffn, H, self.xm, None, "swiglu", c.ffn)
                QB.quant_q8_tiled(self.xm, self.xt2)
            self.resid(L["down"], self.xt2, c.ffn)
        if self._pending:                                       # the last down_proj's further parts
            QB.add_rows(self.h, self.h2[:self._pending])
            self._pending = 0

    def finish(self, pos0: int = 0) -> None:
        """Greedy token after the last prompt token: final norm + LM head on the last row; leaves the wrapped engine
        with tok = first generated token and pos = pos0 + P (ready for `step()`)."""
        m = self.m
        m.h.copy_(self.h[self.P - 1])
        m.pos.fill_(pos0 + self.P - 1)
        if m.head is None:
            m.rms(m.norm, m.x)
            K.head_argmax(m.head16, m.x, m.logits, m.tok, m.pos, m.head_ws)
        else:
            m.norm_gemv(m.norm, m.head, m.logits, None, m.cfg.vocab, m.cfg.hidden, "logits")
            K.finish(m.logits, m.tok, m.pos, m.head_ws)


def prefill(m: FusedQwen, ids, chunk: int = 0, fused: bool = True, linears: str = "q8"):
    """Prefill `ids` (one sequence) in chunks against m's cache (scripts/qwen_prefill.py:262-301).  -> Prefill object."""
    ids = np.asarray(ids, np.int64)
    n = len(ids)
    chunk = chunk or n
    if n % chunk:
        raise ValueError("the prompt length must be a multiple of the chunk")
    pf = Prefill(m, chunk, fused, linears=linears)
    for s0 in range(0, n, chunk):
        pf.tok.copy_(torch.from_numpy(ids[s0:s0 + chunk]).to(pf.tok.device))
        pf.chunk(s0)
    pf.finish(n - chunk)
    pf.status.check("prefill")
    return pf


def perplexity(m: FusedQwen, ids, chunk: int = 0):
    """Mean next-token negative log-likelihood of the sequence `ids` under the two activation paths, the reference's
    quality check of int8 activations (scripts/qwen_prefill.py:315-333: all positions through the final norm and the
    head, NLL of the actual next tokens):
      "i8"     the prefill path (Q8_1 activations, int8 MMQ), in chunks of `chunk` tokens (0 = one chunk);
      "cublas" the fp16 prefill path (`Prefill(linears="f16")`), the reference's yardstick in this check;
      "f16"    the decode path token by token (fp16 activations, exact block dots).
    -> {"i8": nll, "cublas": nll, "f16": nll, "tokens": n - 1}.  Log-softmax and the gather are host-side torch: this is a check, not a
    hot path.  The reference runs it on real text; without a model file any token sequence serves, and what is reported
    is the DIFFERENCE between the two paths."""
    ids = np.asarray(ids, np.int64)
    n = len(ids)
    if n < 2:
        raise ValueError("need at least two tokens")
    c = m.cfg
    tgt = torch.from_numpy(ids[1:]).to(m.device)
    # ---- fp16 activations: one decode step per token, logits of every position but the last
    m.reset()
    nll16 = torch.zeros((), dtype=torch.float64, device=m.device)
    for i in range(n - 1):
        m.tok.fill_(int(ids[i]))
        m.step()
        lp = torch.log_softmax(m.logits.double(), -1)
        nll16 -= lp[tgt[i]]
    m.check_status()
    # ---- int8 activations: prefill, then the head over every row of the residual stream
    m.reset()
    chunk = chunk or n
    if n % chunk:
        raise ValueError("the sequence length must be a multiple of the chunk")
    x = torch.empty(chunk, c.hidden, dtype=torch.float16, device=m.device)
    lg = torch.empty(32, c.vocab, dtype=torch.float32, device=m.device)
    st = QB.Status(m.device)

    def prefill_nll(linears: str) -> float:
        m.reset()
        pf = Prefill(m, chunk, linears=linears)
        nll = torch.zeros((), dtype=torch.float64, device=m.device)
        for s0 in range(0, n, chunk):
            pf.tok.copy_(torch.from_numpy(ids[s0:s0 + chunk]).to(m.device))
            pf.chunk(s0)
            K.rms(pf.h, m.norm, x, c.eps)
            for r0 in range(0, chunk, 32):
                rows = min(32, chunk - r0)
                if m.head is None:
                    QB.head_batched(m.head16, x[r0:r0 + rows], lg[:rows])
                else:
                    Wt, St = m.packed[id(m.head[0])]
                    xq = torch.empty(rows, c.hidden, dtype=torch.int8, device=m.device)
                    xd = torch.empty(rows, c.hidden // 32, dtype=torch.float16, device=m.device)
                    QB.quant_q8(x[r0:r0 + rows], xq, xd)
                    QB.gemm8(Wt, St, xq, xd, lg, None, c.vocab, c.hidden, rows, "logits", c.vocab, st)
                pos = torch.arange(s0 + r0, s0 + r0 + rows, device=m.device)
                keep = pos < n - 1
                if bool(keep.any()):
                    lp = torch.log_softmax(lg[:rows].double(), -1)
                    picked = lp[torch.arange(rows, device=m.device)[keep], tgt[pos[keep]]]
                    nll -= picked.sum()
        pf.status.check("prefill")
        return float(nll / (n - 1))

    out = {"i8": prefill_nll("q8"), "cublas": prefill_nll("f16")}   # the two prefill modes the reference's check compares
    st.check("head")
    out.update({"f16": float(nll16 / (n - 1)), "tokens": n - 1})
    return out
