"""Decode kernels (batch 1 and per-sequence ops), torch-tensor wrappers over the C-ABI.

Mirrors the launch sites of the reference's `lab/qwen_kernels.py` as its engines use them
(`FusedQwen.gemv / rms / step`, scripts/qwen_fused.py:104-145): same epilogue names, same argument meaning, errors
raised as exceptions (the reference's `check()` raises on any CUDA error, scripts/qwen_e2e.py:38-41).  Tensors are
only handles here: every call passes raw device pointers and the current stream to libq4b200."""
from __future__ import annotations

import torch

from . import _ffi

EPILOGUES = ("store", "biasf", "resid", "swiglu", "logits")


def _p(t):
    return 0 if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def init(device: int = 0) -> None:
    _ffi.call("q4b_init", device)


def gemv(W, S, X, Y, aux, N: int, K: int, epi: str = "store") -> None:
    """Y = epilogue(Q4_0(W, S) . X).  W int32 [N, K/8], S fp16 [N, K/32], X fp16 or fp32 [K]
    (reference: gemv_source epilogues, lab/qwen_kernels.py:21-45)."""
    if epi not in _ffi.EPI:
        raise ValueError(f"unknown epilogue {epi!r}; one of {EPILOGUES}")
    if X.dtype == torch.float16:
        xd = _ffi.X_F16
    elif X.dtype == torch.float32:
        xd = _ffi.X_F32
    else:
        raise TypeError("X must be fp16 or fp32")
    _ffi.call("q4b_gemv_q4_0", _p(W), _p(S), _p(X), _p(Y), _p(aux), N, K, _ffi.EPI[epi], xd, _stream())


def rms(h, w, out, eps: float) -> None:
    """out fp16 = RMSNorm(h fp32) * w, for every row of h (RMSNORM_F32W_1P, lab/qwen_kernels.py:683-705)."""
    rows = 1 if h.dim() == 1 else h.shape[0]
    _ffi.call("q4b_rmsnorm", _p(h), _p(w), _p(out), rows, h.shape[-1], float(eps), _stream())


def embed(E, tok, h) -> None:
    """h fp32 [rows, H] = E fp16 [V, H][tok] (EMBED_F32, lab/qwen_kernels.py:284-290)."""
    rows = tok.numel()
    _ffi.call("q4b_embed", _p(E), _p(tok), _p(h), rows, E.shape[1], E.shape[0], _stream())


def attn_workspace(B: int, NH: int, HD: int, max_len: int, device) -> torch.Tensor:
    n = _ffi.lib().q4b_attn_decode_workspace(B, NH, HD, max_len)
    return torch.zeros(n, dtype=torch.uint8, device=device)


def attn(qkv, cosT, sinT, pos, kc, vc, out, NH: int, NKV: int, HD: int, max_len: int, scale: float, ws) -> None:
    """RoPE + K/V append + GQA decode attention for B = pos.numel() sequences (ATTN4, lab/qwen_kernels.py:517-605)."""
    _ffi.call("q4b_attn_decode", _p(qkv), _p(cosT), _p(sinT), _p(pos), _p(kc), _p(vc), _p(out), pos.numel(), NH, NKV, HD,
              max_len, float(scale), _p(ws), ws.numel(), _stream())


def attn_q8(qkv, cosT, sinT, pos, kc, vc, out, xq, xd, NH: int, NKV: int, HD: int, max_len: int, scale: float) -> bool:
    """The same attention with the Q8_1 quantiser of its output fused in (xq int8, xd fp16 as `quant_q8` would write
    them).  Returns False without launching when the shape has no fused kernel; the caller then uses `attn` and the
    quantiser."""
    rc = _ffi.lib().q4b_attn_decode_q8_1(_p(qkv), _p(cosT), _p(sinT), _p(pos), _p(kc), _p(vc), _p(out), _p(xq), _p(xd),
                                         pos.numel(), NH, NKV, HD, max_len, float(scale), _stream())
    if rc == _ffi.E_SHAPE:
        return False
    _ffi.check(rc)
    return True


def head_workspace(V: int, rows: int, device) -> torch.Tensor:
    L = _ffi.lib()
    n = max(L.q4b_head_workspace(V), L.q4b_argmax_workspace(rows, V))
    return torch.zeros(n, dtype=torch.uint8, device=device)


def head_argmax(E, x, logits, tok, pos, ws) -> None:
    """logits = E . x (fp16 table), tok = argmax (lowest index), pos += 1 — the "logits" GEMV + FINISH_MB in one
    launch (lab/qwen_kernels.py:44, 250-282)."""
    _ffi.call("q4b_head_f16_argmax", _p(E), _p(x), _p(logits), E.shape[0], E.shape[1], _p(tok), _p(pos), _p(ws), ws.numel(),
              _stream())


def head_q6_argmax(planes, x, logits, tok, pos, ws) -> None:
    """logits = Q6_K(planes) . x at 6.5625 bits per weight, tok = argmax (lowest index), pos += 1 — gemv_q6_source +
    FINISH_MB in one launch (lab/qwen_kernels.py:608-678, 250-282).  planes = (L, Hb, SC, D) from gguf.q6_k_planes."""
    L, Hb, SC, D = planes
    _ffi.call("q4b_head_q6_k_argmax", _p(L), _p(Hb), _p(SC), _p(D), _p(x), _p(logits), L.shape[0], L.shape[1] * 8, _p(tok),
              _p(pos), _p(ws), ws.numel(), _stream())


def finish(logits, tok, pos, ws) -> None:
    """tok = argmax(logits) per row with the lowest-index tie rule, pos += 1 (FINISH, lab/qwen_kernels.py:222-243)."""
    rows = 1 if logits.dim() == 1 else logits.shape[0]
    _ffi.call("q4b_argmax_advance", _p(logits), rows, logits.shape[-1], _p(tok), _p(pos), _p(ws), ws.numel(), _stream())
