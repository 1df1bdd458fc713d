"""Batched-decode and prefill kernels (Q8_1 activations, int8 tensor-core MMQ), torch-tensor wrappers over the C-ABI.

Mirrors the launch sites of the reference's `lab/qwen_batched.py` as its engines use them (`Batched.step`,
scripts/qwen_batched_decode.py:156-187; `Prefill.chunk`, scripts/qwen_prefill.py:196-246)."""
from __future__ import annotations

import torch

from . import _ffi
from .qwen_kernels import _p, _stream


def blockdot(W, xq, M: int, K: int, mode: int = 0) -> torch.Tensor:
    """Exact int32 dots of every 32-weight Q4_0 block of W with every row of xq (int8 [P, K]) on the int8 tensor cores.
    -> int32 [P, M, K/32].  Raises if a bounded device-side wait expired."""
    P = xq.shape[0]
    out = torch.empty(P, M, K // 32, dtype=torch.int32, device=xq.device)
    status = torch.zeros(1, dtype=torch.int32, device=xq.device)
    _ffi.call("q4b_blockdot_q4_0_q8_1", _p(W), _p(xq), _p(out), M, K, P, mode, _p(status), _stream())
    if int(status.item()) != 0:
        raise _ffi.Q4BError(_ffi.E_TIMEOUT, "blockdot: a bounded wait on the tensor-core pipeline expired")
    return out


def pack_q4(W, S):
    """Canonical Q4_0 (W int32 [N, K/8], S fp16 [N, K/32]) -> tile-packed (Wt int32 [T, K/32, 128, 4], St fp16
    [T, K/32, 128]) for the tensor-core kernels; same bytes, last row tile zero-padded (the reference repacks for its
    tensor-core kernels likewise: pack_q4_mma / pack_q4_i8, lab/qwen_batched.py:394-436, 987-1013)."""
    N, KW = W.shape
    K = KW * 8
    T = (N + 127) // 128
    Wt = torch.empty(T, K // 32, 128, 4, dtype=torch.int32, device=W.device)
    St = torch.empty(T, K // 32, 128, dtype=torch.float16, device=W.device)
    _ffi.call("q4b_pack_q4_0", _p(W), _p(S), _p(Wt), _p(St), N, K, _stream())
    return Wt, St


class Status:
    """The uint32 status word the tensor-core kernels set when a bounded device-side wait expires."""

    def __init__(self, device):
        self.word = torch.zeros(1, dtype=torch.int32, device=device)

    def check(self, what: str = "tensor-core kernel") -> None:
        if int(self.word.item()) != 0:
            self.word.zero_()
            raise _ffi.Q4BError(_ffi.E_TIMEOUT, f"{what}: a bounded wait on the tensor-core pipeline expired")


def gemv_tc(W, S, X, Y, aux, N: int, K: int, epi: str, status: Status) -> None:
    """Exact Q4_0 GEMV of one activation vector on the int8 tensor cores; same contract as qwen_kernels.gemv, with
    (W, S) tile-packed by `pack_q4`."""
    xd = _ffi.X_F16 if X.dtype == torch.float16 else _ffi.X_F32
    if X.dtype not in (torch.float16, torch.float32):
        raise TypeError("X must be fp16 or fp32")
    _ffi.call("q4b_gemv_q4_0_tc", _p(W), _p(S), _p(X), _p(Y), _p(aux), N, K, _ffi.EPI[epi], xd, _p(status.word), _stream())


def gemv_mma(W, S, X, Y, aux, N: int, K: int, epi: str, status: Status) -> None:
    """Exact Q4_0 GEMV of one activation vector by the streaming mma.sync kernel (bulk-copied weight slab, register
    accumulators); same contract as `gemv_tc`, K a multiple of 32."""
    if X.dtype not in (torch.float16, torch.float32):
        raise TypeError("X must be fp16 or fp32")
    xd = _ffi.X_F16 if X.dtype == torch.float16 else _ffi.X_F32
    _ffi.call("q4b_gemv_q4_0_mma", _p(W), _p(S), _p(X), _p(Y), _p(aux), N, K, _ffi.EPI[epi], xd, _p(status.word), _stream())


def gemv_f16mma(W, S, X, Y, aux, N: int, K: int, epi: str, ldy: int, status: Status) -> None:
    """Y[b] = epilogue(X[b] . W^T) for up to 32 fp16 activation rows with fp16-dequantised weights on fp16 tensor-core
    MMAs: the arithmetic of the reference's batched-decode GEMV (gemv_v2_source, lab/qwen_batched.py:467-641).  (W, S)
    tile-packed by `pack_q4`."""
    if X.dtype != torch.float16 or X.dim() != 2:
        raise TypeError("X must be fp16 [B, K]")
    _ffi.call("q4b_gemv_q4_0_f16mma", _p(W), _p(S), _p(X), _p(Y), _p(aux), N, K, X.shape[0], _ffi.EPI[epi], ldy, _p(status.word),
              _stream())


def rmsnorm_gemv_mma(W, S, h, norm_w, eps: float, Y, aux, N: int, K: int, epi: str, status: Status) -> None:
    """RMSNorm(h) * norm_w -> fp16 -> `gemv_mma`, one launch."""
    _ffi.call("q4b_rmsnorm_gemv_q4_0_mma", _p(W), _p(S), _p(h), _p(norm_w), float(eps), _p(Y), _p(aux), N, K, _ffi.EPI[epi],
              _p(status.word), _stream())


def rmsnorm_qkv_rope_kv(W, S, h, norm_w, eps: float, qkv, bias, K: int, cosT, sinT, pos, kc, vc, NH: int, NKV: int, HD: int,
                        max_len: int, status: Status) -> None:
    """The decode QKV projection with bias, rounding, RoPE of q / k and the K/V cache append fused in (the `biasf_kv`
    epilogue, lab/qwen_batched.py:1316-1362, applied to one token).  Follow with `attn_cached`."""
    _ffi.call("q4b_rmsnorm_qkv_rope_kv", _p(W), _p(S), _p(h), _p(norm_w), float(eps), _p(qkv), _p(bias), K, _p(cosT), _p(sinT),
              _p(pos), _p(kc), _p(vc), NH, NKV, HD, max_len, _p(status.word), _stream())


def attn_cached(qkv, pos, kc, vc, out, NH: int, NKV: int, HD: int, max_len: int, scale: float) -> None:
    """Decode attention of one sequence over cache rows 0 .. pos (q already rotated, position pos already appended)."""
    _ffi.call("q4b_attn_decode_cached", _p(qkv), _p(pos), _p(kc), _p(vc), _p(out), NH, NKV, HD, max_len, float(scale), _stream())


def quant_q8(x, xq, xd, xsum=None) -> None:
    """x fp16 [rows, K] -> xq int8 [rows, K], xd fp16 [rows, K/32] (QUANT_Q8, lab/qwen_batched.py:1016-1041)."""
    rows = 1 if x.dim() == 1 else x.shape[0]
    _ffi.call("q4b_quant_q8_1", _p(x), _p(xq), _p(xd), _p(xsum), rows, x.shape[-1], _stream())


def rmsnorm_q8(h, w, xq, xd, eps: float, xsum=None, x16=None) -> None:
    """RMSNorm + Q8_1 quantiser in one pass (rmsnorm_q8_source, lab/qwen_batched.py:1044-1091)."""
    rows = 1 if h.dim() == 1 else h.shape[0]
    _ffi.call("q4b_rmsnorm_q8_1", _p(h), _p(w), _p(xq), _p(xd), _p(xsum), _p(x16), rows, h.shape[-1], float(eps), _stream())


def gemm8(W, S, xq, xd, Y, aux, N: int, K: int, P: int, epi: str, ldy: int, status: Status) -> None:
    """Y[P, :] = epilogue(Q8_1(xq, xd) x Q4_0(W, S)^T) with exact int32 block dots (gemm_q4i8_ms_source,
    lab/qwen_batched.py:1271-1561)."""
    _ffi.call("q4b_mmq_q4_0_q8_1", _p(W), _p(S), _p(xq), _p(xd), _p(Y), _p(aux), N, K, P, _ffi.EPI[epi], ldy,
              _p(status.word), _stream())


def gemm8_mma(W, S, xq, xd, Y, aux, N: int, K: int, P: int, epi: str, ldy: int, status: Status) -> None:
    """`gemm8` for up to 32 rows with register accumulators (mma.sync.m16n8k32.s8, bulk-copied weight slab): same block
    arithmetic, no swiglu_q8 epilogue."""
    _ffi.call("q4b_mmq_q4_0_q8_1_mma", _p(W), _p(S), _p(xq), _p(xd), _p(Y), _p(aux), N, K, P, _ffi.EPI[epi], ldy,
              _p(status.word), _stream())


def quant_gemm8_mma(W, S, x16, Y, aux, N: int, K: int, epi: str, ldy: int, status: Status) -> None:
    """`quant_q8` followed by `gemm8_mma` in one launch: x16 fp16 [P, K] is quantised inside the kernel (same bits).
    Saves a launch, but every CTA requantises its K window after its dependency wait; in the batched decode step the two
    separate launches measured faster, so the engine does not use this form."""
    _ffi.call("q4b_quant_mmq_q4_0_q8_1_mma", _p(W), _p(S), _p(x16), _p(Y), _p(aux), N, K, x16.shape[0], _ffi.EPI[epi], ldy,
              _p(status.word), _stream())


def head_batched(E, x, logits) -> None:
    """logits fp32 [B, V] = x fp16 [B, H] . E^T for the tied fp16 table (head_v2_source, lab/qwen_batched.py:681-833)."""
    _ffi.call("q4b_head_f16_batched", _p(E), _p(x), _p(logits), E.shape[0], E.shape[1], x.shape[0], _stream())


def q8_tiled_buffer(rows: int, K: int, device) -> torch.Tensor:
    """Zero-filled buffer for tiled Q8_1 activations of up to `rows` rows of K values."""
    return torch.zeros(_ffi.lib().q4b_q8_tiled_bytes(rows, K), dtype=torch.uint8, device=device)


def f16_tiled_buffer(rows: int, K: int, device) -> torch.Tensor:
    """Zero-filled buffer for the fp16-mode prefill GEMM's activation operand (up to `rows` rows of K values)."""
    return torch.zeros(_ffi.lib().q4b_f16_tiled_bytes(rows, K), dtype=torch.uint8, device=device)


def f16_tile(x, xt) -> None:
    """x fp16 [rows, K] -> the tensor-core operand order of `gemm16_prefill`."""
    _ffi.call("q4b_f16_tiled", _p(x), _p(xt), x.shape[0], x.shape[1], _stream())


def gemm16_prefill(Wt, St, xt, Y, aux, N: int, K: int, P: int, epi: str, ldy: int, status: Status) -> None:
    """The prefill GEMM in the arithmetic of the reference's `cublas` mode (scripts/qwen_prefill.py:37-53, 156-160): weights
    dequantised to fp16 (`dq`, lab/qwen_batched.py:493-498) inside the kernel, fp16 activations (tiled by `f16_tile` or
    `rmsnorm_f16_tiled`), fp32 accumulation over all of K on tcgen05."""
    _ffi.call("q4b_mm_prefill_q4_0_f16", _p(Wt), _p(St), _p(xt), _p(Y), _p(aux), N, K, P, _ffi.EPI[epi], ldy, _p(status.word), _stream())


def gemm16_prefill_resid_ksplit(Wt, St, xt, Y, Y2, N: int, K: int, P: int, ldy: int, status: Status) -> None:
    """`gemm16_prefill` with the resid epilogue, its launch split along K into 1 + Y2.shape[0] parts (Y += part 0, Y2[z - 1] =
    part z)."""
    _ffi.call("q4b_mm_prefill_f16_resid_ksplit", _p(Wt), _p(St), _p(xt), _p(Y), _p(Y2), 1 + Y2.shape[0], N, K, P, ldy,
              _p(status.word), _stream())


def rmsnorm_f16_tiled(h, w, xt, eps: float, h_add=None) -> None:
    """RMSNorm of every row of h (fp32) as fp16 in the operand order of `gemm16_prefill`; with h_add [n, rows, H] first
    h += h_add[0] + h_add[1] + .. (written back)."""
    n = 0 if h_add is None else h_add.shape[0]
    _ffi.call("q4b_rmsnorm_f16_tiled_add", _p(h), _p(h_add), n, _p(w), _p(xt), h.shape[0], h.shape[1], float(eps), _stream())


def quant_q8_tiled(x, xt) -> None:
    """x fp16 [rows, K] -> tiled Q8_1 (the prefill MMQ's activation operand)."""
    _ffi.call("q4b_quant_q8_1_tiled", _p(x), _p(xt), x.shape[0], x.shape[1], _stream())


def rmsnorm_q8_tiled(h, w, xt, eps: float) -> None:
    _ffi.call("q4b_rmsnorm_q8_1_tiled", _p(h), _p(w), _p(xt), h.shape[0], h.shape[1], float(eps), _stream())


def gemm8_prefill(Wt, St, xt, Y, aux, N: int, K: int, P: int, epi: str, ldy: int, status: Status) -> None:
    """The prefill GEMM: Y[P, :] = epilogue(tiled Q8_1 x tile-packed Q4_0^T) on tcgen05 (gemm_q4i8_ms_source,
    lab/qwen_batched.py:1271-1561)."""
    _ffi.call("q4b_mmq_prefill_q4_0_q8_1", _p(Wt), _p(St), _p(xt), _p(Y), _p(aux), N, K, P, _ffi.EPI[epi], ldy,
              _p(status.word), _stream())


def attn_prefill(qkv, cosT, sinT, kc, vc, out, NH: int, NKV: int, HD: int, max_len: int, pos0: int, scale: float) -> None:
    """RoPE + K/V append + causal GQA flash attention for a chunk of prompt tokens of one sequence
    (flash_prefill_v3_source, lab/qwen_batched.py:1795-2037; K/V write of `biasf_kv`, :1316-1362)."""
    _ffi.call("q4b_attn_prefill", _p(qkv), _p(cosT), _p(sinT), _p(kc), _p(vc), _p(out), qkv.shape[0], NH, NKV, HD, max_len,
              pos0, float(scale), _stream())


def gemm8_prefill_qkv_rope_kv(Wt, St, xt, qkv, bias, K: int, P: int, cosT, sinT, pos0: int, kc, vc, NH: int, NKV: int, HD: int,
                              max_len: int, status: Status) -> None:
    """The prefill QKV GEMM with the `biasf_kv` epilogue (lab/qwen_batched.py:1316-1362): bias, rounding, RoPE of q and k,
    K/V cache rows pos0 .. pos0 + P - 1 written.  Follow with `attn_prefill_cached`."""
    _ffi.call("q4b_mmq_prefill_qkv_rope_kv", _p(Wt), _p(St), _p(xt), _p(qkv), _p(bias), K, P, _p(cosT), _p(sinT), pos0, _p(kc),
              _p(vc), NH, NKV, HD, max_len, _p(status.word), _stream())


def attn_prefill_cached(qkv, kc, vc, out, xt, NH: int, NKV: int, HD: int, max_len: int, pos0: int, scale: float) -> None:
    """Causal flash attention over rotated q rows and a cache that already holds the chunk; `out` (fp16) and / or `xt`
    (tiled Q8_1 of the output, the reference kernel's `q8` mode, lab/qwen_batched.py:1812-1848)."""
    _ffi.call("q4b_attn_prefill_cached", _p(qkv), _p(kc), _p(vc), _p(out), _p(xt), qkv.shape[0], NH, NKV, HD, max_len, pos0,
              float(scale), _stream())


def gemm8_prefill_resid_ksplit(Wt, St, xt, Y, Y2, N: int, K: int, P: int, ldy: int, status: Status) -> None:
    """The residual-adding prefill GEMM with its launch split along K into 1 + Y2.shape[0] parts: Y += part 0, Y2[z - 1] =
    part z (see the header)."""
    _ffi.call("q4b_mmq_prefill_resid_ksplit", _p(Wt), _p(St), _p(xt), _p(Y), _p(Y2), 1 + Y2.shape[0], N, K, P, ldy, _p(status.word),
              _stream())


def rmsnorm_q8_tiled_add(h, h_add, w, xt, eps: float) -> None:
    """h += h_add[0] + h_add[1] + .. (written back), then `rmsnorm_q8_tiled`.  h_add fp32 [n, rows, H]."""
    _ffi.call("q4b_rmsnorm_q8_1_tiled_add", _p(h), _p(h_add), h_add.shape[0], _p(w), _p(xt), h.shape[0], h.shape[1], float(eps),
              _stream())


def add_rows(h, h_add) -> None:
    """h += h_add[0] + h_add[1] + ..; h_add fp32 [n, *h.shape]."""
    _ffi.call("q4b_add_rows", _p(h), _p(h_add), h_add.shape[0], h.numel(), _stream())
