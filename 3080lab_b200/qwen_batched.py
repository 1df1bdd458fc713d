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
