"""ctypes binding of libq4b200.so (the C-ABI declared in include/q4b200.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.  PyTorch is used by the
callers only for device memory and streams; no torch type crosses this boundary (pointers go over as integers, as the
reference's `Kern.launch` passes them, scripts/qwen_fused.py:37-42)."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libq4b200.so"

OK, E_SHAPE, E_ALIGN, E_WORKSPACE, E_CUDA, E_ARG, E_TIMEOUT = 0, -1, -2, -3, -4, -5, -6
EPI = {"store": 0, "biasf": 1, "resid": 2, "swiglu": 3, "logits": 4, "swiglu_q8": 5, "biasf_rope_kv": 6, "swiglu_f16t": 7}
X_F16, X_F32 = 0, 1

_P, _I, _F, _Z = C.c_void_p, C.c_int, C.c_float, C.c_size_t


class Linear(C.Structure):
    _fields_ = [("W", _P), ("S", _P), ("N", _I), ("K", _I), ("Wt", _P), ("St", _P)]


class Layer(C.Structure):
    _fields_ = [("ln1", _P), ("ln2", _P), ("qkv_bias", _P), ("qkv", Linear), ("o", Linear), ("gu", Linear),
                ("down", Linear), ("kc", _P), ("vc", _P)]


class DecodeDesc(C.Structure):
    _fields_ = [("layers", _I), ("hidden", _I), ("ffn", _I), ("n_heads", _I), ("n_kv_heads", _I), ("head_dim", _I),
                ("vocab", _I), ("max_len", _I), ("eps", _F), ("scale", _F), ("embed", _P), ("layer", C.POINTER(Layer)),
                ("norm", _P), ("head", Linear), ("cosT", _P), ("sinT", _P), ("tok", _P), ("pos", _P), ("h", _P),
                ("x", _P), ("qkv", _P), ("att", _P), ("act", _P), ("logits", _P), ("attn_ws", _P), ("attn_ws_bytes", _Z),
                ("head_ws", _P), ("head_ws_bytes", _Z), ("status", _P), ("flags", _I), ("persistent_ws", _P),
                ("persistent_ws_bytes", _Z), ("head16", _P), ("head_q6_L", _P), ("head_q6_H", _P), ("head_q6_SC", _P), ("head_q6_D", _P)]


STEP_TENSOR_CORE = 1
STEP_PERSISTENT = 2
STEP_MMA_GEMV = 4
STEP_LOOKAHEAD = 8


# name -> (restype, argtypes); every symbol include/q4b200.h declares
SIGNATURES = {
    "q4b_version": (_I, []),
    "q4b_last_error": (C.c_char_p, []),
    "q4b_init": (_I, [_I]),
    "q4b_gemv_q4_0": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "q4b_rmsnorm": (_I, [_P, _P, _P, _I, _I, _F, _P]),
    "q4b_embed": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "q4b_attn_decode_workspace": (_Z, [_I, _I, _I, _I]),
    "q4b_attn_decode": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _P, _Z, _P]),
    "q4b_attn_decode_q8_1": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _P]),
    "q4b_head_workspace": (_Z, [_I]),
    "q4b_head_f16_argmax": (_I, [_P, _P, _P, _I, _I, _P, _P, _P, _Z, _P]),
    "q4b_head_q6_k_argmax": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _P, _P, _P, _Z, _P]),
    "q4b_argmax_advance_static": (_I, [_P, _I, _I, _P, _P, _P]),
    "q4b_head_f16_batched": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "q4b_argmax_workspace": (_Z, [_I, _I]),
    "q4b_argmax_advance": (_I, [_P, _I, _I, _P, _P, _P, _Z, _P]),
    "q4b_blockdot_q4_0_q8_1": (_I, [_P, _P, _P, _I, _I, _I, _I, _P, _P]),
    "q4b_gemv_q4_0_tc": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P]),
    "q4b_gemv_q4_0_mma": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P]),
    "q4b_gemv_q4_0_f16mma": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P]),
    "q4b_tp_allreduce_resid_rmsnorm_q8": (_I, [_P, _P, _I, _I, C.c_uint32, _P, _P, _I, _I, _P, _F, _P, _P, _P, _P]),
    "q4b_tp_epoch_advance": (_I, [_P, C.c_uint32, _P]),
    "q4b_debug_tp_allreduce_expired_wait": (_I, [_P, _P, _I, _I, C.c_uint32, _P, _I, _I, _P, _P]),
    "q4b_attn_batched_kernel": (_I, [_I]),
    "q4b_mmq_q4_0_q8_1_mma": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P]),
    "q4b_quant_mmq_q4_0_q8_1_mma": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P]),
    "q4b_rmsnorm_gemv_q4_0_mma": (_I, [_P, _P, _P, _P, _F, _P, _P, _I, _I, _I, _P, _P]),
    "q4b_rmsnorm_qkv_rope_kv": (_I, [_P, _P, _P, _P, _F, _P, _P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P]),
    "q4b_debug_gemv_mma_expired_wait": (_I, [_P, _P, _P, _P, _I, _I, _P, _P]),
    "q4b_attn_decode_cached": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _F, _P]),
    "q4b_pack_q4_0": (_I, [_P, _P, _P, _P, _I, _I, _P]),
    "q4b_q8_tiled_bytes": (_Z, [_I, _I]),
    "q4b_debug_mmq_prefill_expired_wait": (_I, [_P, _P, _P, _P, _I, _I, _I, _P, _P]),
    "q4b_f16_tiled_bytes": (_Z, [_I, _I]),
    "q4b_f16_tiled": (_I, [_P, _P, _I, _I, _P]),
    "q4b_mm_prefill_q4_0_f16": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P]),
    "q4b_mm_prefill_f16_resid_ksplit": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P]),
    "q4b_rmsnorm_f16_tiled_add": (_I, [_P, _P, _I, _P, _P, _I, _I, _F, _P]),
    "q4b_quant_q8_1_tiled": (_I, [_P, _P, _I, _I, _P]),
    "q4b_rmsnorm_q8_1_tiled": (_I, [_P, _P, _P, _I, _I, _F, _P]),
    "q4b_mmq_prefill_q4_0_q8_1": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P]),
    "q4b_mmq_prefill_qkv_rope_kv": (_I, [_P, _P, _P, _P, _P, _I, _I, _P, _P, _I, _P, _P, _I, _I, _I, _I, _P, _P]),
    "q4b_attn_prefill_cached": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P]),
    "q4b_mmq_prefill_resid_ksplit": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P]),
    "q4b_rmsnorm_q8_1_tiled_add": (_I, [_P, _P, _I, _P, _P, _I, _I, _F, _P]),
    "q4b_add_rows": (_I, [_P, _P, _I, _Z, _P]),
    "q4b_mmq_prefill_trace": (_I, [_P, _Z]),
    "q4b_attn_prefill": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P]),
    "q4b_trace_buffer": (_I, [_P, _Z]),
    "q4b_peak_i8_launch": (C.c_double, [_I, _P, _P]),
    "q4b_trace_chain": (_I, [_P, _Z]),
    "q4b_trace_chain_log": (_I, [_P, _I]),
    "q4b_rmsnorm_gemv_q4_0_tc": (_I, [_P, _P, _P, _P, _F, _P, _P, _I, _I, _I, _P, _P]),
    "q4b_mmq_q4_0_q8_1": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P]),
    "q4b_quant_q8_1": (_I, [_P, _P, _P, _P, _I, _I, _P]),
    "q4b_rmsnorm_q8_1": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _F, _P]),
    "q4b_decode_step": (_I, [C.POINTER(DecodeDesc), _P]),
    "q4b_decode_persistent_workspace": (_Z, [C.POINTER(DecodeDesc)]),
    "q4b_decode_persistent_prepare": (_I, [C.POINTER(DecodeDesc), _P, _Z]),
    "q4b_decode_persistent_layers": (_I, [C.POINTER(DecodeDesc), _P, _Z, _P]),
    "q4b_decode_persistent_trace": (_I, [_P, _I]),
}


class Q4BError(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"libq4b200 error {code}: {text}")
        self.code = code


_lib = None


def lib():
    """The loaded library with argument types set.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise FileNotFoundError(f"{LIB_PATH} is missing: build it with `python 3080lab_b200/build.py` "
                                    "(there is no CPU or PyTorch fallback)")
        h = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(h, name)
            fn.restype, fn.argtypes = res, args
        _lib = h
    return _lib


def check(code: int) -> None:
    if code != OK:
        raise Q4BError(code, lib().q4b_last_error().decode("utf-8", "replace"))


def call(name: str, *args):
    """Call an int-returning entry point and raise on a non-zero status."""
    check(getattr(lib(), name)(*args))
