"""Qwen2-architecture models from GGUF files, and back.

`load_model(path)` reads a llama.cpp GGUF (metadata keys `<arch>.embedding_length`, `.block_count`,
`.attention.head_count[_kv]`, `.feed_forward_length`, `.attention.layer_norm_rms_epsilon`, `.rope.freq_base`;
tensors `token_embd`, `blk.N.attn_{q,k,v,output}`, `blk.N.ffn_{gate,up,down}`, `blk.N.{attn,ffn}_norm`, `output_norm`,
`output`) into the model dict `engine.FusedQwen` takes, the way the reference's `GGUFQwen` does
(scripts/qwen_gguf.py:63-91): q, k, v concatenated row-wise into one QKV matrix (and bias), gate and up interleaved row
by row (row 2i = gate i, row 2i + 1 = up i) so the SwiGLU epilogue sees both halves of a pair in one thread pair, all
in the canonical device layout (`gguf.pack_nibbles`).  `GGUFQwen(path)` is `FusedQwen(load_model(path))`.

Supported tensor types: Q4_0 for the layer matrices; Q4_0, Q6_K, F16 or F32 for `token_embd` (kept as an fp16 table:
everything but F16 is rounded to fp16, the reference keeps fp32); `output.weight` absent (tied head), Q4_0 (the Q4_0
head path), or Q6_K / F16 / F32 (dequantised on the host into an untied fp16 head table, `model["head16"]`).  The
reference runs a Q6_K head with its own GEMV kernel at 6.5625 bits per weight (scripts/qwen_gguf.py:92-113); so does the
batch-1 decode step here (`model["head_q6"]`, q4b_head_q6_k_argmax) when hidden is 512 .. 2048; for the other paths such a
head costs 16 bits per weight and its values carry one fp16 rounding (relative 2^-11), which is the documented
difference of this loader.

`export_model(model, path)` writes the same layout back (used for synthetic models and by the tests).
"""
from __future__ import annotations

import numpy as np

from . import gguf as G
from .synth import ModelConfig

_Q4_0, _F16, _F32, _Q6_K = 2, 1, 0, 14      # ggml type ids


def _type_name(t: int) -> str:
    return G.GGML_TYPES[t][0] if t in G.GGML_TYPES else f"ggml type {t}"


def _q4(g: G.GGUF, name: str):
    q, d = G.q4_rows(g, name)
    return q, d


def load_model(path) -> dict:
    g = G.GGUF(path)
    m = g.meta
    arch = m.get("general.architecture", "qwen2")
    key = lambda k: m[f"{arch}.{k}"]                              # noqa: E731
    H, nL = int(key("embedding_length")), int(key("block_count"))
    nh, nkv = int(key("attention.head_count")), int(key("attention.head_count_kv"))
    ffn = int(key("feed_forward_length"))
    eps = float(key("attention.layer_norm_rms_epsilon"))
    theta = float(m.get(f"{arch}.rope.freq_base", 1e6))
    hd = H // nh
    emb_t = g.tensors["token_embd.weight"]
    vocab = int(emb_t.dims[1])
    if emb_t.type == _F16:
        embed = np.ascontiguousarray(g.raw("token_embd.weight")[0]).view(np.float16).reshape(vocab, H).copy()
    elif emb_t.type in (_F32, _Q4_0, _Q6_K):
        embed = g.f32("token_embd.weight").astype(np.float16)
    else:
        raise NotImplementedError(f"token_embd.weight is {_type_name(emb_t.type)}; Q4_0, Q6_K, F16 and F32 are supported")
    head, head16, head_q6 = None, None, None
    if "output.weight" in g.tensors:
        t = g.tensors["output.weight"]
        if t.type == _Q4_0:
            q, d = _q4(g, "output.weight")
            head = (G.pack_nibbles(q), d)
        elif t.type == _F16:
            head16 = np.ascontiguousarray(g.raw("output.weight")[0]).view(np.float16).reshape(vocab, H).copy()
        elif t.type == _Q6_K:
            # kept at 6.5625 bits per weight for the batch-1 head kernel (q4b_head_q6_k_argmax); the fp16 table is what
            # the batched and prefill paths use
            head_q6 = G.q6_k_planes(g.raw("output.weight")[0], vocab, H)
            head16 = g.f32("output.weight").astype(np.float16)
        elif t.type == _F32:
            head16 = g.f32("output.weight").astype(np.float16)
        else:
            raise NotImplementedError(f"output.weight is {_type_name(t.type)}; Q4_0, Q6_K, F16 and F32 are supported")
    layers = []
    for i in range(nL):
        p = f"blk.{i}."
        parts = [_q4(g, p + f"attn_{x}.weight") for x in "qkv"]
        qkv_q = np.concatenate([a for a, _ in parts])
        qkv_d = np.concatenate([b for _, b in parts])
        gq, gd = _q4(g, p + "ffn_gate.weight")
        uq, ud = _q4(g, p + "ffn_up.weight")
        gu_q = np.stack([gq, uq], 1).reshape(-1, gq.shape[1])
        gu_d = np.stack([gd, ud], 1).reshape(-1, gd.shape[1])
        oq, od = _q4(g, p + "attn_output.weight")
        dq, dd = _q4(g, p + "ffn_down.weight")
        bias = [g.f32(p + f"attn_{x}.bias") if p + f"attn_{x}.bias" in g.tensors else
                np.zeros(n, np.float32) for x, n in zip("qkv", (nh * hd, nkv * hd, nkv * hd))]
        layers.append({
            "ln1": g.f32(p + "attn_norm.weight").astype(np.float32).copy(),
            "ln2": g.f32(p + "ffn_norm.weight").astype(np.float32).copy(),
            "qkv": (G.pack_nibbles(qkv_q), np.ascontiguousarray(qkv_d)),
            "qkv_b": np.concatenate(bias).astype(np.float32),
            "o": (G.pack_nibbles(oq), np.ascontiguousarray(od)),
            "gu": (G.pack_nibbles(gu_q), np.ascontiguousarray(gu_d)),
            "down": (G.pack_nibbles(dq), np.ascontiguousarray(dd)),
        })
    cfg = ModelConfig(str(m.get("general.name", arch)), nL, H, ffn, nh, nkv, hd, vocab, eps, theta,
                      tied_fp16_head=head is None)            # True also for an untied fp16 table (model["head16"])
    return {"cfg": cfg, "embed": embed, "layers": layers, "norm": g.f32("output_norm.weight").astype(np.float32).copy(),
            "head": head, "head16": head16, "head_q6": head_q6}


def _q4_tensor(W: np.ndarray, S: np.ndarray):
    """canonical (W int32 [N, K/8], S fp16 [N, K/32]) -> (ggml type, ggml dims, Q4_0 bytes)."""
    q = G.unpack_nibbles(W)
    n, k = q.shape
    return _Q4_0, (k, n), G.q4_0_encode(q.reshape(-1, 32), np.asarray(S, np.float16).reshape(-1)).tobytes()


def _f32_tensor(a: np.ndarray):
    a = np.ascontiguousarray(a, np.float32)
    return _F32, tuple(reversed(a.shape)), a.tobytes()


def export_model(model: dict, path, arch: str = "qwen2") -> None:
    """Write a model dict as a GGUF file with the tensor names and row layouts `load_model` expects."""
    c: ModelConfig = model["cfg"]
    meta = {"general.architecture": arch, "general.name": c.name, f"{arch}.embedding_length": c.hidden,
            f"{arch}.block_count": c.layers, f"{arch}.attention.head_count": c.n_heads,
            f"{arch}.attention.head_count_kv": c.n_kv_heads, f"{arch}.feed_forward_length": c.ffn,
            f"{arch}.attention.layer_norm_rms_epsilon": float(c.eps), f"{arch}.rope.freq_base": float(c.rope_theta)}
    emb = np.ascontiguousarray(model["embed"], np.float16)
    tensors = {"token_embd.weight": (_F16, (c.hidden, c.vocab), emb.tobytes()),
               "output_norm.weight": _f32_tensor(model["norm"])}
    if model["head"] is not None:
        tensors["output.weight"] = _q4_tensor(*model["head"])
    elif model.get("head16") is not None:
        tensors["output.weight"] = (_F16, (c.hidden, c.vocab), np.ascontiguousarray(model["head16"], np.float16).tobytes())
    qr, kr = c.q_rows, c.kv_rows
    for i, L in enumerate(model["layers"]):
        p = f"blk.{i}."
        W, S = L["qkv"]
        for x, (a, b) in zip("qkv", ((0, qr), (qr, qr + kr), (qr + kr, qr + 2 * kr))):
            tensors[p + f"attn_{x}.weight"] = _q4_tensor(W[a:b], S[a:b])
            tensors[p + f"attn_{x}.bias"] = _f32_tensor(L["qkv_b"][a:b])
        W, S = L["gu"]
        tensors[p + "ffn_gate.weight"] = _q4_tensor(W[0::2], S[0::2])
        tensors[p + "ffn_up.weight"] = _q4_tensor(W[1::2], S[1::2])
        tensors[p + "attn_output.weight"] = _q4_tensor(*L["o"])
        tensors[p + "ffn_down.weight"] = _q4_tensor(*L["down"])
        tensors[p + "attn_norm.weight"] = _f32_tensor(L["ln1"])
        tensors[p + "ffn_norm.weight"] = _f32_tensor(L["ln2"])
    G.write_gguf(path, meta, tensors)


def GGUFQwen(path, max_len: int = 1024, device="cuda:0", **kw):
    """The reference's `GGUFQwen(path)` (scripts/qwen_gguf.py:63): a `FusedQwen` built from a GGUF file."""
    from .engine import FusedQwen
    return FusedQwen(load_model(path), max_len=max_len, device=device, **kw)
