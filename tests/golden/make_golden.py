"""Generate the golden fixtures in this folder by running the reference's own Python code.

Run once in a container that has the reference checked out:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's `lab.gguf` (numpy only) and records what that code returns for seeded inputs.  The
fixtures are small .npz files; the tests never need the reference at run time.

Fixtures:
  q4_0_codec.npz   random Q4_0 bytes -> reference q4_0_blocks(d, q) and the GGUF.f32 dequantisation
  gguf_file.npz    a tiny GGUF file (bytes) -> what the reference's GGUF class parses out of it
  gemv_small.npz   a 64 x 256 GEMV drawn like lab/experiments/gemv5.py:40-46, dequantise-and-dot by reference code
  gemv_ffn_up.npz  the 8960 x 1536 ffn_up GEMV: y from the reference's fp32 dequantise-and-dot, and the float64 oracle
  q6_k_codec.npz   random Q6_K blocks -> reference q6_k_parts (q, scales, d) and the GGUF.f32 dequantisation
  tensor_s8_known_answer.npz  the seeded int8 operands of the reference's tensor-core known-answer check
                   (lab/experiments/tensor.py:171-179, which demands exact equality) and its expected A8 @ B8 + C8
  rope_tables.npz  cos / sin rows computed by the reference's own statement (scripts/qwen_gguf.py:111-113, torch double
                   -> float) for head_dim 128, theta 1e6, at a spread of positions
  pack_q4_i8.npz   the same matrix through the reference's `pack_q4_i8` (lab/qwen_batched.py:987-1013): the operand of its
                   int8 MMQ (unsigned nibbles, offset corrected through the planted -8 sum(x) term)
  pack_q4_mma.npz  a seeded 48 x 192 Q4_0 matrix in the canonical device words and what the reference's own
                   `pack_q4_mma` (lab/qwen_batched.py:394-436, torch on the CPU) makes of it: the fragment-ordered
                   operand of its batched-decode GEMV
"""
from __future__ import annotations

import importlib
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]


def gemv_inputs(n: int, k: int, bf16_x: bool):
    """Input recipe of lab/experiments/gemv5.py:40-46 (rng = default_rng(n + k); q, then d, then x)."""
    rng = np.random.default_rng(n + k)
    q = rng.integers(0, 16, size=(n, k), dtype=np.uint32)
    d = rng.uniform(0.002, 0.02, size=(n, k // 32)).astype(np.float16)
    x = rng.standard_normal(k).astype(np.float32)
    if bf16_x:                                   # gemv5 truncates x to bf16; the ffn_up configuration keeps fp32
        x = ((x.view(np.uint32) >> 16) << 16).view(np.float32)
    return q.astype(np.uint8), d, x


def to_q4_0_bytes(q: np.ndarray, d: np.ndarray) -> np.ndarray:
    """Rows of natural-order nibbles -> ggml Q4_0 records (low nibbles = weights 0..15, high = 16..31)."""
    qb = q.reshape(-1, 32)
    rec = np.empty((qb.shape[0], 18), np.uint8)
    rec[:, :2] = d.reshape(-1).view(np.uint8).reshape(-1, 2)
    rec[:, 2:] = qb[:, :16] | (qb[:, 16:] << 4)
    return rec.reshape(-1)


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    ref = importlib.import_module("lab.gguf")
    sys.path.insert(0, str(ROOT))
    ours = importlib.import_module("3080lab_b200.gguf")

    # 1. codec
    rng = np.random.default_rng(1)
    raw = rng.integers(0, 256, size=96 * 18, dtype=np.uint8)
    rec = raw.reshape(-1, 18)
    rec[:, :2] = rng.uniform(-0.05, 0.05, size=96).astype(np.float16).view(np.uint8).reshape(-1, 2)
    d, q = ref.q4_0_blocks(raw)
    deq = (d[:, None] * (q.astype(np.float32) - 8)).reshape(-1)          # the GGUF.f32 Q4_0 branch
    np.savez_compressed(HERE / "q4_0_codec.npz", raw=raw, d=d, q=q, f32=deq)

    # 1b. Q6_K codec: random blocks (every bit pattern of ql / qh / scales is a valid block) with sane fp16 super-scales
    rng6 = np.random.default_rng(6)
    raw6 = rng6.integers(0, 256, size=(40, 210), dtype=np.uint8)
    raw6[:, 208:210] = rng6.uniform(-0.02, 0.02, size=40).astype(np.float16).view(np.uint8).reshape(-1, 2)
    raw6 = raw6.reshape(-1)
    q6, sc6, d6 = ref.q6_k_parts(raw6)
    q6b, s6 = ref.q6_k_blocks(raw6)
    deq6 = (np.repeat(s6, 16, axis=1) * q6b.astype(np.float32)).reshape(-1)   # the GGUF.f32 Q6_K branch (lab/gguf.py:80-82)
    np.savez_compressed(HERE / "q6_k_codec.npz", raw=raw6, q=q6, sc=sc6, d=d6, f32=deq6)

    # 2. a GGUF file parsed by the reference reader
    qs, ds, _ = gemv_inputs(16, 64, False)
    f16t = rng.standard_normal((4, 8)).astype(np.float16)
    f32t = rng.standard_normal(8).astype(np.float32)
    with tempfile.TemporaryDirectory() as tmp:
        path = Path(tmp) / "tiny.gguf"
        ours.write_gguf(path, {"general.architecture": "qwen2", "qwen2.block_count": 2,
                               "qwen2.rope.freq_base": 1e6, "tokens": ["a", "b", "c"]},
                        {"blk.0.attn_q.weight": (2, (64, 16), to_q4_0_bytes(qs, ds).tobytes()),
                         "token_embd.weight": (1, (8, 4), f16t.tobytes()),
                         "output_norm.weight": (0, (8,), f32t.tobytes())})
        blob = np.frombuffer(path.read_bytes(), np.uint8)
        g = ref.GGUF(path)
        np.savez_compressed(
            HERE / "gguf_file.npz", blob=blob, data_start=g.data_start,
            meta_keys=np.array(sorted(g.meta)), meta_block_count=g.meta["qwen2.block_count"],
            meta_freq_base=g.meta["qwen2.rope.freq_base"], meta_tokens=np.array(g.meta["tokens"]),
            names=np.array(list(g.tensors)), dims_q=np.array(g.tensors["blk.0.attn_q.weight"].dims),
            q_f32=g.f32("blk.0.attn_q.weight"), e_f32=g.f32("token_embd.weight"), n_f32=g.f32("output_norm.weight"))
        del g

    # 3/4. GEMV: the reference's numpy dequantise-and-dot on gemv5's input recipe
    for name, n, k, bf in (("gemv_small", 64, 256, True), ("gemv_ffn_up", 8960, 1536, False)):
        q, d, x = gemv_inputs(n, k, bf)
        dd, qq = ref.q4_0_blocks(to_q4_0_bytes(q, d))
        w = (dd[:, None] * (qq.astype(np.float32) - 8)).reshape(n, k)     # lab/gguf.py:77-79
        y32 = w @ x
        y64 = ((q.astype(np.float64) - 8) * np.repeat(d.astype(np.float64), 32, axis=1)) @ x.astype(np.float64)
        out = {"n": n, "k": k, "bf16_x": bf, "y_ref_f32": y32, "y_ref_f64": y64}
        if n * k <= 1 << 16:
            out.update(q=q, d=d, x=x)
        np.savez_compressed(HERE / f"{name}.npz", **out)
    # 5. the s8 known-answer inputs: the draw order of lab/experiments/tensor.py:171-179 (fp16 A, B, fp32 C first, then
    # the int8 operands), expected result as computed there (:178)
    rng = np.random.default_rng(7)
    rng.standard_normal((16, 16)).astype(np.float16)
    rng.standard_normal((16, 8)).astype(np.float16)
    rng.standard_normal((16, 8)).astype(np.float32)
    A8 = rng.integers(-128, 128, (16, 32)).astype(np.int8)
    B8 = rng.integers(-128, 128, (32, 8)).astype(np.int8)
    C8 = rng.integers(-1000, 1000, (16, 8)).astype(np.int32)
    np.savez_compressed(HERE / "tensor_s8_known_answer.npz", A8=A8, B8=B8, C8=C8,
                        ref8=A8.astype(np.int32) @ B8.astype(np.int32) + C8)

    # 6. RoPE tables by the reference's statement, executed with torch on the CPU (scripts/qwen_gguf.py:111-113)
    import torch
    hd, theta = 128, 1e6
    positions = list(range(0, 48)) + [63, 64, 127, 128, 511, 512, 513, 600, 767, 1023, 1024, 2047, 4095]
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2).double() / hd))
    ang = torch.tensor(positions).double()[:, None] * inv[None]
    np.savez_compressed(HERE / "rope_tables.npz", positions=np.array(positions), head_dim=hd, theta=theta,
                        cos=torch.cos(ang).float().numpy(), sin=torch.sin(ang).float().numpy())
    # 7. the reference's fragment-order repack for its batched-decode GEMV, run as is on the CPU
    rb = importlib.import_module("lab.qwen_batched")
    q, d, _ = gemv_inputs(48, 192, False)
    words = np.zeros((48, 192 // 8), np.uint32)
    for i in range(8):                                   # nibble i of word w = weight 8 w + i (scripts/qwen_gguf.py:54-60)
        words |= q[:, i::8].astype(np.uint32) << np.uint32(4 * i)
    W = torch.from_numpy(words.view(np.int32).copy())
    Wp, Sp = rb.pack_q4_mma(W, torch.from_numpy(d.copy()))
    np.savez_compressed(HERE / "pack_q4_mma.npz", W=W.numpy(), S=d, Wp=Wp.numpy(), Sp=Sp.numpy())
    # 8. ... and its repack for the int8 MMQ (unsigned nibbles as the A operand), on the same matrix
    Wi, Si = rb.pack_q4_i8(W, torch.from_numpy(d.copy()))
    np.savez_compressed(HERE / "pack_q4_i8.npz", W=W.numpy(), S=d, Wp=Wi.numpy(), Sp=Si.numpy())
    print("fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
