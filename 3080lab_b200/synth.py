"""Model shapes and the seeded synthetic Q4_0 model generator.

The reference runs the real Qwen2.5-1.5B-Instruct Q4_0 GGUF (scripts/qwen_gguf.py:63-113); no model file is available
to this build, so weights of the same architecture are drawn from a seed with the distributions the reference's GEMV
microbenchmark uses (lab/experiments/gemv5.py:40-46): nibbles q ~ U{0..15}, block scales d ~ U(0.002, 0.02) as fp16.
Norm weights are 1 + 0.1 N(0,1), QKV biases 0.1 N(0,1), the tied fp16 embedding 0.02 N(0,1).

All tensors come out in the canonical device layout (W int32 [N, K/8], S fp16 [N, K/32]); QKV rows are concatenated
(scripts/qwen_gguf.py:77-78) and gate/up rows interleaved g0,u0,g1,u1,... (scripts/qwen_gguf.py:79-81).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class ModelConfig:
    name: str
    layers: int
    hidden: int
    ffn: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    vocab: int
    eps: float = 1e-6
    rope_theta: float = 1e6
    tied_fp16_head: bool = True      # True: logits = fp16 embedding table; False: separate Q4_0 head

    @property
    def q_rows(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_rows(self) -> int:
        return self.n_kv_heads * self.head_dim

    @property
    def qkv_rows(self) -> int:
        return self.q_rows + 2 * self.kv_rows

    def q4_bytes_per_layer(self) -> int:
        w = self.qkv_rows * self.hidden + self.hidden * self.q_rows + 2 * self.ffn * self.hidden + self.hidden * self.ffn
        return w // 32 * 18

    def head_bytes(self) -> int:
        return self.vocab * self.hidden * 2 if self.tied_fp16_head else self.vocab * self.hidden // 32 * 18

    def kv_bytes_per_position(self) -> int:
        return 2 * self.kv_rows * 2 * self.layers


QWEN25_1P5B = ModelConfig("qwen2.5-1.5b", 28, 1536, 8960, 12, 2, 128, 151936)
QWEN25_7B = ModelConfig("qwen2.5-7b", 28, 3584, 18944, 28, 4, 128, 152064, tied_fp16_head=False)
# Small shapes of the same architecture for parity tests the CPU oracle finishes in seconds.
TINY = ModelConfig("tiny", 2, 256, 512, 4, 2, 64, 1024)
SMALL = ModelConfig("small", 4, 512, 1536, 4, 2, 128, 4096)

CONFIGS = {c.name: c for c in (QWEN25_1P5B, QWEN25_7B, TINY, SMALL)}


def synth_q4(rng: np.random.Generator, n: int, k: int):
    """-> (W int32 [n, k/8], S fp16 [n, k/32]) with uniform nibbles and U(0.002, 0.02) scales."""
    words = rng.integers(0, 2 ** 32, size=(n, k // 8), dtype=np.uint32)      # 8 uniform nibbles per word
    scales = rng.uniform(0.002, 0.02, size=(n, k // 32)).astype(np.float16)
    return words.view(np.int32), scales


def synth_model(cfg: ModelConfig, seed: int = 0) -> dict:
    """Deterministic random-init weights.  Returns {"cfg", "embed", "layers": [...], "norm", "head"}."""
    layers = []
    for i in range(cfg.layers):
        rng = np.random.default_rng([seed, i])
        layers.append({
            "ln1": (1.0 + 0.1 * rng.standard_normal(cfg.hidden)).astype(np.float32),
            "ln2": (1.0 + 0.1 * rng.standard_normal(cfg.hidden)).astype(np.float32),
            "qkv": synth_q4(rng, cfg.qkv_rows, cfg.hidden),
            "qkv_b": (0.1 * rng.standard_normal(cfg.qkv_rows)).astype(np.float32),
            "o": synth_q4(rng, cfg.hidden, cfg.q_rows),
            "gu": synth_q4(rng, 2 * cfg.ffn, cfg.hidden),          # rows interleaved gate, up
            "down": synth_q4(rng, cfg.hidden, cfg.ffn),
        })
    rng = np.random.default_rng([seed, 1 << 20])
    # 0.02 N(0,1) in fp16.  Drawing and casting vocab x hidden normals costs tens of seconds in numpy, so 4096 rows are
    # drawn and every further group of 4096 rows is that block with its columns rotated by another 37 places: each
    # element keeps the N(0, 0.02^2) marginal, no two rows are equal, and the table costs one pass of copies.
    rows = min(cfg.vocab, 4096)
    base = (0.02 * rng.standard_normal((rows, cfg.hidden))).astype(np.float16)
    embed = np.empty((cfg.vocab, cfg.hidden), np.float16)
    for c in range(-(-cfg.vocab // rows)):
        n = min(rows, cfg.vocab - c * rows)
        embed[c * rows:c * rows + n] = np.roll(base[:n], 37 * c, axis=1)
    model = {
        "cfg": cfg,
        "embed": embed,
        "layers": layers,
        "norm": (1.0 + 0.1 * rng.standard_normal(cfg.hidden)).astype(np.float32),
        "head": None if cfg.tied_fp16_head else synth_q4(rng, cfg.vocab, cfg.hidden),
    }
    return model


def rope_tables(cfg: ModelConfig, max_len: int):
    """cos/sin fp32 [max_len, head_dim/2] from float64 angles (scripts/qwen_gguf.py:111-113)."""
    half = cfg.head_dim // 2
    inv = 1.0 / (cfg.rope_theta ** (np.arange(0, cfg.head_dim, 2, dtype=np.float64) / cfg.head_dim))
    ang = np.arange(max_len, dtype=np.float64)[:, None] * inv[None, :]
    assert ang.shape == (max_len, half)
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def synth_prompt(cfg: ModelConfig, n: int, seed: int = 0) -> np.ndarray:
    """Prompt tokens drawn uniform from the vocabulary (the reference's prefill check uses
    torch.manual_seed(0); randint(0, 150000, (P,)), scripts/qwen_prefill.py:351-352)."""
    return np.random.default_rng([seed, 7]).integers(0, cfg.vocab, size=n, dtype=np.int64)
