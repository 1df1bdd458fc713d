"""CPU oracle for the Qwen2.5 Q4_0 inference hot path.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only the tests, the smoke check and the benchmark's CPU-baseline leg may import this file; the product package never
does.  It restates, in numpy, the arithmetic of the reference's kernels and host code; every function cites the
reference file:line it follows.  Values are computed in float64 (or exact integers) and rounded where the data path
stores them: fp16 for activations / KV cache / Q8_1 scales, fp32 for the residual stream and logits.  The Q8_1
quantiser is the exception: its fp32 division and round-to-nearest-even decide integer outputs, so it is mirrored
operation by operation in float32.

Pinning: `q4_0_blocks`, `dequant` and `gemv_ref` are checked against the reference's own `lab/gguf.py` code and the
generator/oracle of `lab/experiments/gemv5.py` through fixtures under tests/golden (made by tests/golden/make_golden.py
with the reference imported); the RoPE tables against the reference's statement run with torch on the CPU; `blockdot`
against the reference's s8 known-answer operands and against its own `pack_q4_i8` repack with the planted offset term;
`dequant_f16w` against its `pack_q4_mma` repack read the way its kernel reads it.  The remaining functions restate CUDA source that cannot execute without the
reference's NVRTC toolchain and model files: parity for those is unpinned against a running reference and is
cross-checked against an independent formulation in the tests instead.

Storage deviations from the reference, as the target configuration states them: fp16 (not bf16) activations and KV
cache, Q8_1 activation blocks with an fp16 scale, a tied fp16 LM head for the 1.5B shape.
"""
from __future__ import annotations

import numpy as np

F64, F32, F16 = np.float64, np.float32, np.float16


def f16(x):
    """Round to fp16 storage and return as float64 for further math."""
    return np.asarray(x, F64).astype(F16).astype(F64)


def f32(x):
    return np.asarray(x, F64).astype(F32).astype(F64)


# ----------------------------------------------------------------------------------------------------------- codec
def q4_0_blocks(b):
    """Raw Q4_0 bytes -> (d float32 [nblk], q uint8 [nblk, 32] in weight order).  lab/gguf.py:88-94: byte pair 0-1 is
    the fp16 scale, bytes 2-17 hold weights 0..15 in the low nibbles and 16..31 in the high nibbles."""
    blk = np.asarray(b, np.uint8).reshape(-1, 18)
    d = blk[:, :2].copy().view(F16).astype(F32).reshape(-1)
    qs = blk[:, 2:]
    return d, np.concatenate([qs & 15, qs >> 4], axis=1)


def unpack_words(W):
    """Canonical device words int32 [N, K/8] -> q int64 [N, K] (0..15); nibble i of word w is weight 8w + i
    (scripts/qwen_gguf.py:54-60)."""
    w = np.ascontiguousarray(W).view(np.uint32).astype(np.int64)
    q = np.stack([(w >> (4 * i)) & 15 for i in range(8)], axis=-1)
    return q.reshape(w.shape[0], -1)


def dequant(W, S, dtype=F64):
    """Dense weights (q - 8) * d, the `GGUF.f32` Q4_0 statement (lab/gguf.py:77-79) on the canonical layout."""
    q = unpack_words(W)
    return ((q - 8).astype(dtype) * np.repeat(np.asarray(S).astype(dtype), 32, axis=1))


def dequant_f16w(W, S, dtype=F64):
    """Dense weights as the reference's batched-decode GEMV forms them (`dq`, lab/qwen_batched.py:493-498): q - 8 exact
    in fp16, times the fp16 block scale, rounded ONCE to fp16.  The fp32 product of a 4-bit and an 11-bit significand is
    exact, so rounding it to fp16 is that single rounding."""
    q = unpack_words(W)
    w = (q - 8).astype(F32) * np.repeat(np.asarray(S).astype(F32), 32, axis=1)
    return w.astype(F16).astype(dtype)


def gemv_f16w_ref(W, S, X):
    """The batched-decode GEMV of gemv_v2_source (lab/qwen_batched.py:467-641) in float64: fp16-rounded weights times
    fp16 activations X [B, K] -> [B, N] (the kernel accumulates in fp32)."""
    return np.asarray(X, F16).astype(F64) @ dequant_f16w(W, S, F64).T


def gemv_ref(W, S, x):
    """float64 dequantise-and-dot: ref = ((q - 8) * repeat(d, 32)) @ x  (lab/experiments/gemv5.py:49)."""
    return dequant(W, S, F64) @ np.asarray(x, F64)


def gemv_numpy_f32(W, S, x):
    """The reference's numpy CPU path as it would run it: fp32 dequantise then fp32 matvec (lab/gguf.py:77-79).
    This is the function the CPU baseline times."""
    q = unpack_words(W).astype(F32)
    w = (q - np.float32(8)) * np.repeat(np.asarray(S).astype(F32), 32, axis=1)
    return w @ np.asarray(x, F32)


# ------------------------------------------------------------------------------------------------------- small ops
def rmsnorm(h, w, eps):
    """RMSNORM_F32W_1P (lab/qwen_kernels.py:683-705): r = rsqrt(sum(v^2)/H + eps); out = round16(v * r * w)."""
    h = np.asarray(h, F64)
    r = 1.0 / np.sqrt(np.mean(h * h, axis=-1, keepdims=True) + eps)
    return f16(h * r * np.asarray(w, F64))


def silu_mul(g, u):
    """swiglu epilogue (lab/qwen_kernels.py:27): round16(g / (1 + exp(-g)) * u)."""
    g = np.asarray(g, F64)
    return f16(g / (1.0 + np.exp(-g)) * np.asarray(u, F64))


def argmax_lowest(v):
    """FINISH tie rule (lab/qwen_kernels.py:227-240): the lowest index among the maxima."""
    return int(np.argmax(np.asarray(v)))


def rope_rotate(x, cos, sin):
    """NeoX pairs (d, d + half) (lab/qwen_kernels.py:533-541): first half x_d c - x_{d+half} s, second half
    x_d c + x_{d-half} s, c/s indexed by d mod half; result rounded to fp16.  x [..., heads, head_dim]."""
    x = np.asarray(x, F64)
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    c, s = np.asarray(cos, F64), np.asarray(sin, F64)
    return f16(np.concatenate([a * c - b * s, b * c + a * s], axis=-1))


# ------------------------------------------------------------------------------------------------------------- Q8_1
def quant_q8_1(x):
    """QUANT_Q8 (lab/qwen_batched.py:1030-1039) on fp16-valued input x [..., K]: per 32 values amax = max|x|,
    d = amax / 127 (fp32 division), q = d > 0 ? rint(x / d) : 0 (fp32 division, round half to even), s = sum q.
    Returns (q int8 [..., K], d16 fp16 [..., K/32], s int32 [..., K/32]).  The stored scale is d rounded to fp16 (the
    Q8_1 record of the target configuration); q comes from the unrounded fp32 d, as in the reference."""
    x = np.asarray(x, F32)
    xb = x.reshape(x.shape[:-1] + (x.shape[-1] // 32, 32))
    amax = np.max(np.abs(xb), axis=-1)
    d = (amax / np.float32(127.0)).astype(F32)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(d[..., None] > 0, np.rint(xb / d[..., None]), np.float32(0)).astype(np.int32)
    return q.reshape(x.shape).astype(np.int8), d.astype(F16), q.sum(axis=-1).astype(np.int32)


def blockdot(W, xq):
    """Exact per-block integer dots: dot[n, m, b] = sum_{i<32} (q4[m, 32b+i] - 8) * q8[n, 32b+i]
    (lab/qwen_batched.py:1237-1243: the u8 x s8 MMA plus the -8 sum(q8) correction carried in its C operand).
    W int32 [M, K/8]; xq int8 [P, K] -> int32 [P, M, K/32]."""
    q = (unpack_words(W) - 8).astype(F64)                       # [M, K]
    M, K = q.shape
    xq = np.asarray(xq).astype(F64)                              # [P, K]
    qb = q.reshape(M, K // 32, 32)
    xb = xq.reshape(-1, K // 32, 32)
    out = np.einsum("pbi,mbi->pmb", xb, qb, optimize=True)       # |dot| <= 32*8*127: exact in float64
    return np.rint(out).astype(np.int32)


def mmq(W, S, xq, xd):
    """Q8_1 x Q4_0 matrix product: y[n, m] = sum_b dw[m, b] * dx[n, b] * dot[n, m, b]
    (lab/qwen_batched.py:1237-1243; the reference adds blocks in ascending order in fp32 with dw*dx rounded to fp32
    first; here the sum is float64).  xd fp16 [P, K/32].  -> float64 [P, M]."""
    q = (unpack_words(W) - 8).astype(F64)
    M, K = q.shape
    wd = (q.reshape(M, K // 32, 32) * np.asarray(S).astype(F64)[:, :, None]).reshape(M, K)
    xs = (np.asarray(xq).astype(F64).reshape(-1, K // 32, 32) * np.asarray(xd).astype(F64)[:, :, None]).reshape(-1, K)
    return xs @ wd.T


def mmq_dense(wd, xq, xd):
    """`mmq` with the weight side already dequantised to float64 [M, K] (caches the expensive half)."""
    K = wd.shape[1]
    xs = (np.asarray(xq).astype(F64).reshape(-1, K // 32, 32) * np.asarray(xd).astype(F64)[:, :, None]).reshape(-1, K)
    return xs @ wd.T


# -------------------------------------------------------------------------------------------------------- attention
def attn_decode(q, kc, vc, n_ctx, scale):
    """Decode attention for one sequence (lab/qwen_kernels.py:548-603): s_j = (q . k_j) * scale, softmax over
    j < n_ctx with a running max, o = sum_j e_j v_j / sum_j e_j with e_j unrounded, result rounded to fp16.
    q [NH, HD] (already rotated + rounded), kc/vc [NKV, >= n_ctx, HD] holding the new position too."""
    q = np.asarray(q, F64)
    NH = q.shape[0]
    NKV = kc.shape[0]
    grp = NH // NKV
    out = np.empty_like(q)
    for h in range(NH):
        k = np.asarray(kc[h // grp, :n_ctx], F64)
        v = np.asarray(vc[h // grp, :n_ctx], F64)
        s = (k @ q[h]) * scale
        e = np.exp(s - s.max())
        out[h] = (e @ v) / e.sum()
    return f16(out)


def attn_prefill(q, k, v, scale, pos0=0, round_p=True):
    """Causal GQA attention over a chunk (lab/qwen_batched.py:1601-1711): query row i (absolute position pos0 + i)
    sees keys j <= pos0 + i; probabilities are rounded to 16 bits before the P.V product (pack of P for the MMA,
    :1686), the normaliser uses the unrounded ones; output rounded to fp16.
    q [P, NH, HD]; k, v [>= pos0 + P, NKV, HD] (cache contents, rotated K)."""
    q = np.asarray(q, F64)
    P, NH, HD = q.shape
    NKV = k.shape[1]
    grp = NH // NKV
    n_keys = pos0 + P
    out = np.empty((P, NH, HD), F64)
    mask = np.arange(n_keys)[None, :] <= (pos0 + np.arange(P))[:, None]
    for h in range(NH):
        kk = np.asarray(k[:n_keys, h // grp], F64)
        vv = np.asarray(v[:n_keys, h // grp], F64)
        s = (q[:, h] @ kk.T) * scale
        s = np.where(mask, s, -np.inf)
        e = np.exp(s - s.max(axis=1, keepdims=True))
        l = e.sum(axis=1, keepdims=True)
        p = f16(e) if round_p else e
        out[:, h] = (p @ vv) / l
    return f16(out)


# ------------------------------------------------------------------------------------------------------- the model
class Oracle:
    """Mirrors the reference engines on a synthetic model dict (see the product's synth.synth_model):
    `step` = FusedQwen.step (scripts/qwen_fused.py:113-145), the fp16-activation decode path;
    `step_q8` = Batched.step op order (scripts/qwen_batched_decode.py:156-187) with the linears routed through
    Q8_1 x Q4_0 as the prefill path does (scripts/qwen_prefill.py:196-246);
    `prefill_q8` = Prefill.chunk (scripts/qwen_prefill.py:196-246)."""

    def __init__(self, model, max_len, cos, sin, batch=1, dense_dtype=F64, weights="exact"):
        """dense_dtype: storage of the cached dequantised matrices.  float64 by default; float32 halves the memory for
        the full 1.5B shape (6 GB instead of 12) at ~1e-7 relative error per linear, far below the 1e-3 bar.
        weights: "exact" = (q - 8) * d; "f16w" = that product rounded to fp16, the layer weights of the reference's
        batched-decode GEMV (`dequant_f16w`); `step` is then Batched.step of scripts/qwen_batched_decode.py:156-187."""
        self.dense_dtype = dense_dtype
        self.weights = weights
        self.m, self.cfg = model, model["cfg"]
        self.max_len, self.B = max_len, batch
        c = self.cfg
        self.cos, self.sin = np.asarray(cos, F64), np.asarray(sin, F64)
        self.kc = np.zeros((c.layers, batch, c.n_kv_heads, max_len, c.head_dim), F16)
        self.vc = np.zeros_like(self.kc)
        self.pos = np.zeros(batch, np.int64)
        self.tok = np.zeros(batch, np.int64)
        self.scale = 1.0 / np.sqrt(c.head_dim)
        self._dense = {}
        self.logits = None

    # dense weights are cached: the oracle is about arithmetic, not about re-decoding nibbles every call
    def dense(self, layer, name):
        key = (layer, name)
        if key not in self._dense:
            W, S = self.m["layers"][layer][name] if layer >= 0 else self.m["head"]
            self._dense[key] = (dequant_f16w if self.weights == "f16w" and layer >= 0 else dequant)(W, S, self.dense_dtype)
        return self._dense[key]

    def _mm(self, x, Wd):
        """x [B, K] @ Wd[N, K]^T in the storage type of Wd (no per-call up-conversion of the matrix), result float64."""
        return (np.asarray(x, Wd.dtype) @ Wd.T).astype(F64)

    def head_dense(self):
        if "head" not in self._dense:
            if self.m.get("head_q6") is not None and self.m.get("head") is None:
                # Q6_K head: (d * sc) * (q - 32) with the fp32 scale product formed first (lab/gguf.py:95-113)
                L, Hb, SC, D = (np.asarray(a) for a in self.m["head_q6"])
                lo, hb = L.view(np.uint32), Hb.view(np.uint32)
                n, k = lo.shape[0], lo.shape[1] * 8
                code = np.zeros((n, k), np.int32)
                for i in range(8):
                    code[:, i::8] = (lo >> np.uint32(4 * i)) & 15
                for i in range(16):                            # bit positions of the Hb plane, see the product's gguf._q6_hi_shift
                    sh = 8 * ((i % 8) // 2) + 2 * ((i % 2) + 2 * (i // 8))
                    code[:, i::16] |= ((hb >> np.uint32(sh)) & 3).astype(np.int32) << 4
                scale = np.repeat(D.astype(F32), 16, axis=1) * SC.astype(F32)
                self._dense["head"] = np.repeat(scale, 16, axis=1).astype(self.dense_dtype) * (code - 32).astype(self.dense_dtype)
            elif self.cfg.tied_fp16_head:
                self._dense["head"] = self.m["embed"].astype(self.dense_dtype)
            else:
                self._dense["head"] = (dequant_f16w if self.weights == "f16w" else dequant)(*self.m["head"], self.dense_dtype)
        return self._dense["head"]

    def _attend(self, i, qkv):
        """RoPE, K/V append at pos, decode attention (lab/qwen_kernels.py:517-605) for every sequence.
        qkv [B, qkv_rows] fp16-valued.  -> att [B, q_rows]."""
        c = self.cfg
        att = np.empty((self.B, c.q_rows), F64)
        for b in range(self.B):
            p = int(self.pos[b])
            q = qkv[b, :c.q_rows].reshape(c.n_heads, c.head_dim)
            k = qkv[b, c.q_rows:c.q_rows + c.kv_rows].reshape(c.n_kv_heads, c.head_dim)
            v = qkv[b, c.q_rows + c.kv_rows:].reshape(c.n_kv_heads, c.head_dim)
            q = rope_rotate(q, self.cos[p], self.sin[p])
            self.kc[i, b, :, p] = rope_rotate(k, self.cos[p], self.sin[p]).astype(F16)
            self.vc[i, b, :, p] = v.astype(F16)
            att[b] = attn_decode(q, self.kc[i, b], self.vc[i, b], p + 1, self.scale).reshape(-1)
        return att

    def step(self):
        """One decode token per sequence on the fp16-activation path.  Leaves fp32 logits in self.logits, the greedy
        token in self.tok, and advances self.pos."""
        c, m = self.cfg, self.m
        h = m["embed"][self.tok].astype(F64)                                  # EMBED: h = float(E[tok])
        for i, L in enumerate(m["layers"]):
            x = rmsnorm(h, L["ln1"], c.eps)
            qkv = f16(self._mm(x, self.dense(i, "qkv")) + L["qkv_b"].astype(F64))    # biasf epilogue
            att = self._attend(i, qkv)
            h = f32(h + self._mm(att, self.dense(i, "o")))                    # resid epilogue
            x = rmsnorm(h, L["ln2"], c.eps)
            gu = self._mm(x, self.dense(i, "gu"))
            act = silu_mul(gu[:, 0::2], gu[:, 1::2])                          # swiglu epilogue, rows interleaved g,u
            h = f32(h + self._mm(act, self.dense(i, "down")))
        x = rmsnorm(h, m["norm"], c.eps)
        self.logits = f32(self._mm(x, self.head_dense()))
        self.h_last = h
        self.tok = np.array([argmax_lowest(r) for r in self.logits], np.int64)
        self.pos = self.pos + 1
        return self.tok.copy()

    def _lin_q8(self, i, name, x16):
        xq, xd, _ = quant_q8_1(x16)
        return mmq_dense(self.dense(i, name), xq, xd)

    def step_q8(self):
        """One decode token per sequence with every linear computed as Q8_1 x Q4_0 (int8 activations)."""
        c, m = self.cfg, self.m
        h = m["embed"][self.tok].astype(F64)
        for i, L in enumerate(m["layers"]):
            x = rmsnorm(h, L["ln1"], c.eps)
            qkv = f16(self._lin_q8(i, "qkv", x) + L["qkv_b"].astype(F64))
            att = self._attend(i, qkv)
            h = f32(h + self._lin_q8(i, "o", att))
            x = rmsnorm(h, L["ln2"], c.eps)
            gu = self._lin_q8(i, "gu", x)
            act = silu_mul(gu[:, 0::2], gu[:, 1::2])
            h = f32(h + self._lin_q8(i, "down", act))
        x = rmsnorm(h, m["norm"], c.eps)
        self.logits = f32(self._mm(x, self.head_dense()))
        self.h_last = h
        self.tok = np.array([argmax_lowest(r) for r in self.logits], np.int64)
        self.pos = self.pos + 1
        return self.tok.copy()

    def prefill_q8(self, ids, pos0=0):
        """One chunk of P prompt tokens of sequence 0 at positions pos0.. (scripts/qwen_prefill.py:196-246): fills the
        KV cache and returns the fp32 residual stream h [P, H]."""
        c, m = self.cfg, self.m
        ids = np.asarray(ids, np.int64)
        P = ids.shape[0]
        pos = pos0 + np.arange(P)
        h = m["embed"][ids].astype(F64)
        for i, L in enumerate(m["layers"]):
            x = rmsnorm(h, L["ln1"], c.eps)
            qkv = f16(self._lin_q8(i, "qkv", x) + L["qkv_b"].astype(F64))
            q = qkv[:, :c.q_rows].reshape(P, c.n_heads, c.head_dim)
            k = qkv[:, c.q_rows:c.q_rows + c.kv_rows].reshape(P, c.n_kv_heads, c.head_dim)
            v = qkv[:, c.q_rows + c.kv_rows:].reshape(P, c.n_kv_heads, c.head_dim)
            cs, sn = self.cos[pos][:, None, :], self.sin[pos][:, None, :]
            q = rope_rotate(q, cs, sn)
            self.kc[i, 0, :, pos0:pos0 + P] = rope_rotate(k, cs, sn).astype(F16).transpose(1, 0, 2)
            self.vc[i, 0, :, pos0:pos0 + P] = v.astype(F16).transpose(1, 0, 2)
            kk = self.kc[i, 0].transpose(1, 0, 2)                             # [maxlen, NKV, HD]
            vv = self.vc[i, 0].transpose(1, 0, 2)
            att = attn_prefill(q, kk, vv, self.scale, pos0).reshape(P, -1)
            h = f32(h + self._lin_q8(i, "o", att))
            x = rmsnorm(h, L["ln2"], c.eps)
            gu = self._lin_q8(i, "gu", x)
            act = silu_mul(gu[:, 0::2], gu[:, 1::2])
            h = f32(h + self._lin_q8(i, "down", act))
        self.pos[0] = pos0 + P
        self.h_last = h
        return h

    def logits_of(self, h):
        x = rmsnorm(h, self.m["norm"], self.cfg.eps)
        return f32(self._mm(x, self.head_dense()))

    def greedy(self, prompt, n_new, q8=False):
        """The reference's decode protocol (scripts/qwen_fused.py:148-180): the prompt goes through `step` token by
        token (its argmax overwritten by the next prompt token); generated token 0 is the argmax after the last
        prompt token.  Single sequence.  -> list of n_new tokens."""
        step = self.step_q8 if q8 else self.step
        for t in prompt:
            self.tok[:] = t
            step()
        out = [int(self.tok[0])]
        for _ in range(n_new - 1):
            step()
            out.append(int(self.tok[0]))
        return out


# --------------------------------------------------------------------------------------------- timed CPU baseline
def canonical_to_gguf_bytes(W, S):
    """Canonical device layout -> raw ggml Q4_0 records (inverse of q4_rows + pack, scripts/qwen_gguf.py:44-60), so the
    CPU baseline can start from the bytes the reference's numpy path starts from."""
    q = unpack_words(W).astype(np.uint8).reshape(-1, 32)
    rec = np.empty((q.shape[0], 18), np.uint8)
    rec[:, :2] = np.ascontiguousarray(S).reshape(-1).view(np.uint8).reshape(-1, 2)
    rec[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    return rec.reshape(-1)


def gemv_numpy_bytes(raw, n, k, x):
    """The reference's numpy CPU path for one linear, from raw GGUF bytes: q4_0_blocks, then the GGUF.f32 statement
    d[:, None] * (q.astype(float32) - 8) reshaped [n, k] (lab/gguf.py:77-79, 88-94), then the fp32 matvec."""
    d, q = q4_0_blocks(raw)
    w = (d[:, None] * (q.astype(F32) - 8)).reshape(n, k)
    return w @ np.asarray(x, F32)


class CpuDecoder:
    """fp32 numpy decode of one sequence with every linear going through `gemv_numpy_bytes` (nothing dequantised ahead
    of time).  Only the CPU-baseline timing uses it; `layer()` and `head()` can be timed separately so that a bounded
    sample (a few layers) can be scaled to a whole token."""

    def __init__(self, model, max_len, cos, sin, layers=None):
        self.m, self.c = model, model["cfg"]
        c = self.c
        self.cos, self.sin = np.asarray(cos, F32), np.asarray(sin, F32)
        self.kc = np.zeros((c.layers, c.n_kv_heads, max_len, c.head_dim), F16)
        self.vc = np.zeros_like(self.kc)
        self.raw = {}
        for i in (range(c.layers) if layers is None else layers):
            L = model["layers"][i]
            self.raw[i] = {k: canonical_to_gguf_bytes(*L[k]) for k in ("qkv", "o", "gu", "down")}
        self.head_raw = None if c.tied_fp16_head else canonical_to_gguf_bytes(*model["head"])

    def _rms(self, v, w):
        return (v * (1.0 / np.sqrt(np.mean(v * v) + np.float32(self.c.eps))) * w).astype(F16).astype(F32)

    def layer(self, i, h, p):
        c, L, raw = self.c, self.m["layers"][i], self.raw[i]
        half = c.head_dim // 2
        cs, sn = self.cos[p], self.sin[p]

        def rot(x):
            a, b = x[:, :half], x[:, half:]
            return np.concatenate([a * cs - b * sn, b * cs + a * sn], axis=1).astype(F16)

        x = self._rms(h, L["ln1"])
        qkv = (gemv_numpy_bytes(raw["qkv"], c.qkv_rows, c.hidden, x) + L["qkv_b"]).astype(F16).astype(F32)
        q = rot(qkv[:c.q_rows].reshape(c.n_heads, c.head_dim)).astype(F32)
        self.kc[i, :, p] = rot(qkv[c.q_rows:c.q_rows + c.kv_rows].reshape(c.n_kv_heads, c.head_dim))
        self.vc[i, :, p] = qkv[c.q_rows + c.kv_rows:].reshape(c.n_kv_heads, c.head_dim).astype(F16)
        att = np.empty((c.n_heads, c.head_dim), F32)
        grp = c.n_heads // c.n_kv_heads
        for hh in range(c.n_heads):
            k = self.kc[i, hh // grp, :p + 1].astype(F32)
            v = self.vc[i, hh // grp, :p + 1].astype(F32)
            s = (k @ q[hh]) * np.float32(1.0 / np.sqrt(c.head_dim))
            e = np.exp(s - s.max())
            att[hh] = (e @ v) / e.sum()
        att = att.reshape(-1).astype(F16).astype(F32)
        h = h + gemv_numpy_bytes(raw["o"], c.hidden, c.q_rows, att)
        x = self._rms(h, L["ln2"])
        gu = gemv_numpy_bytes(raw["gu"], 2 * c.ffn, c.hidden, x)
        g, u = gu[0::2], gu[1::2]
        act = (g / (1.0 + np.exp(-g)) * u).astype(F16).astype(F32)
        return h + gemv_numpy_bytes(raw["down"], c.hidden, c.ffn, act)

    def head(self, h):
        x = self._rms(h, self.m["norm"])
        if self.c.tied_fp16_head:
            logits = self.m["embed"].astype(F32) @ x
        else:
            logits = gemv_numpy_bytes(self.head_raw, self.c.vocab, self.c.hidden, x)
        return int(np.argmax(logits)), logits

    def step(self, tok, p):
        h = self.m["embed"][tok].astype(F32)
        for i in range(self.c.layers):
            h = self.layer(i, h, p)
        return self.head(h)
