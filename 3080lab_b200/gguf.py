"""GGUF container reader and the Q4_0 block codec (host side, numpy).

Call surface follows the reference's `lab/gguf.py`: `GGUF(path).meta / .tensors / .raw(name) / .f32(name)`
(lab/gguf.py:27-85) and `q4_0_blocks(bytes) -> (d, q)` (lab/gguf.py:88-94).  Written from the GGUF v2/v3 file
format and the ggml Q4_0 block definition; the device layout helpers restate `q4_rows` / `to_device_q4`
(scripts/qwen_gguf.py:44-60).

Q4_0 block = 18 bytes for 32 weights: an fp16 scale `d` followed by 16 bytes `qs`.  Weight i (i < 16) is the low
nibble of qs[i], weight i + 16 the high nibble; the value is `d * (nibble - 8)`.

Device layout ("canonical" in this package, the reference's): `W` int32 `[N, K/8]`, nibble i of word w is weight
8w + i (natural weight order, not ggml's low-half/high-half order); `S` fp16 `[N, K/32]`.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np

# ggml type id -> (name, weights per block, bytes per block)
GGML_TYPES = {0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 14: ("Q6_K", 256, 210)}

_FIXED = {0: "B", 1: "b", 2: "H", 3: "h", 4: "I", 5: "i", 6: "f", 7: "?", 10: "Q", 11: "q", 12: "d"}
_T_STRING, _T_ARRAY = 8, 9


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dims: tuple          # ggml order: dims[0] is the contiguous (K) axis, dims[1] the rows (N)
    type: int
    offset: int          # relative to the start of the data section


class _Cursor:
    """Little-endian reader over a bytes-like object."""

    def __init__(self, buf):
        self.buf, self.at = buf, 0

    def take(self, fmt: str):
        size = struct.calcsize("<" + fmt)
        out = struct.unpack_from("<" + fmt, self.buf, self.at)
        self.at += size
        return out

    def string(self) -> str:
        n, = self.take("Q")
        s = bytes(self.buf[self.at:self.at + n]).decode("utf-8", "replace")
        self.at += n
        return s

    def value(self, t: int):
        if t == _T_STRING:
            return self.string()
        if t == _T_ARRAY:
            et, n = self.take("IQ")
            return [self.value(et) for _ in range(n)]
        if t not in _FIXED:
            raise ValueError(f"unknown GGUF metadata type {t}")
        return self.take(_FIXED[t])[0]


class GGUF:
    """Parsed GGUF file.  `meta` maps key -> value, `tensors` maps name -> TensorInfo; tensor bytes stay memory-mapped."""

    def __init__(self, path):
        self.path = Path(path)
        self._fh = open(self.path, "rb")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        cur = _Cursor(self._map)
        magic, = cur.take("4s")
        if magic != b"GGUF":
            raise ValueError(f"{self.path}: not a GGUF file (magic {magic!r})")
        version, n_tensors, n_kv = cur.take("IQQ")
        if version not in (2, 3):
            raise ValueError(f"{self.path}: GGUF version {version} not supported")
        self.version = version
        self.meta: dict = {}
        for _ in range(n_kv):
            key = cur.string()
            t, = cur.take("I")
            self.meta[key] = cur.value(t)
        self.tensors: dict[str, TensorInfo] = {}
        for _ in range(n_tensors):
            name = cur.string()
            nd, = cur.take("I")
            dims = cur.take(f"{nd}Q")
            t, off = cur.take("IQ")
            self.tensors[name] = TensorInfo(name, tuple(dims), t, off)
        align = int(self.meta.get("general.alignment", 32))
        self.data_start = -(-cur.at // align) * align
        self.mm = np.frombuffer(self._map, dtype=np.uint8)

    def raw(self, name: str):
        """-> (uint8 view of the tensor's bytes, TensorInfo)."""
        t = self.tensors[name]
        if t.type not in GGML_TYPES:
            raise NotImplementedError(f"ggml type {t.type} of {name}")
        _, per, size = GGML_TYPES[t.type]
        count = int(np.prod(t.dims))
        begin = self.data_start + t.offset
        return self.mm[begin:begin + count // per * size], t

    def f32(self, name: str) -> np.ndarray:
        """Dequantised fp32 array shaped rows-first (reversed ggml dims)."""
        b, t = self.raw(name)
        kind = GGML_TYPES[t.type][0]
        if kind == "F32":
            flat = b.view(np.float32)
        elif kind == "F16":
            flat = b.view(np.float16).astype(np.float32)
        elif kind == "Q6_K":
            flat = q6_k_dequant(b)
        else:
            d, q = q4_0_blocks(b)
            flat = (d[:, None] * (q.astype(np.float32) - 8.0)).reshape(-1)
        return flat.reshape(tuple(reversed(t.dims)))


def q4_0_blocks(b: np.ndarray):
    """Decode raw Q4_0 bytes -> (d float32 [nblk], q uint8 [nblk, 32]); q is in weight order and still carries the
    +8 offset (value = d * (q - 8)).  Same contract as the reference's `q4_0_blocks` (lab/gguf.py:88-94)."""
    rec = np.ascontiguousarray(b, dtype=np.uint8).reshape(-1, 18)
    d = np.ascontiguousarray(rec[:, 0:2]).view(np.float16).reshape(-1).astype(np.float32)
    packed = rec[:, 2:18]
    q = np.empty((rec.shape[0], 32), np.uint8)
    q[:, :16] = packed & 0x0F
    q[:, 16:] = packed >> 4
    return d, q


def q6_k_values(b: np.ndarray):
    """Decode raw Q6_K bytes -> (q int8 [nblk, 256] in -32..31, sc int8 [nblk, 16], d fp16 [nblk]).

    ggml's block_q6_K is 210 bytes for 256 weights: 128 bytes of low nibbles, 64 bytes of 2-bit high parts, 16 signed
    sub-block scales, one fp16 super-scale.  Inside each half of 128 weights, weight 32 j + l (j = 0..3, l = 0..31) takes
    its low nibble from byte 32 (j & 1) + l of the half's 64 nibble bytes (low nibble for j < 2, high nibble otherwise)
    and its two high bits from bits 2j, 2j + 1 of byte l of the half's 32 high bytes; value = 6-bit code - 32, and weight
    w of the block is scaled by d * sc[w // 16].  Same contract as the reference's `q6_k_parts` (lab/gguf.py:95-123)."""
    rec = np.ascontiguousarray(b, dtype=np.uint8).reshape(-1, 210)
    n = rec.shape[0]
    nib = rec[:, 0:128].reshape(n, 2, 2, 32)                 # [block, half, byte group (j & 1), l]
    high = rec[:, 128:192].reshape(n, 2, 1, 32)              # [block, half, -, l]
    code = np.empty((n, 2, 4, 32), np.uint8)                 # [block, half, j, l]
    for j in range(4):
        low = (nib[:, :, j & 1, :] & 0x0F) if j < 2 else (nib[:, :, j & 1, :] >> 4)
        code[:, :, j, :] = low | (((high[:, :, 0, :] >> (2 * j)) & 3) << 4)
    q = (code.reshape(n, 256).astype(np.int16) - 32).astype(np.int8)
    sc = np.ascontiguousarray(rec[:, 192:208]).view(np.int8)
    d = np.ascontiguousarray(rec[:, 208:210]).view(np.float16).reshape(-1)
    return q, sc, d


def q6_k_dequant(b: np.ndarray) -> np.ndarray:
    """Raw Q6_K bytes -> float32 weights [nblk * 256]: d * sc[w // 16] * q[w], evaluated in float32 as (d * sc) * q."""
    q, sc, d = q6_k_values(b)
    scale = d.astype(np.float32)[:, None] * sc.astype(np.float32)            # [nblk, 16]
    return (np.repeat(scale, 16, axis=1) * q.astype(np.float32)).reshape(-1)


def _q6_hi_shift(i: int) -> int:
    """Bit position of the two high bits of weight i (0..15) inside its word of the Hb plane: byte (i % 8) // 2, slot
    (i % 2) + 2 * (i // 8).  With that order ((Hb << 4) & 0x30303030), ((Hb << 2) & ...), (Hb & ...), ((Hb >> 2) & ...)
    are the high bits of weights (0,2,4,6), (1,3,5,7), (8,10,12,14), (9,11,13,15) already sitting at bits 4-5 of the
    bytes that the low-nibble words give for the same weights, so four 6-bit codes cost three instructions."""
    return 8 * ((i % 8) // 2) + 2 * ((i % 2) + 2 * (i // 8))


def q6_k_planes(b: np.ndarray, n_rows: int, k: int):
    """Raw Q6_K bytes of an [n_rows, k] matrix -> the device planes of the Q6_K head kernel: L int32 [N, K/8] (low
    nibbles of q + 32, nibble i of word w = weight 8w+i, as the reference's plane, scripts/qwen_gguf.py:92-104), Hb int32
    [N, K/16] (high two bits of the 16 weights of a sub-block, at the bit positions of `_q6_hi_shift`; the reference uses
    field i = weight i), SC int8 [N, K/16], D fp16 [N, K/256].  Same 6.5625 bits per weight as the file."""
    if k % 256:
        raise ValueError("K must be a multiple of the 256-weight Q6_K block")
    q, sc, d = q6_k_values(b)
    code = (q.astype(np.int16) + 32).reshape(n_rows, k).astype(np.uint32)            # 0..63
    lo = np.zeros((n_rows, k // 8), np.uint32)
    for i in range(8):
        lo |= (code[:, i::8] & 15) << np.uint32(4 * i)
    hi = np.zeros((n_rows, k // 16), np.uint32)
    for i in range(16):
        hi |= (code[:, i::16] >> 4) << np.uint32(_q6_hi_shift(i))
    return (lo.view(np.int32), hi.view(np.int32), np.ascontiguousarray(sc.reshape(n_rows, k // 16)),
            np.ascontiguousarray(d.reshape(n_rows, k // 256)))


def q6_k_planes_dense(L, Hb, SC, D, dtype=np.float64) -> np.ndarray:
    """The planes back to dense weights (d * sc) * (q - 32), the fp32 scale product formed first as in the kernel and in
    the reference's `q6_k_blocks` (lab/gguf.py:95-113).  -> [N, K]."""
    L, Hb = np.asarray(L).view(np.uint32), np.asarray(Hb).view(np.uint32)
    n, k = L.shape[0], L.shape[1] * 8
    code = np.zeros((n, k), np.int32)
    for i in range(8):
        code[:, i::8] = (L >> np.uint32(4 * i)) & 15
    for i in range(16):
        code[:, i::16] |= ((Hb >> np.uint32(_q6_hi_shift(i))) & 3).astype(np.int32) << 4
    scale = np.repeat(np.asarray(D, np.float32), 16, axis=1) * np.asarray(SC, np.float32)   # [N, K/16], fp32 product
    return (np.repeat(scale, 16, axis=1).astype(dtype) * (code - 32).astype(dtype))


def q4_0_encode(q: np.ndarray, d: np.ndarray) -> np.ndarray:
    """Inverse of `q4_0_blocks`: q uint8 [..., 32] in weight order (0..15), d fp16 [...] -> uint8 bytes [nblk * 18]."""
    q = np.asarray(q, np.uint8).reshape(-1, 32)
    d = np.asarray(d, np.float16).reshape(-1)
    rec = np.empty((q.shape[0], 18), np.uint8)
    rec[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    rec[:, 2:18] = (q[:, :16] & 0x0F) | (q[:, 16:] << 4)
    return rec.reshape(-1)


def q4_rows(g: GGUF, name: str):
    """-> (q uint8 [N, K] with values 0..15, d fp16 [N, K/32]) for a Q4_0 tensor (scripts/qwen_gguf.py:44-51)."""
    b, t = g.raw(name)
    if GGML_TYPES[t.type][0] != "Q4_0":
        raise ValueError(f"{name} is not Q4_0")
    K, N = t.dims
    _, q = q4_0_blocks(b)
    d16 = np.ascontiguousarray(np.ascontiguousarray(b).reshape(-1, 18)[:, 0:2]).view(np.float16).reshape(N, K // 32)
    return q.reshape(N, K), d16


def pack_nibbles(q: np.ndarray) -> np.ndarray:
    """q uint8 [N, K] (0..15) -> W int32 [N, K/8]: nibble i of word w = weight 8w + i (scripts/qwen_gguf.py:54-60)."""
    N, K = q.shape
    if K % 32:
        raise ValueError("K must be a multiple of the 32-weight block")
    lanes = q.reshape(N, K // 8, 8).astype(np.uint32)
    words = np.zeros((N, K // 8), np.uint32)
    for i in range(8):
        words |= lanes[:, :, i] << np.uint32(4 * i)
    return words.view(np.int32)


def unpack_nibbles(W: np.ndarray) -> np.ndarray:
    """W int32 [N, K/8] -> q uint8 [N, K] (0..15); inverse of `pack_nibbles`."""
    words = np.ascontiguousarray(W).view(np.uint32)
    N, KW = words.shape
    q = np.empty((N, KW, 8), np.uint8)
    for i in range(8):
        q[:, :, i] = (words >> np.uint32(4 * i)) & np.uint32(15)
    return q.reshape(N, KW * 8)


def write_gguf(path, meta: dict, tensors: dict, alignment: int = 32) -> None:
    """Write a minimal GGUF v3 file (used by the tests and by tools that export synthetic models).

    `meta`: key -> int / float / str / bool / list of those.  `tensors`: name -> (ggml_type, dims_ggml_order, bytes)."""
    def enc_str(s):
        raw = s.encode("utf-8")
        return struct.pack("<Q", len(raw)) + raw

    def enc_val(v):
        if isinstance(v, bool):
            return 7, struct.pack("<?", v)
        if isinstance(v, int):
            return (4, struct.pack("<I", v)) if 0 <= v < 2 ** 32 else (11, struct.pack("<q", v))
        if isinstance(v, float):
            return 6, struct.pack("<f", v)
        if isinstance(v, str):
            return _T_STRING, enc_str(v)
        if isinstance(v, (list, tuple)):
            if not v:
                return _T_ARRAY, struct.pack("<IQ", 4, 0)
            et, _ = enc_val(v[0])
            return _T_ARRAY, struct.pack("<IQ", et, len(v)) + b"".join(enc_val(x)[1] for x in v)
        raise TypeError(type(v))

    meta = dict(meta)
    meta.setdefault("general.alignment", alignment)
    head = struct.pack("<4sIQQ", b"GGUF", 3, len(tensors), len(meta))
    for k, v in meta.items():
        t, payload = enc_val(v)
        head += enc_str(k) + struct.pack("<I", t) + payload
    offset, blobs = 0, []
    for name, (ttype, dims, data) in tensors.items():
        data = bytes(data)
        head += enc_str(name) + struct.pack("<I", len(dims)) + struct.pack(f"<{len(dims)}Q", *dims)
        head += struct.pack("<IQ", ttype, offset)
        pad = -len(data) % alignment
        blobs.append(data + b"\0" * pad)
        offset += len(data) + pad
    head += b"\0" * (-len(head) % alignment)
    Path(path).write_bytes(head + b"".join(blobs))
