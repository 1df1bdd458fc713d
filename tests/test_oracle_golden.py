"""The oracle and the host-side codec against fixtures produced by the reference's own Python code."""
import numpy as np

from conftest import gemv_inputs, oracle, pkg


def test_q4_0_blocks_matches_reference(golden):
    g = golden["q4_0_codec"]
    for impl in (oracle().q4_0_blocks, pkg("gguf").q4_0_blocks):
        d, q = impl(g["raw"])
        assert d.dtype == np.float32 and q.dtype == np.uint8
        np.testing.assert_array_equal(d, g["d"])
        np.testing.assert_array_equal(q, g["q"])
        deq = (d[:, None] * (q.astype(np.float32) - 8)).reshape(-1)
        np.testing.assert_array_equal(deq, g["f32"])


def test_q4_0_encode_round_trip(golden):
    gg = pkg("gguf")
    g = golden["q4_0_codec"]
    d16 = g["raw"].reshape(-1, 18)[:, :2].copy().view(np.float16).reshape(-1)
    np.testing.assert_array_equal(gg.q4_0_encode(g["q"], d16), g["raw"])


def test_gguf_reader_matches_reference(golden, tmp_path):
    gg = pkg("gguf")
    g = golden["gguf_file"]
    path = tmp_path / "tiny.gguf"
    path.write_bytes(g["blob"].tobytes())
    f = gg.GGUF(path)
    assert f.data_start == int(g["data_start"])
    assert sorted(f.meta) == list(g["meta_keys"])
    assert f.meta["qwen2.block_count"] == int(g["meta_block_count"])
    assert abs(f.meta["qwen2.rope.freq_base"] - float(g["meta_freq_base"])) == 0
    assert f.meta["tokens"] == list(g["meta_tokens"])
    assert list(f.tensors) == list(g["names"])
    assert tuple(f.tensors["blk.0.attn_q.weight"].dims) == tuple(g["dims_q"])
    np.testing.assert_array_equal(f.f32("blk.0.attn_q.weight"), g["q_f32"])
    np.testing.assert_array_equal(f.f32("token_embd.weight"), g["e_f32"])
    np.testing.assert_array_equal(f.f32("output_norm.weight"), g["n_f32"])
    q, d = gg.q4_rows(f, "blk.0.attn_q.weight")
    W = gg.pack_nibbles(q)
    np.testing.assert_array_equal(gg.unpack_nibbles(W), q)
    np.testing.assert_array_equal(oracle().dequant(W, d, np.float32), g["q_f32"])


def test_gguf_rejects_bad_magic(tmp_path):
    import pytest
    p = tmp_path / "bad.gguf"
    p.write_bytes(b"GGML" + b"\0" * 64)
    with pytest.raises(ValueError):
        pkg("gguf").GGUF(p)


def test_gemv_oracle_small_matches_reference(golden):
    g = golden["gemv_small"]
    q, d, x = gemv_inputs(int(g["n"]), int(g["k"]), bool(g["bf16_x"]))
    np.testing.assert_array_equal(q, g["q"])
    np.testing.assert_array_equal(d, g["d"])
    np.testing.assert_array_equal(x, g["x"])
    W = pkg("gguf").pack_nibbles(q)
    o = oracle()
    np.testing.assert_array_equal(o.gemv_ref(W, d, x), g["y_ref_f64"])
    y32 = o.gemv_numpy_f32(W, d, x)
    assert np.max(np.abs(y32 - g["y_ref_f32"])) <= 1e-5 * np.max(np.abs(g["y_ref_f32"]))


def test_gemv_oracle_ffn_up_matches_reference(golden):
    """The 8960 x 1536 ffn_up GEMV of the first benchmark configuration."""
    g = golden["gemv_ffn_up"]
    q, d, x = gemv_inputs(8960, 1536, False)
    W = pkg("gguf").pack_nibbles(q)
    o = oracle()
    y = o.gemv_ref(W, d, x)
    np.testing.assert_allclose(y, g["y_ref_f64"], rtol=0, atol=1e-12)
    scale = np.max(np.abs(g["y_ref_f64"]))
    assert np.max(np.abs(g["y_ref_f32"] - y)) / scale < 1e-5          # the reference's fp32 numpy path vs float64


def test_quant_q8_1_properties():
    o = oracle()
    rng = np.random.default_rng(3)
    x = rng.standard_normal((5, 256)).astype(np.float16)
    x[1, 32:64] = 0                                    # an all-zero block: d = 0, q = 0
    x[2, 0] = 60000.0                                  # near the fp16 maximum
    q, d, s = o.quant_q8_1(x)
    assert q.dtype == np.int8 and d.dtype == np.float16 and s.dtype == np.int32
    assert np.all(np.abs(q.astype(int)) <= 127)
    assert np.all(q[1, 32:64] == 0) and d[1, 1] == 0
    np.testing.assert_array_equal(s, q.reshape(5, 8, 32).astype(np.int32).sum(-1))
    amax = np.abs(x.astype(np.float32)).reshape(5, 8, 32).max(-1)
    # the block maximum quantises to +-127 exactly
    hit = np.abs(q.reshape(5, 8, 32).astype(int)).max(-1)
    assert np.all(hit[amax > 0] == 127)
    recon = q.reshape(5, 8, 32) * (amax / np.float32(127))[..., None]
    assert np.max(np.abs(recon - x.astype(np.float32).reshape(5, 8, 32))) <= 0.5 * np.max(amax / 127) * 1.0001


def test_blockdot_and_mmq_consistent():
    o = oracle()
    rng = np.random.default_rng(4)
    M, K, P = 24, 128, 5
    W = rng.integers(0, 2 ** 32, size=(M, K // 8), dtype=np.uint32).view(np.int32)
    S = rng.uniform(0.002, 0.02, size=(M, K // 32)).astype(np.float16)
    x = rng.standard_normal((P, K)).astype(np.float16)
    xq, xd, _ = o.quant_q8_1(x)
    dots = o.blockdot(W, xq)
    q4 = o.unpack_words(W) - 8
    slow = np.zeros((P, M, K // 32), np.int64)
    for p in range(P):
        for m in range(M):
            for b in range(K // 32):
                slow[p, m, b] = int(np.dot(q4[m, 32 * b:32 * b + 32], xq[p, 32 * b:32 * b + 32].astype(np.int64)))
    np.testing.assert_array_equal(dots, slow)
    y = o.mmq(W, S, xq, xd)
    y2 = np.einsum("pmb,mb,pb->pm", dots.astype(np.float64), S.astype(np.float64), xd.astype(np.float64))
    np.testing.assert_allclose(y, y2, rtol=1e-12, atol=1e-12)
    # int8 activations cost about half a percent against the fp16-activation GEMV
    yf = x.astype(np.float64) @ o.dequant(W, S).T
    assert np.max(np.abs(y - yf)) / np.max(np.abs(yf)) < 2e-2


def test_q6_k_codec_matches_reference_vectors(golden):
    """Q6_K block decode against vectors made with the reference's q6_k_parts / GGUF.f32 (lab/gguf.py:80-82, 95-123)."""
    G = pkg("gguf")
    z = golden["q6_k_codec"]
    q, sc, d = G.q6_k_values(z["raw"])
    assert np.array_equal(q, z["q"]) and np.array_equal(sc, z["sc"])
    assert np.array_equal(d.view(np.uint16), z["d"].view(np.uint16))
    assert np.array_equal(G.q6_k_dequant(z["raw"]), z["f32"])
    assert q.min() >= -32 and q.max() <= 31


def test_rope_tables_match_the_reference_statement(golden):
    """cos / sin rows against the reference's own table statement (scripts/qwen_gguf.py:111-113) executed with torch:
    float64 angles, rounded to fp32.  numpy's and torch's double cos / sin may differ in the last double bit, which can
    move the fp32 rounding by one unit on rare entries, never more."""
    g = golden["rope_tables"]
    s = pkg("synth")
    cfg = s.ModelConfig("t", 1, 128, 64, 1, 1, int(g["head_dim"]), 16, rope_theta=float(g["theta"]))
    cos, sin = s.rope_tables(cfg, 4096)
    pos = g["positions"]
    for got, want in ((cos[pos], g["cos"]), (sin[pos], g["sin"])):
        ulp = np.abs(got.view(np.int32).astype(np.int64) - want.view(np.int32).astype(np.int64))
        assert ulp.max() <= 1 and (ulp > 0).mean() < 1e-3
    assert np.array_equal(cos[0], np.ones(64, np.float32)) and np.array_equal(sin[0], np.zeros(64, np.float32))


def test_blockdot_oracle_on_the_reference_known_answer_inputs(golden):
    """The seeded int8 operands of the reference's tensor-core known-answer check (lab/experiments/tensor.py:171-179,
    exact equality demanded there).  The fixture's expected product pins the operands; the Q4_0 block dot takes the low
    nibble of A8 as the weight (value nibble - 8), one 32-wide block per row."""
    o = oracle()
    g = golden["tensor_s8_known_answer"]
    A8, B8, C8 = g["A8"].astype(np.int32), g["B8"].astype(np.int32), g["C8"]
    assert np.array_equal(g["ref8"], A8 @ B8 + C8)
    nib = (A8 & 15).astype(np.uint8)                                # [16 rows, 32]
    W = pkg("gguf").pack_nibbles(nib)                               # canonical words [16, 4]
    got = o.blockdot(W, np.ascontiguousarray(g["B8"].T))            # xq [8 columns, 32] -> [8, 16, 1]
    assert np.array_equal(got[:, :, 0].T, (nib.astype(np.int32) - 8) @ B8)


def test_f16_weight_oracle_reads_the_reference_fragment_pack(golden):
    """`dequant_f16w` against the reference's own repack for its batched-decode GEMV: the fragment-ordered words and
    scales `pack_q4_mma` made are read the way gemv_v2_source reads them (lane (g, t), word s, A register j =
    (w >> 4 j) & 0x000F000F, `dq` with the fp16 ops done one by one in numpy float16) and must give, bit for bit, the
    weights the oracle forms from the canonical words."""
    o = oracle()
    g = golden["pack_q4_mma"]
    W, S, Wp, Sp = g["W"], g["S"], g["Wp"].view(np.uint32), g["Sp"]
    N, K = W.shape[0], W.shape[1] * 8
    w16 = np.zeros((N, K), np.float16)
    for tile in range(N // 16):
        for ch in range(K // 64):
            for lane in range(32):
                gg, t = lane >> 2, lane & 3
                for s in range(4):                        # k-step of 16 inside the 64-k chunk; Q4_0 block s // 2
                    word = int(Wp[tile, ch, lane, s])
                    dA, dB = Sp[tile, ch, gg, 2 * (s // 2)], Sp[tile, ch, gg, 2 * (s // 2) + 1]     # rows g, g + 8
                    for j in range(4):
                        h = (word >> (4 * j)) & 0x000F000F
                        pair = np.array([1024 + (h & 15), 1024 + (h >> 16)], np.float16) - np.float16(1032)
                        pair = pair * (dA if j % 2 == 0 else dB)                                  # __hmul2, one rounding
                        row = 16 * tile + gg + (8 if j % 2 else 0)
                        k = 64 * ch + 16 * s + 2 * t + (8 if j >= 2 else 0)
                        w16[row, k:k + 2] = pair
    want = o.dequant_f16w(W, S, np.float64)
    np.testing.assert_array_equal(w16.astype(np.float64), want)
    # and the rounding is real: the exact product differs from it in a good share of the weights
    exact = o.dequant(W, S)
    assert 0.2 < np.mean(exact != want) < 1.0
    assert np.max(np.abs(exact - want) / np.abs(exact).max()) < 2 ** -11


def test_block_dot_oracle_against_the_reference_int8_repack(golden):
    """The reference's int8 MMQ multiplies UNSIGNED nibbles (its `pack_q4_i8` operand) with the int8 activations and plants
    0x4B400000 - 8 sum(x) in the accumulator (QUANT_Q8, lab/qwen_batched.py:1016-1041), so that the result is the bit
    pattern of 2^23 + 2^22 + sum((q - 8) x).  Reading the reference-made operand the way its kernel does (lane (g, t), word
    2 b + h, byte i = row g | row g + 8 << 4 at k = 32 b + 16 h + 4 t + i) and applying that correction must give the
    oracle's signed block dots, and the planted constant must turn them into exact floats."""
    o = oracle()
    g = golden["pack_q4_i8"]
    W, Wp, Sp, S = g["W"], g["Wp"].view(np.uint32), g["Sp"], g["S"]
    N, K = W.shape[0], W.shape[1] * 8
    q = np.zeros((N, K), np.int64)
    for tile in range(N // 16):
        for ch in range(K // 64):
            for lane in range(32):
                gg, t = lane >> 2, lane & 3
                for b in range(2):
                    for h in range(2):
                        word = int(Wp[tile, ch, lane, 2 * b + h])
                        for i in range(4):
                            k = 64 * ch + 32 * b + 16 * h + 4 * t + i
                            byte = (word >> (8 * i)) & 0xFF
                            q[16 * tile + gg, k] = byte & 15
                            q[16 * tile + gg + 8, k] = byte >> 4
    np.testing.assert_array_equal(q, o.unpack_words(W))
    # scales: [tile][chunk][g][4] = (row g blk 0, row g + 8 blk 0, row g blk 1, row g + 8 blk 1)
    Sv = S.reshape(N // 16, 16, K // 64, 2)
    np.testing.assert_array_equal(Sp[:, :, :, 0], Sv[:, :8, :, 0].transpose(0, 2, 1))
    np.testing.assert_array_equal(Sp[:, :, :, 3], Sv[:, 8:, :, 1].transpose(0, 2, 1))
    rng = np.random.default_rng(3)
    xq = rng.integers(-127, 128, size=(5, K)).astype(np.int8)
    want = o.blockdot(W, xq)                                   # [P, N, K / 32] signed dots
    qb = q.reshape(N, K // 32, 32)
    xb = xq.astype(np.int64).reshape(5, K // 32, 32)
    unsigned = np.einsum("nbk,pbk->pnb", qb, xb)
    planted = 0x4B400000 - 8 * xb.sum(axis=2)                  # per (token, block), as QUANT_Q8 writes it
    acc = (unsigned + planted[:, None, :]).astype(np.int64)
    np.testing.assert_array_equal(acc - 0x4B400000, want)
    as_float = acc.astype(np.uint32).view(np.float32).astype(np.float64) - 12582912.0
    np.testing.assert_array_equal(as_float, want.astype(np.float64))
