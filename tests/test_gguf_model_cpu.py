"""GGUF model files: export -> load round trip of a synthetic Qwen2-architecture model (no GPU needed).

Mirrors what the reference's GGUFQwen constructor does with a file (scripts/qwen_gguf.py:63-91): QKV concatenation,
gate/up row interleave, canonical nibble packing."""
import dataclasses
import importlib

import numpy as np
import pytest

from conftest import pkg


def _same_cfg(a, b):
    da, db = dataclasses.asdict(a), dataclasses.asdict(b)
    for k in da:
        if isinstance(da[k], float):
            assert da[k] == pytest.approx(db[k], rel=1e-6), k      # GGUF stores eps and theta as float32
        elif k != "name":
            assert da[k] == db[k], k


@pytest.mark.parametrize("tied", [True, False])
def test_export_load_round_trip(tmp_path, tied):
    synth, qg = pkg("synth"), pkg("qwen_gguf")
    cfg = synth.ModelConfig("tiny-rt", 2, 256, 512, 4, 2, 64, 1024, tied_fp16_head=tied)
    model = synth.synth_model(cfg, 11)
    path = tmp_path / "model.gguf"
    qg.export_model(model, path)
    back = qg.load_model(path)
    _same_cfg(cfg, back["cfg"])
    assert np.array_equal(model["embed"], back["embed"]) and np.array_equal(model["norm"], back["norm"])
    for a, b in zip(model["layers"], back["layers"]):
        for k in ("ln1", "ln2", "qkv_b"):
            assert np.array_equal(a[k], b[k]), k
        for k in ("qkv", "o", "gu", "down"):
            assert np.array_equal(a[k][0], b[k][0]) and np.array_equal(a[k][1], b[k][1]), k
    if tied:
        assert back["head"] is None
    else:
        assert np.array_equal(model["head"][0], back["head"][0]) and np.array_equal(model["head"][1], back["head"][1])


def test_file_uses_llama_cpp_names_and_row_order(tmp_path):
    synth, qg, G = pkg("synth"), pkg("qwen_gguf"), pkg("gguf")
    cfg = synth.TINY
    model = synth.synth_model(cfg, 2)
    path = tmp_path / "model.gguf"
    qg.export_model(model, path)
    g = G.GGUF(path)
    assert g.meta["general.architecture"] == "qwen2" and g.meta["qwen2.block_count"] == cfg.layers
    for name in ("token_embd.weight", "output_norm.weight", "blk.0.attn_q.weight", "blk.0.attn_k.bias", "blk.1.ffn_gate.weight",
                 "blk.1.ffn_up.weight", "blk.1.ffn_down.weight", "blk.0.attn_output.weight", "blk.0.attn_norm.weight"):
        assert name in g.tensors, name
    assert g.tensors["blk.0.attn_q.weight"].dims == (cfg.hidden, cfg.q_rows)        # ggml order: K first
    assert g.tensors["blk.0.ffn_down.weight"].dims == (cfg.ffn, cfg.hidden)
    # gate rows are the even rows of the interleaved gate/up matrix, k rows follow the q rows of QKV
    q_gate, d_gate = G.q4_rows(g, "blk.0.ffn_gate.weight")
    W, S = model["layers"][0]["gu"]
    assert np.array_equal(G.pack_nibbles(q_gate), W[0::2]) and np.array_equal(d_gate, S[0::2])
    q_k, _ = G.q4_rows(g, "blk.0.attn_k.weight")
    assert np.array_equal(G.pack_nibbles(q_k), model["layers"][0]["qkv"][0][cfg.q_rows:cfg.q_rows + cfg.kv_rows])


def test_q6_k_tensors_load_as_fp16_tables(tmp_path):
    """A file whose embedding and head are Q6_K (the layout of llama.cpp's Q4_0 exports) loads: both become fp16 tables,
    the head an untied one; an unsupported type is refused by name."""
    synth, qg, G = pkg("synth"), pkg("qwen_gguf"), pkg("gguf")
    cfg = synth.TINY
    model = synth.synth_model(cfg, 2)
    path = tmp_path / "model.gguf"
    qg.export_model(model, path)
    g = G.GGUF(path)
    tensors = {n: (t.type, t.dims, bytes(g.raw(n)[0])) for n, t in g.tensors.items()}
    rng = np.random.default_rng(9)
    nblk = cfg.vocab * cfg.hidden // 256

    def q6(seed):
        raw = np.random.default_rng(seed).integers(0, 256, size=(nblk, 210), dtype=np.uint8)
        raw[:, 208:210] = rng.uniform(1e-4, 1e-3, nblk).astype(np.float16).view(np.uint8).reshape(-1, 2)
        return raw.reshape(-1)

    emb_raw, head_raw = q6(1), q6(2)
    tensors["token_embd.weight"] = (14, (cfg.hidden, cfg.vocab), emb_raw.tobytes())
    tensors["output.weight"] = (14, (cfg.hidden, cfg.vocab), head_raw.tobytes())
    G.write_gguf(tmp_path / "q6.gguf", dict(g.meta), tensors)
    back = qg.load_model(tmp_path / "q6.gguf")
    assert back["head"] is None and back["head16"].dtype == np.float16 and back["head16"].shape == (cfg.vocab, cfg.hidden)
    assert np.array_equal(back["embed"], G.q6_k_dequant(emb_raw).reshape(cfg.vocab, cfg.hidden).astype(np.float16))
    assert np.array_equal(back["head16"], G.q6_k_dequant(head_raw).reshape(cfg.vocab, cfg.hidden).astype(np.float16))
    tensors["output.weight"] = (8, (cfg.hidden, cfg.vocab), bytes(cfg.vocab * cfg.hidden // 32 * 34))     # Q8_0: not supported
    G.write_gguf(tmp_path / "q8.gguf", dict(g.meta), tensors)
    with pytest.raises(NotImplementedError, match="ggml type 8"):
        qg.load_model(tmp_path / "q8.gguf")


def test_q6_k_planes_round_trip_against_reference_vectors(golden):
    """The device planes of the Q6_K head (low-nibble, high-two-bit, scale planes) rebuild exactly the weights that the
    reference's own Q6_K decode gives for the golden blocks (fixture made by lab.gguf.q6_k_blocks)."""
    G = pkg("gguf")
    g = golden["q6_k_codec"]
    raw = g["raw"]                                              # 40 blocks = 40 x 256 weights
    L, Hb, SC, D = G.q6_k_planes(raw, 20, 512)
    assert L.shape == (20, 64) and Hb.shape == (20, 32) and SC.shape == (20, 32) and D.shape == (20, 2)
    dense = G.q6_k_planes_dense(L, Hb, SC, D, np.float32)
    assert np.array_equal(dense.reshape(-1), g["f32"])
    with pytest.raises(ValueError):
        G.q6_k_planes(raw[:210 * 3], 1, 3 * 256 + 128)          # K not a multiple of the 256-weight block


def test_q6_k_head_is_kept_at_six_bits_by_the_loader(tmp_path):
    synth, qg, G = pkg("synth"), pkg("qwen_gguf"), pkg("gguf")
    cfg = synth.ModelConfig("q6head", 1, 512, 512, 4, 2, 128, 1024)
    model = synth.synth_model(cfg, 2)
    path = tmp_path / "m.gguf"
    qg.export_model(model, path)
    g = G.GGUF(path)
    tensors = {n: (t.type, t.dims, bytes(g.raw(n)[0])) for n, t in g.tensors.items()}
    rng = np.random.default_rng(4)
    nblk = cfg.vocab * cfg.hidden // 256
    raw = rng.integers(0, 256, size=(nblk, 210), dtype=np.uint8)
    raw[:, 208:210] = rng.uniform(1e-4, 1e-3, nblk).astype(np.float16).view(np.uint8).reshape(-1, 2)
    tensors["output.weight"] = (14, (cfg.hidden, cfg.vocab), raw.tobytes())
    G.write_gguf(tmp_path / "q6.gguf", dict(g.meta), tensors)
    back = qg.load_model(tmp_path / "q6.gguf")
    assert back["head"] is None and back["head_q6"] is not None
    dense = G.q6_k_planes_dense(*back["head_q6"], np.float32)
    assert np.array_equal(dense.reshape(-1), G.q6_k_dequant(raw.reshape(-1)))
    assert np.array_equal(back["head16"], dense.astype(np.float16))
