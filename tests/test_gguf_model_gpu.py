"""A model loaded from a GGUF file decodes exactly like the model it was exported from."""
import pytest
import torch

from conftest import pkg

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tied", [True, False])
def test_gguf_qwen_decodes_like_the_source_model(tmp_path, tied):
    synth, qg, engine = pkg("synth"), pkg("qwen_gguf"), pkg("engine")
    cfg = synth.ModelConfig("small-gguf", 2, 512, 1536, 4, 2, 128, 4096, tied_fp16_head=tied)
    model = synth.synth_model(cfg, 4)
    path = tmp_path / "small.gguf"
    qg.export_model(model, path)
    a = engine.FusedQwen(model, max_len=128)
    b = qg.GGUFQwen(path, max_len=128)
    ids = synth.synth_prompt(cfg, 24, 3)
    for t in ids:
        for m in (a, b):
            m.tok.fill_(int(t))
            m.step()
        torch.cuda.synchronize()
        assert int(a.tok.item()) == int(b.tok.item())
        # weights are bit-identical; eps went through float32 in the file
        assert torch.allclose(a.h, b.h, rtol=1e-5, atol=1e-5 * a.h.abs().max().item())
    a.check_status()
    b.check_status()


def test_untied_fp16_head_from_gguf(tmp_path):
    """`output.weight` kept as an fp16 table (what a Q6_K / F16 head of a file becomes): logits = head16 . x."""
    import numpy as np
    synth, qg = pkg("synth"), pkg("qwen_gguf")
    cfg = synth.ModelConfig("small-head16", 2, 512, 1536, 4, 2, 128, 4096)
    model = synth.synth_model(cfg, 6)
    model["head16"] = (0.05 * np.random.default_rng(3).standard_normal((cfg.vocab, cfg.hidden))).astype(np.float16)
    path = tmp_path / "h16.gguf"
    qg.export_model(model, path)
    m = qg.GGUFQwen(path, max_len=64)
    assert m.head16 is not m.embed
    for t in synth.synth_prompt(cfg, 6, 1):
        m.tok.fill_(int(t))
        m.step()
    torch.cuda.synchronize()
    want = m.head16.float() @ m.x.float()
    assert torch.allclose(m.logits, want, rtol=1e-4, atol=1e-4 * want.abs().max().item())
    assert int(m.tok.item()) == int(want.argmax().item())


def _q6_raw(rng, n_rows, k):
    import numpy as np
    nblk = n_rows * k // 256
    raw = rng.integers(0, 256, size=(nblk, 210), dtype=np.uint8)
    raw[:, 208:210] = rng.uniform(1e-4, 1e-3, nblk).astype(np.float16).view(np.uint8).reshape(-1, 2)
    return raw.reshape(-1)


@pytest.mark.parametrize("V,K", [(1000, 512), (4099, 1536), (33, 2048), (151936, 1536)])
def test_head_q6_k_argmax_matches_dense(V, K):
    """The Q6_K head kernel (6.5625 bits per weight) against the dense weights rebuilt from its planes (which the CPU
    suite pins to the reference's Q6_K decode), fp32 logits within 1e-5 of the largest, lowest-index argmax, twice."""
    import numpy as np
    G, K_ = pkg("gguf"), pkg("qwen_kernels")
    K_.init(0)
    rng = np.random.default_rng(V + K)
    planes = G.q6_k_planes(_q6_raw(rng, V, K), V, K)
    x = rng.standard_normal(K).astype(np.float16)
    if V <= 5000:
        ref = G.q6_k_planes_dense(*planes) @ x.astype(np.float64)
    else:                                                        # the full vocabulary: rows in slabs, float32 is enough
        ref = np.concatenate([G.q6_k_planes_dense(*(p[r:r + 8192] for p in planes), np.float32) @ x.astype(np.float32)
                              for r in range(0, V, 8192)]).astype(np.float64)
    dev = [torch.from_numpy(np.ascontiguousarray(p)).cuda() for p in planes]
    xd = torch.from_numpy(x).cuda()
    logits = torch.full((V,), float("nan"), device="cuda")
    tok = torch.zeros(1, dtype=torch.long, device="cuda")
    pos = torch.full((1,), 5, dtype=torch.long, device="cuda")
    ws = K_.head_workspace(V, 1, "cuda")
    for rep in range(2):
        K_.head_q6_argmax(dev, xd, logits, tok, pos, ws)
        got = logits.cpu().numpy()
        assert np.max(np.abs(got - ref)) / np.max(np.abs(ref)) < (1e-5 if V <= 5000 else 1e-4)
        assert int(tok.item()) == int(np.argmax(got))
        assert int(pos.item()) == 6 + rep


def test_gguf_with_q6_k_head_decodes_through_the_six_bit_kernel(tmp_path):
    """A file whose `output.weight` is Q6_K (the layout of llama.cpp's Q4_0 exports): the batch-1 step runs the head at
    6.5625 bits per weight; greedy tokens and logits against the oracle with the same Q6_K head."""
    import importlib
    import numpy as np
    synth, qg, G = pkg("synth"), pkg("qwen_gguf"), pkg("gguf")
    ora = importlib.import_module("oracle.q4ref")
    cfg = synth.ModelConfig("small-q6", 2, 512, 1536, 4, 2, 128, 4096)
    model = synth.synth_model(cfg, 8)
    path = tmp_path / "m.gguf"
    qg.export_model(model, path)
    g = G.GGUF(path)
    tensors = {n: (t.type, t.dims, bytes(g.raw(n)[0])) for n, t in g.tensors.items()}
    tensors["output.weight"] = (14, (cfg.hidden, cfg.vocab), _q6_raw(np.random.default_rng(1), cfg.vocab, cfg.hidden).tobytes())
    G.write_gguf(tmp_path / "q6.gguf", dict(g.meta), tensors)
    loaded = qg.load_model(tmp_path / "q6.gguf")
    m = pkg("engine").FusedQwen(loaded, max_len=64)
    assert m.head_q6 is not None
    cos, sin = synth.rope_tables(cfg, 64)
    o = ora.Oracle(loaded, 64, cos, sin)
    dense = G.q6_k_planes_dense(*loaded["head_q6"])
    for t in synth.synth_prompt(cfg, 12, 2):
        o.tok[:] = t
        o.step()
        m.tok.fill_(int(t))
        m.step()
        lg, ref = m.logits.cpu().numpy(), o.logits[0]
        # the head itself: exact against the dense Q6_K weights applied to the engine's own activation vector
        own = dense @ m.x.float().cpu().numpy().astype(np.float64)
        assert np.max(np.abs(lg - own)) / np.max(np.abs(own)) < 1e-5
        # against the oracle the residual stream carries the usual 16-bit rounding flips of the layers (2e-3 at most here)
        assert np.max(np.abs(lg - ref)) / np.max(np.abs(ref)) < 5e-3
        assert int(m.tok.item()) == int(o.tok[0])
    m.check_status()
