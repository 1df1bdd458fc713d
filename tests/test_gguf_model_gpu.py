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
