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
