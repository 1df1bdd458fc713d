"""End-to-end parity of the batch-1 decode engine with the oracle on small models of the Qwen2.5 architecture:
identical greedy tokens over 64 steps, logits within 1e-3 of the largest logit, KV cache equal up to fp16 rounding."""
import numpy as np
import pytest

from conftest import oracle, pkg

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def build(cfg_name, seed, max_len, tensor_core=True):
    s = pkg("synth")
    cfg = s.CONFIGS[cfg_name]
    model = s.synth_model(cfg, seed)
    eng = pkg("engine").FusedQwen(model, max_len=max_len, tensor_core=tensor_core)
    cos, sin = s.rope_tables(cfg, max_len)
    orc = oracle().Oracle(model, max_len, cos, sin)
    return s, cfg, model, eng, orc


@pytest.mark.parametrize("tensor_core", [True, False])
@pytest.mark.parametrize("cfg_name,seed", [("tiny", 0), ("small", 1)])
def test_greedy_tokens_match_oracle_64_steps(cfg_name, seed, tensor_core):
    s, cfg, model, eng, orc = build(cfg_name, seed, 128, tensor_core)
    prompt = s.synth_prompt(cfg, 24, seed)
    want = orc.greedy(prompt, 64)
    E = pkg("engine")
    got, _ = E.run_fused(eng, prompt, 64)
    assert got == want


def test_step_logits_and_cache_match_oracle():
    s, cfg, model, eng, orc = build("small", 3, 64)
    prompt = s.synth_prompt(cfg, 20, 3)
    for t in prompt:
        orc.tok[:] = t
        orc.step()
        eng.tok.fill_(int(t))
        eng.step()
        lg = eng.logits.cpu().numpy()
        ref = orc.logits[0]
        assert np.max(np.abs(lg - ref)) / np.max(np.abs(ref)) < 1e-3
        assert int(eng.tok.item()) == int(orc.tok[0])
    assert int(eng.pos.item()) == len(prompt)
    n = len(prompt)
    kc = eng.kc[:, :, :n].float().cpu().numpy()
    vc = eng.vc[:, :, :n].float().cpu().numpy()
    kr = orc.kc[:, 0, :, :n].astype(np.float32)
    vr = orc.vc[:, 0, :, :n].astype(np.float32)
    assert np.max(np.abs(kc - kr)) / np.max(np.abs(kr)) < 2e-3
    assert np.max(np.abs(vc - vr)) / np.max(np.abs(vr)) < 2e-3


def test_one_call_step_equals_per_op_step():
    """q4b_decode_step and the per-op entry points run the same kernels: bit-identical state."""
    s, cfg, model, eng, _ = build("tiny", 5, 64)
    eng2 = pkg("engine").FusedQwen(model, max_len=64)
    assert eng.tensor_core and eng2.tensor_core
    for t in s.synth_prompt(cfg, 10, 5):
        eng.tok.fill_(int(t))
        eng2.tok.fill_(int(t))
        eng.step()
        eng2.step_ops()
    assert torch.equal(eng.logits, eng2.logits) and torch.equal(eng.kc, eng2.kc) and torch.equal(eng.h, eng2.h)
    assert torch.equal(eng.tok, eng2.tok) and torch.equal(eng.pos, eng2.pos)
    eng.check_status()
    eng2.check_status()


def test_graph_replay_equals_eager():
    s, cfg, model, eng, _ = build("tiny", 6, 64)
    prompt = s.synth_prompt(cfg, 8, 6)
    E = pkg("engine")
    toks, _ = E.run_fused(eng, prompt, 16)
    eng.reset()
    eng.feed(prompt)
    eager = [int(eng.tok.item())]
    for _ in range(15):
        eng.step()
        eager.append(int(eng.tok.item()))
    assert toks == eager


def test_qwen15_shape_single_layer_step():
    """Full Qwen2.5-1.5B layer shapes (one layer, reduced vocabulary) for one token at a late position."""
    s = pkg("synth")
    cfg = s.ModelConfig("q15-1layer", 1, 1536, 8960, 12, 2, 128, 8192)
    model = s.synth_model(cfg, 9)
    eng = pkg("engine").FusedQwen(model, max_len=1024)
    cos, sin = s.rope_tables(cfg, 1024)
    orc = oracle().Oracle(model, 1024, cos, sin)
    rng = np.random.default_rng(9)
    kc = rng.standard_normal(orc.kc.shape).astype(np.float16)
    vc = rng.standard_normal(orc.vc.shape).astype(np.float16)
    orc.kc[:], orc.vc[:] = kc, vc
    eng.kc.copy_(torch.from_numpy(kc[:, 0]))
    eng.vc.copy_(torch.from_numpy(vc[:, 0]))
    for p, t in ((700, 123), (701, 4567)):
        orc.pos[:], orc.tok[:] = p, t
        eng.pos.fill_(p)
        eng.tok.fill_(t)
        orc.step()
        eng.step()
        lg, ref = eng.logits.cpu().numpy(), orc.logits[0]
        assert np.max(np.abs(lg - ref)) / np.max(np.abs(ref)) < 1e-3
        assert int(eng.tok.item()) == int(orc.tok[0])


def test_full_qwen15_shape_greedy_64_steps_match_oracle():
    """The benchmark configuration itself: 28 layers, hidden 1536, FFN 8960, 12/2 heads, vocabulary 151 936 with the tied
    fp16 head, the layer kernels at their real grid geometry (split-K over clusters, the 148-CTA head).  A short prompt,
    then 64 greedy tokens by graph replay: identical to the oracle's.  With random weights a greedy sequence soon settles
    on one token, so the same state is then driven for 32 more steps with random input tokens (teacher forcing): at every
    step the greedy pick must equal the oracle's and the logits agree within 1e-3 of the largest.  The oracle keeps its
    dense matrices in float32 here (6 GB instead of 12; ~1e-7 per linear)."""
    s, E = pkg("synth"), pkg("engine")
    cfg = s.QWEN25_1P5B
    model = s.synth_model(cfg, 0)
    eng = E.FusedQwen(model, max_len=128)
    cos, sin = s.rope_tables(cfg, 128)
    orc = oracle().Oracle(model, 128, cos, sin, dense_dtype=np.float32)
    prompt = s.synth_prompt(cfg, 8, 0)
    want = orc.greedy(prompt, 64)
    got, _ = E.run_fused(eng, prompt, 64)
    assert got == want
    eng.check_status()
    # run_fused's second (timed) pass replays 64 steps from the end of the prompt, one more than the 63 that produced
    # the tokens: the oracle takes that step too, then both are at the same position with the same cache
    orc.step()
    assert int(eng.pos.item()) == int(orc.pos[0]) and int(eng.tok.item()) == int(orc.tok[0])
    worst = 0.0
    for t in s.synth_prompt(cfg, 32, 11):
        orc.tok[:] = t
        orc.step()
        eng.tok.fill_(int(t))
        eng.step()
        lg, ref = eng.logits.cpu().numpy(), orc.logits[0]
        worst = max(worst, float(np.max(np.abs(lg - ref)) / np.max(np.abs(ref))))
        assert int(eng.tok.item()) == int(orc.tok[0])
    assert worst < 1e-3
    eng.check_status()
