"""Prefill: causal flash attention against the oracle, and the whole prefill chunk (int8 MMQ path) against the oracle's
int8-activation forward and against token-by-token decode."""
import numpy as np
import pytest

from conftest import oracle, pkg

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("P,pos0,NH,NKV", [(64, 0, 4, 2), (100, 0, 12, 2), (200, 56, 6, 1), (2048, 0, 2, 1), (1, 300, 4, 4)])
def test_flash_prefill_matches_oracle(P, pos0, NH, NKV):
    o, s, QB = oracle(), pkg("synth"), pkg("qwen_batched")
    pkg("qwen_kernels").init(0)
    HD = 128
    max_len = pos0 + P + 7
    rng = np.random.default_rng(P + pos0 + NH)
    cfg = s.ModelConfig("t", 1, NH * HD, 64, NH, NKV, HD, 100)
    cos, sin = s.rope_tables(cfg, max_len)
    qkv = rng.standard_normal((P, (NH + 2 * NKV) * HD)).astype(np.float16)
    kc = np.zeros((NKV, max_len, HD), np.float16)
    vc = np.zeros_like(kc)
    kc[:, :pos0] = rng.standard_normal((NKV, pos0, HD)).astype(np.float16)
    vc[:, :pos0] = rng.standard_normal((NKV, pos0, HD)).astype(np.float16)
    kcd, vcd = dev(kc), dev(vc)
    out = torch.full((P, NH * HD), float("nan"), dtype=torch.float16, device="cuda")
    scale = 1.0 / np.sqrt(HD)
    QB.attn_prefill(dev(qkv), dev(cos), dev(sin), kcd, vcd, out, NH, NKV, HD, max_len, pos0, scale)
    pos = pos0 + np.arange(P)
    cs, sn = cos[pos][:, None, :], sin[pos][:, None, :]
    q = o.rope_rotate(qkv[:, :NH * HD].reshape(P, NH, HD), cs, sn)
    k = o.rope_rotate(qkv[:, NH * HD:(NH + NKV) * HD].reshape(P, NKV, HD), cs, sn).astype(np.float16)
    v = qkv[:, (NH + NKV) * HD:].reshape(P, NKV, HD)
    kc[:, pos0:pos0 + P] = k.transpose(1, 0, 2)
    vc[:, pos0:pos0 + P] = v.transpose(1, 0, 2)
    ref = o.attn_prefill(q, kc.transpose(1, 0, 2), vc.transpose(1, 0, 2), scale, pos0).reshape(P, -1)
    got = out.float().cpu().numpy()
    assert not np.isnan(got).any()
    err = np.max(np.abs(got - ref)) / np.max(np.abs(ref))
    assert err < 2e-3, err                                           # fp16 probabilities; the reference reports ~2e-3 with bf16
    assert np.array_equal(vcd.cpu().numpy(), vc)
    dk = np.abs(kcd.cpu().numpy().view(np.int16).astype(np.int32) - kc.view(np.int16).astype(np.int32))
    assert dk.max() <= 1


def _prefill_pair(layers, seed, n=160):
    s, E = pkg("synth"), pkg("engine")
    cfg = s.ModelConfig("small128", layers, 512, 1536, 4, 2, 128, 4096)
    model = s.synth_model(cfg, seed)
    m = E.FusedQwen(model, max_len=256)
    ids = s.synth_prompt(cfg, n, seed)
    pf = E.prefill(m, ids)
    cos, sin = s.rope_tables(cfg, 256)
    orc = oracle().Oracle(model, 256, cos, sin)
    h_ref = orc.prefill_q8(ids)
    return s, cfg, model, m, pf, orc, h_ref, ids, (cos, sin)


def test_prefill_one_layer_matches_oracle():
    """One layer: everything but a handful of int8 flips (an activation one fp16 ulp apart lands on the other side of
    a rounding boundary) agrees to fp32 rounding; a flip moves an output by a fraction of a percent."""
    s, cfg, model, m, pf, orc, h_ref, ids, _ = _prefill_pair(1, 2)
    h = pf.h.cpu().numpy()
    rel = np.abs(h - h_ref) / np.max(np.abs(h_ref))
    assert np.median(rel) < 1e-6, np.median(rel)
    assert np.quantile(rel, 0.99) < 5e-3 and rel.max() < 2e-2, (np.quantile(rel, 0.99), rel.max())
    n = len(ids)
    kc, kr = m.kc[:, :, :n].float().cpu().numpy(), orc.kc[:, 0, :, :n].astype(np.float32)
    vc, vr = m.vc[:, :, :n].float().cpu().numpy(), orc.vc[:, 0, :, :n].astype(np.float32)
    assert np.max(np.abs(kc - kr)) / np.max(np.abs(kr)) < 2e-3          # layer 0 K/V: one fp16 ulp at most
    assert np.max(np.abs(vc - vr)) / np.max(np.abs(vr)) < 2e-3


def test_prefill_chunk_matches_oracle_and_decode():
    """Three layers.  int8 activation noise is amplified by the random-weight layers, for the oracle exactly as for the
    kernels: the yardstick is the distance between the oracle's int8-activation forward and its own fp16-activation
    forward.  The kernels must be closer to the int8 oracle than that quantisation noise (the reference checks its
    prefill the same way, against its decode path: K err 6e-3, V err 7e-2, logits 2e-2,
    data/night_oct13/ours_pp_r1.txt)."""
    s, cfg, model, m, pf, orc, h_ref, ids, (cos, sin) = _prefill_pair(3, 2)
    n = len(ids)
    orc_fp = oracle().Oracle(model, 256, cos, sin)
    rows = []
    for t in ids:
        orc_fp.tok[:] = t
        orc_fp.step()
        rows.append(orc_fp.h_last[0])
    h_fp = np.stack(rows)
    h = pf.h.cpu().numpy()
    scale = np.max(np.abs(h_ref))
    err = np.abs(h - h_ref) / scale
    noise = np.abs(h_ref - h_fp) / scale
    assert np.median(err) <= np.median(noise), (np.median(err), np.median(noise))
    assert np.quantile(err, 0.99) <= 1.5 * np.quantile(noise, 0.99)
    assert err.max() <= 1.5 * noise.max()
    lg_ref = orc.logits_of(h_ref[-1:])[0]
    lg = m.logits.cpu().numpy()
    lerr = np.max(np.abs(lg - lg_ref))
    assert lerr / np.max(np.abs(lg_ref)) < 5e-2
    assert int(m.pos.item()) == n
    assert lg_ref.max() - lg_ref[int(m.tok.item())] <= 2 * lerr + 1e-6   # same argmax unless the top two are that close
    m.step()                                                             # decode continues from the prefilled cache
    m.check_status()
    assert 0 <= int(m.tok.item()) < cfg.vocab and int(m.pos.item()) == n + 1


def test_chunked_prefill_equals_single_chunk():
    """Two chunks of 64 against one chunk of 128: same cache and logits up to int8 flips at the chunk boundary."""
    s, E = pkg("synth"), pkg("engine")
    cfg = s.ModelConfig("small128", 2, 512, 1536, 4, 2, 128, 4096)
    model = s.synth_model(cfg, 3)
    ids = s.synth_prompt(cfg, 128, 3)
    m1 = E.FusedQwen(model, max_len=128)
    E.prefill(m1, ids)
    m2 = E.FusedQwen(model, max_len=128)
    E.prefill(m2, ids, chunk=64)
    assert torch.equal(m1.vc[0], m2.vc[0])                               # layer 0 sees identical inputs
    rel = (m1.logits - m2.logits).abs().max() / m1.logits.abs().max()
    assert float(rel) < 2e-2


def test_chunked_prefill_equals_single_chunk_on_the_fp16_route():
    """The same for `linears="f16"`: no int8 rounding, so the two agree to the fp16 level (the attention sums differ in
    order between one key range and two)."""
    s, E = pkg("synth"), pkg("engine")
    cfg = s.ModelConfig("small128", 2, 512, 1536, 4, 2, 128, 4096)
    model = s.synth_model(cfg, 3)
    ids = s.synth_prompt(cfg, 128, 3)
    m1 = E.FusedQwen(model, max_len=128)
    E.prefill(m1, ids, linears="f16")
    m2 = E.FusedQwen(model, max_len=128)
    E.prefill(m2, ids, chunk=64, linears="f16")
    assert torch.equal(m1.vc[0], m2.vc[0])
    rel = (m1.logits - m2.logits).abs().max() / m1.logits.abs().max()
    assert float(rel) < 5e-3
    assert int(m1.tok.item()) == int(m2.tok.item())


def test_nll_of_int8_and_fp16_activation_paths_agree():
    """The reference's quality check of int8 activations (scripts/qwen_prefill.py:315-333): mean next-token NLL over all
    positions, prefill path (Q8_1 activations; and the fp16 prefill mode the reference compares it with) against the
    token-by-token decode path (fp16 activations).  On a small
    random-weight model the two must agree to well under one percent of the NLL itself."""
    s, E = pkg("synth"), pkg("engine")
    cfg = s.CONFIGS["small"]
    model = s.synth_model(cfg, 7)
    m = E.FusedQwen(model, max_len=128)
    ids = s.synth_prompt(cfg, 128, 7)
    r = E.perplexity(m, ids, chunk=64)
    assert r["tokens"] == 127
    assert np.isfinite(r["i8"]) and np.isfinite(r["f16"])
    assert 0.5 * np.log(cfg.vocab) < r["f16"] < 2.0 * np.log(cfg.vocab)      # random weights: near the uniform level
    assert abs(r["i8"] - r["f16"]) < 5e-3 * r["f16"]
    assert abs(r["cublas"] - r["f16"]) < 2e-3 * r["f16"]                      # the fp16 prefill mode: no int8 rounding


def _rand_q4(rng, n, k):
    W = rng.integers(0, 2 ** 32, size=(n, k // 8), dtype=np.uint32).view(np.int32)
    S = rng.uniform(0.002, 0.02, size=(n, k // 32)).astype(np.float16)
    return W, S


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("P", [128, 200, 77])
def test_swiglu_q8_epilogue_equals_swiglu_then_quantiser(P):
    """The gate/up GEMM with the `swiglu_q8` epilogue writes, byte for byte, the tiled Q8_1 operand that the `swiglu`
    epilogue followed by the tiled quantiser writes (lab/qwen_batched.py:1363-1396 against :1016-1041)."""
    QB = pkg("qwen_batched")
    pkg("qwen_kernels").init(0)
    rng = np.random.default_rng(P)
    N, K = 1536, 512                                   # 768 product columns = 24 k-blocks
    W, S = _rand_q4(rng, N, K)
    Wt, St = QB.pack_q4(_dev(W), _dev(S))
    x = torch.from_numpy(rng.standard_normal((P, K)).astype(np.float16)).cuda()
    xt = QB.q8_tiled_buffer(P, K, "cuda")
    QB.quant_q8_tiled(x, xt)
    st = QB.Status("cuda")
    act = torch.zeros(P, N // 2, dtype=torch.float16, device="cuda")
    QB.gemm8_prefill(Wt, St, xt, act, None, N, K, P, "swiglu", N // 2, st)
    want = QB.q8_tiled_buffer(P, N // 2, "cuda")
    QB.quant_q8_tiled(act, want)
    got = QB.q8_tiled_buffer(P, N // 2, "cuda")
    QB.gemm8_prefill(Wt, St, xt, got, None, N, K, P, "swiglu_q8", N // 2, st)
    st.check()
    assert torch.equal(got, want)


@pytest.mark.parametrize("P,pos0,NH,NKV", [(128, 0, 4, 2), (200, 56, 6, 1), (77, 3, 12, 2)])
def test_qkv_rope_kv_epilogue_and_cached_flash_equal_the_separate_launches(P, pos0, NH, NKV):
    """QKV GEMM with the `biasf_kv` epilogue + flash attention with the `q8` output against the `biasf` GEMM, the
    RoPE / append launch, flash attention and the tiled quantiser: the same cache rows, the same attention output and the
    same Q8_1 operand for the o projection, bit for bit (lab/qwen_batched.py:1316-1362, 1812-1848)."""
    s, QB = pkg("synth"), pkg("qwen_batched")
    pkg("qwen_kernels").init(0)
    rng = np.random.default_rng(P + NH)
    HD, K, max_len = 128, 512, 320
    N = (NH + 2 * NKV) * HD
    W, S = _rand_q4(rng, N, K)
    Wt, St = QB.pack_q4(_dev(W), _dev(S))
    bias = _dev(rng.standard_normal(N).astype(np.float32))
    x = torch.from_numpy(rng.standard_normal((P, K)).astype(np.float16)).cuda()
    xt = QB.q8_tiled_buffer(P, K, "cuda")
    QB.quant_q8_tiled(x, xt)
    cfg = s.ModelConfig("rope", 1, K, 256, NH, NKV, HD, 1024)
    cos, sin = (_dev(a) for a in s.rope_tables(cfg, max_len))
    st = QB.Status("cuda")
    scale = 1.0 / np.sqrt(HD)
    old = torch.from_numpy(rng.standard_normal((NKV, max_len, HD)).astype(np.float16)).cuda()   # earlier positions of the cache
    # separate launches
    kc1, vc1 = old.clone(), old.flip(1).clone()
    qkv1 = torch.zeros(P, N, dtype=torch.float16, device="cuda")
    QB.gemm8_prefill(Wt, St, xt, qkv1, bias, N, K, P, "biasf", N, st)
    out1 = torch.zeros(P, NH * HD, dtype=torch.float16, device="cuda")
    QB.attn_prefill(qkv1, cos, sin, kc1, vc1, out1, NH, NKV, HD, max_len, pos0, scale)
    xo1 = QB.q8_tiled_buffer(P, NH * HD, "cuda")
    QB.quant_q8_tiled(out1, xo1)
    # fused
    kc2, vc2 = old.clone(), old.flip(1).clone()
    qkv2 = torch.zeros(P, N, dtype=torch.float16, device="cuda")
    QB.gemm8_prefill_qkv_rope_kv(Wt, St, xt, qkv2, bias, K, P, cos, sin, pos0, kc2, vc2, NH, NKV, HD, max_len, st)
    out2 = torch.zeros(P, NH * HD, dtype=torch.float16, device="cuda")
    xo2 = QB.q8_tiled_buffer(P, NH * HD, "cuda")
    QB.attn_prefill_cached(qkv2, kc2, vc2, out2, xo2, NH, NKV, HD, max_len, pos0, scale)
    st.check()
    assert torch.equal(kc1, kc2) and torch.equal(vc1, vc2)
    assert torch.equal(qkv1[:, (NH + NKV) * HD:], qkv2[:, (NH + NKV) * HD:])           # v is passed through
    assert torch.equal(qkv2[:, NH * HD:(NH + NKV) * HD].reshape(P, NKV, HD).transpose(0, 1), kc2[:, pos0:pos0 + P])
    assert torch.equal(out1, out2)
    assert torch.equal(xo1, xo2)
    # the q8-only form (no fp16 output) writes the same operand
    xo3 = QB.q8_tiled_buffer(P, NH * HD, "cuda")
    QB.attn_prefill_cached(qkv2, kc2, vc2, None, xo3, NH, NKV, HD, max_len, pos0, scale)
    assert torch.equal(xo3, xo2)


def test_fused_prefill_equals_ten_launch_prefill():
    """`Prefill(fused=True)` (seven launches per layer, as scripts/qwen_prefill.py:196-246) against the ten-launch form on
    a three-layer model, two chunks: identical residual stream, cache and first generated token."""
    s, E = pkg("synth"), pkg("engine")
    cfg = s.ModelConfig("small128f", 3, 512, 1536, 4, 2, 128, 4096)
    model = s.synth_model(cfg, 21)
    ids = s.synth_prompt(cfg, 192, 9)
    res = []
    for fused in (False, True):
        m = E.FusedQwen(model, max_len=256)
        pf = E.prefill(m, ids, chunk=96, fused=fused)
        assert pf.launches_per_chunk == 1 + (7 if fused else 10) * cfg.layers
        res.append((pf.h.clone(), m.kc.clone(), m.vc.clone(), int(m.tok.item())))
    assert torch.equal(res[0][0], res[1][0])
    assert torch.equal(res[0][1], res[1][1]) and torch.equal(res[0][2], res[1][2])
    assert res[0][3] == res[1][3]


@pytest.mark.parametrize("P,n,k", [(200, 1536, 1536), (256, 1536, 8960), (77, 640, 512)])
def test_resid_gemm_split_along_k_equals_the_two_halves(P, n, k):
    """The K-split launch: Y gets the first K half added, Y2 the second half stored; each must equal the unsplit kernel run
    on that half alone (bit for bit: same k order inside a half), and their sum the oracle's product."""
    o, QB = oracle(), pkg("qwen_batched")
    pkg("qwen_kernels").init(0)
    rng = np.random.default_rng(P + n + k)
    W, S = _rand_q4(rng, n, k)
    x = rng.standard_normal((P, k)).astype(np.float16)
    xq, xd, _ = o.quant_q8_1(x)
    ref = o.mmq(W, S, xq, xd)
    Wt, St = QB.pack_q4(_dev(W), _dev(S))
    xt = QB.q8_tiled_buffer(P, k, "cuda")
    QB.quant_q8_tiled(_dev(x), xt)
    st = QB.Status("cuda")
    h0 = torch.from_numpy(rng.standard_normal((P, n)).astype(np.float32)).cuda()
    y, y2 = h0.clone(), torch.full((1, P, n), float("nan"), device="cuda")
    QB.gemm8_prefill_resid_ksplit(Wt, St, xt, y, y2, n, k, P, n, st)
    st.check()
    got = (y.double() + y2[0].double()).cpu().numpy()
    want = h0.double().cpu().numpy() + ref
    assert np.max(np.abs(got - want)) / np.max(np.abs(want)) < 2e-6
    # the halves against the oracle restricted to their k-blocks
    split = ((k // 32 // 2 + 7) // 8) * 8 * 32
    lo = o.mmq(W[:, :split // 8], S[:, :split // 32], xq[:, :split], xd[:, :split // 32])
    hi = o.mmq(W[:, split // 8:], S[:, split // 32:], xq[:, split:], xd[:, split // 32:])
    assert np.max(np.abs((y - h0).double().cpu().numpy() - lo)) / np.max(np.abs(lo)) < 2e-6
    assert np.max(np.abs(y2[0].double().cpu().numpy() - hi)) / np.max(np.abs(hi)) < 2e-6
    if k >= 768:                                             # three parts: their sum is the whole product again
        y3, p3 = h0.clone(), torch.full((2, P, n), float("nan"), device="cuda")
        QB.gemm8_prefill_resid_ksplit(Wt, St, xt, y3, p3, n, k, P, n, st)
        st.check()
        got3 = (y3.double() + p3[0].double() + p3[1].double()).cpu().numpy()
        assert np.max(np.abs(got3 - want)) / np.max(np.abs(want)) < 2e-6
    # twice the same bits
    ya, yb = h0.clone(), torch.zeros_like(y2)
    QB.gemm8_prefill_resid_ksplit(Wt, St, xt, ya, yb, n, k, P, n, st)
    assert torch.equal(ya, y) and torch.equal(yb, y2)


def test_rmsnorm_q8_tiled_add_equals_add_then_quantiser():
    QB = pkg("qwen_batched")
    pkg("qwen_kernels").init(0)
    g = torch.Generator(device="cuda").manual_seed(1)
    P, H = 200, 1536
    h = torch.randn(P, H, device="cuda", generator=g)
    h2 = torch.randn(2, P, H, device="cuda", generator=g)
    w = 1.0 + 0.1 * torch.randn(H, device="cuda", generator=g)
    want_h = (h + h2[0]) + h2[1]
    want = QB.q8_tiled_buffer(P, H, "cuda")
    QB.rmsnorm_q8_tiled(want_h, w, want, 1e-6)
    got = QB.q8_tiled_buffer(P, H, "cuda")
    QB.rmsnorm_q8_tiled_add(h, h2, w, got, 1e-6)
    assert torch.equal(h, want_h) and torch.equal(got, want)
    a = torch.randn(P, H, device="cuda", generator=g)
    b = a.clone()
    QB.add_rows(b, h2)
    assert torch.equal(b, (a + h2[0]) + h2[1])


def test_prefill_with_split_k_matches_the_unsplit_pass():
    """o_proj / down_proj launched as two half-K CTAs per tile: the residual stream differs from the unsplit pass only by the
    fp32 order of one addition per linear ((h + a) + b against h + (a + b)); fused and ten-launch forms stay identical."""
    s, E = pkg("synth"), pkg("engine")
    cfg = s.ModelConfig("small128s", 3, 512, 1536, 4, 2, 128, 4096)
    model = s.synth_model(cfg, 22)
    ids = s.synth_prompt(cfg, 128, 9)
    res = {}
    for split in (False, True):
        for fused in (False, True):
            m = E.FusedQwen(model, max_len=256)
            pf = E.Prefill(m, 128, fused=fused, split_k=split)
            pf.tok.copy_(torch.from_numpy(ids).cuda())
            pf.chunk(0)
            pf.finish(0)
            pf.status.check("prefill")
            res[(split, fused)] = (pf.h.clone(), m.kc.clone(), int(m.tok.item()))
    for split in (False, True):
        assert torch.equal(res[(split, False)][0], res[(split, True)][0])
        assert torch.equal(res[(split, False)][1], res[(split, True)][1])
    a, b = res[(False, True)][0], res[(True, True)][0]
    # an int8 flip downstream of a last-bit difference is possible, as everywhere on this path: typical rows agree to fp32 level
    err = ((a - b).abs().max(dim=1).values / a.abs().max()).cpu().numpy()
    assert np.median(err) < 1e-5 and err.max() < 5e-2


# ---- fp16 route: weights dequantised to fp16 inside the GEMM, fp16 activations, fp32 accumulation over all of K ----------

def test_f16_tile_layout():
    """The fp16 operand: per (128-token tile, k-block) [8-token group][8-value chunk][token][16 bytes], values of a chunk
    in the order (0,4,1,5,2,6,3,7); rows past P stay zero."""
    QB = pkg("qwen_batched")
    rng = np.random.default_rng(3)
    P, K = 200, 96
    x = rng.standard_normal((P, K)).astype(np.float16)
    xt = QB.f16_tiled_buffer(P, K, "cuda")
    QB.f16_tile(dev(x), xt)
    got = xt.cpu().numpy().view(np.float16).reshape(2, K // 32, 16, 4, 8, 8)      # tile, k-block, group, chunk, token, value
    xp = np.zeros((256, K), np.float16)
    xp[:P] = x
    want = xp.reshape(2, 16, 8, K // 32, 4, 8)[..., [0, 4, 1, 5, 2, 6, 3, 7]].transpose(0, 3, 1, 4, 2, 5)
    assert np.array_equal(got.view(np.uint16), np.ascontiguousarray(want).view(np.uint16))


@pytest.mark.parametrize("P,n,k,epi", [(128, 128, 256, "logits"), (200, 256, 512, "store"), (130, 384, 1536, "biasf"),
                                       (256, 1536, 8960, "resid"), (300, 512, 768, "swiglu"), (1, 128, 256, "logits")])
def test_gemm16_prefill_matches_f16w_oracle(P, n, k, epi):
    """Against the float64 product of the fp16-rounded weights (the reference's `dq`) and the fp16 activations; the kernel
    accumulates in fp32 on the tensor cores, so the bar is north_star's 1e-3 of the output scale, and in practice 1e-5."""
    QB, o = pkg("qwen_batched"), oracle()
    rng = np.random.default_rng(P + n)
    W = rng.integers(0, 2 ** 32, size=(n, k // 8), dtype=np.uint32).view(np.int32)
    S = rng.uniform(0.002, 0.02, size=(n, k // 32)).astype(np.float16)
    x = rng.standard_normal((P, k)).astype(np.float16)
    Wt, St = QB.pack_q4(dev(W), dev(S))
    xt = QB.f16_tiled_buffer(P, k, "cuda")
    QB.f16_tile(dev(x), xt)
    st = QB.Status("cuda")
    ref = o.gemv_f16w_ref(W, S, x)
    scale = np.abs(ref).max()
    if epi == "resid":
        h0 = rng.standard_normal((P, n)).astype(np.float32)
        y = dev(h0)
        QB.gemm16_prefill(Wt, St, xt, y, None, n, k, P, epi, n, st)
        got, want = y.cpu().numpy(), h0 + ref
    elif epi == "swiglu":
        y = torch.full((P, n // 2), float("nan"), dtype=torch.float16, device="cuda")
        QB.gemm16_prefill(Wt, St, xt, y, None, n, k, P, epi, n // 2, st)
        g, u = ref[:, 0::2], ref[:, 1::2]
        got, want = y.float().cpu().numpy(), g / (1 + np.exp(-g)) * u
        scale = np.abs(want).max()
    elif epi == "biasf":
        b = rng.standard_normal(n).astype(np.float32)
        y = torch.full((P, n), float("nan"), dtype=torch.float16, device="cuda")
        QB.gemm16_prefill(Wt, St, xt, y, dev(b), n, k, P, epi, n, st)
        got, want = y.float().cpu().numpy(), ref + b
    else:
        y = torch.full((P, n), float("nan"), dtype=torch.float16 if epi == "store" else torch.float32, device="cuda")
        QB.gemm16_prefill(Wt, St, xt, y, None, n, k, P, epi, n, st)
        got, want = y.float().cpu().numpy(), ref
    st.check()
    assert not np.isnan(got).any()
    tol = 1e-3 if y.dtype == torch.float16 else 1e-4          # fp16 outputs: half an ulp of the largest value is 5e-4 of it
    assert np.abs(got - want).max() / scale < tol


def test_prefill_f16_route_matches_f16w_oracle_and_decode_continues():
    """Three layers through `Prefill(linears="f16")` against the oracle's token-by-token forward with the same fp16-rounded
    weights (statistical: fp16 activations are rounded at every storage point on both sides, the accumulation orders
    differ)."""
    s, E = pkg("synth"), pkg("engine")
    cfg = s.ModelConfig("small128", 3, 512, 1536, 4, 2, 128, 4096)
    model = s.synth_model(cfg, 5)
    m = E.FusedQwen(model, max_len=256)
    ids = s.synth_prompt(cfg, 160, 5)
    pf = E.prefill(m, ids, linears="f16")
    cos, sin = s.rope_tables(cfg, 256)
    orc = oracle().Oracle(model, 256, cos, sin, weights="f16w")
    rows = []
    for t in ids:
        orc.tok[:] = t
        orc.step()
        rows.append(orc.h_last[0])
    h_ref = np.stack(rows)
    h = pf.h.cpu().numpy()
    err = np.abs(h - h_ref) / np.max(np.abs(h_ref))
    assert np.median(err) < 1e-3 and np.quantile(err, 0.9) < 3e-3 and err.max() < 5e-2, (np.median(err), err.max())
    lg_ref = orc.logits_of(h_ref[-1:])[0]
    lg = m.logits.cpu().numpy()
    lerr = np.max(np.abs(lg - lg_ref))
    assert lerr / np.max(np.abs(lg_ref)) < 2e-2
    assert lg_ref.max() - lg_ref[int(m.tok.item())] <= 2 * lerr + 1e-6
    assert int(m.pos.item()) == len(ids)
    m.step()
    m.check_status()
    assert 0 <= int(m.tok.item()) < cfg.vocab and int(m.pos.item()) == len(ids) + 1


def test_prefill_f16_and_q8_routes_agree_statistically():
    s, E = pkg("synth"), pkg("engine")
    cfg = s.ModelConfig("small128", 2, 512, 1536, 4, 2, 128, 4096)
    model = s.synth_model(cfg, 6)
    ids = s.synth_prompt(cfg, 256, 6)
    hs = []
    for lin in ("q8", "f16"):
        m = E.FusedQwen(model, max_len=256)
        hs.append(E.prefill(m, ids, linears=lin).h.cpu().numpy())
    err = np.abs(hs[0] - hs[1]) / np.max(np.abs(hs[1]))
    assert np.median(err) < 5e-3 and err.max() < 0.2, (np.median(err), err.max())


def test_rmsnorm_f16_tiled_equals_rmsnorm_then_tiling_and_adds_parts():
    """Layout exactly that of `f16_tile`, values those of the fp16 RMSNorm kernel to one fp16 ulp (the two kernels sum the
    squares in different orders); with addends: h completed exactly, and the same bits as the plain call on the completed h."""
    QB, K = pkg("qwen_batched"), pkg("qwen_kernels")
    rng = np.random.default_rng(11)
    P, H = 200, 512
    h = rng.standard_normal((P, H)).astype(np.float32)
    add = rng.standard_normal((2, P, H)).astype(np.float32)
    w = rng.uniform(0.5, 1.5, H).astype(np.float32)
    x16 = torch.zeros(P, H, dtype=torch.float16, device="cuda")
    K.rms(dev(h), dev(w), x16, 1e-6)
    want = QB.f16_tiled_buffer(P, H, "cuda")
    QB.f16_tile(x16, want)
    got = QB.f16_tiled_buffer(P, H, "cuda")
    QB.rmsnorm_f16_tiled(dev(h), dev(w), got, 1e-6)
    a = got.cpu().numpy().view(np.int16).astype(np.int32)
    b = want.cpu().numpy().view(np.int16).astype(np.int32)
    assert np.abs(a - b).max() <= 1 and np.mean(a != b) < 0.01
    total = (h + add[0]) + add[1]
    plain = QB.f16_tiled_buffer(P, H, "cuda")
    QB.rmsnorm_f16_tiled(dev(total), dev(w), plain, 1e-6)
    hd = dev(h)
    summed = QB.f16_tiled_buffer(P, H, "cuda")
    QB.rmsnorm_f16_tiled(hd, dev(w), summed, 1e-6, dev(add))
    assert torch.equal(summed, plain)
    assert np.array_equal(hd.cpu().numpy(), total)


@pytest.mark.parametrize("P,n,k,parts", [(256, 1536, 8960, 3), (130, 512, 1536, 2), (2048, 1536, 8960, 3)])
def test_gemm16_resid_split_along_k_matches_the_unsplit_launch(P, n, k, parts):
    QB = pkg("qwen_batched")
    rng = np.random.default_rng(P + parts)
    W = rng.integers(0, 2 ** 32, size=(n, k // 8), dtype=np.uint32).view(np.int32)
    S = rng.uniform(0.002, 0.02, size=(n, k // 32)).astype(np.float16)
    Wt, St = QB.pack_q4(dev(W), dev(S))
    xt = QB.f16_tiled_buffer(P, k, "cuda")
    QB.f16_tile(dev(rng.standard_normal((P, k)).astype(np.float16)), xt)
    st = QB.Status("cuda")
    h0 = rng.standard_normal((P, n)).astype(np.float32)
    y1, y2 = dev(h0), dev(h0)
    y2b = torch.full((parts - 1, P, n), float("nan"), device="cuda")
    QB.gemm16_prefill(Wt, St, xt, y1, None, n, k, P, "resid", n, st)
    QB.gemm16_prefill_resid_ksplit(Wt, St, xt, y2, y2b, n, k, P, n, st)
    QB.add_rows(y2, y2b)
    st.check()
    a, b = y1.cpu().numpy(), y2.cpu().numpy()
    assert not np.isnan(b).any()
    assert np.abs(a - b).max() / np.abs(a).max() < 1e-5        # the same products, summed in parts


@pytest.mark.parametrize("P,n,k", [(200, 256, 512), (2048, 1024, 256), (130, 384, 768)])
def test_swiglu_f16t_epilogue_equals_swiglu_then_tiling(P, n, k):
    """The fused epilogue of the fp16 gate/up GEMM writes the same bits into the next GEMM's operand as the plain swiglu
    epilogue followed by `f16_tile` (also with a last row pair that has only one row tile, n = 384)."""
    QB = pkg("qwen_batched")
    rng = np.random.default_rng(P + k)
    W = rng.integers(0, 2 ** 32, size=(n, k // 8), dtype=np.uint32).view(np.int32)
    S = rng.uniform(0.002, 0.02, size=(n, k // 32)).astype(np.float16)
    Wt, St = QB.pack_q4(dev(W), dev(S))
    xt = QB.f16_tiled_buffer(P, k, "cuda")
    QB.f16_tile(dev(rng.standard_normal((P, k)).astype(np.float16)), xt)
    st = QB.Status("cuda")
    y = torch.zeros(P, n // 2, dtype=torch.float16, device="cuda")
    QB.gemm16_prefill(Wt, St, xt, y, None, n, k, P, "swiglu", n // 2, st)
    want = QB.f16_tiled_buffer(P, n // 2, "cuda")
    QB.f16_tile(y, want)
    got = QB.f16_tiled_buffer(P, n // 2, "cuda")
    QB.gemm16_prefill(Wt, St, xt, got, None, n, k, P, "swiglu_f16t", n // 2, st)
    st.check()
    assert torch.equal(got, want)


def test_prefill_gemm_expired_waits_set_the_status_word_and_return():
    """The bounded waits of the tcgen05 pipeline: with the copy thread issuing nothing every role runs into its limit
    (about a second), the kernel sets the status word, lets its MMAs retire, frees its tensor memory and returns; the
    next launch on the same context computes correctly."""
    QB, ffi, o = pkg("qwen_batched"), pkg("_ffi"), oracle()
    rng = np.random.default_rng(5)
    P, n, k = 128, 128, 256
    W = rng.integers(0, 2 ** 32, size=(n, k // 8), dtype=np.uint32).view(np.int32)
    S = rng.uniform(0.002, 0.02, size=(n, k // 32)).astype(np.float16)
    Wt, St = QB.pack_q4(dev(W), dev(S))
    x = rng.standard_normal((P, k)).astype(np.float16)
    xt = QB.q8_tiled_buffer(P, k, "cuda")
    QB.quant_q8_tiled(dev(x), xt)
    y = torch.zeros(P, n, dtype=torch.float32, device="cuda")
    st = QB.Status("cuda")
    ffi.call("q4b_debug_mmq_prefill_expired_wait", Wt.data_ptr(), St.data_ptr(), xt.data_ptr(), y.data_ptr(), n, k, P,
             st.word.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()                                  # the kernel came back
    assert int(st.word.item()) != 0
    with pytest.raises(ffi.Q4BError) as e:
        st.check("prefill")
    assert e.value.code == ffi.E_TIMEOUT
    QB.gemm8_prefill(Wt, St, xt, y, None, n, k, P, "logits", n, st)
    torch.cuda.synchronize()
    st.check("prefill")
    xq, xd, _ = o.quant_q8_1(x)
    ref = o.mmq(W, S, xq, xd)
    assert np.abs(y.cpu().numpy() - ref).max() / np.abs(ref).max() < 1e-5
