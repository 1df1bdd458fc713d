"""The streaming mma.sync GEMV (bulk-copied slab, register accumulators, exact digit planes) and the fused
RMSNorm -> QKV -> bias -> RoPE -> K/V append launch, against the oracle.  fp32 results within 1e-3 of the largest
reference magnitude (observed ~1e-7); 16-bit outputs within one unit in the last place."""
import numpy as np
import pytest

from conftest import gemv_inputs, oracle, pkg

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def nerr(got, ref):
    ref = np.asarray(ref, np.float64)
    return float(np.max(np.abs(np.asarray(got, np.float64) - ref)) / max(np.max(np.abs(ref)), 1e-30))


def rand_q4(rng, n, k):
    W = rng.integers(0, 2 ** 32, size=(n, k // 8), dtype=np.uint32).view(np.int32)
    S = rng.uniform(0.002, 0.02, size=(n, k // 32)).astype(np.float16)
    return W, S


def ulps16(a, b):
    a = np.asarray(a, np.float16).view(np.int16).astype(np.int32)
    b = np.asarray(b, np.float16).view(np.int16).astype(np.int32)
    return np.abs(a - b)


@pytest.fixture(scope="module")
def QB():
    pkg("qwen_kernels").init(0)
    return pkg("qwen_batched")


# ragged N, K of one block, K not a multiple of 256, every layer shape of both models, a slab of two K windows
@pytest.mark.parametrize("n,k", [(128, 32), (5, 96), (200, 544), (2048, 1536), (1536, 1536), (17920, 1536), (1536, 8960),
                                 (130, 3584), (260, 18944), (4608, 3584)])
@pytest.mark.parametrize("xdt", ["f16", "f32"])
def test_gemv_mma_matches_oracle(QB, n, k, xdt):
    o = oracle()
    rng = np.random.default_rng(n * 7 + k)
    W, S = rand_q4(rng, n, k)
    x = rng.standard_normal(k).astype(np.float16 if xdt == "f16" else np.float32)
    x[::97] *= 1e-3                                           # wide dynamic range inside blocks
    x[5 * 32:6 * 32] = 0 if k > 6 * 32 else x[5 * 32:6 * 32]  # an all-zero block
    ref = o.gemv_ref(W, S, x)
    st = QB.Status("cuda")
    y = torch.full((n + 8,), float("nan"), device="cuda")
    Wd, Sd = QB.pack_q4(dev(W), dev(S))
    xd = dev(x)
    QB.gemv_mma(Wd, Sd, xd, y, None, n, k, "logits", st)
    st.check()
    got = y.cpu().numpy()
    assert np.all(np.isnan(got[n:]))
    assert nerr(got[:n], ref) < 2e-6
    y2 = torch.empty(n, device="cuda")
    QB.gemv_mma(Wd, Sd, xd, y2, None, n, k, "logits", st)
    st.check()
    assert torch.equal(y2, y[:n]), "not bit-repeatable"


def test_gemv_mma_ffn_up_golden(QB, golden):
    """BASELINE configuration 1 on the reference's own seeded inputs (lab/experiments/gemv5.py:40-49)."""
    g = golden["gemv_ffn_up"]
    q, d, x = gemv_inputs(8960, 1536, False)
    W = pkg("gguf").pack_nibbles(q)
    st = QB.Status("cuda")
    y = torch.empty(8960, device="cuda")
    QB.gemv_mma(*QB.pack_q4(dev(W), dev(d)), dev(x), y, None, 8960, 1536, "logits", st)
    st.check()
    got = y.cpu().numpy()
    assert nerr(got, g["y_ref_f64"]) < 2e-6
    assert nerr(got, g["y_ref_f32"]) < 1e-5


@pytest.mark.parametrize("n,k", [(256, 256), (2048, 1536), (1536, 8960), (17920, 1536)])
def test_gemv_mma_epilogues(QB, n, k):
    o = oracle()
    rng = np.random.default_rng(n + k + 1)
    W, S = rand_q4(rng, n, k)
    x = rng.standard_normal(k).astype(np.float16)
    acc = o.gemv_ref(W, S, x)
    Wd, Sd = QB.pack_q4(dev(W), dev(S))
    xd = dev(x)
    st = QB.Status("cuda")
    y = torch.empty(n, dtype=torch.float16, device="cuda")
    big = np.abs(acc) > 0.05 * np.abs(acc).max()              # a unit in the last place only means something away from zero
    QB.gemv_mma(Wd, Sd, xd, y, None, n, k, "store", st)
    assert nerr(y.float().cpu().numpy(), o.f16(acc)) < 1e-3
    assert ulps16(y.cpu().numpy(), o.f16(acc))[big].max() <= 1
    bias = (0.1 * rng.standard_normal(n)).astype(np.float32)
    QB.gemv_mma(Wd, Sd, xd, y, dev(bias), n, k, "biasf", st)
    assert nerr(y.float().cpu().numpy(), o.f16(acc + bias)) < 1e-3
    assert ulps16(y.cpu().numpy(), o.f16(acc + bias))[big].max() <= 1
    h0 = rng.standard_normal(n).astype(np.float32)
    h = dev(h0)
    QB.gemv_mma(Wd, Sd, xd, h, None, n, k, "resid", st)
    assert nerr(h.cpu().numpy(), h0 + acc) < 1e-5
    ys = torch.empty(n // 2, dtype=torch.float16, device="cuda")
    QB.gemv_mma(Wd, Sd, xd, ys, None, n, k, "swiglu", st)
    assert nerr(ys.float().cpu().numpy(), o.silu_mul(acc[0::2], acc[1::2])) < 1e-3
    st.check()


def test_gemv_mma_agrees_with_the_other_two_gemvs(QB):
    """Three independent implementations of the same dequantise-and-dot agree to fp32 rounding."""
    K = pkg("qwen_kernels")
    rng = np.random.default_rng(77)
    n, k = 2048, 1536
    W, S = rand_q4(rng, n, k)
    x = rng.standard_normal(k).astype(np.float16)
    Wd, Sd, xd = dev(W), dev(S), dev(x)
    a, b, c = (torch.empty(n, device="cuda") for _ in range(3))
    st = QB.Status("cuda")
    K.gemv(Wd, Sd, xd, a, None, n, k, "logits")
    Wt, St = QB.pack_q4(Wd, Sd)
    QB.gemv_tc(Wt, St, xd, b, None, n, k, "logits", st)
    QB.gemv_mma(Wt, St, xd, c, None, n, k, "logits", st)
    st.check()
    assert nerr(c.cpu().numpy(), a.cpu().numpy()) < 2e-6
    assert nerr(c.cpu().numpy(), b.cpu().numpy()) < 1e-6


@pytest.mark.parametrize("n,k", [(2048, 1536), (17920, 1536), (512, 256)])
def test_rmsnorm_gemv_mma(QB, n, k):
    o = oracle()
    rng = np.random.default_rng(n + 3 * k)
    W, S = rand_q4(rng, n, k)
    h = (3 * rng.standard_normal(k)).astype(np.float32)
    nw = (1 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    x = o.rmsnorm(h, nw, 1e-6)
    ref = o.gemv_ref(W, S, x)
    st = QB.Status("cuda")
    y = torch.empty(n, device="cuda")
    QB.rmsnorm_gemv_mma(*QB.pack_q4(dev(W), dev(S)), dev(h), dev(nw), 1e-6, y, None, n, k, "logits", st)
    st.check()
    # the normalised row may differ from the oracle's by one fp16 unit on a few elements (fp32 vs float64 rsqrt)
    assert nerr(y.cpu().numpy(), ref) < 1e-3


@pytest.mark.parametrize("NH,NKV,HD,H,max_len,p", [(12, 2, 128, 1536, 1024, 517), (4, 2, 64, 256, 64, 0), (4, 2, 128, 512, 4096, 4095),
                                                   (28, 4, 128, 3584, 256, 255)])
def test_qkv_rope_kv_and_cached_attention(QB, NH, NKV, HD, H, max_len, p):
    """One launch does RMSNorm -> QKV GEMV -> +bias -> round -> RoPE(q, k) -> round -> cache append; the attention that
    follows only reads.  Checked against the oracle's statement of the same chain (rounding points of ATTN4,
    lab/qwen_kernels.py:533-603) and against the two-launch form of this library."""
    o, s, K = oracle(), pkg("synth"), pkg("qwen_kernels")
    rng = np.random.default_rng(NH * 1000 + p)
    n = (NH + 2 * NKV) * HD
    cfg = s.ModelConfig("t", 1, H, 64, NH, NKV, HD, 100)
    cos, sin = s.rope_tables(cfg, max_len)
    W, S = rand_q4(rng, n, H)
    h = (2 * rng.standard_normal(H)).astype(np.float32)
    nw = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    bias = (0.1 * rng.standard_normal(n)).astype(np.float32)
    kc = rng.standard_normal((NKV, max_len, HD)).astype(np.float16)
    vc = rng.standard_normal((NKV, max_len, HD)).astype(np.float16)
    scale = 1.0 / np.sqrt(HD)
    # oracle
    x = o.rmsnorm(h, nw, 1e-6)
    y16 = o.f16(o.gemv_ref(W, S, x) + bias)
    q_ref = o.rope_rotate(y16[:NH * HD].reshape(NH, HD), cos[p], sin[p])
    k_ref = o.rope_rotate(y16[NH * HD:(NH + NKV) * HD].reshape(NKV, HD), cos[p], sin[p])
    v_ref = y16[(NH + NKV) * HD:].reshape(NKV, HD)
    kc_ref, vc_ref = kc.copy(), vc.copy()
    kc_ref[:, p], vc_ref[:, p] = k_ref.astype(np.float16), v_ref.astype(np.float16)
    att_ref = o.attn_decode(q_ref, kc_ref, vc_ref, p + 1, scale)
    # device: fused launch + cached attention
    Wt, St = QB.pack_q4(dev(W), dev(S))
    st = QB.Status("cuda")
    hd, nwd, bd, posd = dev(h), dev(nw), dev(bias), dev(np.array([p], np.int64))
    cosd, sind = dev(cos), dev(sin)
    kcd, vcd = dev(kc), dev(vc)
    qkv = torch.empty(n, dtype=torch.float16, device="cuda")
    att = torch.full((NH * HD,), float("nan"), dtype=torch.float16, device="cuda")
    QB.rmsnorm_qkv_rope_kv(Wt, St, hd, nwd, 1e-6, qkv, bd, H, cosd, sind, posd, kcd, vcd, NH, NKV, HD, max_len, st)
    QB.attn_cached(qkv, posd, kcd, vcd, att, NH, NKV, HD, max_len, scale)
    st.check()
    got_q = qkv[:NH * HD].cpu().numpy().reshape(NH, HD)
    got_k, got_v = kcd.cpu().numpy(), vcd.cpu().numpy()
    assert nerr(got_q, q_ref) < 1e-3 and nerr(got_k[:, p], k_ref) < 1e-3 and nerr(got_v[:, p], v_ref) < 1e-3
    assert (ulps16(got_q, q_ref) > 0).mean() < 0.02           # 16-bit roundings agree except for a few last-place flips
    keep = np.ones(max_len, bool)
    keep[p] = False
    assert np.array_equal(got_k[:, keep], kc[:, keep]) and np.array_equal(got_v[:, keep], vc[:, keep]), "other rows touched"
    assert nerr(att.float().cpu().numpy().reshape(NH, HD), att_ref) < 2e-3
    # device: the two-launch form (plain biasf GEMV, then the attention that rotates and appends itself)
    kc2, vc2 = dev(kc), dev(vc)
    qkv2 = torch.empty_like(qkv)
    att2 = torch.empty_like(att)
    QB.rmsnorm_gemv_mma(Wt, St, hd, nwd, 1e-6, qkv2, bd, n, H, "biasf", st)
    ws = K.attn_workspace(1, NH, HD, max_len, "cuda")
    K.attn(qkv2.view(1, -1), cosd, sind, posd, kc2.unsqueeze(0), vc2.unsqueeze(0), att2.view(1, -1), NH, NKV, HD, max_len, scale, ws)
    st.check()
    # same arithmetic in two kernels; the compiler may contract a*c - b*s differently, so allow one unit in the last place
    assert nerr(kc2.float().cpu().numpy(), got_k) < 1e-3 and torch.equal(vc2, vcd), "fused append differs from the attention kernel's own"
    assert nerr(att2.float().cpu().numpy(), att.float().cpu().numpy()) < 2e-3, "cached attention differs from the self-rotating one"


def test_expired_wait_sets_the_status_word_and_returns(QB):
    """A bounded device-side wait that runs out must end in a status word and an exception on the host, never a hang:
    the debug entry withholds the bulk copies of one chunk and cuts the wait to a few thousand polls."""
    ffi = pkg("_ffi")
    rng = np.random.default_rng(3)
    n, k = 256, 1536
    W, S = rand_q4(rng, n, k)
    Wt, St = QB.pack_q4(dev(W), dev(S))
    x = dev(rng.standard_normal(k).astype(np.float16))
    y = torch.empty(n, device="cuda")
    st = QB.Status("cuda")
    ffi.call("q4b_debug_gemv_mma_expired_wait", Wt.data_ptr(), St.data_ptr(), x.data_ptr(), y.data_ptr(), n, k,
             st.word.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()                                  # the kernel came back
    assert int(st.word.item()) != 0
    with pytest.raises(ffi.Q4BError) as e:
        st.check("gemv")
    assert e.value.code == ffi.E_TIMEOUT
    assert int(st.word.item()) == 0                           # check() clears the word
    # and the context is fine: the same GEMV without the fault gives the right answer
    QB.gemv_mma(Wt, St, x, y, None, n, k, "logits", st)
    st.check()
    assert nerr(y.cpu().numpy(), oracle().gemv_ref(W, S, x.cpu().numpy())) < 2e-6


def test_gemv_mma_rejects_bad_arguments(QB):
    ffi = pkg("_ffi")
    st = QB.Status("cuda")
    W = torch.zeros(1, 1, 128, 4, dtype=torch.int32, device="cuda")
    S = torch.zeros(1, 1, 128, dtype=torch.float16, device="cuda")
    x = torch.zeros(64, dtype=torch.float16, device="cuda")
    y = torch.zeros(4, device="cuda")
    with pytest.raises(ffi.Q4BError) as e:
        QB.gemv_mma(W, S, x, y, None, 4, 31, "logits", st)
    assert e.value.code == ffi.E_SHAPE
    with pytest.raises(ffi.Q4BError) as e:
        QB.gemv_mma(W, S, x[1:], y, None, 4, 32, "logits", st)
    assert e.value.code == ffi.E_ALIGN
    with pytest.raises(ffi.Q4BError) as e:
        QB.gemv_mma(W, S, x, y, None, 4, 32, "biasf", st)         # bias missing
    assert e.value.code == ffi.E_ALIGN
    with pytest.raises(ffi.Q4BError) as e:
        QB.gemv_mma(W, S, x, y, None, 4, 32, "biasf_rope_kv", st)
    assert e.value.code == ffi.E_ARG
    with pytest.raises(ffi.Q4BError) as e:                        # K beyond what one cluster of 8 CTAs can hold in shared memory
        QB.gemv_mma(W, S, x, y, None, 300, 24576, "logits", st)
    assert e.value.code == ffi.E_SHAPE


@pytest.mark.parametrize("max_len", [256, 1024, 2048])
def test_attn_cached_every_chunk_geometry(QB, max_len):
    """The shared-memory-resident attention cuts the ACTUAL context into 8 chunks of whole 16-position warp tiles, so the
    geometry changes with the position: first position, one short of / exactly / one past tile and chunk boundaries,
    the last row of the cache.  Against the oracle's decode attention on the same cache."""
    o = oracle()
    NH, NKV, HD = 12, 2, 128
    rng = np.random.default_rng(max_len)
    kc = rng.standard_normal((NKV, max_len, HD)).astype(np.float16)
    vc = rng.standard_normal((NKV, max_len, HD)).astype(np.float16)
    kcd, vcd = dev(kc), dev(vc)
    scale = 1.0 / np.sqrt(HD)
    qkv = torch.zeros((NH + 2 * NKV) * HD, dtype=torch.float16, device="cuda")
    att = torch.empty(NH * HD, dtype=torch.float16, device="cuda")
    for p in sorted({0, 1, 14, 15, 16, 17, 126, 127, 128, 129, 130, 255, max_len // 2, max_len - 2, max_len - 1}):
        if p >= max_len:
            continue
        q = rng.standard_normal((NH, HD)).astype(np.float16)
        qkv[:NH * HD] = dev(q.reshape(-1))
        att.fill_(float("nan"))
        QB.attn_cached(qkv, dev(np.array([p], np.int64)), kcd, vcd, att, NH, NKV, HD, max_len, scale)
        ref = o.attn_decode(q, kc, vc, p + 1, scale)
        got = att.float().cpu().numpy().reshape(NH, HD)
        assert np.isfinite(got).all(), f"p={p}"
        assert nerr(got, ref) < 2e-3, f"p={p}"
    assert torch.equal(kcd, dev(kc)) and torch.equal(vcd, dev(vc)), "the cached form must not write the cache"
