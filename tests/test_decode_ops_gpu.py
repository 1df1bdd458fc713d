"""Parity of the batch-1 decode kernels with the CPU oracle, through the C-ABI.  Floating point: tolerance 1e-3 of the
largest reference magnitude (the bound the target states for fp32 outputs and logits); observed errors are ~1e-6.
Index outputs (argmax) must be identical."""
import numpy as np
import pytest

from conftest import gemv_inputs, oracle, pkg

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

TOL = 1e-3


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def nerr(got, ref):
    ref = np.asarray(ref, np.float64)
    return float(np.max(np.abs(np.asarray(got, np.float64) - ref)) / max(np.max(np.abs(ref)), 1e-30))


def rand_q4(rng, n, k):
    W = rng.integers(0, 2 ** 32, size=(n, k // 8), dtype=np.uint32).view(np.int32)
    S = rng.uniform(0.002, 0.02, size=(n, k // 32)).astype(np.float16)
    return W, S


@pytest.fixture(scope="module")
def K():
    k = pkg("qwen_kernels")
    k.init(0)
    return k


@pytest.mark.parametrize("n,k", [(4, 32), (1, 64), (7, 96), (64, 256), (2048, 1536), (1536, 8960), (130, 3584), (36, 18944)])
@pytest.mark.parametrize("xdt", ["f16", "f32"])
def test_gemv_logits_matches_oracle(K, n, k, xdt):
    o = oracle()
    rng = np.random.default_rng(n * 131 + k)
    W, S = rand_q4(rng, n, k)
    x = rng.standard_normal(k).astype(np.float16 if xdt == "f16" else np.float32)
    ref = o.gemv_ref(W, S, x)
    y = torch.full((n + 8,), float("nan"), device="cuda")            # guard band behind the output
    K.gemv(dev(W), dev(S), dev(x), y, None, n, k, "logits")
    torch.cuda.synchronize()
    got = y.cpu().numpy()
    assert np.all(np.isnan(got[n:])), "wrote past the end of Y"
    assert nerr(got[:n], ref) < 1e-5
    y2 = torch.empty(n, device="cuda")
    K.gemv(dev(W), dev(S), dev(x), y2, None, n, k, "logits")
    assert torch.equal(y2, y[:n]), "GEMV is not bit-repeatable"


def test_gemv_ffn_up_golden(K, golden):
    """The 8960 x 1536 ffn_up GEMV against the reference's own numpy dequantise-and-dot (fixture)."""
    g = golden["gemv_ffn_up"]
    q, d, x = gemv_inputs(8960, 1536, False)
    W = pkg("gguf").pack_nibbles(q)
    y = torch.empty(8960, device="cuda")
    K.gemv(dev(W), dev(d), dev(x), y, None, 8960, 1536, "logits")
    got = y.cpu().numpy()
    assert nerr(got, g["y_ref_f64"]) < 1e-5
    assert nerr(got, g["y_ref_f32"]) < 1e-5
    # the reference's own acceptance bound for this kernel family (lab/experiments/gemv5.py:66-69)
    assert nerr(got, g["y_ref_f64"]) < 1e-4


@pytest.mark.parametrize("n,k", [(64, 256), (2048, 1536), (1536, 8960)])
def test_gemv_epilogues(K, n, k):
    o = oracle()
    rng = np.random.default_rng(n + k)
    W, S = rand_q4(rng, n, k)
    x = rng.standard_normal(k).astype(np.float16)
    acc = o.gemv_ref(W, S, x)
    Wd, Sd, xd = dev(W), dev(S), dev(x)
    # store
    y = torch.empty(n, dtype=torch.float16, device="cuda")
    K.gemv(Wd, Sd, xd, y, None, n, k, "store")
    assert nerr(y.float().cpu().numpy(), o.f16(acc)) < TOL
    # biasf
    bias = (0.1 * rng.standard_normal(n)).astype(np.float32)
    K.gemv(Wd, Sd, xd, y, dev(bias), n, k, "biasf")
    assert nerr(y.float().cpu().numpy(), o.f16(acc + bias)) < TOL
    # resid
    h0 = rng.standard_normal(n).astype(np.float32)
    h = dev(h0)
    K.gemv(Wd, Sd, xd, h, None, n, k, "resid")
    assert nerr(h.cpu().numpy(), h0 + acc) < 1e-5
    # swiglu: rows interleaved gate, up
    ys = torch.empty(n // 2, dtype=torch.float16, device="cuda")
    K.gemv(Wd, Sd, xd, ys, None, n, k, "swiglu")
    assert nerr(ys.float().cpu().numpy(), o.silu_mul(acc[0::2], acc[1::2])) < TOL


def test_gemv_rejects_bad_arguments(K):
    ffi = pkg("_ffi")
    W = torch.zeros(4, 4, dtype=torch.int32, device="cuda")
    S = torch.zeros(4, 1, dtype=torch.float16, device="cuda")
    x = torch.zeros(32, dtype=torch.float16, device="cuda")
    y = torch.zeros(4, device="cuda")
    with pytest.raises(ffi.Q4BError) as e:
        K.gemv(W, S, x, y, None, 4, 31, "logits")
    assert e.value.code == ffi.E_SHAPE
    with pytest.raises(ValueError):
        K.gemv(W, S, x, y, None, 4, 32, "nope")
    with pytest.raises(ffi.Q4BError) as e:
        K.gemv(W, S, x[1:], y, None, 4, 32, "logits")        # x no longer 16-byte aligned
    assert e.value.code == ffi.E_ALIGN


@pytest.mark.parametrize("rows,H", [(1, 1536), (3, 256), (2, 3584), (1, 4100), (5, 40)])
def test_rmsnorm(K, rows, H):
    o = oracle()
    rng = np.random.default_rng(H + rows)
    h = (3 * rng.standard_normal((rows, H))).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    out = torch.empty(rows, H, dtype=torch.float16, device="cuda")
    K.rms(dev(h), dev(w), out, 1e-6)
    ref = o.rmsnorm(h, w, 1e-6)
    got = out.float().cpu().numpy()
    assert nerr(got, ref) < TOL
    # 16-bit rounding may differ by one unit in the last place on a few elements, never more
    ulp = np.abs(got.astype(np.float16).view(np.int16).astype(np.int32) - ref.astype(np.float16).view(np.int16).astype(np.int32))
    assert ulp.max() <= 1 and (ulp > 0).mean() < 0.01


def test_embed(K):
    rng = np.random.default_rng(5)
    E = (0.02 * rng.standard_normal((1000, 256))).astype(np.float16)
    tok = np.array([0, 999, 17, 2 ** 40, -3], np.int64)              # out-of-range ids are clamped
    h = torch.empty(5, 256, device="cuda")
    K.embed(dev(E), dev(tok), h)
    ref = E[np.clip(tok, 0, 999)].astype(np.float32)
    assert np.array_equal(h.cpu().numpy(), ref)


@pytest.mark.parametrize("rows,V", [(1, 151936), (3, 1000), (2, 63), (8, 4096)])
def test_argmax_lowest_index_tie_rule(K, rows, V):
    rng = np.random.default_rng(V)
    lg = rng.standard_normal((rows, V)).astype(np.float32)
    top = lg.max()
    lg[0, [V // 3, V // 2, V - 1]] = top + 1.0                        # three-way tie: the lowest index wins
    if rows > 1:
        lg[1, :] = -5.0                                              # all equal: index 0
    tok = torch.full((rows,), -1, dtype=torch.long, device="cuda")
    pos = torch.arange(rows, dtype=torch.long, device="cuda") * 10
    ws = K.head_workspace(V, rows, "cuda")
    for rep in range(2):                                             # twice: the counters reset themselves
        K.finish(dev(lg), tok, pos, ws)
        assert tok.cpu().tolist() == [int(np.argmax(r)) for r in lg]
        assert pos.cpu().tolist() == [10 * r + rep + 1 for r in range(rows)]
    assert int(ws.view(torch.int32)[:rows].abs().sum()) == 0


@pytest.mark.parametrize("V,H", [(151936, 1536), (1000, 256), (4099, 512), (33, 64)])
def test_head_f16_argmax(K, V, H):
    o = oracle()
    rng = np.random.default_rng(V + H)
    E = (0.02 * rng.standard_normal((V, H))).astype(np.float16)
    x = rng.standard_normal(H).astype(np.float16)
    ref = E.astype(np.float64) @ x.astype(np.float64)
    logits = torch.empty(V, device="cuda")
    tok = torch.zeros(1, dtype=torch.long, device="cuda")
    pos = torch.full((1,), 7, dtype=torch.long, device="cuda")
    ws = K.head_workspace(V, 1, "cuda")
    Ed, xd = dev(E), dev(x)
    for rep in range(2):
        K.head_argmax(Ed, xd, logits, tok, pos, ws)
        got = logits.cpu().numpy()
        assert nerr(got, ref) < 1e-5
        assert int(tok.item()) == int(np.argmax(got))                # lowest index among the maxima of what it wrote
        assert int(pos.item()) == 8 + rep
    assert int(tok.item()) == o.argmax_lowest(ref) or abs(ref[int(tok.item())] - ref.max()) < 1e-5 * abs(ref).max()


def _attn_case(K, B, NH, NKV, HD, max_len, positions, seed):
    o = oracle()
    s = pkg("synth")
    rng = np.random.default_rng(seed)
    cfg = s.ModelConfig("t", 1, NH * HD, 64, NH, NKV, HD, 100)
    cos, sin = s.rope_tables(cfg, max_len)
    kc = rng.standard_normal((B, NKV, max_len, HD)).astype(np.float16)
    vc = rng.standard_normal((B, NKV, max_len, HD)).astype(np.float16)
    qkv = rng.standard_normal((B, (NH + 2 * NKV) * HD)).astype(np.float16)
    pos = np.asarray(positions, np.int64)
    kcd, vcd = dev(kc), dev(vc)
    out = torch.full((B, NH * HD), float("nan"), dtype=torch.float16, device="cuda")
    ws = K.attn_workspace(B, NH, HD, max_len, "cuda")
    scale = 1.0 / np.sqrt(HD)
    K.attn(dev(qkv), dev(cos), dev(sin), dev(pos), kcd, vcd, out, NH, NKV, HD, max_len, scale, ws)
    torch.cuda.synchronize()
    got = out.float().cpu().numpy()
    kc_ref, vc_ref = kc.copy(), vc.copy()
    for b in range(B):
        p = int(pos[b])
        q = o.rope_rotate(qkv[b, :NH * HD].reshape(NH, HD), cos[p], sin[p])
        kc_ref[b, :, p] = o.rope_rotate(qkv[b, NH * HD:(NH + NKV) * HD].reshape(NKV, HD), cos[p], sin[p]).astype(np.float16)
        vc_ref[b, :, p] = qkv[b, (NH + NKV) * HD:].reshape(NKV, HD)
        ref = o.attn_decode(q, kc_ref[b], vc_ref[b], p + 1, scale).reshape(-1)
        assert nerr(got[b], ref) < TOL, (b, p)
    # the cache holds the appended K/V and nothing else changed
    kg, vg = kcd.cpu().numpy(), vcd.cpu().numpy()
    assert np.array_equal(vg, vc_ref)
    dk = np.abs(kg.view(np.int16).astype(np.int32) - kc_ref.view(np.int16).astype(np.int32))
    assert dk.max() <= 1                                             # rotated K: one fp16 ulp at most (fp32 vs float64 rope)
    assert int(ws.view(torch.int32)[:B * NH].abs().sum()) == 0       # counters back to zero
    return got


@pytest.fixture(params=["cached", "streaming"])
def batched_kernel(request):
    """Both kernels that serve several sequences: the shared-memory-resident form (default where max_len <= 2048) and the
    streaming tensor-core kernel."""
    ffi = pkg("_ffi")
    ffi.call("q4b_attn_batched_kernel", 1 if request.param == "streaming" else 0)
    yield request.param
    ffi.call("q4b_attn_batched_kernel", 0)


@pytest.mark.parametrize("pos", [0, 1, 127, 128, 129, 511, 767, 1023])
def test_attn_decode_qwen_shape(K, pos):
    _attn_case(K, 1, 12, 2, 128, 1024, [pos], pos)


@pytest.mark.parametrize("NH,NKV,HD", [(4, 2, 64), (7, 1, 128), (14, 2, 128), (8, 8, 64), (8, 1, 128), (6, 2, 64)])
def test_attn_decode_head_groups(K, NH, NKV, HD, batched_kernel):
    _attn_case(K, 3, NH, NKV, HD, 300, [0, 130, 299], NH * HD)


def test_attn_decode_repeatable(K, batched_kernel):
    a = _attn_case(K, 2, 12, 2, 128, 2048, [2047, 1000], 11)
    b = _attn_case(K, 2, 12, 2, 128, 2048, [2047, 1000], 11)
    assert np.array_equal(a, b)


def test_attn_decode_batched_ragged_positions(K, batched_kernel):
    """32 sequences at different positions (tile and chunk boundaries of the tensor-core kernel: 64-position tiles,
    chunks of max_len / 8 rounded to tiles), Qwen2.5-1.5B head shape."""
    positions = [0, 1, 62, 63, 64, 65, 127, 128, 159, 160, 161, 191, 192, 319, 320, 321, 479, 480, 639, 640, 641, 799, 800, 959,
                 960, 1000, 1023, 1024, 1119, 1120, 1278, 1279]
    _attn_case(K, 32, 12, 2, 128, 1280, positions, 5)


def test_attn_decode_batched_long_context(K):
    """Chunks of several tiles (max_len 4100 -> 576-position chunks) and a 7-head group."""
    _attn_case(K, 4, 14, 2, 128, 4100, [4099, 2048, 5, 3000], 9)


@pytest.mark.parametrize("B,NH,NKV,positions", [(3, 12, 2, [0, 130, 299]), (8, 4, 2, [5, 64, 100, 191, 192, 200, 250, 299]),
                                                (2, 16, 2, [17, 298]), (2, 14, 2, [3, 200])])
def test_attn_decode_fused_q8_equals_attention_then_quantiser(K, B, NH, NKV, positions, batched_kernel):
    """The attention entry with the fused Q8_1 quantiser writes exactly what the same kernel's attention followed by the
    quantiser launch writes, for the shared-memory-resident kernel (every head group) and the streaming one (head groups
    whose 32-value blocks fall inside a cluster CTA's share; otherwise it reports that it has no fused form)."""
    QB = pkg("qwen_batched")
    s = pkg("synth")
    HD, max_len = 128, 300
    rng = np.random.default_rng(B * 100 + NH)
    cfg = s.ModelConfig("t", 1, NH * HD, 64, NH, NKV, HD, 100)
    cos, sin = s.rope_tables(cfg, max_len)
    kc = rng.standard_normal((B, NKV, max_len, HD)).astype(np.float16)
    vc = rng.standard_normal((B, NKV, max_len, HD)).astype(np.float16)
    qkv = dev(rng.standard_normal((B, (NH + 2 * NKV) * HD)).astype(np.float16))
    pos = dev(np.asarray(positions, np.int64))
    scale = 1.0 / np.sqrt(HD)
    nq = NH * HD
    outs = []
    for fused in (False, True):
        kcd, vcd = dev(kc), dev(vc)
        out = torch.zeros(B, nq, dtype=torch.float16, device="cuda")
        xq = torch.zeros(B * nq, dtype=torch.int8, device="cuda")
        xd = torch.zeros(B * nq // 32, dtype=torch.float16, device="cuda")
        if fused:
            ok = K.attn_q8(qkv, dev(cos), dev(sin), pos, kcd, vcd, out, xq, xd, NH, NKV, HD, max_len, scale)
            if batched_kernel == "streaming" and (NH // NKV) * HD % 256:
                assert not ok                      # no fused form for this head group there: the caller falls back
                return
            assert ok
        else:
            K.attn(qkv, dev(cos), dev(sin), pos, kcd, vcd, out, NH, NKV, HD, max_len, scale, K.attn_workspace(B, NH, HD, max_len, "cuda"))
            QB.quant_q8(out, xq, xd)
        torch.cuda.synchronize()
        outs.append((out.clone(), xq.clone(), xd.clone(), kcd, vcd))
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a, b)
