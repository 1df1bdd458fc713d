"""The prefill MMQ (tcgen05, 128 x 128 tiles, warp-specialised) and the tiled Q8_1 quantisers against the oracle."""
import numpy as np
import pytest

from conftest import oracle, pkg

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


def untile(buf, P, K):
    """Tiled Q8_1 bytes -> (q int8 [P, K], d float32 [P, K/32])."""
    KB = K // 32
    TT = (P + 127) // 128
    b = buf.reshape(TT, KB, 4608)
    i = np.arange(32)
    pos = 4 * (2 * (i >> 3) + (i & 1)) + ((i & 7) >> 1)
    n = np.arange(128)
    off = ((n[:, None] >> 3) * 2 + (pos[None, :] >> 4)) * 128 + (n[:, None] & 7) * 16 + (pos[None, :] & 15)   # [128, 32]
    q = b[:, :, :4096][:, :, off].view(np.int8)                      # [TT, KB, 128, 32]
    q = q.transpose(0, 2, 1, 3).reshape(TT * 128, K)[:P]
    d = b[:, :, 4096:].copy().view(np.float32).reshape(TT, KB, 128).transpose(0, 2, 1).reshape(TT * 128, KB)[:P]
    return q, d


@pytest.fixture(scope="module")
def QB():
    pkg("qwen_kernels").init(0)
    return pkg("qwen_batched")


@pytest.mark.parametrize("P,K", [(1, 256), (130, 1536), (128, 512), (300, 8960)])
def test_quant_tiled_layout(QB, P, K):
    o = oracle()
    rng = np.random.default_rng(P + K)
    x = (rng.standard_normal((P, K)) * rng.uniform(0.01, 30, size=(P, 1))).astype(np.float16)
    xt = QB.q8_tiled_buffer(P, K, "cuda")
    QB.quant_q8_tiled(dev(x), xt)
    q, d = untile(xt.cpu().numpy(), P, K)
    qr, dr, _ = o.quant_q8_1(x)
    assert np.array_equal(q, qr)
    assert np.array_equal(d, dr.astype(np.float32))


def test_rmsnorm_q8_tiled_equals_untiled(QB):
    rng = np.random.default_rng(3)
    P, H = 200, 1536
    h = dev((3 * rng.standard_normal((P, H))).astype(np.float32))
    w = dev((1 + 0.1 * rng.standard_normal(H)).astype(np.float32))
    xt = QB.q8_tiled_buffer(P, H, "cuda")
    QB.rmsnorm_q8_tiled(h, w, xt, 1e-6)
    xq = torch.empty(P, H, dtype=torch.int8, device="cuda")
    xd = torch.empty(P, H // 32, dtype=torch.float16, device="cuda")
    QB.rmsnorm_q8(h, w, xq, xd, 1e-6)
    q, d = untile(xt.cpu().numpy(), P, H)
    assert np.array_equal(q, xq.cpu().numpy())
    assert np.array_equal(d, xd.float().cpu().numpy())


@pytest.mark.parametrize("P,n,k", [(1, 128, 256), (100, 200, 512), (128, 2048, 1536), (300, 1536, 8960), (2048, 512, 1536),
                                   (257, 17920, 1536)])
def test_mmq_prefill_matches_oracle(QB, P, n, k):
    o = oracle()
    rng = np.random.default_rng(P + n + k)
    W, S = rand_q4(rng, n, k)
    x = rng.standard_normal((P, k)).astype(np.float16)
    xq, xd, _ = o.quant_q8_1(x)
    wd = o.dequant(W, S)
    ref = o.mmq_dense(wd, xq, xd)
    xt = QB.q8_tiled_buffer(P, k, "cuda")
    QB.quant_q8_tiled(dev(x), xt)
    Wt, St = QB.pack_q4(dev(W), dev(S))
    st = QB.Status("cuda")
    y = torch.full((P, n), float("nan"), device="cuda")
    QB.gemm8_prefill(Wt, St, xt, y, None, n, k, P, "logits", n, st)
    st.check()
    got = y.cpu().numpy()
    assert nerr(got, ref) < 2e-6
    y2 = torch.empty(P, n, device="cuda")
    QB.gemm8_prefill(Wt, St, xt, y2, None, n, k, P, "logits", n, st)
    st.check()
    assert torch.equal(y, y2), "not bit-repeatable"


def test_mmq_prefill_equals_streaming_kernel(QB):
    """The two tensor-core MMQ kernels (128-column tiles vs the decode streaming kernel) give the same numbers."""
    o = oracle()
    rng = np.random.default_rng(17)
    P, n, k = 32, 1536, 1536
    W, S = rand_q4(rng, n, k)
    x = rng.standard_normal((P, k)).astype(np.float16)
    xq, xd, _ = o.quant_q8_1(x)
    Wt, St = QB.pack_q4(dev(W), dev(S))
    st = QB.Status("cuda")
    a = torch.empty(P, n, device="cuda")
    QB.gemm8(Wt, St, dev(xq), dev(xd), a, None, n, k, P, "logits", n, st)
    xt = QB.q8_tiled_buffer(P, k, "cuda")
    QB.quant_q8_tiled(dev(x), xt)
    b = torch.empty(P, n, device="cuda")
    QB.gemm8_prefill(Wt, St, xt, b, None, n, k, P, "logits", n, st)
    st.check()
    assert nerr(b.cpu().numpy(), a.cpu().numpy()) < 1e-6


def test_mmq_prefill_epilogues(QB):
    o = oracle()
    rng = np.random.default_rng(5)
    P, n, k = 200, 512, 1536
    W, S = rand_q4(rng, n, k)
    x = rng.standard_normal((P, k)).astype(np.float16)
    xq, xd, _ = o.quant_q8_1(x)
    acc = o.mmq(W, S, xq, xd)
    Wt, St = QB.pack_q4(dev(W), dev(S))
    xt = QB.q8_tiled_buffer(P, k, "cuda")
    QB.quant_q8_tiled(dev(x), xt)
    st = QB.Status("cuda")
    bias = (0.1 * rng.standard_normal(n)).astype(np.float32)
    y = torch.empty(P, n, dtype=torch.float16, device="cuda")
    QB.gemm8_prefill(Wt, St, xt, y, dev(bias), n, k, P, "biasf", n, st)
    assert nerr(y.float().cpu().numpy(), o.f16(acc + bias)) < 1e-3
    h0 = rng.standard_normal((P, n)).astype(np.float32)
    h = dev(h0)
    QB.gemm8_prefill(Wt, St, xt, h, None, n, k, P, "resid", n, st)
    assert nerr(h.cpu().numpy(), h0 + acc) < 1e-5
    ys = torch.empty(P, n // 2, dtype=torch.float16, device="cuda")
    QB.gemm8_prefill(Wt, St, xt, ys, None, n, k, P, "swiglu", n // 2, st)
    assert nerr(ys.float().cpu().numpy(), o.silu_mul(acc[:, 0::2], acc[:, 1::2])) < 1e-3
    st.check()
