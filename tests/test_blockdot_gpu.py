"""Per-block int32 dot products from the tcgen05 int8 path must equal the oracle's exactly (bit-exact item of the
parity contract), for both operand placements and every tile width."""
import numpy as np
import pytest

from conftest import oracle, pkg

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def case(M, K, P, mode, seed=0, extreme=False):
    o = oracle()
    rng = np.random.default_rng(seed + M + K + P)
    W = rng.integers(0, 2 ** 32, size=(M, K // 8), dtype=np.uint32)
    xq = rng.integers(-127, 128, size=(P, K), dtype=np.int8)
    if extreme:                      # largest magnitudes: nibble 0 (weight -8) against -127 / +127
        W[: M // 2] = 0
        W[M // 2:] = 0xFFFFFFFF
        xq[0::2] = -127
        xq[1::2] = 127
    W = W.view(np.int32)
    QB = pkg("qwen_batched")
    got = QB.blockdot(torch.from_numpy(W).cuda(), torch.from_numpy(xq).cuda(), M, K, mode).cpu().numpy()
    want = o.blockdot(W, xq)
    assert got.shape == want.shape
    bad = np.argwhere(got != want)
    assert bad.size == 0, f"{len(bad)} mismatches, first {bad[:4].tolist()} got {got[tuple(bad[0])]} want {want[tuple(bad[0])]}"


@pytest.mark.parametrize("a_tmem", [0, 1])
@pytest.mark.parametrize("nt", [8, 16, 32])
def test_blockdot_exact_one_tile(a_tmem, nt):
    case(128, 64, nt, a_tmem | (nt << 1))


@pytest.mark.parametrize("a_tmem", [0, 1])
@pytest.mark.parametrize("M,K,P", [(128, 32, 1), (100, 96, 5), (300, 256, 19), (1536, 1536, 8), (256, 8960, 33)])
def test_blockdot_exact_ragged(a_tmem, M, K, P):
    case(M, K, P, a_tmem)


@pytest.mark.parametrize("a_tmem", [0, 1])
def test_blockdot_extreme_values(a_tmem):
    case(256, 128, 16, a_tmem, extreme=True)


@pytest.mark.parametrize("a_tmem", [0, 1])
def test_blockdot_reference_known_answer_inputs(golden, a_tmem):
    """The seeded int8 operands of the reference's own tensor-core known-answer check
    (lab/experiments/tensor.py:171-179; exact equality required there) through the tcgen05 block-dot entry: the low
    nibble of A8 is the Q4_0 weight (nibble - 8), B8 the int8 activations, one 32-wide block."""
    g = golden["tensor_s8_known_answer"]
    A8, B8 = g["A8"].astype(np.int32), g["B8"]
    nib = (A8 & 15).astype(np.uint8)
    W = pkg("gguf").pack_nibbles(nib)
    xq = np.ascontiguousarray(B8.T)                                 # [8 columns, 32]
    got = pkg("qwen_batched").blockdot(torch.from_numpy(W).cuda(), torch.from_numpy(xq).cuda(), 16, 32, a_tmem).cpu().numpy()
    assert np.array_equal(got[:, :, 0].T, (nib.astype(np.int32) - 8) @ B8.astype(np.int32))
