"""The allocation-free greedy pick (scratch inside the library image) against the workspace-based entry point.

The file name sorts last on purpose, because the order of first use matters for a scratch array that lives in the
library image: in a whole-suite run its first call comes after every other kernel of the library has run in the
process, and run alone it is the first call in a fresh process.  Both orders must pass."""
import ctypes

import numpy as np
import pytest

from conftest import pkg

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def test_static_scratch_argmax_matches_workspace_version_twice():
    ffi = pkg("_ffi")
    K = pkg("qwen_kernels")
    K.init(0)
    lib = ffi.lib()
    stream = torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(123)
    for call, (rows, V) in enumerate([(8, 151936), (64, 5000)]):      # two calls in a row share the built-in scratch
        lg = rng.standard_normal((rows, V)).astype(np.float32)
        lg[0, [V // 4, V // 2]] = lg.max() + 1.0                      # a tie: the lowest index must win in both
        lgd = torch.from_numpy(lg).cuda()
        tok_a = torch.full((rows,), -1, dtype=torch.long, device="cuda")
        pos_a = torch.arange(rows, dtype=torch.long, device="cuda")
        tok_b, pos_b = tok_a.clone(), pos_a.clone()
        ws = K.head_workspace(V, rows, "cuda")
        K.finish(lgd, tok_a, pos_a, ws)                               # existing entry point, caller-owned workspace
        ffi.check(lib.q4b_argmax_advance_static(lgd.data_ptr(), rows, V, tok_b.data_ptr(), pos_b.data_ptr(), stream))
        torch.cuda.synchronize()
        assert torch.equal(tok_a, tok_b), f"call {call}: tokens differ"
        assert torch.equal(pos_a, pos_b), f"call {call}: positions differ"
        assert tok_b.cpu().tolist() == [int(np.argmax(r)) for r in lg]


def test_static_scratch_rejects_too_many_rows():
    ffi = pkg("_ffi")
    lib = ffi.lib()
    x = torch.zeros(65, 10, device="cuda")
    rc = lib.q4b_argmax_advance_static(x.data_ptr(), 65, 10, None, None, None)
    assert rc == ffi.E_SHAPE
    assert b"64 rows" in lib.q4b_last_error()
