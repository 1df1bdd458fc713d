"""Shared fixtures.  Tests that need a GPU are marked `gpu`; everything else runs on CPU."""
import importlib
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pkg(sub: str = ""):
    """Import the product package (its directory name starts with a digit)."""
    return importlib.import_module("3080lab_b200" + ("." + sub if sub else ""))


def oracle():
    return importlib.import_module("oracle.q4ref")


def gemv_inputs(n: int, k: int, bf16_x: bool = False):
    """Input recipe of the reference's GEMV microbenchmark (lab/experiments/gemv5.py:40-46)."""
    rng = np.random.default_rng(n + k)
    q = rng.integers(0, 16, size=(n, k), dtype=np.uint32)
    d = rng.uniform(0.002, 0.02, size=(n, k // 32)).astype(np.float16)
    x = rng.standard_normal(k).astype(np.float32)
    if bf16_x:
        x = ((x.view(np.uint32) >> 16) << 16).view(np.float32)
    return q.astype(np.uint8), d, x


@pytest.fixture(scope="session")
def golden():
    return {p.stem: np.load(p, allow_pickle=False) for p in GOLDEN.glob("*.npz")}
