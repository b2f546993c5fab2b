"""Shared fixtures.  Tests marked ``gpu`` need a B200; everything else runs on CPU."""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (numpy front end over oracle/exl3_oracle.c)."""
    from oracle import exl3_oracle

    exl3_oracle.lib()
    return exl3_oracle


@pytest.fixture(scope="session")
def golden():
    """Golden vectors produced by the reference (tests/golden/make_golden.py)."""
    return {name: np.load(GOLDEN / f"{name}.npz") for name in
            ("codebook", "trellis", "tiles", "hadamard", "forward")}


def synthetic_layer(k: int, in_features: int, out_features: int, seed: int, *, bias: bool = False):
    """Seeded synthetic layer: arbitrary uint16 bitstream (every bitstream is a
    valid tail-biting tile), random +-1 sign vectors, as the benchmark uses."""
    rng = np.random.default_rng(seed)
    trellis = rng.integers(0, 65536, size=(in_features // 16, out_features // 16, 16 * k),
                           dtype=np.uint16)
    suh = np.where(rng.random(in_features) > 0.5, -1.0, 1.0).astype(np.float16)
    svh = np.where(rng.random(out_features) > 0.5, -1.0, 1.0).astype(np.float16)
    b = (rng.standard_normal(out_features) * 0.01).astype(np.float16) if bias else None
    return trellis, suh, svh, b


def rel_err(a: np.ndarray, b: np.ndarray) -> float:
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))
