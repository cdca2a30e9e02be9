"""Shared test set-up: import paths, the `gpu` marker, fixtures for golden vectors and the GPU."""

from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import pytest

REPO = Path(__file__).resolve().parent.parent
PACKAGE = REPO / "5_b200"
GOLDEN = REPO / "tests" / "golden"
# Checkout of the reference project, for the few tests that run its own code (skipped without it)
# and for tests/golden/make_golden.py: $HC_REFERENCE_DIR, else this location.
REFERENCE = Path(os.environ.get("HC_REFERENCE_DIR") or "/root/reference")

for entry in (str(REPO), str(PACKAGE)):
    if entry not in sys.path:
        sys.path.insert(0, entry)


def pytest_configure(config: pytest.Config) -> None:
    config.addinivalue_line("markers", "gpu: needs a B200 (run with `-m gpu` on the GPU box)")


def load_golden(name: str) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """(A, B, C) of a fixture written by tests/golden/make_golden.py."""
    with np.load(GOLDEN / f"{name}.npz") as data:
        dtype = np_dtype(str(data["dtype"]))
        return data["a_bits"].view(dtype), data["b_bits"].view(dtype), data["c"]


GOLDEN_NAMES = sorted(p.stem for p in GOLDEN.glob("sim_*.npz"))


@pytest.fixture(scope="session")
def gpu_ctx():
    """Context of GPU 0; the tests that use it are marked `gpu`."""
    from hc import cuda

    ctx = cuda.default_context(0)
    yield ctx


def np_dtype(name: str):
    if name in ("bfloat16", "float8_e4m3fn", "float8_e5m2"):
        import ml_dtypes

        return getattr(ml_dtypes, name)
    return np.dtype(name).type
