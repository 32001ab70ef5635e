"""pytest configuration: the `gpu` marker, library builds, shared helpers."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session", autouse=True)
def _native_libs():
    """Build the product library and the CPU oracle if they are stale or missing."""
    from shflbw_sparse_nn_b200.build import build_library
    import oracle_api

    build_library()
    oracle_api.build_oracle()


@pytest.fixture(scope="session")
def golden_dir() -> Path:
    return ROOT / "tests" / "golden"


def assert_close_fp16(got, ref, rel=1e-2, abs_=1e-3, what=""):
    """The parity bar for floating-point outputs: |got - ref| <= max(rel*|ref|, abs_).

    rel = 1e-2 and abs_ = 1e-3 are the stated tolerances of the hot path (fp16 inputs and
    outputs, fp32 accumulation).  fp16 output rounding alone is 2^-11 relative.
    """
    got = np.asarray(got, dtype=np.float32)
    ref = np.asarray(ref, dtype=np.float32)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    err = np.abs(got - ref)
    tol = np.maximum(rel * np.abs(ref), abs_)
    bad = err > tol
    if bad.any():
        idx = np.unravel_index(np.argmax(err - tol), err.shape)
        raise AssertionError(f"{what}: {int(bad.sum())}/{bad.size} elements out of tolerance; worst at {idx}: "
                             f"got {got[idx]} ref {ref[idx]}")
