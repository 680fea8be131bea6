"""Shared test plumbing: the ``gpu`` marker, fixture loading, tolerances."""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = Path(__file__).resolve().parent / "golden"
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# Tolerance of 16-bit results against the fp32 oracle (the bar the hot path is held to).
BF16_TOL = dict(rtol=2e-2, atol=2e-2)
# fp32 kernels against the oracle.
FP32_TOL = dict(rtol=1e-4, atol=1e-5)
LOSS_REL = 1e-3


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name: str):
    return np.load(GOLDEN / name, allow_pickle=False)


@pytest.fixture(scope="session")
def lib():
    from bastile_b200 import _lib

    return _lib.get_lib()


def to_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def assert_close(actual, expected, rtol, atol, what=""):
    a = to_np(actual) if isinstance(actual, torch.Tensor) else np.asarray(actual, np.float32)
    e = to_np(expected) if isinstance(expected, torch.Tensor) else np.asarray(expected, np.float32)
    assert a.shape == e.shape, f"{what}: shape {a.shape} vs {e.shape}"
    assert np.isfinite(a).all(), f"{what}: non-finite values"
    err = np.abs(a - e)
    bound = atol + rtol * np.abs(e)
    bad = err > bound
    if bad.any():
        i = np.unravel_index(np.argmax(err - bound), err.shape)
        raise AssertionError(
            f"{what}: {int(bad.sum())}/{bad.size} elements off; worst at {i}: got {a[i]!r}, want {e[i]!r} "
            f"(|err| {err[i]:.3e} > {bound[i]:.3e})"
        )
