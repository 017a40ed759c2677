"""Shared fixtures: the `gpu` marker, golden-vector loading and the oracle import."""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

import ml_dtypes  # noqa: E402

BF16 = np.dtype(ml_dtypes.bfloat16)
F16, F32 = np.dtype(np.float16), np.dtype(np.float32)

# (atol, rtol) by output dtype: the reference's own differential-test tolerances (tests/conftest.py:75-79).
TOLERANCES = {F32: (1e-5, 1e-5), F16: (1e-3, 2e-3), BF16: (1e-2, 1.6e-2)}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name: str) -> dict[str, np.ndarray]:
    z = np.load(ROOT / "tests" / "golden" / f"{name}.npz")
    out = {}
    for k in z.files:
        out[k[:-6] if k.endswith("__bf16") else k] = z[k].view(BF16) if k.endswith("__bf16") else z[k]
    return out


def bits(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a)
    return a.view(np.uint16) if a.dtype == BF16 else a


def assert_close(actual, expected, atol=None, rtol=None, what="output"):
    """Equal shape and dtype, then closeness with dtype-aware tolerances; integers must be equal."""
    actual, expected = np.asarray(actual), np.asarray(expected)
    assert actual.shape == expected.shape, f"{what}: shape {actual.shape} != {expected.shape}"
    assert actual.dtype == expected.dtype, f"{what}: dtype {actual.dtype} != {expected.dtype}"
    if actual.dtype.kind in "iub":
        np.testing.assert_array_equal(actual, expected, err_msg=what)
        return
    d_atol, d_rtol = TOLERANCES.get(actual.dtype, (1e-5, 1e-5))
    np.testing.assert_allclose(actual.astype(np.float64), expected.astype(np.float64),
                               atol=d_atol if atol is None else atol, rtol=d_rtol if rtol is None else rtol,
                               equal_nan=True, err_msg=what)


@pytest.fixture(scope="session")
def oracle():
    from oracle import enceladus_oracle

    return enceladus_oracle
