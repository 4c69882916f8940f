import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden", "sdpa_golden.npz")

# Tolerances of the path (stated by the task for this kernel family):
#   fp32 kernels vs the CPU reference: max-abs <= 1e-5
#   fp16 inputs, fp32 accumulation:    max-abs <= 2e-3 and relative <= 1e-2, where
#   "relative" is the error norm over the output norm, ||got-ref|| / ||ref||
FP32_ATOL = 1e-5
FP16_ATOL = 2e-3
FP16_REL = 1e-2


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    return np.load(GOLDEN)


def seeded(seed, *shape):
    """Same generator as tests/golden/make_golden.py."""
    return np.random.Generator(np.random.PCG64(seed)).standard_normal(shape, dtype=np.float32)


def assert_close_fp32(got, ref, atol=FP32_ATOL):
    assert got.shape == ref.shape
    nan_ref = np.isnan(ref)
    assert np.array_equal(np.isnan(got), nan_ref), "NaN rows differ from the reference"
    err = np.abs(got[~nan_ref] - ref[~nan_ref])
    assert err.size == 0 or float(err.max()) <= atol, f"max-abs {float(err.max()):.3e} > {atol}"


def assert_close_fp16(got, ref, atol=FP16_ATOL, rel=FP16_REL):
    assert got.shape == ref.shape
    assert np.isfinite(got).all(), "non-finite values in the kernel output"
    err = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    assert float(err.max()) <= atol, f"max-abs {float(err.max()):.3e} > {atol}"
    r = float(np.linalg.norm(err.ravel()) / max(np.linalg.norm(ref.astype(np.float64).ravel()), 1e-30))
    assert r <= rel, f"relative error {r:.3e} > {rel}"
