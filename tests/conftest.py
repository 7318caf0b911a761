import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# Tolerances of the parity tests.  BASELINE.json: rtol 1e-4 for fp32, 2e-2 for fp16 with fp32
# accumulation.  The reference always pairs its rtol with an absolute term
# (daceml/testing/utils.py:54: rtol 1e-5 / atol 1e-4); the absolute terms here are one fp32 /
# fp16 rounding step of an O(1) value.
RTOL = {torch.float32: 1e-4, torch.float16: 2e-2}
ATOL = {torch.float32: 1e-5, torch.float16: 2e-3}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def assert_close(got, ref, dtype=None, rtol=None, atol=None, what=""):
    """Element-wise |got - ref| <= atol + rtol * |ref| on float64 copies."""
    if isinstance(got, torch.Tensor):
        dtype = dtype or got.dtype
        got = got.detach().float().cpu().numpy()
    if isinstance(ref, torch.Tensor):
        ref = ref.detach().float().cpu().numpy()
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    dtype = dtype or torch.float32
    rtol = RTOL[dtype] if rtol is None else rtol
    atol = ATOL[dtype] if atol is None else atol
    err = np.abs(got - ref)
    bound = atol + rtol * np.abs(ref)
    bad = err > bound
    if bad.any():
        i = np.unravel_index(np.argmax(err - bound), err.shape)
        raise AssertionError(f"{what}: {bad.sum()} of {bad.size} elements out of tolerance (rtol {rtol}, atol {atol}); "
                             f"worst at {i}: got {got[i]}, ref {ref[i]}")


@pytest.fixture
def rng():
    return np.random.default_rng(20240611)


@pytest.fixture
def device():
    return torch.device("cuda:0")
