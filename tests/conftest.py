import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


def _have_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _have_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Output tolerance of the attention path against Granite's CPU arithmetic:
# max |gpu - ref| <= 2e-3 and max |gpu - ref| / max(|ref|, 1e-3) <= 1e-2.
ABS_TOL = 2e-3
REL_TOL = 1e-2
REL_FLOOR = 1e-3


def assert_attention_close(got: np.ndarray, ref: np.ndarray, what: str = "") -> tuple[float, float]:
    got = np.asarray(got, np.float32)
    ref = np.asarray(ref, np.float32)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    diff = np.abs(got - ref)
    max_abs = float(diff.max()) if diff.size else 0.0
    max_rel = float((diff / np.maximum(np.abs(ref), REL_FLOOR)).max()) if diff.size else 0.0
    assert max_abs <= ABS_TOL, f"{what}: max abs error {max_abs:.3e} > {ABS_TOL}"
    assert max_rel <= REL_TOL, f"{what}: max rel error {max_rel:.3e} > {REL_TOL}"
    return max_abs, max_rel


@pytest.fixture(scope="session")
def compute():
    """One compute object on cuda:0, enqueueing on torch's current stream."""
    import torch
    import granite_b200 as g
    torch.cuda.set_device(0)
    c = g.CudaCompute(0, torch.cuda.current_stream().cuda_stream)
    yield c
    c.shutdown()
