import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def _has_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device in this environment")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def kat():
    with open(os.path.join(GOLDEN, "reference_kat.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def golden_steps():
    return np.load(os.path.join(GOLDEN, "mlp_small_steps.npz"))


@pytest.fixture(scope="session")
def oc():
    from oracle import oracle_c
    oracle_c.load()
    return oracle_c


@pytest.fixture(scope="session")
def ctx():
    import rstorch_b200 as rt
    c = rt.Context(0)
    yield c
    c.synchronize()
    c.check_device()


def rel_err(a, b) -> float:
    """max|a-b| / max|b|: the per-tensor relative error the 1e-9 bar is judged on."""
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    assert a.shape == b.shape, (a.shape, b.shape)
    if a.size == 0:
        return 0.0
    denom = np.max(np.abs(b))
    num = np.max(np.abs(a - b))
    if denom == 0.0:
        return float(num)
    return float(num / denom)


REL_TOL = 1e-9   # BASELINE north_star: loss, gradients, updated weights within relative 1e-9
