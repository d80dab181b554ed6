import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


def _has_gpu() -> bool:
    try:
        from juno_b200.matvec import GpuContext
        return GpuContext.device_count() > 0
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


def rel_err(got, ref) -> float:
    """max|got-ref| / max|ref| — the norm-wise relative error the parity bar (1e-3) is stated in."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as o
    o.build()
    return o


@pytest.fixture(scope="session")
def ctx():
    from juno_b200.matvec import GpuContext
    return GpuContext.shared(0)


@pytest.fixture(scope="session")
def mv(ctx):
    from juno_b200.matvec import B200MatVec
    return B200MatVec(ctx)
