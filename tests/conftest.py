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
def layout_host():
    """Test-only host build (C++ compiler, no CUDA) of the tile-layout index maps the device kernels use."""
    import ctypes as C
    import subprocess
    src = os.path.join(ROOT, "tests", "native", "layout_host.cpp")
    so = os.path.join(ROOT, "tests", "native", "liblayout_host.so")
    deps = [src] + [os.path.join(ROOT, "juno_b200", "csrc", f) for f in ("layout.cuh", "dequant.cuh", "repack.cuh")]
    if not os.path.exists(so) or os.path.getmtime(so) < max(os.path.getmtime(d) for d in deps):
        subprocess.check_call(["g++", "-O2", "-std=c++17", "-ffp-contract=off", "-shared", "-fPIC", "-o", so, src])
    L = C.CDLL(so)
    L.layout_tiled_bytes.restype = C.c_int64
    L.layout_tiled_bytes.argtypes = [C.c_int, C.c_int64, C.c_int64]
    L.layout_repack.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]
    L.layout_dequant_tiled.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]
    return L


@pytest.fixture(scope="session")
def ctx():
    from juno_b200.matvec import GpuContext
    return GpuContext.shared(0)


@pytest.fixture(scope="session")
def mv(ctx):
    from juno_b200.matvec import B200MatVec
    return B200MatVec(ctx)
