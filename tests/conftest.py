"""Shared fixtures. `-m gpu` tests need a B200 and call the kernels through the C ABI; everything else
runs on CPU (oracle pinning, host logic, ABI surface)."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import ref as R
    R.port()
    return R


@pytest.fixture(scope="session")
def cuda_lib():
    """The built C-ABI library; builds it in-tree if it is missing or stale."""
    from skainet_b200 import build, _lib
    build.build()
    return _lib.lib()


@pytest.fixture(scope="session")
def gpu(cuda_lib):
    """Fails (not skips) when a test marked gpu runs without a usable device: no silent fallback."""
    n = cuda_lib.skainet_cuda_device_count()
    assert n > 0, "test marked gpu but no CUDA device is visible"
    from skainet_b200 import device
    device.set_device(0)
    return device


def rel_err_ok(got: np.ndarray, ref: np.ndarray, rtol: float = 1e-3) -> None:
    """The parity bar for floating-point outputs: |got - ref| <= rtol * max(|ref|, rms(ref)) for every
    element (the scale-aware form of the reference's own `diff <= atol or rel < rtol` check,
    NativeQ4KMatmulKernelParityTest.kt:125-134)."""
    got = np.asarray(got, dtype=np.float64).reshape(-1)
    ref = np.asarray(ref, dtype=np.float64).reshape(-1)
    assert got.shape == ref.shape
    assert np.all(np.isfinite(got)), "non-finite output"
    rms = float(np.sqrt(np.mean(ref * ref))) if ref.size else 0.0
    bound = rtol * np.maximum(np.abs(ref), rms) + 1e-30
    bad = np.abs(got - ref) > bound
    assert not bad.any(), (
        f"{int(bad.sum())}/{ref.size} elements outside rel {rtol}: worst |d|={np.abs(got - ref).max():.3e}, rms(ref)={rms:.3e}")
