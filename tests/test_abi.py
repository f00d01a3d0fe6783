"""CPU: the C-ABI library builds for sm_100a, loads, and exports every symbol include/*.h declares.
No compute call is made here unless it is expected to fail before touching a device."""
import ctypes as C
import glob
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        names |= set(re.findall(r"\b(skainet_cuda_\w+)\s*\(", open(h).read()))
    return sorted(names)


def test_header_declares_the_drop_in_twins():
    names = declared_symbols()
    for twin in ("smoke_double", "q4k_matmul", "q4k_matmul_rm", "q8_0_matmul", "q8_0_matmul_rm", "q6k_matmul", "q6k_matmul_rm", "q5k_matmul", "q5k_matmul_rm",
                 "f32_rms_norm", "f32_sdpa"):
        assert "skainet_cuda_" + twin in names


def test_library_exports_every_declared_symbol(cuda_lib):
    for name in declared_symbols():
        assert hasattr(cuda_lib, name), f"libskainet_cuda.so lacks {name}"


def test_python_binding_covers_every_declared_symbol():
    from skainet_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_every_declaration_cites_what_it_replaces():
    text = open(os.path.join(ROOT, "include", "skainet_cuda.h")).read()
    for twin in ("smoke_double", "q4k_matmul", "q4k_matmul_rm", "q8_0_matmul", "q8_0_matmul_rm", "q6k_matmul", "q6k_matmul_rm", "q5k_matmul", "q5k_matmul_rm",
                 "f32_rms_norm", "f32_sdpa"):
        i = text.index("skainet_cuda_" + twin + "(")
        assert "skainet_kernels.h:" in text[max(0, i - 900):i], twin


def test_invalid_dims_raise_before_any_device_work(cuda_lib):
    # Q4KMatmulKernel contract: inputDim % 256 != 0 -> IllegalArgumentException (NativeQ4KMatmulKernelParityTest.kt:179-190)
    from skainet_b200.provider import CudaQ4KMatmulKernel, CudaQ8_0MatmulKernel
    x = np.zeros(300, np.float32); w = np.zeros(4 * 144 * 2, np.uint8); out = np.zeros(4, np.float32)
    with pytest.raises(ValueError, match="multiple of 256"):
        CudaQ4KMatmulKernel().matmul(x, 0, w, 0, 300, 4, out, 0)
    with pytest.raises(ValueError, match="multiple of 32"):
        CudaQ8_0MatmulKernel().matmul(x, 0, w, 0, 33, 4, out, 0)
    from skainet_b200.provider import CudaQ6KMatmulKernel, CudaQ5KMatmulKernel
    for kern in (CudaQ6KMatmulKernel(), CudaQ5KMatmulKernel(), CudaQ6KMatmulKernel(row_major=True), CudaQ5KMatmulKernel(row_major=True)):
        with pytest.raises(ValueError, match="multiple of 256"):
            kern.matmul(x, 0, w, 0, 300, 4, out, 0)


def test_zero_dims_keep_each_formats_edge_behaviour(cuda_lib):
    # inputDim == 0: Q8_0 zeroes the output (q8_0_matmul.c:175-179), native Q4_K leaves it (q4k_matmul.c:326)
    from skainet_b200.provider import CudaQ4KMatmulKernel, CudaQ8_0MatmulKernel
    x = np.zeros(1, np.float32); w = np.zeros(1, np.uint8)
    out = np.full(3, 7.0, np.float32)
    CudaQ4KMatmulKernel().matmul(x, 0, w, 0, 0, 3, out, 0)
    assert (out == 7.0).all()
    CudaQ8_0MatmulKernel().matmul(x, 0, w, 0, 0, 3, out, 0)
    assert (out == 0.0).all()
    # the other K-quant kernels return early like Q4_K (q6k_matmul.c:284, q5k_matmul.c:264)
    from skainet_b200.provider import CudaQ6KMatmulKernel, CudaQ5KMatmulKernel
    out[:] = 7.0
    CudaQ6KMatmulKernel().matmul(x, 0, w, 0, 0, 3, out, 0)
    CudaQ5KMatmulKernel(row_major=True).matmul(x, 0, w, 0, 0, 3, out, 0)
    assert (out == 7.0).all()


def test_no_gpu_means_unavailable_not_fallback(cuda_lib):
    from skainet_b200 import _lib
    from skainet_b200.provider import CudaKernelProvider
    p = CudaKernelProvider()
    if cuda_lib.skainet_cuda_device_count() > 0:
        assert p.isAvailable()
        return
    assert not p.isAvailable() and p.matmulQ4K() is None and not p.supports("matmul", ["Float32", "Q4_K"])
    assert p.matmulQ6K() is None and p.matmulQ5K() is None and not p.supports("matmul", ["Float32", "Q6_K"])
    x = np.ones(4, np.float32); out = np.zeros(4, np.float32)
    st = cuda_lib.skainet_cuda_smoke_double(x.ctypes.data_as(_lib.f32p), out.ctypes.data_as(_lib.f32p), 4)
    assert st == _lib.ERR_NODEVICE and not out.any()
    assert "no usable CUDA device" in _lib.last_error() or "no CUDA device" in _lib.last_error()


def test_bad_handle_is_an_error_status(cuda_lib):
    from skainet_b200 import _lib
    out = (C.c_int64 * 4)()
    assert cuda_lib.skainet_cuda_weight_info(12345, out) == _lib.ERR_HANDLE
    assert cuda_lib.skainet_cuda_weight_free(0) == _lib.ERR_HANDLE


def test_provider_supports_table():
    from skainet_b200.provider import CudaKernelProvider
    p = CudaKernelProvider()
    assert not p.supports("matmul", ["Float32", "Float32"])
    assert not p.supports("softmax", ["Float32"])
    assert not p.supports("matmul", ["Q8_0", "Q8_0"])
    assert p.priority > 100
