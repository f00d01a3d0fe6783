"""The allocation-free decode-attention entry point, called through the C ABI.

Some hosts of this library may not allocate device memory once they are running: a decode loop held to
a fixed memory plan, a latency-critical thread that cannot afford the device-wide stall inside
cudaMalloc, a process whose allocator hooks forbid it. For them `skainet_cuda_attn_decode_noalloc_dev`
keeps the split-K partial results in a 4 MiB array that is part of the library image instead of in
scratch that grows on demand. This file checks that it returns exactly what the ordinary entry point
returns, twice in a row on different problems (the second smaller, so stale partials of the first call
would show), and that a problem beyond the built-in area is refused before anything is launched.
It is collected last on purpose and passes both alone in a fresh process and after the other tests.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def run_both(gpu, rng, B, H, Hkv, D, L, stride):
    q = rng.standard_normal((B, H, D)).astype(np.float32)
    k = rng.standard_normal((B, Hkv, stride, D)).astype(np.float16)
    v = rng.standard_normal((B, Hkv, stride, D)).astype(np.float16)
    lens = np.array([max(1, L - 29 * b) for b in range(B)], np.int32)
    dq, dk, dv, dl = (gpu.DeviceBuffer.from_host(a) for a in (q, k, v, lens))
    d_ref, d_new = gpu.DeviceBuffer(q.nbytes), gpu.DeviceBuffer(q.nbytes)
    scale = float(1.0 / np.sqrt(D))
    gpu.attn_decode(dq.ptr, dk.ptr, dv.ptr, d_ref.ptr, B, H, Hkv, D, stride, dl.ptr, L, scale)
    gpu.attn_decode_noalloc(dq.ptr, dk.ptr, dv.ptr, d_new.ptr, B, H, Hkv, D, stride, dl.ptr, L, scale)
    ref, new = d_ref.download(np.float32, q.size), d_new.download(np.float32, q.size)
    assert np.isfinite(new).all() and np.abs(ref).max() > 0
    # same kernels, same fixed reduction order: the tolerance of the other attention tests (rel 1e-3) is met with zero error
    np.testing.assert_allclose(new, ref, rtol=1e-3, atol=1e-3 * float(np.sqrt(np.mean(ref ** 2))))
    np.testing.assert_array_equal(new, ref)


def test_noalloc_decode_attention_equals_the_scratch_version_on_two_calls_in_a_row(gpu):
    rng = np.random.default_rng(2024)
    run_both(gpu, rng, B=2, H=32, Hkv=8, D=128, L=3000, stride=3008)    # many key splits: uses a large part of the area
    run_both(gpu, rng, B=3, H=16, Hkv=4, D=64, L=200, stride=256)       # fewer, smaller records over the same area
    from skainet_b200 import _lib
    assert _lib.lib().skainet_cuda_device_status() == 0


def test_noalloc_refuses_sizes_beyond_the_builtin_area(gpu):
    # batch 128 x 64 heads needs 128*64*1*130 floats of partials > 2^20 even unsplit: refused, nothing launched
    dummy = gpu.DeviceBuffer(1 << 16)
    with pytest.raises(ValueError, match="built-in area"):
        gpu.attn_decode_noalloc(dummy.ptr, dummy.ptr, dummy.ptr, dummy.ptr, 128, 64, 8, 128, 32768, dummy.ptr, 32768, 0.088)
