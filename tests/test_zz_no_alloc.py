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
    run_both(gpu, rng, B=2, H=32, Hkv=8, D=128, L=3000, stride=3008)    # nine key splits per sequence and kv head: 74,880 floats of partial records
    run_both(gpu, rng, B=3, H=16, Hkv=4, D=64, L=200, stride=256)       # fewer, smaller records over the same area
    from skainet_b200 import _lib
    assert _lib.lib().skainet_cuda_device_status() == 0


def test_noalloc_refuses_sizes_beyond_the_builtin_area(gpu):
    # batch 128 x 64 heads needs 128*64*1*130 floats of partials > 2^20 even unsplit: refused, nothing launched
    dummy = gpu.DeviceBuffer(1 << 16)
    with pytest.raises(ValueError, match="built-in area"):
        gpu.attn_decode_noalloc(dummy.ptr, dummy.ptr, dummy.ptr, dummy.ptr, 128, 64, 8, 128, 32768, dummy.ptr, 32768, 0.088)


def test_noalloc_allocates_nothing_at_the_capacity_edge_and_with_a_window(gpu):
    """The property the entry exists for, checked directly: after one warm-up call (which resolves the array's address),
    calls of growing size leave the device's free memory where it was, while the ordinary entry grows its scratch on
    the same sizes. Also: a windowed call, and the capacity rule at its edge (126 x 64 heads x 1 split x 130 floats
    = 1,048,320 fits the 2^20-float area, 127 x 64 does not)."""
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(7)

    def make(B, H, Hkv, D, L):
        q = rng.standard_normal((B, H, D)).astype(np.float32)
        k = rng.standard_normal((B, Hkv, L, D)).astype(np.float16); v = rng.standard_normal((B, Hkv, L, D)).astype(np.float16)
        bufs = [gpu.DeviceBuffer.from_host(a) for a in (q, k, v, np.full(B, L, np.int32))]
        return q, bufs + [gpu.DeviceBuffer(q.nbytes), gpu.DeviceBuffer(q.nbytes)]

    shapes = [(1, 8, 2, 64, 300), (1, 32, 8, 128, 2000), (2, 64, 8, 128, 4000), (1, 64, 8, 128, 9000)]
    made = [make(*s) for s in shapes]                      # every input and output buffer exists before anything is measured
    q0, b0 = made[0]
    gpu.attn_decode_noalloc(b0[0].ptr, b0[1].ptr, b0[2].ptr, b0[4].ptr, *shapes[0][:4], shapes[0][4], b0[3].ptr, shapes[0][4], 0.125)
    gpu.sync()
    free_before = torch.cuda.mem_get_info(0)[0]
    for (B, H, Hkv, D, L), (q, b) in zip(shapes, made):
        sc = float(1.0 / np.sqrt(D))
        gpu.attn_decode_noalloc(b[0].ptr, b[1].ptr, b[2].ptr, b[4].ptr, B, H, Hkv, D, L, b[3].ptr, L, sc)
        gpu.attn_decode_noalloc(b[0].ptr, b[1].ptr, b[2].ptr, b[5].ptr, B, H, Hkv, D, L, b[3].ptr, L, sc, window=77)
    gpu.sync()
    assert torch.cuda.mem_get_info(0)[0] == free_before, "the allocation-free entry changed the device's free memory"
    for (B, H, Hkv, D, L), (q, b) in zip(shapes, made):   # same results as the ordinary entry, plain and windowed
        sc = float(1.0 / np.sqrt(D))
        ref = gpu.DeviceBuffer(q.nbytes)
        gpu.attn_decode(b[0].ptr, b[1].ptr, b[2].ptr, ref.ptr, B, H, Hkv, D, L, b[3].ptr, L, sc)
        np.testing.assert_array_equal(b[4].download(np.float32, q.size), ref.download(np.float32, q.size))
        gpu.attn_decode(b[0].ptr, b[1].ptr, b[2].ptr, ref.ptr, B, H, Hkv, D, L, b[3].ptr, L, sc, window=77)
        np.testing.assert_array_equal(b[5].download(np.float32, q.size), ref.download(np.float32, q.size))
    # the capacity rule at its edge
    _, e = make(126, 64, 8, 128, 16)
    gpu.attn_decode_noalloc(e[0].ptr, e[1].ptr, e[2].ptr, e[4].ptr, 126, 64, 8, 128, 16, e[3].ptr, 16, 0.088)
    with pytest.raises(ValueError, match="built-in area"):
        gpu.attn_decode_noalloc(e[0].ptr, e[1].ptr, e[2].ptr, e[4].ptr, 127, 64, 8, 128, 16, e[3].ptr, 16, 0.088)
    # heads per kv head outside {1, 2, 4, 8} is refused by the launcher, not silently mishandled
    with pytest.raises(ValueError):
        gpu.attn_decode_noalloc(e[0].ptr, e[1].ptr, e[2].ptr, e[4].ptr, 1, 12, 4, 128, 16, e[3].ptr, 16, 0.088)
