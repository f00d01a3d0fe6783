"""GPU parity of the fp32 row kernels and decode attention against the oracle / reference C outputs."""
import os

import numpy as np
import pytest

from conftest import rel_err_ok

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
VEC = np.load(os.path.join(HERE, "golden", "ref_vectors.npz"))


def test_smoke_probe(gpu, cuda_lib):
    from skainet_b200.provider import CudaKernelProvider
    assert CudaKernelProvider().isAvailable()


def test_rms_norm_twin(gpu):
    from skainet_b200.provider import CudaKernelProvider
    k = CudaKernelProvider().normFp32()
    out = np.zeros_like(VEC["rms_x"])
    k.rmsNorm(VEC["rms_x"], 0, VEC["rms_g"], out, 0, 3, 320, 1e-5)
    rel_err_ok(out, VEC["rms_y"], 1e-4)        # NativeFusedKernelsTest.kt:92-138 tolerance
    out2 = np.zeros(320, np.float32)
    k.rmsNorm(VEC["rms_x"], 320, None, out2, 0, 1, 320, 1e-5)
    x = VEC["rms_x"][1].astype(np.float64)
    rel_err_ok(out2, x / np.sqrt((x * x).mean() + 1e-5), 1e-4)


def test_sdpa_twin_matches_reference_c(gpu):
    from skainet_b200.provider import CudaKernelProvider
    k = CudaKernelProvider().attentionFp32()
    out = np.zeros_like(VEC["sdpa_dec_q"])
    k.sdpa(VEC["sdpa_dec_q"], VEC["sdpa_dec_k"], VEC["sdpa_dec_v"], out, 2, 8, 2, 1, 40, 64, 0.125, True, 0, 0, None, None, None)
    rel_err_ok(out, VEC["sdpa_dec_o"], 1e-4)
    out = np.zeros_like(VEC["sdpa_win_q"])
    k.sdpa(VEC["sdpa_win_q"], VEC["sdpa_win_k"], VEC["sdpa_win_v"], out, 1, 4, 2, 9, 9, 32, 0.2, True, 4, 0, None, None, None)
    rel_err_ok(out, VEC["sdpa_win_o"], 1e-4)


@pytest.mark.parametrize("case", ["lengths", "mask_full", "mask_bcast", "right_context", "fully_masked", "noncausal"])
def test_sdpa_twin_mask_rules_match_oracle(gpu, oracle, case):
    # every rule of AttentionMask.kt:57-78, as NativeFusedKernelsTest.kt:166-195 sweeps them
    from skainet_b200.provider import CudaKernelProvider
    rng = np.random.default_rng(hash(case) % 1000)
    B, H, Hkv, Sq, Skv, D = 2, 4, 2, 5, 11, 64
    q = rng.standard_normal((B, H, Sq, D)).astype(np.float32)
    k = rng.standard_normal((B, Hkv, Skv, D)).astype(np.float32); v = rng.standard_normal((B, Hkv, Skv, D)).astype(np.float32)
    kw = dict(causal=True, window=0, right_context=0, lengths=None, mask=None)
    if case == "lengths": kw["lengths"] = np.array([7, 11], np.int32)
    if case == "mask_full": kw["mask"] = rng.standard_normal((B, H, Sq, Skv)).astype(np.float32)
    if case == "mask_bcast": kw["mask"] = rng.standard_normal((1, Hkv, 1, Skv)).astype(np.float32)
    if case == "right_context": kw.update(causal=False, window=3, right_context=2)
    if case == "fully_masked": kw["lengths"] = np.array([0, 3], np.int32)
    if case == "noncausal": kw["causal"] = False
    ref = oracle.sdpa(q, k, v, 0.125, **kw)
    out = np.zeros_like(q)
    md = None if kw["mask"] is None else kw["mask"].shape
    CudaKernelProvider().attentionFp32().sdpa(q, k, v, out, B, H, Hkv, Sq, Skv, D, 0.125, kw["causal"], kw["window"],
                                              kw["right_context"], kw["lengths"], kw["mask"], md)
    assert np.isfinite(out).all()
    rel_err_ok(out, ref, 1e-4)


def test_sdpa_empty_kv_zeroes_output(gpu):
    from skainet_b200.provider import CudaKernelProvider
    q = np.ones((1, 2, 1, 64), np.float32); out = np.full_like(q, 5.0)
    e = np.zeros((1, 2, 0, 64), np.float32)
    CudaKernelProvider().attentionFp32().sdpa(q, e, e, out, 1, 2, 2, 1, 0, 64, 1.0, True, 0, 0, None, None, None)
    assert not out.any()


def test_unary_binary_twins(gpu, cuda_lib, oracle):
    from skainet_b200 import _lib as L
    x = VEC["silu_x"]; out = np.zeros_like(x)
    L.check(cuda_lib.skainet_cuda_f32_unary(2, x.ctypes.data_as(L.f32p), out.ctypes.data_as(L.f32p), x.size))
    rel_err_ok(out, VEC["silu_y"], 1e-5)
    a = np.arange(12, dtype=np.float32); b = np.array([1, 2, 3], np.float32); o = np.zeros(12, np.float32)
    L.check(cuda_lib.skainet_cuda_f32_binary(0, a.ctypes.data_as(L.f32p), 0, b.ctypes.data_as(L.f32p), 2, o.ctypes.data_as(L.f32p), 12, 3))
    np.testing.assert_array_equal(o, a + np.tile(b, 4))
    L.check(cuda_lib.skainet_cuda_f32_binary(2, a.ctypes.data_as(L.f32p), 0, b.ctypes.data_as(L.f32p), 1, o.ctypes.data_as(L.f32p), 12, 1))
    np.testing.assert_array_equal(o, a * 1.0)


def test_rope_swiglu_argmax_embed_resident(gpu, oracle):
    rng = np.random.default_rng(11)
    # RoPE, both conventions, several positions
    for mode in (0, 1):
        x = rng.standard_normal((3, 4, 128)).astype(np.float32)
        pos = np.array([0, 17, 4095], np.int32)
        dx = gpu.DeviceBuffer.from_host(x); dp = gpu.DeviceBuffer.from_host(pos)
        gpu.rope(dx.ptr, dp.ptr, 3, 4, 128, 1e4, mode)
        got = dx.download(np.float32, x.size).reshape(x.shape)
        want = np.stack([oracle.rope(x[r], 4, 128, int(pos[r]), 1e4, mode) for r in range(3)])
        rel_err_ok(got, want, 1e-5)
    # SwiGLU
    g = (3 * rng.standard_normal(1000)).astype(np.float32); u = rng.standard_normal(1000).astype(np.float32)
    dg, du, do = gpu.DeviceBuffer.from_host(g), gpu.DeviceBuffer.from_host(u), gpu.DeviceBuffer(4000)
    gpu.swiglu(dg.ptr, du.ptr, do.ptr, 1000)
    rel_err_ok(do.download(np.float32, 1000), oracle.swiglu(g, u), 1e-5)
    # arg max with ties -> lowest index
    lg = rng.standard_normal((2, 32000)).astype(np.float32); lg[0, 500] = lg[0, 20000] = 99.0; lg[1, 31999] = 50.0
    dl, di = gpu.DeviceBuffer.from_host(lg), gpu.DeviceBuffer(8)
    gpu.argmax(dl.ptr, 2, 32000, di.ptr)
    assert list(di.download(np.int32, 2)) == [500, 31999]
    # embedding rows of a packed Q8_0 table == bit-exact dequant of those rows
    tbl = oracle.quantize_q8_0((0.02 * rng.standard_normal((50, 256))).astype(np.float32))
    w = gpu.Weight.upload(tbl, "Q8_0", 50, 256)
    ids = np.array([3, 49, 0, 3], np.int32)
    dids, dout = gpu.DeviceBuffer.from_host(ids), gpu.DeviceBuffer(4 * 256 * 4)
    gpu.embed(w, dids.ptr, 4, dout.ptr)
    np.testing.assert_array_equal(dout.download(np.float32, 4 * 256).reshape(4, 256), oracle.dequant("Q8_0", tbl).reshape(50, 256)[ids])


@pytest.mark.parametrize("B,H,Hkv,D,L", [(1, 32, 8, 128, 512), (2, 32, 8, 128, 777), (3, 8, 8, 128, 100), (2, 16, 2, 64, 300),
                                         (1, 64, 8, 128, 4096), (2, 4, 2, 128, 1)])
def test_decode_attention_f16_cache_matches_oracle(gpu, oracle, B, H, Hkv, D, L):
    """The decode-attention benchmark shape in miniature: q fp32, K/V binary16 in a cache longer than the visible length,
    per-batch lengths; the oracle is the reference SDPA on the exact f16->f32 values."""
    rng = np.random.default_rng(B * 1000 + L)
    stride = L + 13
    q = rng.standard_normal((B, H, 1, D)).astype(np.float32)
    k = rng.standard_normal((B, Hkv, stride, D)).astype(np.float16); v = rng.standard_normal((B, Hkv, stride, D)).astype(np.float16)
    lens = np.array([max(1, L - 37 * b) for b in range(B)], np.int32)
    scale = 1.0 / np.sqrt(D)
    dq, dk, dv = gpu.DeviceBuffer.from_host(q), gpu.DeviceBuffer.from_host(k), gpu.DeviceBuffer.from_host(v)
    dlen, dout = gpu.DeviceBuffer.from_host(lens), gpu.DeviceBuffer(q.nbytes)
    gpu.attn_decode(dq.ptr, dk.ptr, dv.ptr, dout.ptr, B, H, Hkv, D, stride, dlen.ptr, L, scale)
    got = dout.download(np.float32, q.size).reshape(B, H, D)
    for b in range(B):
        n = int(lens[b])
        ref = oracle.sdpa(q[b:b + 1], k[b:b + 1, :, :n].astype(np.float32), v[b:b + 1, :, :n].astype(np.float32), scale, causal=True,
                          use_ref=oracle.ref() is not None)
        rel_err_ok(got[b], ref[0, :, 0, :])
    # sliding window keeps the last `window` keys
    gpu.attn_decode(dq.ptr, dk.ptr, dv.ptr, dout.ptr, B, H, Hkv, D, stride, dlen.ptr, L, scale, window=5)
    got = dout.download(np.float32, q.size).reshape(B, H, D)
    n = int(lens[0]); lo = max(0, n - 5)
    ref = oracle.sdpa(q[0:1], k[0:1, :, lo:n].astype(np.float32), v[0:1, :, lo:n].astype(np.float32), scale, causal=True)
    rel_err_ok(got[0], ref[0, :, 0, :])


def test_bounded_wait_gives_up_reports_and_leaves_the_context_usable(gpu, cuda_lib):
    """Failure detection without a fault: a kernel waits on a barrier nothing completes; the wait is bounded, the
    kernel reaches its end, the device flag is raised exactly once, and the next kernel computes correctly."""
    import ctypes as C
    outcome = C.c_int32(0)
    assert cuda_lib.skainet_cuda_selftest_bounded_wait(C.byref(outcome)) == 0
    assert outcome.value == 2
    assert cuda_lib.skainet_cuda_device_status() == -6          # SKAINET_CUDA_ERR_TIMEOUT, and the condition is cleared
    assert cuda_lib.skainet_cuda_device_status() == 0
    x = np.array([1.0, -2.5, 3.25], np.float32); y = np.zeros(3, np.float32)
    from skainet_b200 import _lib
    assert cuda_lib.skainet_cuda_smoke_double(x.ctypes.data_as(_lib.f32p), y.ctypes.data_as(_lib.f32p), 3) == 0
    np.testing.assert_array_equal(y, 2 * x)
