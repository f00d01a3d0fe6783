"""The graph-level fused ops fused_qkv_proj and fused_swiglu_ffn through the C ABI, against the CPU decomposition the
reference's fallback handlers perform (LLMFusedOpHandlers.kt:86-127,143-196: separate matmuls, silu, multiply), each
step computed with the reference's own kernels on the same packed bytes."""
import numpy as np
import pytest

from conftest import rel_err_ok

pytestmark = pytest.mark.gpu


def _weights(gpu, oracle, enc, shapes, seed):
    rng = np.random.default_rng(seed)
    packed = []
    for n, k in shapes:
        wf = (0.03 * rng.standard_normal((n, k))).astype(np.float32)
        packed.append(oracle.quantize_q4k(wf) if enc == "Q4_K" else oracle.quantize_q8_0(wf))
    return packed, [gpu.Weight.upload(p, enc, n, k) for p, (n, k) in zip(packed, shapes)]


@pytest.mark.parametrize("enc,d,qr,kr,m,norm", [("Q4_K", 1024, 1024, 256, 1, True), ("Q4_K", 4096, 4096, 1024, 1, False), ("Q4_K", 8192, 256, 128, 1, True),
                                                ("Q4_K", 1024, 512, 128, 5, True), ("Q8_0", 1024, 1024, 256, 1, True), ("Q8_0", 512, 256, 256, 9, False),
                                                ("Q4_K", 2048, 768, 256, 150, True)])
def test_fused_qkv_proj_equals_three_reference_matmuls(gpu, oracle, enc, d, qr, kr, m, norm):
    use_ref = oracle.ref() is not None
    (pq, pk, pv), (wq, wk, wv) = _weights(gpu, oracle, enc, [(qr, d), (kr, d), (kr, d)], seed=d + m)
    merged = gpu.concat_rows(wq, wk, wv)
    assert merged.rows == qr + 2 * kr
    np.testing.assert_array_equal(merged.export(), np.concatenate([pq, pk, pv]))      # a pure row concatenation of the packed bytes
    rng = np.random.default_rng(m)
    x = (2 * rng.standard_normal((m, d))).astype(np.float32)
    gamma = (1 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    dx, dg = gpu.DeviceBuffer.from_host(x), gpu.DeviceBuffer.from_host(gamma)
    # one row: outputs back to back in one buffer (written directly); several rows: three separate buffers
    if m == 1:
        dall = gpu.DeviceBuffer((qr + 2 * kr) * 4)
        ptrs = (dall.ptr, dall.ptr + qr * 4, dall.ptr + (qr + kr) * 4)
    else:
        bufs = [gpu.DeviceBuffer(m * r * 4) for r in (qr, kr, kr)]
        ptrs = tuple(b.ptr for b in bufs)
    gpu.fused_qkv_proj(merged, qr, kr, kr, dx.ptr, m, *ptrs, gamma_ptr=dg.ptr if norm else 0, eps=1e-5)
    xin = oracle.rms_norm(x, gamma, 1e-5, use_ref=use_ref) if norm else x
    tol = 2e-3 if norm else 1e-3          # behind a norm one activation code may flip
    for (p, r, name), ptr in zip(((pq, qr, "q"), (pk, kr, "k"), (pv, kr, "v")), ptrs):
        got = np.empty(m * r, np.float32)
        from skainet_b200 import _lib as L
        L.check(L.lib().skainet_cuda_memcpy_d2h(got.ctypes.data, ptr, got.nbytes, 0))
        rel_err_ok(got.reshape(m, r), oracle.matmul(enc, xin, p, d, r, "rm", use_ref=use_ref).reshape(m, r), tol)
    with pytest.raises(ValueError):
        gpu.fused_qkv_proj(merged, qr, kr, kr + 1, dx.ptr, m, *ptrs)
    for w in (wq, wk, wv, merged):
        w.free()


@pytest.mark.parametrize("enc,d,f,m,norm,resid", [("Q4_K", 1024, 2816, 1, True, True), ("Q4_K", 4096, 11008, 1, False, False), ("Q4_K", 1024, 2048, 6, True, True),
                                                  ("Q8_0", 512, 1024, 1, True, True), ("Q8_0", 512, 768, 4, False, True), ("Q4_K", 512, 1024, 140, False, False),
                                                  # one row into a down projection of 4 MB or more with at most 8192 inputs: SwiGLU inside the ring kernel's prologue
                                                  ("Q4_K", 2048, 4096, 1, True, True), ("Q4_K", 2048, 8192, 1, False, False),
                                                  # a small batch over weights of 4 MB or more: the persistent ring with the tile arithmetic, with and without residual
                                                  ("Q4_K", 2048, 4096, 6, True, True), ("Q4_K", 2048, 4096, 3, False, False),
                                                  # the same over a down projection whose rows are too long to stage: the ring's consumers fetch the activation, residual epilogue
                                                  ("Q4_K", 1024, 12288, 6, True, True)])
def test_fused_swiglu_ffn_equals_the_reference_decomposition(gpu, oracle, enc, d, f, m, norm, resid):
    use_ref = oracle.ref() is not None
    (pg, pu, pd), (wg, wu, wd) = _weights(gpu, oracle, enc, [(f, d), (f, d), (d, f)], seed=f + m)
    wgu = gpu.concat_rows(wg, wu)
    rng = np.random.default_rng(f)
    x = (2 * rng.standard_normal((m, d))).astype(np.float32)
    gamma = (1 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    r = rng.standard_normal((m, d)).astype(np.float32)
    dx, dg, dr = gpu.DeviceBuffer.from_host(x), gpu.DeviceBuffer.from_host(gamma), gpu.DeviceBuffer.from_host(r)
    dout = gpu.DeviceBuffer(m * d * 4)
    gpu.fused_swiglu_ffn(wgu, wd, dx.ptr, m, dout.ptr, resid_ptr=dr.ptr if resid else 0, gamma_ptr=dg.ptr if norm else 0, eps=1e-5)
    got = dout.download(np.float32, m * d).reshape(m, d)
    xin = oracle.rms_norm(x, gamma, 1e-5, use_ref=use_ref) if norm else x
    gate = oracle.matmul(enc, xin, pg, d, f, "rm", use_ref=use_ref).reshape(m, f)
    up = oracle.matmul(enc, xin, pu, d, f, "rm", use_ref=use_ref).reshape(m, f)
    ref = oracle.matmul(enc, oracle.swiglu(gate, up), pd, f, d, "rm", use_ref=use_ref).reshape(m, d)
    # two chained quantizers: a code flip in the first moves the second's input slightly; the bar stays at the one-flip level
    rel_err_ok(got - (r if resid else 0), ref, 5e-3)
    err = np.sqrt(np.mean((got - (r if resid else 0) - ref) ** 2) / np.mean(ref ** 2))
    assert err < 1e-3, err
    # in place: out == resid
    if resid:
        gpu.fused_swiglu_ffn(wgu, wd, dx.ptr, m, dr.ptr, resid_ptr=dr.ptr, gamma_ptr=dg.ptr if norm else 0, eps=1e-5)
        np.testing.assert_array_equal(dr.download(np.float32, m * d).reshape(m, d), got)
    for w in (wg, wu, wd, wgu):
        w.free()


def _q6k(oracle, rows, cols, seed, d_scale=6e-5):
    blk = oracle.random_kquant_blocks("Q6_K", rows, cols, seed=seed).reshape(-1, 210)
    rng = np.random.default_rng(seed + 1)
    blk[:, 208:210] = np.abs(d_scale * (1 + 0.3 * rng.standard_normal(blk.shape[0]))).astype(np.float16).view(np.uint8).reshape(-1, 2)
    return blk.reshape(-1)


@pytest.mark.parametrize("d,f,m,resid", [(1024, 2816, 1, True), (512, 1024, 12, True), (1024, 2048, 5, False), (512, 1280, 70, True)])
def test_fused_swiglu_ffn_with_a_q6k_down_projection(gpu, oracle, d, f, m, resid):
    """ffn_down as Q6_K behind Q4_K gate and up (the mix K-quant files carry): the down projection runs on the Q6_K row
    kernel (up to eight rows) or its tensor-core tile kernel, both with the residual in their epilogue; reference =
    the same decomposition with native/src/q6k_matmul.c for the last product."""
    use_ref = oracle.ref() is not None
    (pg, pu), (wg, wu) = _weights(gpu, oracle, "Q4_K", [(f, d), (f, d)], seed=f + m)
    pd = _q6k(oracle, d, f, seed=3 * f + m)
    wd = gpu.Weight.upload(pd, "Q6_K", d, f)
    wgu = gpu.concat_rows(wg, wu)
    rng = np.random.default_rng(f)
    x = (2 * rng.standard_normal((m, d))).astype(np.float32)
    gamma = (1 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    r = rng.standard_normal((m, d)).astype(np.float32)
    dx, dg, dr = gpu.DeviceBuffer.from_host(x), gpu.DeviceBuffer.from_host(gamma), gpu.DeviceBuffer.from_host(r)
    dout = gpu.DeviceBuffer(m * d * 4)
    gpu.fused_swiglu_ffn(wgu, wd, dx.ptr, m, dout.ptr, resid_ptr=dr.ptr if resid else 0, gamma_ptr=dg.ptr, eps=1e-5)
    got = dout.download(np.float32, m * d).reshape(m, d)
    xin = oracle.rms_norm(x, gamma, 1e-5, use_ref=use_ref)
    gate = oracle.matmul("Q4_K", xin, pg, d, f, "rm", use_ref=use_ref).reshape(m, f)
    up = oracle.matmul("Q4_K", xin, pu, d, f, "rm", use_ref=use_ref).reshape(m, f)
    ref = oracle.matmul("Q6_K", oracle.swiglu(gate, up), pd, f, d, "rm", use_ref=use_ref).reshape(m, d)
    err = np.sqrt(np.mean((got - (r if resid else 0) - ref) ** 2) / np.mean(ref ** 2))
    assert err < 2e-3, err
    if resid:                              # in place: out == resid
        gpu.fused_swiglu_ffn(wgu, wd, dx.ptr, m, dr.ptr, resid_ptr=dr.ptr, gamma_ptr=dg.ptr, eps=1e-5)
        np.testing.assert_array_equal(dr.download(np.float32, m * d).reshape(m, d), got)
    with pytest.raises(ValueError):        # the two-term Q8_0 activation and the K-quant one cannot share a call
        w8 = gpu.Weight.upload(oracle.quantize_q8_0(np.zeros((d, f), np.float32)), "Q8_0", d, f)
        try:
            gpu.fused_swiglu_ffn(wgu, w8, dx.ptr, m, dout.ptr)
        finally:
            w8.free()
    for w in (wg, wu, wd, wgu):
        w.free()


@pytest.mark.parametrize("m", [1, 10])
def test_fused_qkv_proj_over_q6k_weights(gpu, oracle, m):
    use_ref = oracle.ref() is not None
    d, qr, kr = 1024, 512, 128
    packed = [_q6k(oracle, r, d, seed=9 * r + m) for r in (qr, kr, kr)]
    ws = [gpu.Weight.upload(p, "Q6_K", r, d) for p, r in zip(packed, (qr, kr, kr))]
    merged = gpu.concat_rows(*ws)
    np.testing.assert_array_equal(merged.export(), np.concatenate(packed))
    x = (2 * np.random.default_rng(m).standard_normal((m, d))).astype(np.float32)
    dx = gpu.DeviceBuffer.from_host(x)
    bufs = [gpu.DeviceBuffer(m * r * 4) for r in (qr, kr, kr)]
    gpu.fused_qkv_proj(merged, qr, kr, kr, dx.ptr, m, *(b.ptr for b in bufs))
    for p, r, b in zip(packed, (qr, kr, kr), bufs):
        rel_err_ok(b.download(np.float32, m * r).reshape(m, r), oracle.matmul("Q6_K", x, p, d, r, "rm", use_ref=use_ref).reshape(m, r), 1e-5)
    for w in ws + [merged]:
        w.free()
