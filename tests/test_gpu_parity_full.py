"""GPU parity at the sizes the benchmark runs, against the reference's own compiled C kernels
(oracle/_ref; the restatement in oracle/port.c where that binary is absent):

* the ring matvec kernels (weights of 20 MiB and more) on the Q4_K sweep shapes, the four linears of the
  70B-class layer and the Q8_0 32000 x 4096 table, plain and with the residual epilogue;
* the Q4_K sweep at M in {2, 5, 8, 64, 512} on both shapes plus ragged M = 130 and 300: the ring with the tile arithmetic up to
  8 rows, `mma.sync` tiles below 288 rows, the tcgen05 kernel from 288 rows;
* GQA decode attention (32 query / 8 KV heads, head_dim 128) at context 32768 x batch 1, 4096 x 16 and
  512 x 64, with RoPE (theta 1e4) applied to q and to every key before it is cached.

Weights are generated and packed on the device (seeded), exported, and the same bytes are handed to the
reference. Bar: |got - ref| <= 1e-3 * max(|ref|, rms(ref)) for every element (conftest.rel_err_ok).
"""
import numpy as np
import pytest

from conftest import rel_err_ok

pytestmark = pytest.mark.gpu

# (rows = out, cols = in): benchmark config 2, then q|k|v, o, gate|up, down of the 70B-class layer
Q4K_RING_SHAPES = [(11008, 4096), (4096, 11008), (10240, 8192), (8192, 8192), (57344, 8192), (8192, 28672)]


def _ref_matmul(oracle, enc, x, packed, k, n):
    return oracle.matmul(enc, x, packed, k, n, "rm", use_ref=oracle.ref() is not None)


@pytest.mark.parametrize("n,k", Q4K_RING_SHAPES)
def test_q4k_ring_matvec_at_benchmark_sizes(gpu, cuda_lib, oracle, n, k):
    """One activation row against a weight of 25 to 264 MB: the ring kernel with the activation quantized in its
    prologue (store and residual epilogues) and RMS-normalised in its prologue. The form that takes an already
    quantized row is what the decoder's o and down projections use; the full-width model test covers it."""
    w = gpu.Weight.synth("Q4_K", n, k, seed=n + k, std=0.02)
    assert w.packed_bytes >= 20 << 20
    packed = w.export()
    rng = np.random.default_rng(n * 3 + k)
    x = rng.standard_normal(k).astype(np.float32)
    ref = _ref_matmul(oracle, "Q4_K", x, packed, k, n)
    # plain: y = W . quantize(x)
    rel_err_ok(gpu.matmul_host(w, x), ref)
    # residual epilogue: y = resid + W . quantize(x), in place
    resid = rng.standard_normal(n).astype(np.float32)
    dx, dr = gpu.DeviceBuffer.from_host(x), gpu.DeviceBuffer.from_host(resid)
    gpu.matvec_fused(w, dx.ptr, 0, 0.0, dr.ptr, dr.ptr)
    rel_err_ok(dr.download(np.float32, n) - resid, ref, 2e-3)      # the difference of two fp32 sums loses a few bits
    # RMSNorm in the prologue
    gamma = (1 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    xs = (3 * x).astype(np.float32)
    dxs, dg, dy = gpu.DeviceBuffer.from_host(xs), gpu.DeviceBuffer.from_host(gamma), gpu.DeviceBuffer(n * 4)
    gpu.matvec_fused(w, dxs.ptr, dg.ptr, 1e-5, 0, dy.ptr)
    xn = oracle.rms_norm(xs, gamma, 1e-5, use_ref=oracle.ref() is not None)
    rel_err_ok(dy.download(np.float32, n), _ref_matmul(oracle, "Q4_K", xn, packed, k, n), 2e-3)   # one activation code may flip
    assert cuda_lib.skainet_cuda_device_status() == 0
    w.free()


def test_q8_0_ring_matvec_output_table(gpu, cuda_lib, oracle):
    n, k = 32000, 4096          # the 7B-class output head: 139 MB of Q8_0
    w = gpu.Weight.synth("Q8_0", n, k, seed=17, std=0.02)
    packed = w.export()
    rng = np.random.default_rng(5)
    x = rng.standard_normal(k).astype(np.float32)
    ref = _ref_matmul(oracle, "Q8_0", x, packed, k, n)
    rel_err_ok(gpu.matmul_host(w, x), ref)
    resid = rng.standard_normal(n).astype(np.float32)
    dx, dr = gpu.DeviceBuffer.from_host(x), gpu.DeviceBuffer.from_host(resid)
    gpu.matvec_fused(w, dx.ptr, 0, 0.0, dr.ptr, dr.ptr)
    rel_err_ok(dr.download(np.float32, n) - resid, ref, 2e-3)
    assert cuda_lib.skainet_cuda_device_status() == 0
    w.free()


def test_q8_0_matvec_config1_shape(gpu, oracle):
    n, k = 4096, 4096           # benchmark config 1, quantized by the reference's Q8_0 rule on the host
    rng = np.random.default_rng(1)
    packed = oracle.quantize_q8_0((0.02 * rng.standard_normal((n, k))).astype(np.float32))
    x = np.random.default_rng(2).standard_normal(k).astype(np.float32)
    w = gpu.Weight.upload(packed, "Q8_0", n, k)
    rel_err_ok(gpu.matmul_host(w, x), _ref_matmul(oracle, "Q8_0", x, packed, k, n))
    w.free()


@pytest.mark.parametrize("n,k", [(11008, 4096), (4096, 11008)])
def test_q4k_batched_rows_sweep(gpu, cuda_lib, oracle, n, k):
    """Benchmark config 2 at M = 8 (and 2, 5: the persistent ring with the tile arithmetic), 64 (mma.sync tiles) and 512
    (tcgen05), plus ragged 130 (mma.sync) and 300 (tcgen05) on the first shape. The reference computes M rows as M matvecs; the tile kernels use the
    same integer arithmetic, so the bar is the matvec bar."""
    w = gpu.Weight.synth("Q4_K", n, k, seed=3 if n > k else 4, std=0.02)
    packed = w.export()
    rng = np.random.default_rng(5)
    ms = [2, 5, 8, 64, 512] + ([130, 300] if n > k else [])
    x = rng.standard_normal((max(ms), k)).astype(np.float32)
    ref = _ref_matmul(oracle, "Q4_K", x, packed, k, n)
    for m in ms:
        rel_err_ok(gpu.matmul_host(w, x[:m]), ref[:m])
    assert cuda_lib.skainet_cuda_device_status() == 0
    w.free()


@pytest.mark.parametrize("L,B", [(32768, 1), (4096, 16), (512, 64)])
def test_gqa_decode_attention_config3(gpu, cuda_lib, oracle, L, B):
    """q and K are rotated on the device (skainet_cuda_rope_dev; q at position L-1, key t at position t), K and V
    are rounded to binary16 into the cache, then the split-K decode attention runs. The oracle rotates with the
    restatement, rounds K/V through binary16 and calls the reference SDPA per batch element."""
    H, Hkv, D = 32, 8, 128
    rng = np.random.default_rng(L + B)
    q = rng.standard_normal((B, H, D)).astype(np.float32)
    scale = float(1.0 / np.sqrt(D))
    stride = L
    dk16, dv16 = gpu.DeviceBuffer(B * Hkv * stride * D * 2), gpu.DeviceBuffer(B * Hkv * stride * D * 2)
    pos_q = np.full(B, L - 1, np.int32)
    pos_k = np.tile(np.arange(L, dtype=np.int32), Hkv)
    dpos_k = gpu.DeviceBuffer.from_host(pos_k)
    refs = []
    for b in range(B):           # one batch element at a time keeps the host arrays small (134 MB of fp32 K at L = 32768)
        k = rng.standard_normal((Hkv, L, D)).astype(np.float32)
        v = rng.standard_normal((Hkv, L, D)).astype(np.float32)
        dk = gpu.DeviceBuffer.from_host(k)
        gpu.rope(dk.ptr, dpos_k.ptr, Hkv * L, 1, D, 1e4, 0)
        gpu.f32_to_f16(dk.ptr, dk16.ptr + b * Hkv * stride * D * 2, Hkv * L * D)
        dv = gpu.DeviceBuffer.from_host(v)
        gpu.f32_to_f16(dv.ptr, dv16.ptr + b * Hkv * stride * D * 2, Hkv * L * D)
        gpu.sync()
        dk.free(); dv.free()
        kr = oracle.round_f16(oracle.rope_seq(k, 0, 1e4, 0))
        qr = oracle.rope(q[b], H, D, L - 1, 1e4, 0)
        refs.append(oracle.sdpa(qr.reshape(1, H, 1, D), kr[None], oracle.round_f16(v)[None], scale, causal=True,
                                use_ref=oracle.ref() is not None)[0, :, 0, :])
    dq, dpos_q = gpu.DeviceBuffer.from_host(q), gpu.DeviceBuffer.from_host(pos_q)
    gpu.rope(dq.ptr, dpos_q.ptr, B, H, D, 1e4, 0)
    lens = np.full(B, L, np.int32)
    dlen, dout = gpu.DeviceBuffer.from_host(lens), gpu.DeviceBuffer(q.nbytes)
    gpu.attn_decode(dq.ptr, dk16.ptr, dv16.ptr, dout.ptr, B, H, Hkv, D, stride, dlen.ptr, L, scale)
    got = dout.download(np.float32, q.size).reshape(B, H, D)
    for b in range(B):
        rel_err_ok(got[b], refs[b])
    assert cuda_lib.skainet_cuda_device_status() == 0
