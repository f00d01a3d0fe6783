"""GPU parity: dequant (bit-exact) and the dequant-fused matvec (rel 1e-3) against the oracle and
against outputs of the reference's own compiled C, all through the C ABI."""
import json
import os

import numpy as np
import pytest

from conftest import rel_err_ok

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
DIGESTS = json.load(open(os.path.join(HERE, "golden", "reference_digests.json")))
VEC = np.load(os.path.join(HERE, "golden", "ref_vectors.npz"))


def host_dequant(lib, enc, packed):
    from skainet_b200 import _lib as L
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    nb = packed.size // L.BLOCK_BYTES[enc]
    out = np.empty(nb * L.BLOCK_ELEMS[enc], dtype=np.float32)
    L.check(lib.skainet_cuda_dequant(L.ENC[enc], packed.ctypes.data_as(L.u8p), nb, out.ctypes.data_as(L.f32p)))
    return out


@pytest.mark.parametrize("enc", ["Q8_0", "Q4_K", "Q5_K", "Q6_K"])
def test_dequant_reproduces_reference_golden_digest(gpu, cuda_lib, oracle, enc):
    blocks = oracle.golden_weight_blocks(enc, 4, 3, 0x5EED0001)
    got = host_dequant(cuda_lib, enc, oracle.golden_row_major(blocks))
    assert oracle.golden_digest(got) == DIGESTS[f"decode/{enc}"]


@pytest.mark.parametrize("enc", ["Q8_0", "Q4_K", "Q5_K", "Q6_K"])
def test_dequant_bit_exact_on_random_bytes(gpu, cuda_lib, oracle, enc):
    # every byte random, f16 fields sane (the reference's own fixture builder), 64 blocks
    blocks = oracle.golden_weight_blocks(enc, 8, 8, 1234)
    packed = oracle.golden_row_major(blocks)
    np.testing.assert_array_equal(host_dequant(cuda_lib, enc, packed).view(np.uint32), oracle.dequant(enc, packed).view(np.uint32))


@pytest.mark.parametrize("enc", ["Q8_0", "Q4_K", "Q5_K", "Q6_K"])
@pytest.mark.parametrize("order", [0, 1])
def test_upload_split_export_is_the_identity_and_resident_dequant_is_bit_exact(gpu, oracle, enc, order):
    rows, bpr = 5, 3
    blocks = oracle.golden_weight_blocks(enc, rows, bpr, 77)
    rm = oracle.golden_row_major(blocks)
    given = rm if order == 0 else oracle.golden_block_major(blocks)
    w = gpu.Weight.upload(given, enc, rows, bpr * oracle.BLOCK_ELEMS[enc], order)
    np.testing.assert_array_equal(w.export(), rm)
    np.testing.assert_array_equal(w.dequant().reshape(-1).view(np.uint32), oracle.dequant(enc, rm).view(np.uint32))
    w.free()


@pytest.mark.parametrize("tag", ["Q4_K_1024x37", "Q4_K_2816x16", "Q8_0_512x45", "Q8_0_96x7"])
def test_host_twins_match_reference_c_outputs(gpu, oracle, tag):
    from skainet_b200.provider import CudaKernelProvider
    enc = tag[:4]; k, n = (int(t) for t in tag[5:].split("x"))
    p = CudaKernelProvider()
    assert p.isAvailable()
    w, x = VEC[tag + "_w"], VEC[tag + "_x"]
    for row_major in (True, False):
        kern = (p.matmulQ4KRowMajor() if row_major else p.matmulQ4K()) if enc == "Q4_K" else \
               (p.matmulQ8_0RowMajor() if row_major else p.matmulQ8_0())
        wb = w if row_major else oracle.to_feed_order(w, enc, n, k)
        # offsets exercised like the SPI allows: activation, weight and output all start mid-array
        xin = np.concatenate([np.full(5, 9.0, np.float32), x])
        wbuf = np.concatenate([np.full(16, 0xEE, np.uint8), wb])
        out = np.full(n + 3, -7.0, np.float32)
        x_before, w_before = xin.copy(), wbuf.copy()
        kern.matmul(xin, 5, wbuf, 16, k, n, out, 3)
        assert (out[:3] == -7.0).all()
        np.testing.assert_array_equal(xin, x_before); np.testing.assert_array_equal(wbuf, w_before)
        rel_err_ok(out[3:], VEC[tag + ("_y_rm" if row_major else "_y_feed")])


@pytest.mark.parametrize("enc,n,k", [("Q6_K", 37, 1024), ("Q6_K", 130, 2816), ("Q5_K", 37, 1024), ("Q5_K", 130, 2816)])
def test_k_quant_host_twins_match_the_reference_c(gpu, oracle, enc, n, k):
    """skainet_cuda_q6k_matmul / _rm and skainet_cuda_q5k_matmul / _rm through the provider's Q6_K / Q5_K slots
    (KernelProvider.kt:86,92) in both weight orders, offsets mid-array, against the reference's own C kernels."""
    from skainet_b200.provider import CudaKernelProvider
    p = CudaKernelProvider()
    assert p.isAvailable() and p.supports("matmul", ["Float32", enc])
    w = oracle.random_kquant_blocks(enc, n, k, seed=n + k)
    x = np.random.default_rng(n).standard_normal(k).astype(np.float32)
    ref = oracle.matmul(enc, x, w, k, n, "rm", use_ref=oracle.ref() is not None).reshape(-1)
    for row_major in (True, False):
        kern = {("Q6_K", True): p.matmulQ6KRowMajor, ("Q6_K", False): p.matmulQ6K, ("Q5_K", True): p.matmulQ5KRowMajor, ("Q5_K", False): p.matmulQ5K}[(enc, row_major)]()
        wb = w if row_major else oracle.to_feed_order(w, enc, n, k)
        xin = np.concatenate([np.full(5, 9.0, np.float32), x])
        wbuf = np.concatenate([np.full(16, 0xEE, np.uint8), wb])
        out = np.full(n + 3, -7.0, np.float32)
        x_before, w_before = xin.copy(), wbuf.copy()
        kern.matmul(xin, 5, wbuf, 16, k, n, out, 3)
        assert (out[:3] == -7.0).all()
        np.testing.assert_array_equal(xin, x_before); np.testing.assert_array_equal(wbuf, w_before)
        rel_err_ok(out[3:], ref, 1e-5 if enc == "Q6_K" else 1e-4)
    with pytest.raises(ValueError):
        p.matmulQ6K().matmul(x, 0, w, 0, 100, n, np.zeros(n, np.float32), 0)
    untouched = np.full(4, 3.0, np.float32)
    p.matmulQ5K().matmul(x, 0, w, 0, 0, 4, untouched, 0)            # inputDim 0: output left as it was (q5k_matmul.c:264)
    assert (untouched == 3.0).all()


@pytest.mark.parametrize("enc,n,k", [("Q4_K", 64, 256), ("Q4_K", 129, 4096), ("Q4_K", 33, 11008), ("Q4_K", 1, 512),
                                     ("Q4_K", 520, 16384),       # 4.8 MB with rows too long to stage: 3..8 rows take the ring whose consumers fetch the activation
                                     ("Q8_0", 64, 32), ("Q8_0", 130, 4096), ("Q8_0", 9, 11008), ("Q8_0", 1, 64)])
@pytest.mark.parametrize("m", [1, 3, 8, 13, 40, 130])
def test_resident_matvec_matches_oracle(gpu, oracle, enc, n, k, m):
    rng = np.random.default_rng(n * 131 + k + m)
    wf = (0.02 * rng.standard_normal((n, k))).astype(np.float32)
    packed = oracle.quantize_q4k(wf) if enc == "Q4_K" else oracle.quantize_q8_0(wf)
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = gpu.Weight.upload(packed, enc, n, k)
    ref = oracle.matmul(enc, x, packed, k, n, "rm", use_ref=oracle.ref() is not None)
    rel_err_ok(gpu.matmul_host(w, x), ref)
    # F32 mode = the exact-float arithmetic of the scalar Kotlin kernels
    exact = x.astype(np.float64) @ oracle.dequant(enc, packed).reshape(n, k).astype(np.float64).T
    rel_err_ok(gpu.matmul_host(w, x, act_mode=1), exact, 1e-4)
    w.free()


def test_q4k_saturated_codes_and_adversarial_activation(gpu, oracle):
    # all nibbles 15, all scales/mins 63, activation alternating +-max: integer partial sums at their extremes
    n, k = 8, 1024
    blk = np.zeros(144, np.uint8)
    blk[0:2] = np.array([0.01], np.float16).view(np.uint8); blk[2:4] = np.array([0.02], np.float16).view(np.uint8)
    blk[4:16] = oracle.pack_k4_scales(np.full((1, 8), 63), np.full((1, 8), 63))[0]
    blk[16:] = 0xFF
    packed = np.tile(blk, n * (k // 256))
    for x in (np.full(k, 3.0, np.float32), np.where(np.arange(k) % 2 == 0, 5.0, -5.0).astype(np.float32)):
        w = gpu.Weight.upload(packed, "Q4_K", n, k)
        rel_err_ok(gpu.matmul_host(w, x), oracle.matmul("Q4_K", x, packed, k, n, "rm"))
        w.free()


def test_zero_activation_blocks(gpu, oracle):
    rng = np.random.default_rng(9)
    n, k = 16, 1024
    packed = oracle.quantize_q4k((0.02 * rng.standard_normal((n, k))).astype(np.float32))
    x = rng.standard_normal(k).astype(np.float32); x[256:512] = 0.0
    w = gpu.Weight.upload(packed, "Q4_K", n, k)
    rel_err_ok(gpu.matmul_host(w, x), oracle.matmul("Q4_K", x, packed, k, n, "rm"))
    assert not gpu.matmul_host(w, np.zeros(k, np.float32)).any()
    w.free()


def test_linearity_at_full_size_q4k(gpu):
    """Size-independent property at the full benchmark shape (11008 x 4096, F32 mode is linear in x):
    W(a + b) == W a + W b within fp32 rounding, on a device-generated weight."""
    w = gpu.Weight.synth("Q4_K", 11008, 4096, seed=3, std=0.02)
    rng = np.random.default_rng(10)
    a = rng.standard_normal(4096).astype(np.float32); b = rng.standard_normal(4096).astype(np.float32)
    ya, yb, yab = (gpu.matmul_host(w, v, act_mode=1) for v in (a, b, a + b))
    rel_err_ok(yab, ya.astype(np.float64) + yb, 1e-4)
    # and the native (int8-activation) mode stays within its documented distance of the exact product
    yn = gpu.matmul_host(w, a)
    rel_rms = np.sqrt(np.mean((yn - ya) ** 2) / np.mean(ya ** 2))
    assert rel_rms < 0.03
    w.free()


def test_synth_weights_are_valid_and_match_oracle_on_exported_bytes(gpu, oracle):
    for enc, n, k in (("Q4_K", 40, 2048), ("Q8_0", 24, 1024)):
        w = gpu.Weight.synth(enc, n, k, seed=5, std=0.02)
        packed = w.export()
        deq = oracle.dequant(enc, packed)
        assert np.isfinite(deq).all() and 0.015 < deq.std() < 0.025 and abs(deq.mean()) < 2e-3
        np.testing.assert_array_equal(w.dequant().reshape(-1).view(np.uint32), deq.view(np.uint32))
        x = np.random.default_rng(6).standard_normal(k).astype(np.float32)
        rel_err_ok(gpu.matmul_host(w, x), oracle.matmul(enc, x, packed, k, n, "rm"))
        w.free()


@pytest.mark.parametrize("enc,n,k", [("Q4_K", 4096, 4096), ("Q4_K", 333, 11008), ("Q4_K", 37, 28672), ("Q4_K", 5, 256),
                                     ("Q8_0", 1000, 4096), ("Q8_0", 77, 2304), ("Q8_0", 9, 256)])
def test_fused_norm_quant_matvec_residual(gpu, oracle, enc, n, k):
    """One launch = RMSNorm + activation quantization + matvec + residual add, against the same chain
    built from the reference kernels (f32_fused.c rms norm -> q4k/q8_0 matmul -> add)."""
    rng = np.random.default_rng(n + k)
    wf = (0.02 * rng.standard_normal((n, k))).astype(np.float32)
    packed = oracle.quantize_q4k(wf) if enc == "Q4_K" else oracle.quantize_q8_0(wf)
    x = (3 * rng.standard_normal(k)).astype(np.float32); gamma = (1 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    resid = rng.standard_normal(n).astype(np.float32)
    w = gpu.Weight.upload(packed, enc, n, k)
    dx, dg, dr, dy = (gpu.DeviceBuffer.from_host(a) for a in (x, gamma, resid, np.zeros(n, np.float32)))
    use_ref = oracle.ref() is not None
    xn = oracle.rms_norm(x, gamma, 1e-5, use_ref=use_ref)
    # norm + residual
    gpu.matvec_fused(w, dx.ptr, dg.ptr, 1e-5, dr.ptr, dy.ptr)
    rel_err_ok(dy.download(np.float32, n) - resid, oracle.matmul(enc, xn, packed, k, n, "rm", use_ref=use_ref), 2e-3)
    # plain (no norm, no residual) and in-place residual
    gpu.matvec_fused(w, dx.ptr, 0, 0.0, 0, dy.ptr)
    plain = oracle.matmul(enc, x, packed, k, n, "rm", use_ref=use_ref)
    rel_err_ok(dy.download(np.float32, n), plain)
    gpu.matvec_fused(w, dx.ptr, 0, 0.0, dr.ptr, dr.ptr)
    rel_err_ok(dr.download(np.float32, n) - resid, plain, 2e-3)
    from skainet_b200 import _lib
    assert _lib.lib().skainet_cuda_device_status() == 0
    w.free()


@pytest.mark.parametrize("n,k,m,runs", [(300, 2048, 290, 10), (129, 4096, 300, 30), (260, 2816, 300, 30), (140, 256, 400, 10)])
def test_tcgen05_rows_tile_kernel_is_exact_and_repeatable(gpu, oracle, n, k, m, runs):
    """From 288 rows the tcgen05 kernel runs: several row and column tiles, ragged on both sides. The integer sums
    are exact in f16 x f16 -> f32, so the result equals the reference's to fp32 rounding, and repeated runs are
    bit-identical (a race between the roles of the kernel shows up as a run that differs). Shapes: an even and an odd
    number of super-blocks per row (8, 16, 11) and a single one, where the two accumulator sets and the two block-scale
    slots are reused with and without a parity change."""
    rng = np.random.default_rng(77)
    wf = (0.02 * rng.standard_normal((n, k))).astype(np.float32)
    packed = oracle.quantize_q4k(wf)
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = gpu.Weight.upload(packed, "Q4_K", n, k)
    ref = oracle.matmul("Q4_K", x, packed, k, n, "rm", use_ref=oracle.ref() is not None)
    first = gpu.matmul_host(w, x)
    rel_err_ok(first, ref, 1e-5)
    for _ in range(runs - 1):
        np.testing.assert_array_equal(gpu.matmul_host(w, x), first)
    from skainet_b200 import _lib
    assert _lib.lib().skainet_cuda_device_status() == 0
    w.free()


@pytest.mark.parametrize("enc", ["Q6_K", "Q5_K"])
@pytest.mark.parametrize("n,k,m", [(64, 256, 1), (129, 4096, 1), (33, 2048, 5), (4096, 11008, 1), (1001, 4096, 3), (515, 2304, 8),
                                   (130, 1280, 11), (77, 256, 20), (11008, 4096, 2), (300, 2816, 16), (200, 1024, 70), (4096, 11008, 130),
                                   (1000, 4096, 512), (11008, 1024, 130), (64, 512, 9)])
def test_k_quant_next_formats_matvec(gpu, oracle, enc, n, k, m):
    """Q6_K / Q5_K over resident planes against the reference's C kernels (native mode: Q6_K quantizes the
    activation to int8 per 256 and is integer-exact per block; Q5_K keeps fp32) and, in F32 mode, against the
    dequantised product in float64. The shapes cover rows that are not a multiple of the CTA's four, block counts per row
    that are not a multiple of the four a warp step takes (43, 9, 5, 1), every activation-row group size, batches that
    need more than one pass over the weight and the tensor-core tile kernels (Q6_K from nine rows, Q5_K from five) (ragged in both
    directions: 300 / 200 / 1000 weight rows against tiles of 32, 11008 against tiles of 64, 9 / 70 / 130 activation rows
    against tiles of 64)."""
    w_bytes = oracle.random_kquant_blocks(enc, n, k, seed=n + k + m)
    x = np.random.default_rng(n * 7 + m).standard_normal((m, k)).astype(np.float32)
    w = gpu.Weight.upload(w_bytes, enc, n, k)
    ref = oracle.matmul(enc, x, w_bytes, k, n, "rm", use_ref=oracle.ref() is not None)
    rel_err_ok(gpu.matmul_host(w, x), ref, 1e-5 if enc == "Q6_K" else 1e-4)
    if n * k <= 1 << 21:                       # the exact-float mode is a plain kernel; small shapes only
        exact = x.astype(np.float64) @ oracle.dequant(enc, w_bytes).reshape(n, k).astype(np.float64).T
        rel_err_ok(gpu.matmul_host(w, x, act_mode=1), exact, 1e-4)
    w.free()


@pytest.mark.parametrize("n,k,m", [(300, 2816, 8), (64, 4096, 8), (300, 2816, 70), (129, 1024, 200)])
def test_q6k_rows_of_a_batch_equal_single_rows(gpu, oracle, n, k, m):
    """Rows of a batch are independent matvecs (native/src/q6k_matmul.c:289-357): the eight-row pass and the tensor-core
    tile kernel (nine rows and more) must give each row the very bits a single-row call gives it, and a second call
    must repeat them."""
    w_bytes = oracle.random_kquant_blocks("Q6_K", n, k, seed=3 * n + m)
    x = np.random.default_rng(n + m).standard_normal((m, k)).astype(np.float32)
    w = gpu.Weight.upload(w_bytes, "Q6_K", n, k)
    full = gpu.matmul_host(w, x)
    assert np.array_equal(full, gpu.matmul_host(w, x))
    for i in (0, 3, 7, m - 1):
        assert np.array_equal(full[i], gpu.matmul_host(w, x[i:i + 1])[0])
    assert np.array_equal(full[:5], gpu.matmul_host(w, x[:5]))
    w.free()
