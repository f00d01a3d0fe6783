"""The lane-to-element maps of the Q6_K / Q5_K kernels (skainet_b200/csrc/matvec_kq.cu, gemm_kq.cu), restated in numpy
and checked against the formats' element definitions (native/src/q6k_matmul.c:83-128, native/src/q5k_matmul.c:93-160): every
element of a super-block is covered exactly once, with the right code bits and the right scale group. Host arithmetic only."""
import numpy as np


def q6k_codes(ql, qh):
    code = np.zeros(256, np.int64)
    for n in range(2):
        for q in range(4):
            for l in range(32):
                lb = ql[64 * n + 32 + l] if (q & 1) else ql[64 * n + l]
                low = (lb >> 4) if (q & 2) else (lb & 0xf)
                code[128 * n + 32 * q + l] = (int(low) | (((int(qh[32 * n + l]) >> (2 * q)) & 3) << 4)) - 32
    return code


def q5k_codes(qs, qh):
    code = np.zeros(256, np.int64)
    for g in range(4):
        for hi in range(2):
            sb = 2 * g + hi
            for l in range(32):
                byte = int(qs[32 * g + l])
                code[32 * sb + l] = ((byte >> 4) if hi else (byte & 0xf)) | (((int(qh[l]) >> sb) & 1) << 4)
    return code


def test_q6k_row_kernel_lane_map():
    """q6k_rows_kernel: part j of a block = ql bytes [16 j, 16 j + 16): elements 128 (j >> 2) + 16 (j & 3) .. in the low
    nibbles, 64 further in the high ones; fifth and sixth bits from qh bytes 32 (j >> 2) + 16 (j & 1) .. at bit 2 ((j >> 1) & 1)
    and four above; scale bytes 8 (j >> 2) + (j & 3) and + 4."""
    rng = np.random.default_rng(1)
    ql = rng.integers(0, 256, 128, dtype=np.uint8); qh = rng.integers(0, 256, 64, dtype=np.uint8)
    sc = rng.integers(-128, 128, 16, dtype=np.int8); q8 = rng.integers(-127, 128, 256, dtype=np.int8)
    code = q6k_codes(ql, qh)
    ref = sum(int(sc[e // 16]) * int(code[e]) * int(q8[e]) for e in range(256))
    seen, tot = np.zeros(256, int), 0
    for j in range(8):
        e_lo = 128 * (j >> 2) + 16 * (j & 3); sh = 2 * ((j >> 1) & 1)
        a = ql[16 * j:16 * j + 16].astype(int)
        h = qh[32 * (j >> 2) + 16 * (j & 1):32 * (j >> 2) + 16 * (j & 1) + 16].astype(int) >> sh
        s8 = sc[8 * (j >> 2):8 * (j >> 2) + 8]
        lo_c = ((a & 0xf) | ((h & 3) << 4)) - 32
        hi_c = (((a >> 4) & 0xf) | (((h >> 4) & 3) << 4)) - 32
        assert (lo_c == code[e_lo:e_lo + 16]).all() and (hi_c == code[e_lo + 64:e_lo + 80]).all(), j
        assert e_lo // 16 == 8 * (j >> 2) + (j & 3)
        seen[e_lo:e_lo + 16] += 1; seen[e_lo + 64:e_lo + 80] += 1
        tot += int(s8[j & 3]) * int((lo_c * q8[e_lo:e_lo + 16].astype(int)).sum()) + int(s8[4 + (j & 3)]) * int((hi_c * q8[e_lo + 64:e_lo + 80].astype(int)).sum())
    assert (seen == 1).all() and tot == ref


def test_q6k_tile_kernel_fragment_map():
    """q6k_gemm_mma_kernel: for (n, h, par, nib) the MMA's 16 contraction elements are 128 n + 32 q + 16 h .. with
    q = par + 2 nib, thread t supplying bytes 4 t .. 4 t + 3 of ql[64 n + 32 par + 16 h ..] and qh[32 n + 16 h ..] >> 2 q;
    the scale group is 8 n + 2 q + h."""
    rng = np.random.default_rng(2)
    ql = rng.integers(0, 256, 128, dtype=np.uint8); qh = rng.integers(0, 256, 64, dtype=np.uint8)
    code = q6k_codes(ql, qh)
    seen = np.zeros(256, int)
    for n in range(2):
        for h in range(2):
            for par in range(2):
                for nib in range(2):
                    q = par + 2 * nib; e = 128 * n + 32 * q + 16 * h
                    assert e // 16 == 8 * n + 2 * q + h
                    for t in range(4):
                        lw = ql[64 * n + 32 * par + 16 * h + 4 * t:64 * n + 32 * par + 16 * h + 4 * t + 4].astype(int)
                        hw = qh[32 * n + 16 * h + 4 * t:32 * n + 16 * h + 4 * t + 4].astype(int)
                        c = (((lw >> (4 * nib)) & 0xf) | (((hw >> (2 * q)) & 3) << 4)) - 32
                        assert (c == code[e + 4 * t:e + 4 * t + 4]).all()
                        seen[e + 4 * t:e + 4 * t + 4] += 1
    assert (seen == 1).all()


def test_q5k_row_and_tile_kernel_maps():
    """q5k_rows_kernel: lane l takes word l of the 128 nibble bytes: run g = l >> 3, elements 64 g + 4 (l & 7) .. + 3 of
    sub-block 2 g (low nibbles) and of sub-block 2 g + 1 (high nibbles), fifth bits at bits 2 g, 2 g + 1 of qh bytes 4 (l & 7) ...
    q5k_gemm_mma_kernel: for (hh, run, nib) the 16 elements 32 sb + 16 hh .. with sb = 2 run + nib, thread t bytes
    32 run + 16 hh + 4 t .. of the nibbles and 16 hh + 4 t .. of qh >> sb."""
    rng = np.random.default_rng(3)
    qs = rng.integers(0, 256, 128, dtype=np.uint8); qh = rng.integers(0, 256, 32, dtype=np.uint8)
    code = q5k_codes(qs, qh)
    seen = np.zeros(256, int)
    for l in range(32):
        g, p = l >> 3, 4 * (l & 7)
        a = qs[4 * l:4 * l + 4].astype(int); hb = qh[p:p + 4].astype(int) >> (2 * g)
        wa = (a & 0xf) | ((hb & 1) << 4); wb = ((a >> 4) & 0xf) | (((hb >> 1) & 1) << 4)
        assert (wa == code[64 * g + p:64 * g + p + 4]).all() and (wb == code[64 * g + 32 + p:64 * g + 32 + p + 4]).all()
        seen[64 * g + p:64 * g + p + 4] += 1; seen[64 * g + 32 + p:64 * g + 32 + p + 4] += 1
    assert (seen == 1).all()
    seen[:] = 0
    for hh in range(2):
        for run in range(4):
            for nib in range(2):
                sb = 2 * run + nib; e0 = 32 * sb + 16 * hh
                for t in range(4):
                    lw = qs[32 * run + 16 * hh + 4 * t:32 * run + 16 * hh + 4 * t + 4].astype(int)
                    hw = qh[16 * hh + 4 * t:16 * hh + 4 * t + 4].astype(int)
                    c = ((lw >> (4 * nib)) & 0xf) | (((hw >> sb) & 1) << 4)
                    assert (c == code[e0 + 4 * t:e0 + 4 * t + 4]).all()
                    seen[e0 + 4 * t:e0 + 4 * t + 4] += 1
    assert (seen == 1).all()


def test_f16_code_times_scale_is_exact():
    """The A operand of the Q5_K tile kernel: f16(1024 + code) * sc - 1024 * sc under one rounding equals code * sc for
    every 5-bit code and 6-bit scale (largest product 1953 < 2048), and the two-term f16 split of an fp32 activation
    loses less than 2^-21 of its magnitude."""
    codes, scs = np.arange(32, dtype=np.float64), np.arange(64, dtype=np.float64)
    prod = (1024 + codes)[:, None] * scs[None, :] - 1024 * scs[None, :]      # exact in float64, rounded once to f16
    assert (prod.astype(np.float16).astype(np.float64) == codes[:, None] * scs[None, :]).all()
    x = np.random.default_rng(4).standard_normal(4096).astype(np.float32) * np.float32(3.0)
    hi = x.astype(np.float16); lo = (x - hi.astype(np.float32)).astype(np.float16)
    err = np.abs(hi.astype(np.float64) + lo.astype(np.float64) - x.astype(np.float64))
    assert (err <= np.abs(x) * 2.0 ** -21 + 6e-8).all()
