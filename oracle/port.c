/*
 * CPU restatement of the reference's packed-quantized decode path, in plain C.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing the product ships may link, load or call this file: it is the
 * checker the CUDA kernels are compared against (tests, the smoke check, and the CPU-baseline leg of
 * the bench). Build: `make -C oracle port` (strict fp32: -ffp-contract=off, no -ffast-math).
 *
 * Every function names the reference file:line it follows (paths relative to the reference tree).
 * Pinning: oracle_dequant_* and oracle_scalar_matmul_* reproduce, bit for bit, the digests recorded
 * in skainet-backends/skainet-backend-cpu/src/goldenTest/kotlin/sk/ainet/exec/golden/Goldens.kt
 * (keys decode/Q8_0, decode/Q4_K, decode/Q5_K, decode/Q6_K, scalar-matmul/Q8_0, scalar-matmul/Q4_K);
 * the Q8-activation matvec, RMSNorm, SDPA and elementwise functions are checked against the
 * reference's compiled C (oracle/_ref) in tests/test_oracle.py. RoPE has no reference code: parity
 * unpinned, the convention is declared at oracle_rope below.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------------
 * binary16 -> binary32, exact for every input.
 * Follows skainet-backends/skainet-backend-native-cpu/native/src/q8_0_matmul.c:31-56 and
 * skainet-lang/skainet-lang-core/src/commonMain/kotlin/sk/ainet/lang/tensor/data/Q4_KTensorData.kt:278-311.
 */
static inline float half_to_float(uint16_t h) {
    uint32_t sign = ((uint32_t)(h & 0x8000u)) << 16, exp = (h >> 10) & 0x1Fu, mant = h & 0x3FFu, bits;
    if (exp == 0) {
        if (mant == 0) bits = sign;
        else {
            int e = -14;
            while ((mant & 0x400u) == 0) { mant <<= 1; --e; }
            bits = sign | ((uint32_t)(e + 127) << 23) | ((mant & 0x3FFu) << 13);
        }
    } else if (exp == 0x1Fu) bits = sign | 0x7F800000u | (mant << 13);
    else bits = sign | ((exp - 15 + 127) << 23) | (mant << 13);
    float r; memcpy(&r, &bits, 4); return r;
}
API float oracle_half_to_float(uint16_t h) { return half_to_float(h); }

/* binary32 -> binary16, round to nearest even (the rule of
 * skainet-lang/skainet-lang-core/src/commonMain/kotlin/sk/ainet/lang/types/NarrowFloatCodec.kt:87-128,
 * used for the stored Q8_0 scale and for the f16 KV cache). */
static inline uint16_t float_to_half(float f) {
    uint32_t x; memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u; x &= 0x7FFFFFFFu;
    if (x >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | (x > 0x7F800000u ? 0x200u : 0));
    if (x >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);          /* rounds to inf */
    if (x < 0x33000001u) return (uint16_t) sign;                        /* rounds to zero */
    int e = (int)(x >> 23) - 127;
    uint32_t m = (x & 0x7FFFFFu) | 0x800000u;
    int shift = (e < -14) ? (13 + (-14 - e)) : 13;
    uint32_t half_m = m >> shift, rem = m & ((1u << shift) - 1), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half_m & 1))) half_m++;
    uint32_t he = (e < -14) ? 0 : (uint32_t)(e + 15);
    /* half_m carries the implicit bit for normals (bit 10); adding folds mantissa overflow into exp */
    uint32_t out = (e < -14) ? half_m : ((he << 10) + (half_m - 0x400u));
    return (uint16_t)(sign | out);
}
API uint16_t oracle_float_to_half(float f) { return float_to_half(f); }

/* ------------------------------------------------------------------------------------------------
 * ggml get_scale_min_k4: 12 packed bytes -> 8 x (6-bit scale, 6-bit min).
 * Follows native/src/q4k_matmul.c:47-65 and
 * skainet-io/skainet-io-gguf/src/commonMain/kotlin/sk/ainet/io/gguf/dequant/DequantOps.kt:585-598.
 */
static inline void k4_scales(const uint8_t* s, int* sc, int* mn) {
    for (int j = 0; j < 4; ++j) { sc[j] = s[j] & 0x3F; mn[j] = s[j + 4] & 0x3F; }
    for (int j = 4; j < 8; ++j) {
        sc[j] = (s[j + 4] & 0x0F) | (((s[j - 4] >> 6) & 3) << 4);
        mn[j] = ((s[j + 4] >> 4) & 0x0F) | (((s[j] >> 6) & 3) << 4);
    }
}

/* Q8_0 dequant: w = d * (float)code. DequantOps.kt:338-355. */
API void oracle_dequant_q8_0(const uint8_t* bytes, int64_t nblocks, float* out) {
    for (int64_t b = 0; b < nblocks; ++b) {
        const uint8_t* blk = bytes + b * 34;
        const float d = half_to_float((uint16_t)(blk[0] | (blk[1] << 8)));
        for (int j = 0; j < 32; ++j) out[b * 32 + j] = d * (float)(int8_t) blk[2 + j];
    }
}

/* Q4_K dequant: w = fl(fl(d*sc)*q) - fl(dmin*m), element order sub-block major.
 * DequantOps.kt:600-644; Q4_KTensorData.kt:120-136,215-226. */
API void oracle_dequant_q4k(const uint8_t* bytes, int64_t nblocks, float* out) {
    for (int64_t b = 0; b < nblocks; ++b) {
        const uint8_t* blk = bytes + b * 144;
        const float d = half_to_float((uint16_t)(blk[0] | (blk[1] << 8)));
        const float dmin = half_to_float((uint16_t)(blk[2] | (blk[3] << 8)));
        int sc[8], mn[8]; k4_scales(blk + 4, sc, mn);
        const uint8_t* qs = blk + 16;
        float* o = out + b * 256;
        for (int g = 0; g < 4; ++g) {
            const float d1 = d * (float) sc[2 * g], m1 = dmin * (float) mn[2 * g];
            const float d2 = d * (float) sc[2 * g + 1], m2 = dmin * (float) mn[2 * g + 1];
            for (int l = 0; l < 32; ++l) o[64 * g + l] = d1 * (float)(qs[32 * g + l] & 0x0F) - m1;
            for (int l = 0; l < 32; ++l) o[64 * g + 32 + l] = d2 * (float)(qs[32 * g + l] >> 4) - m2;
        }
    }
}

/* Q5_K dequant (176-byte block: d, dmin, 12 scale bytes, 32 qh bytes, 128 qs bytes).
 * DequantOps.kt dequantQ5KFromBytes (after :644): w = fl(fl(d*sc)*q) - fl(dmin*m), q = nibble + 16*bit. */
API void oracle_dequant_q5k(const uint8_t* bytes, int64_t nblocks, float* out) {
    for (int64_t b = 0; b < nblocks; ++b) {
        const uint8_t* blk = bytes + b * 176;
        const float d = half_to_float((uint16_t)(blk[0] | (blk[1] << 8)));
        const float dmin = half_to_float((uint16_t)(blk[2] | (blk[3] << 8)));
        int sc[8], mn[8]; k4_scales(blk + 4, sc, mn);
        const uint8_t* qh = blk + 16; const uint8_t* qs = blk + 48;
        float* o = out + b * 256;
        for (int g = 0; g < 4; ++g) {
            const float d1 = d * (float) sc[2 * g], m1 = dmin * (float) mn[2 * g];
            const float d2 = d * (float) sc[2 * g + 1], m2 = dmin * (float) mn[2 * g + 1];
            const int u1 = 1 << (2 * g), u2 = 2 << (2 * g);
            for (int l = 0; l < 32; ++l)
                o[64 * g + l] = d1 * (float)((qs[32 * g + l] & 0x0F) + ((qh[l] & u1) ? 16 : 0)) - m1;
            for (int l = 0; l < 32; ++l)
                o[64 * g + 32 + l] = d2 * (float)((qs[32 * g + l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - m2;
        }
    }
}

/* Q6_K dequant (210-byte block: 128 ql, 64 qh, 16 int8 scales, f16 d at byte 208).
 * DequantOps.kt dequantQ6KFromBytes: w = fl(fl(d*scale)*q), q in [-32, 31]. */
API void oracle_dequant_q6k(const uint8_t* bytes, int64_t nblocks, float* out) {
    for (int64_t b = 0; b < nblocks; ++b) {
        const uint8_t* blk = bytes + b * 210;
        const uint8_t* ql = blk; const uint8_t* qh = blk + 128; const int8_t* sc = (const int8_t*)(blk + 192);
        const float d = half_to_float((uint16_t)(blk[208] | (blk[209] << 8)));
        float* o = out + b * 256;
        for (int n = 0; n < 2; ++n) {
            for (int l = 0; l < 32; ++l) {
                const int is = l / 16;
                const int q1 = (int)((ql[l] & 0x0F) | (((qh[l] >> 0) & 3) << 4)) - 32;
                const int q2 = (int)((ql[l + 32] & 0x0F) | (((qh[l] >> 2) & 3) << 4)) - 32;
                const int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                const int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                o[l]      = (d * (float) sc[is + 0]) * (float) q1;
                o[l + 32] = (d * (float) sc[is + 2]) * (float) q2;
                o[l + 64] = (d * (float) sc[is + 4]) * (float) q3;
                o[l + 96] = (d * (float) sc[is + 6]) * (float) q4;
            }
            o += 128; ql += 64; qh += 32; sc += 8;
        }
    }
}

/* ------------------------------------------------------------------------------------------------
 * The exact-float scalar kernels (feed order, strictly sequential fp32): the Kotlin reference tier.
 * skainet-backends/skainet-backend-cpu/src/commonMain/kotlin/sk/ainet/exec/kernel/ScalarQ8_0MatmulKernel.kt:28-63
 */
API void oracle_scalar_matmul_q8_0(const float* in, const uint8_t* w, int32_t input_dim, int32_t output_dim, float* out) {
    const int32_t nb = input_dim / 32;
    for (int32_t o = 0; o < output_dim; ++o) {
        float acc = 0.0f;
        for (int32_t b = 0; b < nb; ++b) {
            const uint8_t* blk = w + ((size_t) b * output_dim + o) * 34;
            const float d = half_to_float((uint16_t)(blk[0] | (blk[1] << 8)));
            for (int k = 0; k < 32; ++k) acc += in[b * 32 + k] * (float)(int8_t) blk[2 + k] * d;
        }
        out[o] = acc;
    }
}

/* .../exec/kernel/ScalarQ4_KMatmulKernel.kt:21-81 */
API void oracle_scalar_matmul_q4k(const float* in, const uint8_t* w, int32_t input_dim, int32_t output_dim, float* out) {
    const int32_t nb = input_dim / 256;
    for (int32_t o = 0; o < output_dim; ++o) {
        float acc = 0.0f;
        for (int32_t b = 0; b < nb; ++b) {
            const uint8_t* blk = w + ((size_t) b * output_dim + o) * 144;
            const float d = half_to_float((uint16_t)(blk[0] | (blk[1] << 8)));
            const float dmin = half_to_float((uint16_t)(blk[2] | (blk[3] << 8)));
            int sc[8], mn[8]; k4_scales(blk + 4, sc, mn);
            for (int g = 0; g < 4; ++g) for (int h = 0; h < 2; ++h) {
                const int sb = 2 * g + h;
                const float* x = in + b * 256 + sb * 32;
                float code_sum = 0.0f, in_sum = 0.0f;
                for (int i = 0; i < 32; ++i) {
                    const uint8_t pb = blk[16 + 32 * g + i];
                    const int code = h == 0 ? (pb & 0x0F) : (pb >> 4);
                    code_sum += x[i] * (float) code;
                    in_sum += x[i];
                }
                acc += code_sum * (d * (float) sc[sb]) - in_sum * (dmin * (float) mn[sb]);
            }
        }
        out[o] = acc;
    }
}

/* ------------------------------------------------------------------------------------------------
 * The native path: Q8 activation quantization + integer dots.
 * native/src/q4k_matmul.c:74-92 (quantize), :143-198 (block dot), :211-251 (block term),
 * :273-307 (row loops), :315-357 (run).
 */
API float oracle_q8_quantize_block(const float* in, int8_t* q8) {
    float maxabs = 0.0f;
    for (int i = 0; i < 256; ++i) { const float a = fabsf(in[i]); if (a > maxabs) maxabs = a; }
    if (maxabs == 0.0f) { memset(q8, 0, 256); return 0.0f; }
    const float d_in = maxabs / 127.0f, inv = 127.0f / maxabs;
    for (int i = 0; i < 256; ++i) {
        int v = (int) lrintf(in[i] * inv);
        if (v > 127) v = 127; else if (v < -127) v = -127;
        q8[i] = (int8_t) v;
    }
    return d_in;
}

static float q4k_block_term(const uint8_t* blk, const int8_t* q8, float di) {
    const float d = half_to_float((uint16_t)(blk[0] | (blk[1] << 8)));
    const float dmin = half_to_float((uint16_t)(blk[2] | (blk[3] << 8)));
    int sc[8], mn[8]; k4_scales(blk + 4, sc, mn);
    int64_t sdot = 0, msum = 0;
    for (int g = 0; g < 4; ++g) {
        const uint8_t* qs = blk + 16 + 32 * g;
        const int8_t* lo = q8 + 64 * g; const int8_t* hi = lo + 32;
        int32_t dl = 0, sl = 0, dh = 0, sh = 0;
        for (int i = 0; i < 32; ++i) {
            dl += (int) lo[i] * (int)(qs[i] & 0x0F); sl += lo[i];
            dh += (int) hi[i] * (int)(qs[i] >> 4);   sh += hi[i];
        }
        sdot += (int64_t) sc[2 * g] * dl + (int64_t) sc[2 * g + 1] * dh;
        msum += (int64_t) mn[2 * g] * sl + (int64_t) mn[2 * g + 1] * sh;
    }
    return di * (d * (float) sdot - dmin * (float) msum);
}

/* order: 0 = row-major (o*bpr+b), 1 = feed order (b*output_dim+o). input_dim<=0 is a no-op
 * (q4k_matmul.c:326) — the native Q4_K kernel leaves the output untouched. */
API void oracle_q4k_matmul(const float* in, const uint8_t* w, int32_t input_dim, int32_t output_dim,
                           float* out, int32_t order) {
    if (output_dim <= 0 || input_dim <= 0) return;
    const int32_t nb = input_dim / 256;
    int8_t* q8 = (int8_t*) malloc((size_t) input_dim);
    float* di = (float*) malloc(sizeof(float) * (size_t) nb);
    for (int32_t b = 0; b < nb; ++b) di[b] = oracle_q8_quantize_block(in + (size_t) b * 256, q8 + (size_t) b * 256);
    for (int32_t o = 0; o < output_dim; ++o) {
        float acc = 0.0f;
        for (int32_t b = 0; b < nb; ++b) {
            const size_t idx = order == 0 ? (size_t) o * nb + b : (size_t) b * output_dim + o;
            acc += q4k_block_term(w + idx * 144, q8 + (size_t) b * 256, di[b]);
        }
        out[o] = acc;
    }
    free(q8); free(di);
}

/* Q6_K matvec, row-major. native/src/q6k_matmul.c:53-67 (activation quantizer = the Q4_K one), :83-128 (centered
 * codes in element order), :155-177 (weighted dot over sixteen 16-element scale groups, gs = half*8 + is + 2k),
 * :187-215 (block term d * d_in * (float) wdot), :252-268 (row loop). */
API void oracle_q6k_matmul(const float* in, const uint8_t* w, int32_t input_dim, int32_t output_dim, float* out) {
    if (output_dim <= 0 || input_dim <= 0) return;
    const int32_t nb = input_dim / 256;
    int8_t* q8 = (int8_t*) malloc((size_t) input_dim);
    float* di = (float*) malloc(sizeof(float) * (size_t) nb);
    for (int32_t b = 0; b < nb; ++b) di[b] = oracle_q8_quantize_block(in + (size_t) b * 256, q8 + (size_t) b * 256);
    for (int32_t o = 0; o < output_dim; ++o) {
        float acc = 0.0f;
        for (int32_t b = 0; b < nb; ++b) {
            const uint8_t* blk = w + ((size_t) o * nb + b) * 210;
            const int8_t* sc = (const int8_t*)(blk + 192);
            const float d = half_to_float((uint16_t)(blk[208] | (blk[209] << 8)));
            int8_t codes[256];
            for (int half = 0; half < 2; ++half) {
                const uint8_t* ql = blk + half * 64; const uint8_t* qh = blk + 128 + half * 32;
                int8_t* c = codes + half * 128;
                for (int l = 0; l < 32; ++l) {
                    c[l]      = (int8_t)((int)((ql[l] & 0x0F) | (((qh[l] >> 0) & 3) << 4)) - 32);
                    c[l + 32] = (int8_t)((int)((ql[l + 32] & 0x0F) | (((qh[l] >> 2) & 3) << 4)) - 32);
                    c[l + 64] = (int8_t)((int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32);
                    c[l + 96] = (int8_t)((int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32);
                }
            }
            int64_t wdot = 0;
            const int8_t* a = q8 + (size_t) b * 256;
            for (int half = 0; half < 2; ++half)
                for (int k = 0; k < 4; ++k)
                    for (int is = 0; is < 2; ++is) {
                        const int start = half * 128 + 32 * k + is * 16, gs = half * 8 + is + 2 * k;
                        int32_t dot = 0;
                        for (int j = 0; j < 16; ++j) dot += (int) a[start + j] * (int) codes[start + j];
                        wdot += (int64_t) sc[gs] * dot;
                    }
            acc += d * di[b] * (float) wdot;
        }
        out[o] = acc;
    }
    free(q8); free(di);
}

/* Q5_K matvec, row-major, fp32 activations. native/src/q5k_matmul.c:93-215 (portable body): per 64-element group
 * the low- and high-nibble sub-blocks accumulate code_sum = sum v*code and input_sum = sum v, then
 * acc += code_sum * (d*sc) - input_sum * (dmin*mn), low then high; :242-254 (row loop). */
API void oracle_q5k_matmul(const float* in, const uint8_t* w, int32_t input_dim, int32_t output_dim, float* out) {
    if (output_dim <= 0) return;
    if (input_dim <= 0) { for (int32_t o = 0; o < output_dim; ++o) out[o] = 0.0f; return; }
    const int32_t nb = input_dim / 256;
    for (int32_t o = 0; o < output_dim; ++o) {
        float acc_row = 0.0f;
        for (int32_t b = 0; b < nb; ++b) {
            const uint8_t* blk = w + ((size_t) o * nb + b) * 176;
            const float d = half_to_float((uint16_t)(blk[0] | (blk[1] << 8)));
            const float dmin = half_to_float((uint16_t)(blk[2] | (blk[3] << 8)));
            int sc[8], mn[8]; k4_scales(blk + 4, sc, mn);
            const uint8_t* qh = blk + 16; const uint8_t* qs = blk + 48;
            const float* x = in + (size_t) b * 256;
            float acc = 0.0f;
            for (int g = 0; g < 4; ++g) {
                float cs_lo = 0.0f, is_lo = 0.0f, cs_hi = 0.0f, is_hi = 0.0f;
                for (int i = 0; i < 32; ++i) {
                    const uint8_t by = qs[32 * g + i], h = qh[i];
                    const float c_lo = (float)((by & 0x0F) | (((h >> (2 * g)) & 1) << 4));
                    const float c_hi = (float)((by >> 4) | (((h >> (2 * g + 1)) & 1) << 4));
                    const float v_lo = x[64 * g + i], v_hi = x[64 * g + 32 + i];
                    cs_lo += v_lo * c_lo; is_lo += v_lo; cs_hi += v_hi * c_hi; is_hi += v_hi;
                }
                acc += cs_lo * (d * (float) sc[2 * g]) - is_lo * (dmin * (float) mn[2 * g]);
                acc += cs_hi * (d * (float) sc[2 * g + 1]) - is_hi * (dmin * (float) mn[2 * g + 1]);
            }
            acc_row += acc;
        }
        out[o] = acc_row;
    }
}

/* native/src/q8_0_matmul.c:68-118 (block term: fp32 activations, per-block sum then * d),
 * :134-165 (row loops), :168-187 (run; input_dim<=0 zeroes the output). */
API void oracle_q8_0_matmul(const float* in, const uint8_t* w, int32_t input_dim, int32_t output_dim,
                            float* out, int32_t order) {
    if (output_dim <= 0) return;
    if (input_dim <= 0) { for (int32_t o = 0; o < output_dim; ++o) out[o] = 0.0f; return; }
    const int32_t nb = input_dim / 32;
    for (int32_t o = 0; o < output_dim; ++o) {
        float acc = 0.0f;
        for (int32_t b = 0; b < nb; ++b) {
            const size_t idx = order == 0 ? (size_t) o * nb + b : (size_t) b * output_dim + o;
            const uint8_t* blk = w + idx * 34;
            const float d = half_to_float((uint16_t)(blk[0] | (blk[1] << 8)));
            float s = 0.0f;
            for (int k = 0; k < 32; ++k) s += in[b * 32 + k] * (float)(int8_t) blk[2 + k];
            acc += s * d;
        }
        out[o] = acc;
    }
}

/* ------------------------------------------------------------------------------------------------
 * Fused fp32 row kernels. native/src/f32_fused.c:255-286 (rms norm). */
API void oracle_rms_norm(const float* in, const float* gamma, float* out, int32_t rows, int32_t cols, float eps) {
    for (int32_t r = 0; r < rows; ++r) {
        const float* x = in + (size_t) r * cols; float* o = out + (size_t) r * cols;
        float ss = 0.0f;
        for (int32_t i = 0; i < cols; ++i) ss += x[i] * x[i];
        const float scale = 1.0f / sqrtf(ss * (1.0f / (float) cols) + eps);
        for (int32_t i = 0; i < cols; ++i) { float y = x[i] * scale; if (gamma) y *= gamma[i]; o[i] = y; }
    }
}

/* native/src/f32_fused.c:304-360 (one query row), :375-396 (entry). Key range rules as
 * skainet-lang/skainet-lang-core/src/commonMain/kotlin/sk/ainet/lang/tensor/ops/AttentionMask.kt:57-78. */
#define SDPA_MASKED (-1.0e30f)
API void oracle_sdpa(const float* q, const float* k, const float* v, float* out,
                     int32_t batch, int32_t heads, int32_t kv_heads, int32_t seq_q, int32_t seq_kv, int32_t d,
                     float scale, int32_t causal, int32_t window, int32_t right_context, const int32_t* lengths,
                     const float* mask, int32_t mask_b, int32_t mask_h, int32_t mask_q, int32_t mask_k) {
    if (batch <= 0 || heads <= 0 || kv_heads <= 0 || seq_q <= 0 || d <= 0) return;
    if (seq_kv <= 0) { memset(out, 0, sizeof(float) * (size_t) batch * heads * seq_q * d); return; }
    float* s = (float*) malloc(sizeof(float) * (size_t) seq_kv);
    for (int32_t b = 0; b < batch; ++b) for (int32_t h = 0; h < heads; ++h) for (int32_t qi = 0; qi < seq_q; ++qi) {
        const int32_t kvh = h / (heads / kv_heads);
        const float* qr = q + (((size_t) b * heads + h) * seq_q + qi) * d;
        const float* kb = k + ((size_t) b * kv_heads + kvh) * seq_kv * d;
        const float* vb = v + ((size_t) b * kv_heads + kvh) * seq_kv * d;
        float* o = out + (((size_t) b * heads + h) * seq_q + qi) * d;
        const int32_t abs_q = seq_kv - seq_q + qi;
        int32_t first = 0, end = seq_kv;
        if (window > 0) {
            if (abs_q - window + 1 > first) first = abs_q - window + 1;
            if (abs_q + right_context + 1 < end) end = abs_q + right_context + 1;
        }
        if (causal && abs_q + 1 < end) end = abs_q + 1;
        if (lengths && lengths[b] < end) end = lengths[b];
        if (end < 0) end = 0;
        if (first > end) first = end;
        for (int32_t ki = 0; ki < seq_kv; ++ki) s[ki] = SDPA_MASKED;
        for (int32_t ki = first; ki < end; ++ki) {
            float acc = 0.0f;
            for (int32_t x = 0; x < d; ++x) acc += qr[x] * kb[(size_t) ki * d + x];
            s[ki] = acc * scale;
        }
        int32_t pf = first, pe = end;
        if (mask) {
            const int32_t bi = mask_b == 1 ? 0 : b;
            const int32_t hi = mask_h == 1 ? 0 : (mask_h == heads ? h : kvh);
            const float* m = mask + ((((size_t) bi * mask_h + hi) * mask_q) + (mask_q == 1 ? 0 : qi)) * mask_k;
            for (int32_t ki = 0; ki < seq_kv; ++ki) s[ki] += mask_k == 1 ? m[0] : m[ki];
            pf = 0; pe = seq_kv;
        }
        if (first >= end) { pf = 0; pe = seq_kv; }
        float mx = s[0];
        for (int32_t ki = 1; ki < seq_kv; ++ki) if (s[ki] > mx) mx = s[ki];
        float sum = 0.0f;
        for (int32_t ki = 0; ki < seq_kv; ++ki) { s[ki] = expf(s[ki] - mx); sum += s[ki]; }
        if (sum > 0.0f) { const float inv = 1.0f / sum; for (int32_t ki = 0; ki < seq_kv; ++ki) s[ki] *= inv; }
        for (int32_t x = 0; x < d; ++x) o[x] = 0.0f;
        for (int32_t ki = pf; ki < pe; ++ki) for (int32_t x = 0; x < d; ++x) o[x] += s[ki] * vb[(size_t) ki * d + x];
    }
    free(s);
}

/* native/src/f32_ops.c:222,243-245 (silu = x * 1/(1+exp(-x))). */
API void oracle_silu(const float* in, float* out, int32_t n) {
    for (int32_t i = 0; i < n; ++i) out[i] = in[i] * (1.0f / (1.0f + expf(-in[i])));
}
/* SwiGLU gate as the model composes it from the reference's elementwise kernels:
 * silu(gate) (f32_ops.c:243-245) then mul (f32_ops.c:107-114). */
API void oracle_swiglu(const float* gate, const float* up, float* out, int32_t n) {
    for (int32_t i = 0; i < n; ++i) out[i] = (gate[i] * (1.0f / (1.0f + expf(-gate[i])))) * up[i];
}

/* RoPE. NO REFERENCE CODE EXISTS (the only mentions are comments,
 * skainet-lang/skainet-lang-core/src/commonMain/kotlin/sk/ainet/context/ExecutionContext.kt:42,90,
 * which say "interleaved rotation"): parity unpinned. Declared convention: for pair index i of a head
 * of width d, angle = pos * theta^(-2i/d) evaluated in double, cos/sin rounded to float once;
 * mode 0 rotates elements (2i, 2i+1) ("interleaved"), mode 1 rotates (i, i + d/2) ("half split"):
 *   x' = x*c - y*s ; y' = x*s + y*c   (each product and sum individually rounded in fp32). */
API void oracle_rope_table(int32_t max_pos, int32_t d, float theta, float* cos_out, float* sin_out) {
    for (int32_t p = 0; p < max_pos; ++p) for (int32_t i = 0; i < d / 2; ++i) {
        const double a = (double) p * pow((double) theta, -2.0 * (double) i / (double) d);
        cos_out[(size_t) p * (d / 2) + i] = (float) cos(a);
        sin_out[(size_t) p * (d / 2) + i] = (float) sin(a);
    }
}
API void oracle_rope(float* x, int32_t heads, int32_t d, int32_t pos, float theta, int32_t mode) {
    for (int32_t h = 0; h < heads; ++h) for (int32_t i = 0; i < d / 2; ++i) {
        const double a = (double) pos * pow((double) theta, -2.0 * (double) i / (double) d);
        const float c = (float) cos(a), s = (float) sin(a);
        float* px = x + (size_t) h * d + (mode == 0 ? 2 * i : i);
        float* py = x + (size_t) h * d + (mode == 0 ? 2 * i + 1 : i + d / 2);
        const float a0 = *px, b0 = *py;
        *px = a0 * c - b0 * s;
        *py = a0 * s + b0 * c;
    }
}

/* The same rotation applied to a cache-shaped block x[heads][len][d]: the row at index t of every head is
 * rotated for position pos0 + t (what a decoder has applied to each key before it was cached). */
API void oracle_rope_seq(float* x, int32_t heads, int32_t len, int32_t d, int32_t pos0, float theta, int32_t mode) {
    for (int32_t t = 0; t < len; ++t) for (int32_t i = 0; i < d / 2; ++i) {
        const double a = (double) (pos0 + t) * pow((double) theta, -2.0 * (double) i / (double) d);
        const float c = (float) cos(a), s = (float) sin(a);
        for (int32_t h = 0; h < heads; ++h) {
            float* row = x + ((size_t) h * len + t) * d;
            float* px = row + (mode == 0 ? 2 * i : i);
            float* py = row + (mode == 0 ? 2 * i + 1 : i + d / 2);
            const float a0 = *px, b0 = *py;
            *px = a0 * c - b0 * s;
            *py = a0 * s + b0 * c;
        }
    }
}

/* arg max, lowest index on ties:
 * skainet-backends/skainet-backend-cpu/src/commonMain/kotlin/sk/ainet/exec/tensor/ops/DefaultCpuOps.kt:3042-3078 */
API int32_t oracle_argmax(const float* x, int32_t n) {
    int32_t best = 0;
    for (int32_t i = 1; i < n; ++i) if (x[i] > x[best]) best = i;
    return best;
}

/* Round a float vector through binary16 (the f16 KV cache of the backend; f16->f32 is exact). */
API void oracle_round_f16(const float* in, float* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = half_to_float(float_to_half(in[i]));
}
API void oracle_to_f16(const float* in, uint16_t* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = float_to_half(in[i]);
}
