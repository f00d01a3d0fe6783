// Q6_K and Q5_K matvec over resident planes (the formats real Q4_K_M files mix in for some tensors).
//
// The kernels that carry the traffic (q6k_rows_kernel, q5k_rows_kernel): one warp per output row, four super-blocks per
// step, the next step's weight words requested before the current one is worked on (and the first step's before the wait
// on the preceding kernel). Up to eight (Q6_K) or four (Q5_K) activation rows ride on one pass over the weight: the codes
// are decoded once and reused; larger batches take the tensor-core tile kernels of gemm_kq.cu (Q6_K from nine rows, Q5_K
// from five). Both formats interleave their bit fields in runs
// of 32 elements. Q6_K: eight lanes per super-block, 16 bytes per lane = 16 consecutive elements of one run in the low
// nibbles and of the run 64 elements later in the high nibbles, one scale group each. Q5_K: see its kernel.
//
// Q6_K, native mode (reference: native/src/q6k_matmul.c:53-67 activation quantizer, :83-128 code layout,
// :155-177 weighted dot, :187-215 block term): the activation is int8 per 256 (the Q4_K quantizer), a block
// contributes d * d_in * float( sum_g sc[g] * sum_{i in g} q8[i] * (code[i] - 32) ) with 16-element scale groups;
// the integer sum is exact (dp4a on code - 32 as signed bytes, added across the block's eight lanes), the two fp32
// products and the running sum over blocks are done in the reference's order, so a row is bit-identical to the C kernel.
// Q5_K (reference: native/src/q5k_matmul.c:93-215) keeps fp32 activations: per sub-block
// code_sum * (d * sc) - input_sum * (dmin * mn); here each lane forms those two sums over its 16 elements and the
// warp adds the lanes at the end (fp32 rounding order differs from the CPU's vector lanes; parity is to tolerance).
// F32 mode for Q6_K is the plain dequantised dot product (q6k_matvec_kernel<false>: one lane per element of a run,
// the exact-float mode is not a streaming path).
#include "common.cuh"
#include "actquant.cuh"
#include "tma.cuh"

namespace sk {

namespace {

constexpr int KQ_WARPS = 8;

__device__ __forceinline__ float h2f(const uint8_t* p) { return __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(p))); }

// code - 32 of element 128n + 32q + l from the ql / qh bytes of half n
__device__ __forceinline__ int q6_code(uint32_t ql_a, uint32_t ql_b, uint32_t qh, int q) {
    const uint32_t lb = (q & 1) ? ql_b : ql_a;
    const int low = (q & 2) ? (int) (lb >> 4) : (int) (lb & 0x0f);
    return (low | (int) (((qh >> (2 * q)) & 3) << 4)) - 32;
}

// F32 mode of Q6_K: one lane per element of a 32-element run.
__global__ void __launch_bounds__(KQ_WARPS * 32)
q6k_matvec_f32_kernel(const uint8_t* __restrict__ ql, const uint8_t* __restrict__ qh, const int8_t* __restrict__ sc, const uint8_t* __restrict__ dd,
                      int rows, int bpr, const float* __restrict__ x, float* __restrict__ y) {
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    const int lane = threadIdx.x & 31, row = blockIdx.x * KQ_WARPS + (threadIdx.x >> 5), mrow = blockIdx.y;
    if (row >= rows) return;
    const int cols = bpr * 256;
    float acc = 0.0f;
    for (int b = 0; b < bpr; ++b) {
        const size_t pblk = (size_t) row * bpr + b;
        const float d = h2f(dd + pblk * 2);
        float fsum = 0.0f;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            const uint32_t a = ql[pblk * 128 + n * 64 + lane], bb = ql[pblk * 128 + n * 64 + 32 + lane], h = qh[pblk * 64 + n * 32 + lane];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int code = q6_code(a, bb, h, q);
                const int s = (int) sc[pblk * 16 + n * 8 + 2 * q + (lane >> 4)];
                const size_t e = (size_t) mrow * cols + (size_t) b * 256 + n * 128 + q * 32 + lane;
                fsum += (d * (float) s) * (float) code * x[e];
            }
        }
        acc += fsum;
    }
    acc = skd::warp_sum(acc);
    if (lane == 0) y[(size_t) mrow * rows + row] = acc;
}

// Activation rows from which the tensor-core tile kernel (gemm_kq.cu) takes a Q6_K product: 11008 x 4096 at 9 / 12 rows
// 52 / 50 us there against 57 / 71 us in two passes of the row kernel (8 rows: 47 us in one pass).
constexpr int Q6K_GEMM_MIN_ROWS = 9;
constexpr int KQR_WARPS = 4;       // small CTAs: a 4096-row weight still spreads evenly over the SMs

__device__ __forceinline__ uint32_t word_of(const uint4& v, int k) { return k == 0 ? v.x : k == 1 ? v.y : k == 2 ? v.z : v.w; }

// Native Q6_K over MT activation rows (act rows m0 .. m0 + mm - 1 of the quantized batch).
// Lane = (block of the step: lane >> 3, part j = lane & 7). Part j holds ql bytes [16 j, 16 j + 16) of its block: half
// n = j >> 2, run pair (j >> 1) & 1, bytes 16 (j & 1) .. + 15 of the run, i.e. elements e_lo = 128 n + 16 (j & 3) .. + 15
// in the low nibbles (scale group e_lo / 16) and e_lo + 64 .. in the high nibbles (scale group + 4); the high bits of
// both sit in qh bytes 32 n + 16 (j & 1) .. at bit 2 * ((j >> 1) & 1) and four bits above.
// The weight bytes of step b0 + 4 are requested before step b0 is worked on, and those of the first step before the
// wait on the preceding kernel (the weights depend on nothing), so a warp keeps two steps of loads in flight.
struct Q6Step { uint4 a, h; uint2 s8; float d; };

template <int MT>
__global__ void __launch_bounds__(KQR_WARPS * 32)
q6k_rows_kernel(const uint8_t* __restrict__ ql, const uint8_t* __restrict__ qh, const int8_t* __restrict__ sc, const uint8_t* __restrict__ dd,
                int rows, int bpr, ActQ8K act, int m0, int mm, float* y, const float* resid) {
    skd::pdl_launch_dependents();
    const int lane = threadIdx.x & 31, row = min((int) (blockIdx.x * KQR_WARPS + (threadIdx.x >> 5)), rows - 1);   // a warp past the end repeats the last row
    const int cols = bpr * 256, j = lane & 7, bq = lane >> 3;
    const int e_lo = 128 * (j >> 2) + 16 * (j & 3), sh = 2 * ((j >> 1) & 1), sbyte = 8 * (j & 3);
    auto fetch = [&](int b0) {
        const size_t pblk = (size_t) row * bpr + min(b0 + bq, bpr - 1);       // lanes past the row's last block repeat it and are left out below
        Q6Step r;
        r.a = skd::ld_stream(ql + pblk * 128 + 16 * j);
        r.h = skd::ld_stream(qh + pblk * 64 + 32 * (j >> 2) + 16 * (j & 1));
        r.s8 = __ldg(reinterpret_cast<const uint2*>(sc + pblk * 16 + 8 * (j >> 2)));
        r.d = h2f(dd + pblk * 2);
        return r;
    };
    Q6Step cur = fetch(0);
    skd::pdl_wait();                     // the quantized activation is the preceding kernel's output
    float acc[MT];
#pragma unroll
    for (int i = 0; i < MT; ++i) acc[i] = 0.0f;
#pragma unroll 1
    for (int b0 = 0; b0 < bpr; b0 += 4) {
        Q6Step nxt = cur;
        if (b0 + 4 < bpr) nxt = fetch(b0 + 4);
        const int blk = min(b0 + bq, bpr - 1);
        const int s_lo = (int) (int8_t) (cur.s8.x >> sbyte), s_hi = (int) (int8_t) (cur.s8.y >> sbyte);
        uint32_t lo_c[4], hi_c[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t aw = word_of(cur.a, k), hw = word_of(cur.h, k) >> sh;
            lo_c[k] = __vsub4((aw & 0x0f0f0f0fu) | ((hw & 0x03030303u) << 4), 0x20202020u);
            hi_c[k] = __vsub4(((aw >> 4) & 0x0f0f0f0fu) | (((hw >> 4) & 0x03030303u) << 4), 0x20202020u);
        }
#pragma unroll
        for (int i = 0; i < MT; ++i) {
            if (i < mm) {
                const int8_t* xq = act.q + (size_t) (m0 + i) * cols + (size_t) blk * 256 + e_lo;
                const uint4 xl = skd::ld_ro(xq), xh = skd::ld_ro(xq + 64);
                int gl = 0, gh = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    gl = __dp4a((int) lo_c[k], (int) word_of(xl, k), gl);
                    gh = __dp4a((int) hi_c[k], (int) word_of(xh, k), gh);
                }
                int isum = s_lo * gl + s_hi * gh;
                isum += __shfl_xor_sync(0xffffffffu, isum, 1);
                isum += __shfl_xor_sync(0xffffffffu, isum, 2);
                isum += __shfl_xor_sync(0xffffffffu, isum, 4);
                const float term = __fmul_rn(__fmul_rn(cur.d, __ldg(act.d + (size_t) (m0 + i) * bpr + blk)), (float) isum);
#pragma unroll
                for (int jb = 0; jb < 4; ++jb) {                    // the reference adds the blocks of a row in order
                    const float t = __shfl_sync(0xffffffffu, term, 8 * jb);
                    if (b0 + jb < bpr) acc[i] = __fadd_rn(acc[i], t);
                }
            }
        }
        cur = nxt;
    }
    if ((int) (blockIdx.x * KQR_WARPS + (threadIdx.x >> 5)) >= rows) return;
#pragma unroll
    for (int i = 0; i < MT; ++i)
        if (i < mm && lane == i) {
            const size_t o = (size_t) (m0 + i) * rows + row;
            y[o] = resid ? __fadd_rn(resid[o], acc[i]) : acc[i];       // resid may be y itself: read and written by this thread only
        }
}

// Q5_K over MT fp32 activation rows. The fp32 activation is sixteen times the weight bytes, so its loads decide
// the mapping: lane l takes the 4-byte word l of a block's 128 nibble bytes, i.e. elements 64 g + 4 (l & 7) .. + 3 of
// sub-block 2 g (g = l >> 3) in the low nibbles and the same offsets of sub-block 2 g + 1 in the high ones, so the two
// float4 activation loads of a block are 128 contiguous bytes per eight lanes; the fifth bits are bits 2 g and 2 g + 1
// of qh bytes 4 (l & 7) .. + 3. Four blocks per step, the next step's words requested before the current one is worked on;
// the four headers of a step are decoded in one pass, each lane one sub-block's scale and min, and handed round by shuffles.
struct Q5Step { uint32_t a[4], hb[4]; uint4 hd; };       // hd: the header of block (lane >> 3) of the step

// code bytes of a word as floats: 0x4B000000 | byte is 2^23 + byte as an fp32 bit pattern
__device__ __forceinline__ float byte_to_float(uint32_t w, int t) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650 + t)) - 8388608.0f;
}

template <int MT>
__global__ void __launch_bounds__(KQR_WARPS * 32)
q5k_rows_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ hdr, const uint8_t* __restrict__ qh,
                int rows, int bpr, const float* __restrict__ x, int mm, float* __restrict__ y) {
    skd::pdl_launch_dependents();
    const int lane = threadIdx.x & 31, row = min((int) (blockIdx.x * KQR_WARPS + (threadIdx.x >> 5)), rows - 1);   // a warp past the end repeats the last row
    const int cols = bpr * 256, g = lane >> 3, p = 4 * (lane & 7);
    auto fetch = [&](int b0) {
        Q5Step r;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const size_t pblk = (size_t) row * bpr + min(b0 + u, bpr - 1);      // steps past the row's last block repeat it with zero scales
            r.a[u] = __ldg(reinterpret_cast<const uint32_t*>(qs + pblk * 128) + lane);
            r.hb[u] = __ldg(reinterpret_cast<const uint32_t*>(qh + pblk * 32) + (lane & 7));
        }
        r.hd = skd::ld_ro(hdr + ((size_t) row * bpr + min(b0 + g, bpr - 1)) * 16);
        return r;
    };
    Q5Step cur = fetch(0);
    skd::pdl_wait();                     // the activation may be the preceding kernel's output
    float acc[MT];
#pragma unroll
    for (int i = 0; i < MT; ++i) acc[i] = 0.0f;
#pragma unroll 1
    for (int b0 = 0; b0 < bpr; b0 += 4) {
        Q5Step nxt = cur;
        if (b0 + 4 < bpr) nxt = fetch(b0 + 4);
        // the headers of the step's four blocks are decoded in one pass: lane 8 u + sb holds d * sc and dmin * mn of sub-block sb of block u
        float s_mine, o_mine;
        {
            const uint4 hd = cur.hd;
            const float d = __half2float(__ushort_as_half((unsigned short) (hd.x & 0xffff)));
            const float dmin = __half2float(__ushort_as_half((unsigned short) (hd.x >> 16)));
            uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
            skd::k4_unpack(hd.y, hd.z, hd.w, sc_lo, sc_hi, mn_lo, mn_hi);
            const int sb = lane & 7;
            const bool live = b0 + g < bpr;
            s_mine = live ? d * (float) skd::byte_of(sb < 4 ? sc_lo : sc_hi, sb & 3) : 0.0f;
            o_mine = live ? dmin * (float) skd::byte_of(sb < 4 ? mn_lo : mn_hi, sb & 3) : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int blk = min(b0 + u, bpr - 1);
            const float s_a = __shfl_sync(0xffffffffu, s_mine, 8 * u + 2 * g), s_b = __shfl_sync(0xffffffffu, s_mine, 8 * u + 2 * g + 1);
            const float o_a = __shfl_sync(0xffffffffu, o_mine, 8 * u + 2 * g), o_b = __shfl_sync(0xffffffffu, o_mine, 8 * u + 2 * g + 1);
            const uint32_t hw = cur.hb[u] >> (2 * g);
            const uint32_t wa = (cur.a[u] & 0x0f0f0f0fu) | ((hw & 0x01010101u) << 4), wb = ((cur.a[u] >> 4) & 0x0f0f0f0fu) | (((hw >> 1) & 0x01010101u) << 4);
            const float ca0 = byte_to_float(wa, 0), ca1 = byte_to_float(wa, 1), ca2 = byte_to_float(wa, 2), ca3 = byte_to_float(wa, 3);
            const float cb0 = byte_to_float(wb, 0), cb1 = byte_to_float(wb, 1), cb2 = byte_to_float(wb, 2), cb3 = byte_to_float(wb, 3);
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                if (i < mm) {
                    const float* xb = x + (size_t) i * cols + (size_t) blk * 256 + 64 * g + p;
                    const float4 va = __ldg(reinterpret_cast<const float4*>(xb)), vb = __ldg(reinterpret_cast<const float4*>(xb + 32));
                    const float cs_a = (va.x * ca0 + va.y * ca1) + (va.z * ca2 + va.w * ca3), is_a = (va.x + va.y) + (va.z + va.w);
                    const float cs_b = (vb.x * cb0 + vb.y * cb1) + (vb.z * cb2 + vb.w * cb3), is_b = (vb.x + vb.y) + (vb.z + vb.w);
                    acc[i] += (cs_a * s_a - is_a * o_a) + (cs_b * s_b - is_b * o_b);
                }
            }
        }
        cur = nxt;
    }
    if ((int) (blockIdx.x * KQR_WARPS + (threadIdx.x >> 5)) >= rows) return;
#pragma unroll
    for (int i = 0; i < MT; ++i) {
        if (i < mm) {
            const float v = skd::warp_sum(acc[i]);
            if (lane == 0) y[(size_t) i * rows + row] = v;
        }
    }
}

template <int MT>
cudaError_t launch_q6k_rows(const Weight& w, ActQ8K a, int m0, int mm, float* y, const float* resid, cudaStream_t s) {
    return launch_pdl(q6k_rows_kernel<MT>, dim3((w.rows + KQR_WARPS - 1) / KQR_WARPS), dim3(KQR_WARPS * 32), 0, s, (const uint8_t*) w.qs,
                      (const uint8_t*) w.extra, (const int8_t*) w.hdr, (const uint8_t*) w.aux, w.rows, w.bpr, a, m0, mm, y, resid);
}
template <int MT>
cudaError_t launch_q5k_rows(const Weight& w, const float* x, int mm, float* y, cudaStream_t s) {
    return launch_pdl(q5k_rows_kernel<MT>, dim3((w.rows + KQR_WARPS - 1) / KQR_WARPS), dim3(KQR_WARPS * 32), 0, s, (const uint8_t*) w.qs,
                      (const uint8_t*) w.hdr, (const uint8_t*) w.extra, w.rows, w.bpr, x, mm, y);
}

}  // namespace

// y[m][w.rows] for Q6_K (native int8 activations already quantized into `a`, or fp32 x) and Q5_K (always fp32 x).
// Activation rows go through in groups of up to eight (Q6_K) or four (Q5_K) per pass over the weight (the callers send
// larger batches to the tile kernels of gemm_kq.cu first). resid (native Q6_K
// only; may be y itself): y = resid + W x.
int32_t launch_matvec_kq(const Weight& w, const float* x, ActQ8K a, int m, float* y, int act_mode, cudaStream_t s, const float* resid) {
    if (m <= 0 || w.rows <= 0) return SKAINET_CUDA_OK;
    if (resid && !(w.enc == SKAINET_ENC_Q6_K && act_mode == SKAINET_ACT_NATIVE)) {
        set_error("matmul: the residual epilogue exists for native Q6_K only");
        return SKAINET_CUDA_ERR_INVALID;
    }
    if (w.enc == SKAINET_ENC_Q6_K && act_mode == SKAINET_ACT_NATIVE) {
        if (m >= Q6K_GEMM_MIN_ROWS) {
            const int32_t st = launch_gemm_q6k(w, a, m, y, resid, s);
            if (st != 1) return st;
        }
        for (int m0 = 0; m0 < m; m0 += 8) {
            const int mm = std::min(8, m - m0);
            if (mm == 1) SK_CUDA(launch_q6k_rows<1>(w, a, m0, mm, y, resid, s));
            else if (mm == 2) SK_CUDA(launch_q6k_rows<2>(w, a, m0, mm, y, resid, s));
            else if (mm <= 4) SK_CUDA(launch_q6k_rows<4>(w, a, m0, mm, y, resid, s));
            else SK_CUDA(launch_q6k_rows<8>(w, a, m0, mm, y, resid, s));
        }
        return SKAINET_CUDA_OK;
    }
    if (w.enc == SKAINET_ENC_Q6_K) {
        if (m > 65535) { set_error("matmul: %d activation rows exceed what the Q6_K F32 mode takes per call", m); return SKAINET_CUDA_ERR_INVALID; }
        SK_CUDA(launch_pdl(q6k_matvec_f32_kernel, dim3((w.rows + KQ_WARPS - 1) / KQ_WARPS, m), dim3(KQ_WARPS * 32), 0, s, (const uint8_t*) w.qs,
                           (const uint8_t*) w.extra, (const int8_t*) w.hdr, (const uint8_t*) w.aux, w.rows, w.bpr, x, y));
        return SKAINET_CUDA_OK;
    }
    if (w.enc == SKAINET_ENC_Q5_K) {
        for (int m0 = 0; m0 < m; m0 += 4) {
            const int mm = std::min(4, m - m0);
            const float* xr = x + (size_t) m0 * w.cols;
            float* yr = y + (size_t) m0 * w.rows;
            if (mm == 1) SK_CUDA(launch_q5k_rows<1>(w, xr, mm, yr, s));
            else if (mm == 2) SK_CUDA(launch_q5k_rows<2>(w, xr, mm, yr, s));
            else SK_CUDA(launch_q5k_rows<4>(w, xr, mm, yr, s));
        }
        return SKAINET_CUDA_OK;
    }
    return 1;
}

}  // namespace sk
