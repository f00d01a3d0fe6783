// Q6_K and Q5_K matvec over resident planes (the formats real Q4_K_M files mix in for some tensors).
// One warp per (output row, activation row); lane l takes the l-th element of every 32-element run of a
// super-block, which is how both formats interleave their bit fields, so all plane reads are 32 consecutive
// bytes per warp. First versions: correct and HBM-streaming, not yet staged through TMA like the Q4_K kernels.
//
// Q6_K, native mode (reference: native/src/q6k_matmul.c:53-67 activation quantizer, :83-128 code layout,
// :155-177 weighted dot, :187-215 block term): the activation is int8 per 256 (the Q4_K quantizer), a block
// contributes d * d_in * float( sum_g sc[g] * sum_{i in g} q8[i] * (code[i] - 32) ) with 16-element scale groups;
// the integer sum is exact, the two fp32 products and the running sum over blocks are done in the reference's
// order, so a row is bit-identical to the C kernel.
// Q5_K (reference: native/src/q5k_matmul.c:93-215) keeps fp32 activations: per sub-block
// code_sum * (d * sc) - input_sum * (dmin * mn); here one fused sum per lane and a warp reduction (fp32
// rounding order differs from the CPU's vector lanes; parity is to tolerance).
// F32 mode for Q6_K is the plain dequantised dot product.
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

template <bool NATIVE>
__global__ void __launch_bounds__(KQ_WARPS * 32)
q6k_matvec_kernel(const uint8_t* __restrict__ ql, const uint8_t* __restrict__ qh, const int8_t* __restrict__ sc, const uint8_t* __restrict__ dd,
                  int rows, int bpr, const float* __restrict__ x, ActQ8K act, float* __restrict__ y) {
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    const int lane = threadIdx.x & 31, row = blockIdx.x * KQ_WARPS + (threadIdx.x >> 5), mrow = blockIdx.y;
    if (row >= rows) return;
    const int cols = bpr * 256;
    float acc = 0.0f;
    for (int b = 0; b < bpr; ++b) {
        const size_t pblk = (size_t) row * bpr + b;
        const float d = h2f(dd + pblk * 2);
        int isum = 0; float fsum = 0.0f;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            const uint32_t a = ql[pblk * 128 + n * 64 + lane], bb = ql[pblk * 128 + n * 64 + 32 + lane], h = qh[pblk * 64 + n * 32 + lane];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int code = q6_code(a, bb, h, q);
                const int s = (int) sc[pblk * 16 + n * 8 + 2 * q + (lane >> 4)];
                const size_t e = (size_t) mrow * cols + (size_t) b * 256 + n * 128 + q * 32 + lane;
                if (NATIVE) isum += s * code * (int) act.q[e];
                else fsum += (d * (float) s) * (float) code * x[e];
            }
        }
        if (NATIVE) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) isum += __shfl_xor_sync(0xffffffffu, isum, o);
            const float di = act.d[(size_t) mrow * bpr + b];
            acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(d, di), (float) isum));     // d * d_in * float(wdot), summed block by block
        } else acc += fsum;
    }
    if (!NATIVE) acc = skd::warp_sum(acc);
    if (lane == 0) y[(size_t) mrow * rows + row] = acc;
}

__global__ void __launch_bounds__(KQ_WARPS * 32)
q5k_matvec_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ hdr, const uint8_t* __restrict__ qh,
                  int rows, int bpr, const float* __restrict__ x, float* __restrict__ y) {
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    const int lane = threadIdx.x & 31, row = blockIdx.x * KQ_WARPS + (threadIdx.x >> 5), mrow = blockIdx.y;
    if (row >= rows) return;
    const int cols = bpr * 256;
    float acc = 0.0f;
    for (int b = 0; b < bpr; ++b) {
        const size_t pblk = (size_t) row * bpr + b;
        const uint4 hd = *reinterpret_cast<const uint4*>(hdr + pblk * 16);
        const float d = __half2float(__ushort_as_half((unsigned short) (hd.x & 0xffff)));
        const float dmin = __half2float(__ushort_as_half((unsigned short) (hd.x >> 16)));
        uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
        skd::k4_unpack(hd.y, hd.z, hd.w, sc_lo, sc_hi, mn_lo, mn_hi);
        const uint32_t hb = qh[pblk * 32 + lane];
        const float* xb = x + (size_t) mrow * cols + (size_t) b * 256;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const uint32_t byte = qs[pblk * 128 + 32 * g + lane];
#pragma unroll
            for (int hi = 0; hi < 2; ++hi) {
                const int sb = 2 * g + hi;
                const int code = (int) (hi ? (byte >> 4) : (byte & 0x0f)) | (int) (((hb >> sb) & 1) << 4);
                const float s = d * (float) skd::byte_of(sb < 4 ? sc_lo : sc_hi, sb & 3);
                const float o = dmin * (float) skd::byte_of(sb < 4 ? mn_lo : mn_hi, sb & 3);
                const float v = xb[32 * sb + lane];
                acc += (v * (float) code) * s - v * o;
            }
        }
    }
    acc = skd::warp_sum(acc);
    if (lane == 0) y[(size_t) mrow * rows + row] = acc;
}

}  // namespace

// y[m][w.rows] for Q6_K (native int8 activations already quantized into `a`, or fp32 x) and Q5_K (always fp32 x).
int32_t launch_matvec_kq(const Weight& w, const float* x, ActQ8K a, int m, float* y, int act_mode, cudaStream_t s) {
    if (m <= 0 || w.rows <= 0) return SKAINET_CUDA_OK;
    if (m > 65535) { set_error("matmul: %d activation rows exceed what the Q5_K/Q6_K kernels take per call", m); return SKAINET_CUDA_ERR_INVALID; }
    dim3 grid((w.rows + KQ_WARPS - 1) / KQ_WARPS, m);
    if (w.enc == SKAINET_ENC_Q6_K) {
        if (act_mode == SKAINET_ACT_NATIVE)
            SK_CUDA(launch_pdl(q6k_matvec_kernel<true>, grid, dim3(KQ_WARPS * 32), 0, s, (const uint8_t*) w.qs, (const uint8_t*) w.extra, (const int8_t*) w.hdr,
                               (const uint8_t*) w.aux, w.rows, w.bpr, x, a, y));
        else
            SK_CUDA(launch_pdl(q6k_matvec_kernel<false>, grid, dim3(KQ_WARPS * 32), 0, s, (const uint8_t*) w.qs, (const uint8_t*) w.extra, (const int8_t*) w.hdr,
                               (const uint8_t*) w.aux, w.rows, w.bpr, x, a, y));
        return SKAINET_CUDA_OK;
    }
    if (w.enc == SKAINET_ENC_Q5_K) {
        SK_CUDA(launch_pdl(q5k_matvec_kernel, grid, dim3(KQ_WARPS * 32), 0, s, (const uint8_t*) w.qs, (const uint8_t*) w.hdr, (const uint8_t*) w.extra, w.rows,
                           w.bpr, x, y));
        return SKAINET_CUDA_OK;
    }
    return 1;
}

}  // namespace sk
