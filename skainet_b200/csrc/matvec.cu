// Dequant-fused matvec over packed Q4_K / Q8_0 weights resident in HBM, and the activation
// quantizers that feed it. HBM-bound: each weight byte is read once with 128-bit coalesced loads,
// nibbles/codes stay packed for __dp4a, scales and mins are decoded in registers, accumulation is
// fp32 per lane and rows are reduced with warp shuffles (no atomics: results are deterministic).
//
// Reference arithmetic followed here:
//   Q4_K: native/src/q4k_matmul.c:74-92 (per-256 int8 activation quantization),
//         :143-198 (integer sub-block dots), :211-251 (di * (d*sum_sc_dot - dmin*sum_mn_sum)).
//   Q8_0: native/src/q8_0_matmul.c:68-118 (fp32 activation x int8 code, block sum times d).
//   F32 mode: skainet-backends/skainet-backend-cpu/src/commonMain/kotlin/sk/ainet/exec/kernel/
//         ScalarQ4_KMatmulKernel.kt:66-75 and ScalarQ8_0MatmulKernel.kt:56-59.
#include "common.cuh"
#include "actquant.cuh"
#include "matvec_fused.cuh"
#include "tma.cuh"

#include <cstdlib>
#include <cstring>

namespace sk {

// ---- scratch layout of a quantized activation [m][cols] -----------------------------------------------
static inline size_t align256(size_t x) { return (x + 255) & ~(size_t) 255; }

size_t act_scratch_bytes(int enc, int act_mode, int m, int cols) {
    if (act_mode == SKAINET_ACT_F32) return 0;
    if (enc == SKAINET_ENC_Q5_K) return m >= Q5K_GEMM_MIN_ROWS ? act_f16split_bytes(m, cols) : 0;      // fp32 activations: only the tile kernel wants them prepared
    if (enc == SKAINET_ENC_Q8_0) return align256((size_t) m * cols) * 2 + align256((size_t) m * (cols / 32) * 4);
    return align256((size_t) m * cols) + align256((size_t) m * (cols / 256) * 4) + align256((size_t) m * (cols / 32) * 2);
}

ActQ8K act_q8k_layout(void* scratch, int m, int cols) {
    ActQ8K a;
    uint8_t* p = (uint8_t*) scratch;
    a.q = (int8_t*) p; p += align256((size_t) m * cols);
    a.d = (float*) p; p += align256((size_t) m * (cols / 256) * 4);
    a.bsums = (int16_t*) p;
    return a;
}
ActSplit act_split_layout(void* scratch, int m, int cols) {
    ActSplit a;
    uint8_t* p = (uint8_t*) scratch;
    a.hi = (int8_t*) p; p += align256((size_t) m * cols);
    a.lo = (int8_t*) p; p += align256((size_t) m * cols);
    a.d = (float*) p;
    return a;
}

// ---- activation quantizers ----------------------------------------------------------------------------
// One warp per 256-element block of one activation row.
__global__ void act_quant_q8k_kernel(const float* x, int64_t nblocks, ActQ8K a) {
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    const int64_t warp = (blockIdx.x * (int64_t) blockDim.x + threadIdx.x) >> 5;
    if (warp >= nblocks) return;
    skd::quant_q8k_block(x + warp * 256, a.q + warp * 256, a.d + warp, a.bsums + warp * 8, threadIdx.x & 31);
}
// One warp per 8 blocks of 32 (lane group of 4 per block).
__global__ void act_quant_split_kernel(const float* x, int64_t nblocks32, ActSplit a) {
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    const int64_t t = blockIdx.x * (int64_t) blockDim.x + threadIdx.x;
    const int64_t blk = t >> 2;
    const bool live = blk < nblocks32;
    skd::quant_split_block(x, a, live ? blk : nblocks32 - 1, threadIdx.x & 3, live);
}

int32_t launch_act_quant(int enc, int act_mode, const float* x, int m, int cols, void* scratch, cudaStream_t s) {
    if (act_mode == SKAINET_ACT_F32 || m == 0 || cols == 0) return SKAINET_CUDA_OK;
    if (enc == SKAINET_ENC_Q5_K) return m >= Q5K_GEMM_MIN_ROWS ? launch_act_f16split(x, m, cols, scratch, s) : SKAINET_CUDA_OK;
    if (enc == SKAINET_ENC_Q8_0) {
        const int64_t nb = (int64_t) m * (cols / 32);
        SK_CUDA(launch_pdl(act_quant_split_kernel, dim3((unsigned) ((nb * 4 + 255) / 256)), dim3(256), 0, s, x, nb, act_split_layout(scratch, m, cols)));
    } else {
        const int64_t nb = (int64_t) m * (cols / 256);
        SK_CUDA(launch_pdl(act_quant_q8k_kernel, dim3((unsigned) ((nb * 32 + 255) / 256)), dim3(256), 0, s, x, nb, act_q8k_layout(scratch, m, cols)));
    }
    SK_CUDA(cudaGetLastError());
    return SKAINET_CUDA_OK;
}

// ---- Q4_K matvec, int8 activations ----------------------------------------------------------------------
// One warp per output row. A lane pair (slot = lane/2) owns one 256-element super-block per step:
// lane parity h reads bytes [32g + 16h, 32g + 16h + 16) of each 32-byte group g, i.e. elements
// 64g+16h.. of the low-nibble sub-block 2g and 64g+32+16h.. of the high-nibble sub-block 2g+1.
// Per step the warp issues four fully used 16-byte loads per lane (2 KB of codes) plus the 16-byte
// headers, so a 4096-wide row is a single step.
constexpr int MV_WARPS = 8;

template <int M>
__global__ void __launch_bounds__(MV_WARPS * 32)
q4k_matvec_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ hdr, int rows, int bpr,
                  ActQ8K act, int cols, float* __restrict__ y) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x * MV_WARPS + warp;
    if (row >= rows) return;
    const int h = lane & 1, slot = lane >> 1;
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.0f;

    for (int b = slot; b < bpr; b += 16) {
        const int64_t blk = (int64_t) row * bpr + b;
        const uint8_t* qp = qs + blk * 128 + h * 16;
        uint4 w[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) w[g] = skd::ld_stream(qp + 32 * g);
        const uint4 hd = skd::ld_ro(hdr + blk * 16);
        const float d = __half2float(__ushort_as_half((unsigned short) (hd.x & 0xffff)));
        const float dmin = __half2float(__ushort_as_half((unsigned short) (hd.x >> 16)));
        uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
        skd::k4_unpack(hd.y, hd.z, hd.w, sc_lo, sc_hi, mn_lo, mn_hi);
        // scale of sub-block s: byte s of sc_lo (s < 4) or byte s-4 of sc_hi
        int sc[8];
#pragma unroll
        for (int s = 0; s < 4; ++s) { sc[s] = skd::byte_of(sc_lo, s); sc[s + 4] = skd::byte_of(sc_hi, s); }
        const uint32_t mn_mine = h ? mn_hi : mn_lo;   // lane h accounts the mins of sub-blocks 4h..4h+3

#pragma unroll
        for (int m = 0; m < M; ++m) {
            const int8_t* qa = act.q + (int64_t) m * cols + b * 256 + 16 * h;
            int sdot = 0;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const uint4 a_lo = skd::ld_ro(qa + 64 * g);
                const uint4 a_hi = skd::ld_ro(qa + 64 * g + 32);
                int dl = 0, dh = 0;
                dl = __dp4a((int) (w[g].x & 0x0f0f0f0fu), (int) a_lo.x, dl);
                dl = __dp4a((int) (w[g].y & 0x0f0f0f0fu), (int) a_lo.y, dl);
                dl = __dp4a((int) (w[g].z & 0x0f0f0f0fu), (int) a_lo.z, dl);
                dl = __dp4a((int) (w[g].w & 0x0f0f0f0fu), (int) a_lo.w, dl);
                dh = __dp4a((int) ((w[g].x >> 4) & 0x0f0f0f0fu), (int) a_hi.x, dh);
                dh = __dp4a((int) ((w[g].y >> 4) & 0x0f0f0f0fu), (int) a_hi.y, dh);
                dh = __dp4a((int) ((w[g].z >> 4) & 0x0f0f0f0fu), (int) a_hi.z, dh);
                dh = __dp4a((int) ((w[g].w >> 4) & 0x0f0f0f0fu), (int) a_hi.w, dh);
                sdot += sc[2 * g] * dl + sc[2 * g + 1] * dh;
            }
            // mins: sum_s mn[s] * (sum of the sub-block's int8 activations), four sub-blocks per lane
            const uint2 bs = __ldg((const uint2*) (act.bsums + ((int64_t) m * (cols / 32) + b * 8 + 4 * h)));
            const int msum = skd::byte_of(mn_mine, 0) * (int) (short) (bs.x & 0xffff) + skd::byte_of(mn_mine, 1) * (int) (short) (bs.x >> 16)
                           + skd::byte_of(mn_mine, 2) * (int) (short) (bs.y & 0xffff) + skd::byte_of(mn_mine, 3) * (int) (short) (bs.y >> 16);
            const float di = __ldg(act.d + (int64_t) m * (cols / 256) + b);
            acc[m] += di * (d * (float) sdot - dmin * (float) msum);
        }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
        const float r = skd::warp_sum(acc[m]);
        if (lane == 0) y[(int64_t) m * rows + row] = r;
    }
}

// ---- Q4_K matvec, exact-float activations (F32 mode) ---------------------------------------------------
__global__ void __launch_bounds__(MV_WARPS * 32)
q4k_matvec_f32_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ hdr, int rows, int bpr,
                      const float* __restrict__ x, int cols, float* __restrict__ y) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x * MV_WARPS + warp;
    const int m = blockIdx.y;
    if (row >= rows) return;
    const int h = lane & 1, slot = lane >> 1;
    const float* xr = x + (int64_t) m * cols;
    float acc = 0.0f;
    for (int b = slot; b < bpr; b += 16) {
        const int64_t blk = (int64_t) row * bpr + b;
        const uint8_t* qp = qs + blk * 128 + h * 16;
        const uint4 hd = skd::ld_ro(hdr + blk * 16);
        const float d = __half2float(__ushort_as_half((unsigned short) (hd.x & 0xffff)));
        const float dmin = __half2float(__ushort_as_half((unsigned short) (hd.x >> 16)));
        uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
        skd::k4_unpack(hd.y, hd.z, hd.w, sc_lo, sc_hi, mn_lo, mn_hi);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const uint4 wq = skd::ld_stream(qp + 32 * g);
            const uint32_t ww[4] = {wq.x, wq.y, wq.z, wq.w};
            const float* xl = xr + b * 256 + 64 * g + 16 * h;
            float cs_lo = 0.f, cs_hi = 0.f, xs_lo = 0.f, xs_hi = 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const uint32_t byte = (ww[i >> 2] >> (8 * (i & 3))) & 0xff;
                const float a = __ldg(xl + i), c = __ldg(xl + 32 + i);
                cs_lo += a * (float) (byte & 15); xs_lo += a;
                cs_hi += c * (float) (byte >> 4); xs_hi += c;
            }
            const int s0 = 2 * g, s1 = 2 * g + 1;
            const float sc0 = (float) skd::byte_of(s0 < 4 ? sc_lo : sc_hi, s0 & 3), sc1 = (float) skd::byte_of(s1 < 4 ? sc_lo : sc_hi, s1 & 3);
            const float mn0 = (float) skd::byte_of(s0 < 4 ? mn_lo : mn_hi, s0 & 3), mn1 = (float) skd::byte_of(s1 < 4 ? mn_lo : mn_hi, s1 & 3);
            acc += cs_lo * (d * sc0) - xs_lo * (dmin * mn0);
            acc += cs_hi * (d * sc1) - xs_hi * (dmin * mn1);
        }
    }
    acc = skd::warp_sum(acc);
    if (lane == 0) y[(int64_t) m * rows + row] = acc;
}

// ---- Q8_0 matvec, two-term int8 activations -------------------------------------------------------------
// One warp per output row; a lane owns 16 codes (half a block) per step, 512 contiguous bytes per
// warp load. The fp32 activation is carried as hi*128 + lo (two int8 planes, one scale per 32), so
// a block costs eight dp4a instead of 32 convert+FMA pairs; the 15-bit split keeps the result within
// ~4e-5 relative RMS of the reference's fp32 product.
template <int M>
__global__ void __launch_bounds__(MV_WARPS * 32)
q8_0_matvec_kernel(const int8_t* __restrict__ codes, const __half* __restrict__ scales, int rows, int cols,
                   ActSplit act, float* __restrict__ y) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x * MV_WARPS + warp;
    if (row >= rows) return;
    const int nchunks = cols >> 4, bpr = cols >> 5;
    const int8_t* wr = codes + (int64_t) row * cols;
    const __half* sr = scales + (int64_t) row * bpr;
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.0f;
#pragma unroll 4
    for (int c = lane; c < nchunks; c += 32) {
        const uint4 w = skd::ld_stream(wr + c * 16);
        const float dw = __half2float(sr[c >> 1]);
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const uint4 ah = skd::ld_ro(act.hi + (int64_t) m * cols + c * 16);
            const uint4 al = skd::ld_ro(act.lo + (int64_t) m * cols + c * 16);
            int dh = 0, dl = 0;
            dh = __dp4a((int) w.x, (int) ah.x, dh); dh = __dp4a((int) w.y, (int) ah.y, dh);
            dh = __dp4a((int) w.z, (int) ah.z, dh); dh = __dp4a((int) w.w, (int) ah.w, dh);
            dl = __dp4a((int) w.x, (int) al.x, dl); dl = __dp4a((int) w.y, (int) al.y, dl);
            dl = __dp4a((int) w.z, (int) al.z, dl); dl = __dp4a((int) w.w, (int) al.w, dl);
            const float dx = __ldg(act.d + (int64_t) m * bpr + (c >> 1));
            acc[m] += (dw * dx) * (float) (dh * 128 + dl);
        }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
        const float r = skd::warp_sum(acc[m]);
        if (lane == 0) y[(int64_t) m * rows + row] = r;
    }
}

// ---- Q8_0 matvec, fp32 activations exactly as the reference multiplies them (F32 mode) -----------
__global__ void __launch_bounds__(MV_WARPS * 32)
q8_0_matvec_f32_kernel(const int8_t* __restrict__ codes, const __half* __restrict__ scales, int rows, int cols,
                       const float* __restrict__ x, float* __restrict__ y) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x * MV_WARPS + warp;
    const int m = blockIdx.y;
    if (row >= rows) return;
    const int nchunks = cols >> 4, bpr = cols >> 5;
    const int8_t* wr = codes + (int64_t) row * cols;
    const float* xr = x + (int64_t) m * cols;
    float acc = 0.0f;
    for (int c = lane; c < nchunks; c += 32) {
        const uint4 w = skd::ld_stream(wr + c * 16);
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int code = (int) (int8_t) ((ww[i >> 2] >> (8 * (i & 3))) & 0xff);
            s += __ldg(xr + c * 16 + i) * (float) code;
        }
        acc += s * __half2float(scales[(int64_t) row * bpr + (c >> 1)]);
    }
    acc = skd::warp_sum(acc);
    if (lane == 0) y[(int64_t) m * rows + row] = acc;
}

// ---- dispatch -------------------------------------------------------------------------------------------
template <int M>
static void launch_q4k_m(const Weight& w, ActQ8K act, float* y, cudaStream_t s) {
    const int grid = (w.rows + MV_WARPS - 1) / MV_WARPS;
    q4k_matvec_kernel<M><<<grid, MV_WARPS * 32, 0, s>>>(w.qs, w.hdr, w.rows, w.bpr, act, w.cols, y);
}
template <int M>
static void launch_q8_m(const Weight& w, ActSplit act, float* y, cudaStream_t s) {
    const int grid = (w.rows + MV_WARPS - 1) / MV_WARPS;
    q8_0_matvec_kernel<M><<<grid, MV_WARPS * 32, 0, s>>>((const int8_t*) w.qs, (const __half*) w.hdr, w.rows, w.cols, act, y);
}

// y[m][rows] = x[m][cols] . W^T. Activation rows are taken in groups of up to 8 per pass over the
// weight (later passes of a large m are served from L2 when the weight fits there).
int32_t launch_matvec(const Weight& w, const float* x, const void* act_scratch, int m, float* y, int act_mode,
                      cudaStream_t s) {
    if (m == 0 || w.rows == 0) return SKAINET_CUDA_OK;
    if (w.enc == SKAINET_ENC_Q6_K || w.enc == SKAINET_ENC_Q5_K) {
        if (x == nullptr && (w.enc == SKAINET_ENC_Q5_K || act_mode == SKAINET_ACT_F32)) {      // Q6_K in the native mode reads the quantized rows only
            set_error("matmul: Q5_K (and Q6_K in the F32 mode) take the fp32 activation pointer");
            return SKAINET_CUDA_ERR_INVALID;
        }
        if (w.enc == SKAINET_ENC_Q5_K && act_mode == SKAINET_ACT_NATIVE && m >= Q5K_GEMM_MIN_ROWS && act_scratch) {
            const int32_t st = launch_gemm_q5k(w, act_scratch, m, y, s);
            if (st != 1) return st;
        }
        return launch_matvec_kq(w, x, act_q8k_layout(const_cast<void*>(act_scratch), m, w.cols), m, y, act_mode, s);
    }
    if (w.enc != SKAINET_ENC_Q4_K && w.enc != SKAINET_ENC_Q8_0) {
        set_error("matmul: encoding %d has no matvec kernel", w.enc);
        return SKAINET_CUDA_ERR_INVALID;
    }
    const int grid = (w.rows + MV_WARPS - 1) / MV_WARPS;
    if (act_mode == SKAINET_ACT_F32) {
        for (int m0 = 0; m0 < m; m0 += 65535) {
            const int mm = std::min(m - m0, 65535);
            dim3 g(grid, mm);
            if (w.enc == SKAINET_ENC_Q4_K)
                q4k_matvec_f32_kernel<<<g, MV_WARPS * 32, 0, s>>>(w.qs, w.hdr, w.rows, w.bpr, x + (int64_t) m0 * w.cols, w.cols, y + (int64_t) m0 * w.rows);
            else
                q8_0_matvec_f32_kernel<<<g, MV_WARPS * 32, 0, s>>>((const int8_t*) w.qs, (const __half*) w.hdr, w.rows, w.cols, x + (int64_t) m0 * w.cols, y + (int64_t) m0 * w.rows);
        }
        SK_CUDA(cudaGetLastError());
        return SKAINET_CUDA_OK;
    }
    if (m >= 2) {       // several activation rows: tensor-core tile kernel
        const int32_t st = w.enc == SKAINET_ENC_Q8_0
            ? launch_gemm_mma_q8(w, act_split_layout(const_cast<void*>(act_scratch), m, w.cols), m, y, nullptr, s)
            : launch_gemm_mma(w, act_q8k_layout(const_cast<void*>(act_scratch), m, w.cols), m, y, nullptr, s);
        if (st != 1) return st;
    }
    for (int m0 = 0; m0 < m;) {
        const int left = m - m0;
        const int mm = left >= 8 ? 8 : (left >= 4 ? 4 : (left >= 2 ? 2 : 1));
        float* yo = y + (int64_t) m0 * w.rows;
        {   // shapes the tile kernels decline: the streaming kernel, then direct loads
            const int32_t st = launch_matvec_stream(w, act_scratch, m, m0, mm, yo, s);
            if (st == SKAINET_CUDA_OK) { m0 += mm; continue; }
            if (st != 1) return st;
        }
        if (w.enc == SKAINET_ENC_Q4_K) {
            ActQ8K a = act_q8k_layout(const_cast<void*>(act_scratch), m, w.cols);
            a.q += (int64_t) m0 * w.cols; a.d += (int64_t) m0 * (w.cols / 256); a.bsums += (int64_t) m0 * (w.cols / 32);
            switch (mm) {
                case 8: launch_q4k_m<8>(w, a, yo, s); break;
                case 4: launch_q4k_m<4>(w, a, yo, s); break;
                case 2: launch_q4k_m<2>(w, a, yo, s); break;
                default: launch_q4k_m<1>(w, a, yo, s); break;
            }
        } else {
            ActSplit a = act_split_layout(const_cast<void*>(act_scratch), m, w.cols);
            a.hi += (int64_t) m0 * w.cols; a.lo += (int64_t) m0 * w.cols; a.d += (int64_t) m0 * (w.cols / 32);
            switch (mm) {
                case 8: launch_q8_m<8>(w, a, yo, s); break;
                case 4: launch_q8_m<4>(w, a, yo, s); break;
                case 2: launch_q8_m<2>(w, a, yo, s); break;
                default: launch_q8_m<1>(w, a, yo, s); break;
            }
        }
        m0 += mm;
    }
    SK_CUDA(cudaGetLastError());
    return SKAINET_CUDA_OK;
}

}  // namespace sk
