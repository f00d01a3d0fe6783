// Batched rows (m >= 2): Q4_K weights x int8-quantized activations on the tensor cores
// (mma.sync m16n8k32, u8 x s8 -> s32). Used by prefill (m = prompt tokens) and by decode with several
// sequences in a batch; one activation row is left to the matvec kernels.
//
// Arithmetic is the reference's integer path (native/src/q4k_matmul.c:143-251): per 32-element sub-block
// an exact integer dot of the 4-bit codes with the activation codes, scaled by the 6-bit sub-block scale,
// minus the 6-bit min times the sum of the activation codes, then d_in * (d * sum_sc - dmin * sum_mn) in
// fp32. The MMA's A tile is 16 weight rows x 32 codes of one sub-block, its B tile the same 32 codes of
// 8 activation rows, so an output tile reuses every weight byte for all its activation rows.
//
// CTA = NW warps x 16 weight rows, MT = 8*NT activation rows, looping over the 256-element super-blocks
// of the contraction through an NS-stage cp.async pipeline:
//   weight stage  [16*NW rows][144 B]: 128 B of nibbles then the 16-byte header; the 144-byte row stride
//                 makes ldmatrix (8 rows x 16 B) and the header reads bank-conflict free;
//   activation stage [MT rows][272 B]: 256 codes then the 8 int16 sub-block sums; 272-byte stride makes the
//                 B-fragment reads (8 rows x 4 words) conflict free; plus [MT] fp32 block scales.
// A lane's ldmatrix.x4 of 32 raw bytes per row yields the A fragments of two sub-blocks: low nibbles are
// sub-block 2g, high nibbles sub-block 2g+1 of 64-element group g.
#include "common.cuh"
#include "actquant.cuh"
#include "tma.cuh"
#include "matvec_fused.cuh"

#include <cstdlib>

namespace sk {

namespace {

constexpr int GW_STRIDE = 144;      // bytes per weight row per stage
constexpr int GX_STRIDE = 272;      // bytes per activation row per stage

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(skd::smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(skd::smem_u32(dst)), "l"(src) : "memory");
}
// 16 bytes, or zeros when `bytes` is 0 (activation rows past the batch)
__device__ __forceinline__ void cp_async16_zfill(void* dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(skd::smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(skd::smem_u32(p)));
}
__device__ __forceinline__ void mma_u8s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int NW, int NT, int NS, int EPI>
__global__ void __launch_bounds__(NW * 32)
q4k_gemm_mma_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ hdr, int rows, int bpr, ActQ8K act, int m,
                    float* __restrict__ y, const float* __restrict__ resid) {
    constexpr int RT = NW * 16, MT = NT * 8;
    constexpr int W_BYTES = RT * GW_STRIDE, X_BYTES = MT * GX_STRIDE, S_BYTES = W_BYTES + X_BYTES + MT * 4;
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * RT, col0 = blockIdx.y * MT;
    const int cols = bpr * 256;
    skd::pdl_launch_dependents();

    // Each thread copies the same chunks of every stage: its sources advance by one super-block per stage, so the
    // row / chunk arithmetic (divisions by 9 and 17) is done once, not per copy.
    constexpr int WSLOTS = (RT * 9 + NW * 32 - 1) / (NW * 32), XSLOTS = (MT * 17 + NW * 32 - 1) / (NW * 32);
    const uint8_t* wsrc[WSLOTS]; int wdst[WSLOTS], wstep[WSLOTS];
    const uint8_t* xsrc[XSLOTS]; int xdst[XSLOTS], xstep[XSLOTS], xbytes[XSLOTS];
#pragma unroll
    for (int i = 0; i < WSLOTS; ++i) {
        const int c = threadIdx.x + i * NW * 32;
        const int r = c / 9, ch = c % 9;
        const size_t blk0 = (size_t) min(row0 + r, rows - 1) * bpr;
        wdst[i] = c < RT * 9 ? r * GW_STRIDE + ch * 16 : -1;
        wsrc[i] = ch < 8 ? qs + blk0 * 128 + ch * 16 : hdr + blk0 * 16;
        wstep[i] = ch < 8 ? 128 : 16;
    }
#pragma unroll
    for (int i = 0; i < XSLOTS; ++i) {
        const int c = threadIdx.x + i * NW * 32;
        const int r = c / 17, ch = c % 17;
        const size_t arow = (size_t) min(col0 + r, m - 1);
        xdst[i] = c < MT * 17 ? r * GX_STRIDE + ch * 16 : -1;
        xsrc[i] = ch < 16 ? (const uint8_t*) (act.q + arow * cols + ch * 16) : (const uint8_t*) (act.bsums + arow * bpr * 8);
        xstep[i] = ch < 16 ? 256 : 16;
        // rows past the batch are zero-filled, not fetched: every CTA re-reading the last row's addresses cost 57344 x 8192
        // at five rows 82.7 us against 67.7 us
        xbytes[i] = col0 + r < m ? 16 : 0;
    }
    const float* dsrc = act.d + (size_t) min(col0 + (int) threadIdx.x, m - 1) * bpr;
    auto issue_w = [&](int kb) {
        uint8_t* st = smem + (size_t) (kb % NS) * S_BYTES;
#pragma unroll
        for (int i = 0; i < WSLOTS; ++i)
            if (wdst[i] >= 0) cp_async16(st + wdst[i], wsrc[i] + (size_t) kb * wstep[i]);
    };
    auto issue_x = [&](int kb) {
        uint8_t* st = smem + (size_t) (kb % NS) * S_BYTES + W_BYTES;
#pragma unroll
        for (int i = 0; i < XSLOTS; ++i)
            if (xdst[i] >= 0) cp_async16_zfill(st + xdst[i], xsrc[i] + (size_t) kb * xstep[i], xbytes[i]);
        if (threadIdx.x < MT) cp_async4(st + X_BYTES + threadIdx.x * 4, dsrc + kb);
    };

    // The weights depend on no predecessor: their first stages are in flight before the wait.
    for (int s = 0; s < NS - 1 && s < bpr; ++s) issue_w(s);
    skd::pdl_wait();
    for (int s = 0; s < NS - 1; ++s) {
        if (s < bpr) issue_x(s);
        cp_async_commit();
    }

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) { acc[nt][0] = 0.f; acc[nt][1] = 0.f; acc[nt][2] = 0.f; acc[nt][3] = 0.f; }

    // ldmatrix source of this lane: matrix (lane/8): rows +8 for odd matrices, bytes +16 for matrices 2, 3
    const int lm_row = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), lm_byte = 16 * (lane >> 4);

    for (int kb = 0; kb < bpr; ++kb) {
        cp_async_wait<NS - 2>();
        __syncthreads();
        if (kb + NS - 1 < bpr) { issue_w(kb + NS - 1); issue_x(kb + NS - 1); }
        cp_async_commit();

        const uint8_t* ws = smem + (size_t) (kb % NS) * S_BYTES;
        const uint8_t* xs = ws + W_BYTES;
        const float* xd = (const float*) (xs + X_BYTES);

        // headers of rows g and g+8 of this warp's tile
        float dw[2], dminw[2];
        uint32_t sc_lo[2], sc_hi[2], mn_lo[2], mn_hi[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint4 hd = skd::lds128(ws + (warp * 16 + g + 8 * r) * GW_STRIDE + 128);
            dw[r] = __half2float(__ushort_as_half((unsigned short) (hd.x & 0xffff)));
            dminw[r] = __half2float(__ushort_as_half((unsigned short) (hd.x >> 16)));
            skd::k4_unpack(hd.y, hd.z, hd.w, sc_lo[r], sc_hi[r], mn_lo[r], mn_hi[r]);
        }
        int isum[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) { isum[nt][0] = 0; isum[nt][1] = 0; isum[nt][2] = 0; isum[nt][3] = 0; }

#pragma unroll
        for (int gq = 0; gq < 4; ++gq) {
            uint32_t raw[4], lo[4], hi[4];
            ldmatrix_x4(raw, ws + lm_row * GW_STRIDE + 32 * gq + lm_byte);
#pragma unroll
            for (int i = 0; i < 4; ++i) { lo[i] = raw[i] & 0x0f0f0f0fu; hi[i] = (raw[i] >> 4) & 0x0f0f0f0fu; }
            // scales of sub-blocks 2gq (low nibbles) and 2gq+1 (high nibbles) for rows g, g+8
            int s_lo[2], s_hi[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const uint32_t word = gq < 2 ? sc_lo[r] : sc_hi[r];
                s_lo[r] = (int) ((word >> (16 * (gq & 1))) & 0xff);
                s_hi[r] = (int) ((word >> (16 * (gq & 1) + 8)) & 0xff);
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint8_t* xr = xs + (nt * 8 + g) * GX_STRIDE + 64 * gq + 4 * t;
                int c[4] = {0, 0, 0, 0};
                mma_u8s8(c, lo, *(const uint32_t*) xr, *(const uint32_t*) (xr + 16));
                isum[nt][0] += s_lo[0] * c[0]; isum[nt][1] += s_lo[0] * c[1];
                isum[nt][2] += s_lo[1] * c[2]; isum[nt][3] += s_lo[1] * c[3];
                int e[4] = {0, 0, 0, 0};
                mma_u8s8(e, hi, *(const uint32_t*) (xr + 32), *(const uint32_t*) (xr + 48));
                isum[nt][0] += s_hi[0] * e[0]; isum[nt][1] += s_hi[0] * e[1];
                isum[nt][2] += s_hi[1] * e[2]; isum[nt][3] += s_hi[1] * e[3];
            }
        }
        // mins and the fp32 update; accumulator j: row g + 8*(j/2), activation row 2t + (j&1)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                const int col = nt * 8 + 2 * t + cc;
                const uint4 bs = skd::lds128(xs + col * GX_STRIDE + 256);     // eight int16 sums
                const float dx = xd[col];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    int ms = __dp2a_lo((int) bs.x, (int) mn_lo[r], 0);
                    ms = __dp2a_hi((int) bs.y, (int) mn_lo[r], ms);
                    ms = __dp2a_lo((int) bs.z, (int) mn_hi[r], ms);
                    ms = __dp2a_hi((int) bs.w, (int) mn_hi[r], ms);
                    acc[nt][2 * r + cc] += dx * (dw[r] * (float) isum[nt][2 * r + cc] - dminw[r] * (float) ms);
                }
            }
        }
    }
    cp_async_wait<0>();

    // y[activation row][weight row]
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int row = row0 + warp * 16 + g + 8 * (j >> 1), col = col0 + nt * 8 + 2 * t + (j & 1);
            if (row < rows && col < m) {
                const size_t o = (size_t) col * rows + row;
                y[o] = EPI == EPI_ADD ? resid[o] + acc[nt][j] : acc[nt][j];
            }
        }
}

template <int NW, int NT, int NS>
int32_t launch_cfg(const Weight& w, ActQ8K a, int m, float* y, const float* resid, cudaStream_t s) {
    constexpr int RT = NW * 16, MT = NT * 8;
    constexpr size_t smem = (size_t) NS * (RT * GW_STRIDE + MT * GX_STRIDE + MT * 4);
    dim3 grid((w.rows + RT - 1) / RT, (m + MT - 1) / MT);
    if (resid) {
        SK_TRY(ensure_dynamic_smem((const void*) q4k_gemm_mma_kernel<NW, NT, NS, EPI_ADD>, (int) smem));
        SK_CUDA(launch_pdl(q4k_gemm_mma_kernel<NW, NT, NS, EPI_ADD>, grid, dim3(NW * 32), smem, s, (const uint8_t*) w.qs, (const uint8_t*) w.hdr, w.rows,
                           w.bpr, a, m, y, resid));
    } else {
        SK_TRY(ensure_dynamic_smem((const void*) q4k_gemm_mma_kernel<NW, NT, NS, EPI_STORE>, (int) smem));
        SK_CUDA(launch_pdl(q4k_gemm_mma_kernel<NW, NT, NS, EPI_STORE>, grid, dim3(NW * 32), smem, s, (const uint8_t*) w.qs, (const uint8_t*) w.hdr, w.rows,
                           w.bpr, a, m, y, resid));
    }
    return SKAINET_CUDA_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Q8_0 weights x two-term int8 activations (hi*128 + lo per 32 values, ActSplit): mma.sync m16n8k32 s8 x s8.
// One Q8_0 block (32 codes) is one MMA against `hi` and one against `lo`; the block contributes
// d_w * d_x * float(128*dot_hi + dot_lo), the same 15-bit arithmetic as the matvec (reference:
// native/src/q8_0_matmul.c:68-118 keeps fp32 activations; deviation of the split is ~4e-5 relative).
// Stage = 256 columns (8 blocks): weights [16*NW rows][272 B] = 256 codes + 8 f16 scales; activations
// hi [MT][272 B] and lo [MT][272 B], each 256 codes + four of the row's eight fp32 block scales in the pad.
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_s8s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int NW, int NT, int NS, int EPI>
__global__ void __launch_bounds__(NW * 32)
q8_0_gemm_mma_kernel(const int8_t* __restrict__ codes, const __half* __restrict__ scales, int rows, int cols, ActSplit act, int m,
                     float* __restrict__ y, const float* __restrict__ resid) {
    constexpr int RT = NW * 16, MT = NT * 8, ST = 272;
    constexpr int W_BYTES = RT * ST, X_BYTES = MT * ST, S_BYTES = W_BYTES + 2 * X_BYTES;
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * RT, col0 = blockIdx.y * MT;
    const int nst = cols >> 8, b32 = cols >> 5;
    skd::pdl_launch_dependents();

    // fixed copy slots per thread (see the Q4_K kernel): weights 17 chunks per row, activations 34 per row
    constexpr int WSLOTS = (RT * 17 + NW * 32 - 1) / (NW * 32), XSLOTS = (MT * 34 + NW * 32 - 1) / (NW * 32);
    const uint8_t* wsrc[WSLOTS]; int wdst[WSLOTS], wstep[WSLOTS];
    const uint8_t* xsrc[XSLOTS]; int xdst[XSLOTS], xstep[XSLOTS], xbytes[XSLOTS];
#pragma unroll
    for (int i = 0; i < WSLOTS; ++i) {
        const int c = threadIdx.x + i * NW * 32;
        const int r = c / 17, ch = c % 17;
        const size_t grow = (size_t) min(row0 + r, rows - 1);
        wdst[i] = c < RT * 17 ? r * ST + ch * 16 : -1;
        wsrc[i] = ch < 16 ? (const uint8_t*) (codes + grow * cols + ch * 16) : (const uint8_t*) (scales + grow * b32);
        wstep[i] = ch < 16 ? 256 : 16;
    }
#pragma unroll
    for (int i = 0; i < XSLOTS; ++i) {
        const int c = threadIdx.x + i * NW * 32;
        const int r = c / 34, ch = c % 34;
        const size_t arow = (size_t) min(col0 + r, m - 1);
        xbytes[i] = col0 + r < m ? 16 : 0;             // rows past the batch are zero-filled, not fetched
        // ch 0..15 hi codes, 16 = scales 0..3 (hi pad), 17..32 lo codes, 33 = scales 4..7 (lo pad)
        const bool lo_half = ch >= 17;
        const int cc = lo_half ? ch - 17 : ch;
        xdst[i] = c < MT * 34 ? (lo_half ? X_BYTES : 0) + r * ST + cc * 16 : -1;
        if (cc < 16) { xsrc[i] = (const uint8_t*) ((lo_half ? act.lo : act.hi) + arow * cols + cc * 16); xstep[i] = 256; }
        else { xsrc[i] = (const uint8_t*) (act.d + arow * b32 + (lo_half ? 4 : 0)); xstep[i] = 32; }
    }
    auto issue_w = [&](int kb) {
        uint8_t* st = smem + (size_t) (kb % NS) * S_BYTES;
#pragma unroll
        for (int i = 0; i < WSLOTS; ++i)
            if (wdst[i] >= 0) cp_async16(st + wdst[i], wsrc[i] + (size_t) kb * wstep[i]);
    };
    auto issue_x = [&](int kb) {
        uint8_t* st = smem + (size_t) (kb % NS) * S_BYTES + W_BYTES;
#pragma unroll
        for (int i = 0; i < XSLOTS; ++i)
            if (xdst[i] >= 0) cp_async16_zfill(st + xdst[i], xsrc[i] + (size_t) kb * xstep[i], xbytes[i]);
    };
    for (int s = 0; s < NS - 1 && s < nst; ++s) issue_w(s);
    skd::pdl_wait();
    for (int s = 0; s < NS - 1; ++s) {
        if (s < nst) issue_x(s);
        cp_async_commit();
    }

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) { acc[nt][0] = 0.f; acc[nt][1] = 0.f; acc[nt][2] = 0.f; acc[nt][3] = 0.f; }
    const int lm_row = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), lm_byte = 16 * (lane >> 4);

    for (int kb = 0; kb < nst; ++kb) {
        cp_async_wait<NS - 2>();
        __syncthreads();
        if (kb + NS - 1 < nst) { issue_w(kb + NS - 1); issue_x(kb + NS - 1); }
        cp_async_commit();
        const uint8_t* ws = smem + (size_t) (kb % NS) * S_BYTES;
        const uint8_t* xh = ws + W_BYTES;
        const uint8_t* xl = xh + X_BYTES;
#pragma unroll
        for (int blk = 0; blk < 8; ++blk) {
            uint32_t a[4];
            ldmatrix_x4(a, ws + lm_row * ST + 32 * blk + lm_byte);
            const float dw0 = __half2float(*reinterpret_cast<const __half*>(ws + (warp * 16 + g) * ST + 256 + 2 * blk));
            const float dw1 = __half2float(*reinterpret_cast<const __half*>(ws + (warp * 16 + g + 8) * ST + 256 + 2 * blk));
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint8_t* rh = xh + (nt * 8 + g) * ST + 32 * blk + 4 * t;
                const uint8_t* rl = xl + (nt * 8 + g) * ST + 32 * blk + 4 * t;
                int ch[4] = {0, 0, 0, 0}, cl[4] = {0, 0, 0, 0};
                mma_s8s8(ch, a, *(const uint32_t*) rh, *(const uint32_t*) (rh + 16));
                mma_s8s8(cl, a, *(const uint32_t*) rl, *(const uint32_t*) (rl + 16));
                // block scale of activation rows 2t, 2t+1: four in the hi pad, four in the lo pad
                const uint8_t* pad = (blk < 4 ? xh : xl) + 256 + 4 * (blk & 3);
                const float dx0 = *reinterpret_cast<const float*>(pad + (nt * 8 + 2 * t) * ST);
                const float dx1 = *reinterpret_cast<const float*>(pad + (nt * 8 + 2 * t + 1) * ST);
                acc[nt][0] += (dw0 * dx0) * (float) (ch[0] * 128 + cl[0]);
                acc[nt][1] += (dw0 * dx1) * (float) (ch[1] * 128 + cl[1]);
                acc[nt][2] += (dw1 * dx0) * (float) (ch[2] * 128 + cl[2]);
                acc[nt][3] += (dw1 * dx1) * (float) (ch[3] * 128 + cl[3]);
            }
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int row = row0 + warp * 16 + g + 8 * (j >> 1), col = col0 + nt * 8 + 2 * t + (j & 1);
            if (row < rows && col < m) {
                const size_t o = (size_t) col * rows + row;
                y[o] = EPI == EPI_ADD ? resid[o] + acc[nt][j] : acc[nt][j];
            }
        }
}

template <int NW, int NT, int NS>
int32_t launch_cfg_q8(const Weight& w, ActSplit a, int m, float* y, const float* resid, cudaStream_t s) {
    constexpr int RT = NW * 16, MT = NT * 8;
    constexpr size_t smem = (size_t) NS * (RT * 272 + 2 * MT * 272);
    dim3 grid((w.rows + RT - 1) / RT, (m + MT - 1) / MT);
    if (resid) {
        SK_TRY(ensure_dynamic_smem((const void*) q8_0_gemm_mma_kernel<NW, NT, NS, EPI_ADD>, (int) smem));
        SK_CUDA(launch_pdl(q8_0_gemm_mma_kernel<NW, NT, NS, EPI_ADD>, grid, dim3(NW * 32), smem, s, (const int8_t*) w.qs, (const __half*) w.hdr, w.rows, w.cols,
                           a, m, y, resid));
    } else {
        SK_TRY(ensure_dynamic_smem((const void*) q8_0_gemm_mma_kernel<NW, NT, NS, EPI_STORE>, (int) smem));
        SK_CUDA(launch_pdl(q8_0_gemm_mma_kernel<NW, NT, NS, EPI_STORE>, grid, dim3(NW * 32), smem, s, (const int8_t*) w.qs, (const __half*) w.hdr, w.rows, w.cols,
                           a, m, y, resid));
    }
    return SKAINET_CUDA_OK;
}

}  // namespace

// y[m][w.rows] (= resid +) act . W^T for m >= 2 activation rows already quantized (ActQ8K). Returns 1 when
// the weight is not Q4_K (the caller falls back to the per-row kernels).
int32_t launch_gemm_mma(const Weight& w, ActQ8K a, int m, float* y, const float* resid, cudaStream_t s) {
    if (w.enc != SKAINET_ENC_Q4_K) return 1;
    if (m >= TC_MIN_ROWS) {
        const int32_t st = launch_gemm_tc(w, a, m, y, resid, s);
        if (st != 1) return st;
    }
    // One or two activation rows stay with the streaming matvec kernels (faster there; from three rows the tile
    // kernel wins: 13.6 vs 15.7 us on 11008x4096). Few rows: weight streaming decides, so 64-row tiles and a deep
    // pipeline; many rows: 128 x 32 output tiles.
    // A small batch over a weight with few columns or few rows: the persistent ring with the same tile arithmetic
    // (gemm_ring.cu). Measured at 8 rows: 4096 x 4096 5.5 against 8.6 us, 22016 x 4096 18.2 against 22.6, 4096 x 11008 18.2
    // against 20.7, 8192 x 8192 19.8 against 19.4 (at 4 rows 15.4 against 21.4; inside the 70B decode step at batch 8 / 4:
    // 16.43 against 16.55 / 18.57 against 19.10 ms); on 8192-column weights of more than 8192 rows this kernel's cp.async
    // pipeline is the faster one (57344 x 8192: 66 against 100 us, 10240 x 8192: 21 against 27). 8192 x 28672 is faster through
    // the ring when timed alone (54.6 against 70.3 us) but slower inside the decode step (17.9 against 16.6 ms at batch 8:
    // the ring's CTAs fill the SMs' shared memory, so the kernel that follows cannot start beside their tail), and stays here.
    if (m >= 3 && m <= 8 && (w.cols <= 4096 || w.rows <= 4096 || (w.rows <= 8192 && w.cols <= 8192))) {
        const int32_t st = launch_rows_ring(w, a, m, y, resid, s);
        if (st != 1) return st;
    }
    // Two rows: two passes of the streaming matvec, except over weights of 64 MB and more, where one pass of the tile kernel
    // is faster (57344 x 8192: 64 against 69 us, 8192 x 28672: 66 against 81; 10240 x 8192: 22 against 18 the other way).
    if (m <= 1 || (m == 2 && w.packed_bytes < ((int64_t) 64 << 20))) return 1;
    // (row tiles of 32 or 16 for weights with few rows were measured slower: more activation re-fetch per weight byte)
    // Up to eight rows: a grid of at least one 64-row tile per SM keeps enough bytes in flight with three stages and six
    // CTAs per SM (57344 x 8192: 65.7 against 77.4 us with eight stages and two CTAs per SM; 10240 x 8192: 21.0 against
    // 22.2); fewer tiles than SMs need the deep pipeline (8192 x 28672: 70 against 117 us, 8192 x 8192: 19.4 against 20.5).
    if (m <= 8) return (w.rows + 63) / 64 >= sm_count() ? launch_cfg<4, 1, 3>(w, a, m, y, resid, s) : launch_cfg<4, 1, 8>(w, a, m, y, resid, s);
    if (m <= 16) return launch_cfg<4, 2, 6>(w, a, m, y, resid, s);
    // 64-row tiles until 128-row tiles give about two CTAs per SM (measured on both decoder shapes at batch 32: +3 % / +20 %)
    if ((int64_t) ((w.rows + 127) / 128) * ((m + 31) / 32) < 2 * sm_count()) return launch_cfg<4, 4, 4>(w, a, m, y, resid, s);
    return launch_cfg<8, 4, 4>(w, a, m, y, resid, s);
}

// The same for Q8_0 weights and the two-term activation split; needs whole 256-column stages. 1 = not taken.
int32_t launch_gemm_mma_q8(const Weight& w, ActSplit a, int m, float* y, const float* resid, cudaStream_t s) {
    if (w.enc != SKAINET_ENC_Q8_0 || w.cols % 256 != 0 || m < 2) return 1;     // from two rows up: the per-pass Q8_0 matvec is slower
    if (m <= 8) return launch_cfg_q8<4, 1, 4>(w, a, m, y, resid, s);
    if (m <= 16) return launch_cfg_q8<4, 2, 4>(w, a, m, y, resid, s);
    if ((int64_t) ((w.rows + 127) / 128) * ((m + 31) / 32) < 2 * sm_count()) return launch_cfg_q8<4, 4, 3>(w, a, m, y, resid, s);
    return launch_cfg_q8<8, 4, 3>(w, a, m, y, resid, s);
}

}  // namespace sk
