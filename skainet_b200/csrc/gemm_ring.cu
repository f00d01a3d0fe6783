// Q4_K weights x three to eight int8-quantized activation rows (a small decode batch): the persistent ring of the
// single-row matvec (matvec_ring.cu: one CTA per SM, groups of one producer warp and consumer warps, cp.async.bulk stages,
// full / empty mbarriers counted in bytes, static row-group schedule) with the tile arithmetic of the mma.sync kernel
// (gemm_mma.cu: m16n8k32 u8 x s8 -> s32 per 32-element sub-block, integer sub-block scales, mins by dp2a on the
// activation's sub-block sums, fp32 combine) as its consumer. It is the faster of the two on weights with few columns or
// few rows, where the general tile kernel's per-super-block CTA barrier and cp.async pipeline do not reach steady state
// (the dispatcher in gemm_mma.cu holds the measured rule); both are bound by the integer scale application at about
// 2-3 TB/s of weights. Reference arithmetic: native/src/q4k_matmul.c:143-251 (rows of a batch are independent matvecs there).
//
// Stage = 16 weight rows (one MMA tile) x 8 super-blocks: row r's 1024 bytes of nibbles at r * 1040 (the 16-byte pad makes
// ldmatrix over eight rows hit 32 distinct banks), then the rows' 128 bytes of headers at stride 144. Consumer warp w takes
// super-block w of the stage for all 16 rows; the eight warps' partial tiles are added once per row group, in warp order.
// Two groups per CTA. The quantized activation rows (codes, sub-block sums, block scales) are staged once per CTA in the
// layout the B fragments read without bank conflicts; where eight rows do not fit beside three stages per group (rows of
// more than 8192 elements) every consumer warp fetches its super-block's slice of the activation from global memory (L2)
// into registers one stage ahead instead, and the rings take all of the shared memory. Four super-blocks per stage and
// four groups measured the same (184 against 193 us over twelve 25 MB weights).
#include "common.cuh"
#include "actquant.cuh"
#include "tma.cuh"
#include "matvec_fused.cuh"

#include <algorithm>

namespace sk {

namespace {

constexpr int GR_ROWS = 16, GR_BLKS = 8, GR_MT = 8;       // GR_BLKS = consumer warps per group = super-blocks per stage
constexpr int GR_GW = GR_BLKS + 1;                                 // warps per group
constexpr int GR_QS_STRIDE = GR_BLKS * 128 + 16, GR_HDR_STRIDE = GR_BLKS * 16 + 16;
constexpr int GR_HDR_OFF = GR_ROWS * GR_QS_STRIDE, GR_STAGE = GR_HDR_OFF + GR_ROWS * GR_HDR_STRIDE;
constexpr int GR_MAX_STAGES = 8;
constexpr size_t GR_BUDGET = 190 * 1024;

__device__ __forceinline__ void gr_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(skd::smem_u32(p)));
}
__device__ __forceinline__ void gr_mma_u8s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void gr_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(skd::smem_u32(bar)) : "memory");
}
// the consumer warps of group `grp` (barriers 2..5; 1 = the consumer warps of all groups)
__device__ __forceinline__ void gr_group_sync(int grp) {
    if (grp == 0) asm volatile("bar.sync 2, %0;" ::"n"(GR_BLKS * 32) : "memory");
    else if (grp == 1) asm volatile("bar.sync 3, %0;" ::"n"(GR_BLKS * 32) : "memory");
    else if (grp == 2) asm volatile("bar.sync 4, %0;" ::"n"(GR_BLKS * 32) : "memory");
    else asm volatile("bar.sync 5, %0;" ::"n"(GR_BLKS * 32) : "memory");
}

// x_stride: bytes between activation rows in shared memory (bpr * 272, + 16 when that is a multiple of 128 bytes' worth of banks)
template <int NG, int EPI, bool XG>
__global__ void __launch_bounds__(NG * GR_GW * 32)
q4k_rows_ring_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ hdr, int rows, int bpr, ActQ8K act, int m,
                     float* __restrict__ y, const float* __restrict__ resid, int nstages, int x_stride, int* __restrict__ timeout_flag) {
    extern __shared__ __align__(128) uint8_t smem[];
    // layout: rings [NG][nstages][GR_STAGE] | activation rows [8][x_stride] | block scales [8][bpr] | partial tiles [NG][2][4][128] | barriers
    const int lane = threadIdx.x & 31;
    const int grp = (int) (threadIdx.x >> 5) / GR_GW, warp = (int) (threadIdx.x >> 5) - grp * GR_GW;       // warp GR_BLKS = the group's producer
    uint8_t* s_ring = smem + (size_t) grp * nstages * GR_STAGE;
    // XG: the activation rows are too long to stage; every consumer warp fetches its super-block's slice from global
    // memory (L2) into registers one stage ahead instead
    uint8_t* s_x = smem + (size_t) NG * nstages * GR_STAGE;
    float* s_d = (float*) (s_x + (XG ? 0 : (size_t) GR_MT * x_stride));
    const int nd = XG ? 0 : ((GR_MT * bpr + 3) & ~3);
    float* s_part = s_d + nd + grp * 2 * GR_BLKS * 128;
    uint64_t* full = (uint64_t*) (s_d + nd + NG * 2 * GR_BLKS * 128) + grp * 2 * GR_MAX_STAGES;
    uint64_t* empty = full + GR_MAX_STAGES;

    const int vcta = (int) blockIdx.x * NG + grp, vgrid = (int) gridDim.x * NG;
    const int nrg = (rows + GR_ROWS - 1) / GR_ROWS, ncg = (bpr + GR_BLKS - 1) / GR_BLKS;
    const int my_rgs = vcta < nrg ? (nrg - 1 - vcta) / vgrid + 1 : 0;
    const int cols = bpr * 256;

    if (warp == GR_BLKS && lane == 0) {
        for (int s = 0; s < nstages; ++s) { skd::mbar_init(full + s, 1); skd::mbar_init(empty + s, GR_BLKS); }
        skd::mbar_fence_init();
    }
    __syncthreads();
    skd::pdl_launch_dependents();

    if (warp == GR_BLKS) {
        // ---------------- producer: the weights depend on no predecessor ----------------
        const int r = lane & 15;
        int stage = 0, round = 0;
        for (int rgi = 0; rgi < my_rgs; ++rgi) {
            const int row0 = (vcta + rgi * vgrid) * GR_ROWS;
            const size_t srow = (size_t) min(row0 + r, rows - 1);         // rows past the end repeat the last one (never written)
            for (int cg = 0; cg < ncg; ++cg) {
                if (round > 0 && !skd::mbar_wait_bounded(empty + stage, (round - 1) & 1, timeout_flag)) return;
                const int b0 = cg * GR_BLKS, nb = min(GR_BLKS, bpr - b0);
                uint8_t* dst = s_ring + (size_t) stage * GR_STAGE;
                if (lane == 0) skd::mbar_expect_tx(full + stage, (uint32_t) GR_ROWS * nb * 144);
                __syncwarp();
                if (lane < 16) skd::bulk_g2s(dst + r * GR_QS_STRIDE, qs + (srow * bpr + b0) * 128, (uint32_t) nb * 128, full + stage);
                else skd::bulk_g2s(dst + GR_HDR_OFF + r * GR_HDR_STRIDE, hdr + (srow * bpr + b0) * 16, (uint32_t) nb * 16, full + stage);
                if (++stage == nstages) { stage = 0; ++round; }
            }
        }
        skd::pdl_wait();
        return;
    }

    // ---------------- consumers ----------------
    skd::pdl_wait();                                   // the quantized activation rows are the predecessor's output
    if (!XG) {
        const int ct = (grp * GR_BLKS + warp) * 32 + lane, nct = NG * GR_BLKS * 32;          // this thread among the consumer threads of the CTA
        for (int c = ct; c < GR_MT * (cols >> 4); c += nct) {                 // 16 codes
            const int row = c / (cols >> 4), ch = c % (cols >> 4), blk = ch >> 4, k16 = ch & 15;
            const uint4 v = row < m ? skd::ld_ro(act.q + (size_t) row * cols + (size_t) ch * 16) : make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(s_x + (size_t) row * x_stride + blk * 272 + k16 * 16) = v;
        }
        for (int c = ct; c < GR_MT * bpr; c += nct) {                         // a block's eight int16 sums and its scale
            const int row = c / bpr, blk = c % bpr;
            const uint4 v = row < m ? skd::ld_ro(act.bsums + ((size_t) row * bpr + blk) * 8) : make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(s_x + (size_t) row * x_stride + blk * 272 + 256) = v;
            s_d[row * bpr + blk] = row < m ? __ldg(act.d + (size_t) row * bpr + blk) : 0.0f;
        }
    }
    if (!XG) asm volatile("bar.sync 1, %0;" ::"n"(NG * GR_BLKS * 32) : "memory");

    const int g = lane >> 2, t = lane & 3;
    const int lm_row = (lane & 7) + 8 * ((lane >> 3) & 1), lm_byte = 16 * (lane >> 4);
    int stage = 0, phase = 0, pbuf = 0;
    // XG: B fragments of activation row g (words 4 t .. of every 16 codes), sub-block sums and block scales of rows 2 t, 2 t + 1
    uint32_t xw[16], xw_n[16];
    uint4 xbs[2], xbs_n[2];
    float xd[2], xd_n[2];
    auto fetch_x = [&](int b, uint32_t (&w)[16], uint4 (&bs2)[2], float (&d2)[2]) {
        const int bb = min(b, bpr - 1);
        const bool live = g < m;
        const int8_t* src = act.q + (size_t) min(g, m - 1) * cols + (size_t) bb * 256 + 4 * t;
#pragma unroll
        for (int i = 0; i < 16; ++i) w[i] = live ? __ldg(reinterpret_cast<const uint32_t*>(src + 16 * i)) : 0u;
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
            const int col = 2 * t + cc;
            const bool cl = col < m;
            bs2[cc] = cl ? skd::ld_ro(act.bsums + ((size_t) col * bpr + bb) * 8) : make_uint4(0, 0, 0, 0);
            d2[cc] = cl ? __ldg(act.d + (size_t) col * bpr + bb) : 0.0f;
        }
    };
    if (XG && my_rgs > 0) fetch_x(warp, xw_n, xbs_n, xd_n);
    for (int rgi = 0; rgi < my_rgs; ++rgi) {
        const int row0 = (vcta + rgi * vgrid) * GR_ROWS;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int cg = 0; cg < ncg; ++cg) {
            const int b = cg * GR_BLKS + warp;
            const bool live = b < bpr;
            if (XG) {
#pragma unroll
                for (int i = 0; i < 16; ++i) xw[i] = xw_n[i];
                xbs[0] = xbs_n[0]; xbs[1] = xbs_n[1]; xd[0] = xd_n[0]; xd[1] = xd_n[1];
                fetch_x((cg + 1 < ncg ? cg + 1 : 0) * GR_BLKS + warp, xw_n, xbs_n, xd_n);     // the slice the next stage needs (the same for every row group)
            }
            if (!skd::mbar_wait_bounded(full + stage, phase, timeout_flag)) return;
            if (live) {
                const uint8_t* st = s_ring + (size_t) stage * GR_STAGE;
                float dw[2], dminw[2];
                uint32_t sc_lo[2], sc_hi[2], mn_lo[2], mn_hi[2];
#pragma unroll
                for (int r = 0; r < 2; ++r) {                       // headers of rows g and g + 8
                    const uint4 hd = skd::lds128(st + GR_HDR_OFF + (g + 8 * r) * GR_HDR_STRIDE + warp * 16);
                    dw[r] = __half2float(__ushort_as_half((unsigned short) (hd.x & 0xffff)));
                    dminw[r] = __half2float(__ushort_as_half((unsigned short) (hd.x >> 16)));
                    skd::k4_unpack(hd.y, hd.z, hd.w, sc_lo[r], sc_hi[r], mn_lo[r], mn_hi[r]);
                }
                int isum[4] = {0, 0, 0, 0};
                const uint8_t* xb = s_x + (size_t) g * x_stride + b * 272 + 4 * t;
#pragma unroll
                for (int gq = 0; gq < 4; ++gq) {
                    uint32_t raw[4], lo[4], hi[4];
                    gr_ldmatrix_x4(raw, st + lm_row * GR_QS_STRIDE + warp * 128 + 32 * gq + lm_byte);
#pragma unroll
                    for (int i = 0; i < 4; ++i) { lo[i] = raw[i] & 0x0f0f0f0fu; hi[i] = (raw[i] >> 4) & 0x0f0f0f0fu; }
                    int s_lo[2], s_hi[2];
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        const uint32_t word = gq < 2 ? sc_lo[r] : sc_hi[r];
                        s_lo[r] = (int) ((word >> (16 * (gq & 1))) & 0xff);
                        s_hi[r] = (int) ((word >> (16 * (gq & 1) + 8)) & 0xff);
                    }
                    const uint8_t* xr = xb + 64 * gq;
                    const uint32_t b0 = XG ? xw[4 * gq] : *(const uint32_t*) xr, b1 = XG ? xw[4 * gq + 1] : *(const uint32_t*) (xr + 16);
                    const uint32_t b2 = XG ? xw[4 * gq + 2] : *(const uint32_t*) (xr + 32), b3 = XG ? xw[4 * gq + 3] : *(const uint32_t*) (xr + 48);
                    int c[4] = {0, 0, 0, 0};
                    gr_mma_u8s8(c, lo, b0, b1);
                    isum[0] += s_lo[0] * c[0]; isum[1] += s_lo[0] * c[1]; isum[2] += s_lo[1] * c[2]; isum[3] += s_lo[1] * c[3];
                    int e[4] = {0, 0, 0, 0};
                    gr_mma_u8s8(e, hi, b2, b3);
                    isum[0] += s_hi[0] * e[0]; isum[1] += s_hi[0] * e[1]; isum[2] += s_hi[1] * e[2]; isum[3] += s_hi[1] * e[3];
                }
                // mins and the fp32 update; accumulator j: weight row g + 8 (j / 2), activation row 2 t + (j & 1)
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    const int col = 2 * t + cc;
                    const uint4 bs = XG ? xbs[cc] : skd::lds128(s_x + (size_t) col * x_stride + b * 272 + 256);
                    const float dx = XG ? xd[cc] : s_d[col * bpr + b];
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        int ms = __dp2a_lo((int) bs.x, (int) mn_lo[r], 0);
                        ms = __dp2a_hi((int) bs.y, (int) mn_lo[r], ms);
                        ms = __dp2a_lo((int) bs.z, (int) mn_hi[r], ms);
                        ms = __dp2a_hi((int) bs.w, (int) mn_hi[r], ms);
                        acc[2 * r + cc] += dx * (dw[r] * (float) isum[2 * r + cc] - dminw[r] * (float) ms);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) gr_arrive(empty + stage);     // this warp is done reading the stage
            if (++stage == nstages) { stage = 0; phase ^= 1; }
        }
        // the eight warps' partial tiles -> one; two buffers, so one barrier per row group is enough
        float* part = s_part + pbuf * GR_BLKS * 128;
        *reinterpret_cast<float4*>(part + warp * 128 + lane * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        gr_group_sync(grp);
        if (warp == 0) {
            float4 v = *reinterpret_cast<const float4*>(part + lane * 4);
#pragma unroll
            for (int w = 1; w < GR_BLKS; ++w) {
                const float4 o = *reinterpret_cast<const float4*>(part + w * 128 + lane * 4);
                v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
            }
            const float out[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int row = row0 + g + 8 * (j >> 1), col = 2 * t + (j & 1);
                if (row < rows && col < m) {
                    const size_t o = (size_t) col * rows + row;
                    y[o] = EPI == EPI_ADD ? resid[o] + out[j] : out[j];
                }
            }
        }
        pbuf ^= 1;
    }
}

template <int NG, bool XG>
int32_t launch_rows_ring_ng(const Weight& w, ActQ8K a, int m, float* y, const float* resid, size_t fixed, int x_stride, cudaStream_t s) {
    if (GR_BUDGET <= fixed) return 1;
    const int ns = (int) std::min<size_t>(GR_MAX_STAGES, (GR_BUDGET - fixed - (size_t) NG * (2 * GR_BLKS * 128 * 4 + 2 * GR_MAX_STAGES * 8)) / ((size_t) NG * GR_STAGE));
    if (ns < 3) return 1;
    const size_t smem = (size_t) NG * ns * GR_STAGE + fixed + (size_t) NG * (2 * GR_BLKS * 128 * 4 + 2 * GR_MAX_STAGES * 8) + 128;
    const int nrg = (w.rows + GR_ROWS - 1) / GR_ROWS, grid = std::min(sm_count(), (nrg + NG - 1) / NG);
    int* flag = device_timeout_flag();
    if (resid) {
        auto kernel = q4k_rows_ring_kernel<NG, EPI_ADD, XG>;
        SK_TRY(ensure_dynamic_smem((const void*) kernel, 200 * 1024));
        SK_CUDA(launch_pdl(kernel, dim3(grid), dim3(NG * GR_GW * 32), smem, s, (const uint8_t*) w.qs, (const uint8_t*) w.hdr, w.rows, w.bpr, a, m, y, resid, ns, x_stride, flag));
    } else {
        auto kernel = q4k_rows_ring_kernel<NG, EPI_STORE, XG>;
        SK_TRY(ensure_dynamic_smem((const void*) kernel, 200 * 1024));
        SK_CUDA(launch_pdl(kernel, dim3(grid), dim3(NG * GR_GW * 32), smem, s, (const uint8_t*) w.qs, (const uint8_t*) w.hdr, w.rows, w.bpr, a, m, y, resid, ns, x_stride, flag));
    }
    return SKAINET_CUDA_OK;
}

}  // namespace

// y[m][w.rows] (= resid +) for 2 <= m <= 8 quantized activation rows over a Q4_K weight of 4 MB or more.
// Returns 1 when the shape is not taken (the caller then uses the general tile kernel).
int32_t launch_rows_ring(const Weight& w, ActQ8K a, int m, float* y, const float* resid, cudaStream_t s) {
    if (w.enc != SKAINET_ENC_Q4_K || m < 2 || m > GR_MT || w.bpr < 1 || w.packed_bytes < ((int64_t) 4 << 20)) return 1;
    // activation row stride: the B-fragment reads of eight rows must fall into distinct banks
    const int x_stride = w.bpr * 272 + ((w.bpr & 1) ? 0 : 16);
    const size_t fixed = (size_t) GR_MT * x_stride + (((size_t) GR_MT * w.bpr + 3) & ~(size_t) 3) * 4;
    constexpr int NG0 = 16 / GR_BLKS;                  // sixteen consumer warps per SM
    // staged activation rows where eight of them fit beside three stages per group (11008 x 4096 at 8 rows: 11.3 us staged,
    // 16.4 us fetched); longer rows are fetched from global memory by the consumers (4096 x 11008: 13.8 us against 18.2 us
    // for one group with staged rows; 7B decode at batch 8 / 4: 3117 / 1846 against 2931 / 1734 tokens/s)
    const int32_t st = launch_rows_ring_ng<NG0, false>(w, a, m, y, resid, fixed, x_stride, s);
    if (st != 1) return st;
    return launch_rows_ring_ng<NG0, true>(w, a, m, y, resid, 0, x_stride, s);
}

}  // namespace sk
