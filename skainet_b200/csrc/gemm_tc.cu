// Batched rows on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM) for Q4_K weights
// and many activation rows (the dispatcher sends 288 and more here): the prefill GEMM.
//
// The reference's arithmetic for one 256-element super-block (native/src/q4k_matmul.c:143-251) is
//     y += d_x * ( d_w * S1 - dmin_w * S2 ),   S1 = sum_sb sc[sb] * <codes_sb, xq_sb>,   S2 = sum_sb mn[sb] * sum(xq_sb)
// with 4-bit codes, 6-bit sc / mn and int8 activation codes xq. Both sums are products of small integers,
// so they are exact in f16 x f16 -> f32: the A operand carries code*sc (<= 945 < 2048, exact in f16), the
// B operand the activation codes, and one super-block is 16 MMAs of K = 16 accumulated in TMEM. S2 is one
// more K = 16 MMA of (mn[sb] twice) x (sums of 16 codes, <= 2032). The CUDA cores only unpack nibbles into
// the A operand (one LOP3 + one HFMA2 per two elements, using the 0x6400|n trick: f16(1024+n)*s - 1024*s
// is n*s exactly under the fused rounding) and apply the three fp32 block scales once per super-block.
//
// CTA = 128 weight rows (TMEM lanes) x 128 activation rows (TMEM columns), 18 warps:
//   warps 0-15 four threads per weight row: per 64-element group each writes a quarter of that row's 64 f16 of
//              the A stage (weights fetched one super-block ahead); after producing super-block kb they fold
//              super-block kb-1 out of TMEM (tcgen05.ld) into 32 fp32 accumulators per thread (each of the four
//              takes a quarter of the columns);
//   warp 17    one lane posts the bulk copies of the B stages and of the S2 / scale pieces as soon as their slots
//              free up, independently of the other warps;
//   warp 16    one lane issues the MMAs and commits: stage barriers back to the producers, accumulator
//              barriers to the epilogue; two TMEM accumulator sets so MMAs of kb+1 overlap the fold of kb.
// The stage operands use the K-major 128-byte-swizzle canonical layout (a 64-element group is exactly one
// 128-byte row; 16-byte chunks XOR the row index), the small S2 operands the no-swizzle one (8 rows x 16 B
// core matrices). A stage holds two such groups (128 k). The activation side is prepared once per call by
// act_f16_tiles_kernel in exactly that order, so a B stage is one contiguous 32 KB bulk copy.
// Every mbarrier wait is bounded; a wait that runs out raises the device flag, and the CTA still reaches
// the common exit where TMEM is freed.
// Measured and not kept: every CTA walking its super-blocks in a rotated order (so that CTAs sharing an activation tile do
// not ask L2 for the same stage at the same moment): 138.6 against 134.0 us per call at 512 rows.
#include "common.cuh"
#include "actquant.cuh"
#include "tma.cuh"
#include "matvec_fused.cuh"

#include <cuda_fp16.h>
#include <mutex>

namespace sk {

namespace {

constexpr int TC_M = 128, TC_N = 128, TC_KS = 128, TC_STAGES = 3;     // a stage holds two 64-element groups
constexpr int TC_A_BYTES = TC_M * TC_KS * 2, TC_B_BYTES = TC_N * TC_KS * 2, TC_STAGE_BYTES = TC_A_BYTES + TC_B_BYTES;
constexpr int TC_S2A_BYTES = TC_M * 16 * 2, TC_S2B_BYTES = TC_N * 16 * 2, TC_S2_BYTES = TC_S2A_BYTES + TC_S2B_BYTES;
constexpr int TC_OFF_S2 = TC_STAGES * TC_STAGE_BYTES;
constexpr int TC_OFF_DX = TC_OFF_S2 + 2 * TC_S2_BYTES;
constexpr int TC_DX_SLOTS = 2;                   // block-scale slots: one per accumulator set
constexpr int TC_OFF_BAR = TC_OFF_DX + TC_DX_SLOTS * TC_N * 4;
constexpr int TC_NBARS = 2 * TC_STAGES + 6;      // full, empty per stage; s2_full, acc_full, acc_empty per accumulator set
constexpr int TC_SMEM = TC_OFF_BAR + TC_NBARS * 8 + 16;
constexpr uint32_t TC_IDESC = (1u << 4) | ((uint32_t) (TC_N >> 3) << 17) | ((uint32_t) (TC_M >> 4) << 24);   // f16 x f16 -> f32, K-major both

// K-major operand in the 128-byte swizzle: rows of 128 B (64 f16), groups of 8 rows 1024 B apart; a K = 16 step
// moves the start address by 32 B inside the swizzle atom.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
    return (uint64_t) ((saddr & 0x3ffffu) >> 4) | (1ull << 16) | ((uint64_t) (1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// K-major operand without swizzle: 8 rows x 16 B core matrices, lbo = next 8 k-elements, sbo = next 8 rows.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t) ((saddr & 0x3ffffu) >> 4) | ((uint64_t) (lbo_bytes >> 4) << 16) | ((uint64_t) (sbo_bytes >> 4) << 32) | (1ull << 46);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(skd::smem_u32(bar)) : "memory");
}
// 8-byte weight load as volatile asm: the compiler keeps it where it is written (ahead of the barrier waits of the
// current super-block), so the next super-block's bytes really are in flight one iteration early.
__device__ __forceinline__ uint2 ld_nc_v2(const void* p) {
    uint2 r;
    asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));    // L1-allocating: the four threads of a row share sectors
    return r;
}
__device__ __forceinline__ uint4 ld_nc_v4(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive1(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(skd::smem_u32(bar)) : "memory");
}
// Two 16-column TMEM loads and the wait for them in ONE asm statement: the destination registers are only defined
// for the compiler once the wait has been issued, so no use of them can be scheduled ahead of it.
__device__ __forceinline__ void tmem_ld16x2(uint32_t ta, uint32_t tb, float (&u)[16], float (&v)[16]) {
    uint32_t r[16], q[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%32];\n\t"
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%33];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(q[0]), "=r"(q[1]), "=r"(q[2]), "=r"(q[3]), "=r"(q[4]), "=r"(q[5]), "=r"(q[6]), "=r"(q[7]), "=r"(q[8]), "=r"(q[9]),
          "=r"(q[10]), "=r"(q[11]), "=r"(q[12]), "=r"(q[13]), "=r"(q[14]), "=r"(q[15])
        : "r"(ta), "r"(tb)
        : "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) { u[i] = __uint_as_float(r[i]); v[i] = __uint_as_float(q[i]); }
}

// Bounded wait for the many producer / epilogue warps: between polls the warp sleeps, so sixteen waiting warps do
// not take the shared-memory pipe away from the tensor core's operand reads.
__device__ __forceinline__ bool wait_backoff(uint64_t* bar, uint32_t parity, int* timeout_flag) {
    for (int i = 0; i < (1 << 21); ++i) {
        if (skd::mbar_try_wait(bar, parity)) return true;
        __nanosleep(64);
    }
    if (timeout_flag) *timeout_flag = 1;
    return false;
}

// ---- activation side: int8 codes -> f16 in core-matrix order, sums of 16 codes, transposed block scales ----
//   xh  [m_pad/128][cols/64][16][8 rows][8][8]  f16: one 16 KB B stage (128 rows x 64 k) is contiguous, rows of 128 B
//                                               whose 16-byte chunks are XOR-swizzled with the row (128B swizzle);
//                                               inside every group of four k the order is (0,2,1,3), matching the
//                                               order in which the weight nibbles leave a 32-bit word
//   hs  [m_pad/128][bpr][16][2][8 rows][8]      f16 sums of 16 consecutive codes: 4 KB per (tile, super-block)
//   dxt [bpr][m_pad]                            fp32 block scales
__global__ void __launch_bounds__(256)
act_f16_tiles_kernel(ActQ8K act, int m, int m_pad, int cols, __half* __restrict__ xh, __half* __restrict__ hs, float* __restrict__ dxt) {
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    const int per_row = cols >> 4;
    const int64_t idx = (int64_t) blockIdx.x * 256 + threadIdx.x;
    if (idx >= (int64_t) m_pad * per_row) return;
    const int n = (int) (idx / per_row), seg = (int) (idx % per_row);        // 16 codes: elements 16*seg ..
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (n < m) raw = *reinterpret_cast<const uint4*>(act.q + (size_t) n * cols + (size_t) seg * 16);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    int sum = 0;
    __half out[16];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int b0 = (int8_t) (w[j] & 0xff), b1 = (int8_t) ((w[j] >> 8) & 0xff), b2 = (int8_t) ((w[j] >> 16) & 0xff), b3 = (int8_t) (w[j] >> 24);
        sum += b0 + b1 + b2 + b3;
        out[4 * j] = __int2half_rn(b0); out[4 * j + 1] = __int2half_rn(b2); out[4 * j + 2] = __int2half_rn(b1); out[4 * j + 3] = __int2half_rn(b3);
    }
    const int tile = n >> 7, ng = (n & 127) >> 3, r = n & 7;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const int kcg = seg * 2 + c, it = kcg >> 3, kc = kcg & 7;            // 8-element chunk: stage it, chunk kc of the stage
        *reinterpret_cast<uint4*>(xh + (((((size_t) tile * (cols >> 6) + it) * 16 + ng) * 8 + r) * 8 + (kc ^ r)) * 8) = *reinterpret_cast<const uint4*>(out + 8 * c);
    }
    const int kb = seg >> 4, j = seg & 15;
    hs[(((((size_t) tile * (cols >> 8) + kb) * 16 + ng) * 2 + (j >> 3)) * 8 + r) * 8 + (j & 7)] = __int2half_rn(sum);
    if (j == 0) dxt[(size_t) kb * m_pad + n] = n < m ? act.d[(size_t) n * (cols >> 8) + kb] : 0.0f;
}

constexpr int TC_PROD_WARPS = 8;     // two threads per weight row convert the A stages
constexpr int TC_EPI_WARPS = 16;     // four threads per weight row (= TMEM lane) fold a quarter of the columns each
constexpr int TC_WORKERS = (TC_PROD_WARPS + TC_EPI_WARPS) * 32;

__global__ void __launch_bounds__(TC_WORKERS + 64, 1)
q4k_gemm_tc_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ hdr, int rows, int bpr, const __half* __restrict__ xh,
                   const __half* __restrict__ hs, const float* __restrict__ dxt, int m, int m_pad, float* __restrict__ y,
                   const float* __restrict__ resid, int* __restrict__ timeout_flag) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* full = (uint64_t*) (smem + TC_OFF_BAR);        // stage ready: one arrival per producer warp + the bulk copy's bytes
    uint64_t* empty = full + TC_STAGES;
    uint64_t* s2_full = empty + TC_STAGES;
    uint64_t* acc_full = s2_full + 2;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = (uint32_t*) (acc_empty + 2);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile_m = blockIdx.x, tile_n = blockIdx.y;
    const int row0 = tile_m * TC_M, col0 = tile_n * TC_N;
    constexpr int MMA_WARP = TC_WORKERS / 32, TMA_WARP = MMA_WARP + 1;
    const int nst = bpr * 2;                           // stages of 128 k: two per super-block
    skd::pdl_launch_dependents();

    if (warp == MMA_WARP) {
        if (lane == 0) {
            for (int s = 0; s < TC_STAGES; ++s) { skd::mbar_init(full + s, TC_PROD_WARPS + 1); skd::mbar_init(empty + s, 1); }
            for (int b = 0; b < 2; ++b) {
                skd::mbar_init(s2_full + b, TC_PROD_WARPS + 1); skd::mbar_init(acc_full + b, 1); skd::mbar_init(acc_empty + b, TC_EPI_WARPS);
            }
            skd::mbar_fence_init();
        }
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(skd::smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;                  // set S at columns 256*S: S1 in 0..127, S2 in 128..255

    if (warp == MMA_WARP) {
        // ------------------------------------------------ MMA issuer ------------------------------------------------
        if (lane == 0) {
            bool ok = true;
            const uint64_t d_a = smem_desc_sw128(skd::smem_u32(smem)), d_b = smem_desc_sw128(skd::smem_u32(smem + TC_A_BYTES));
            int s = 0, par = 0;
            for (int kb = 0; kb < bpr && ok; ++kb) {
                const int set = kb & 1;
                if (kb >= 2) ok = skd::mbar_wait_bounded(acc_empty + set, ((kb >> 1) - 1) & 1, timeout_flag);
                for (int j = 0; j < 2 && ok; ++j) {
                    ok = skd::mbar_wait_bounded(full + s, par, timeout_flag);
                    if (!ok) break;
                    tc_fence_after();
                    // descriptors move in 16-byte units: a stage is 64 KB, a 64-k half 16 KB, a K = 16 step 32 B
                    const uint64_t off = (uint64_t) ((s * TC_STAGE_BYTES) >> 4);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint64_t o = off + (uint64_t) (((i >> 2) * (TC_A_BYTES / 2) + (i & 3) * 32) >> 4);
                        umma_f16(tmem + set * 256, d_a + o, d_b + o, TC_IDESC, (j | i) != 0 ? 1u : 0u);
                    }
                    umma_commit(empty + s);            // the stage may be overwritten once these MMAs have read it
                    if (++s == TC_STAGES) { s = 0; par ^= 1; }
                }
                if (!ok) break;
                ok = skd::mbar_wait_bounded(s2_full + set, (kb >> 1) & 1, timeout_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a2 = skd::smem_u32(smem + TC_OFF_S2 + set * TC_S2_BYTES), b2 = a2 + TC_S2A_BYTES;
                umma_f16(tmem + set * 256 + 128, smem_desc(a2, 128, 256), smem_desc(b2, 128, 256), TC_IDESC, 0u);
                umma_commit(acc_full + set);
            }
        }
        __syncwarp();
    } else if (warp == TMA_WARP) {
        // ------------------------- bulk copies of the activation side, running ahead of everyone -------------------------
        if (lane == 0) {
            skd::pdl_wait();                           // the activation tiles are the predecessor's output
            bool ok = true;
            int s = 0, round = 0;
            for (int kb = 0; kb < bpr && ok; ++kb) {
                const int set = kb & 1;
                for (int j = 0; j < 2 && ok; ++j) {
                    const int it = kb * 2 + j;
                    if (round > 0) ok = skd::mbar_wait_bounded(empty + s, (round - 1) & 1, timeout_flag);
                    if (!ok) break;
                    skd::mbar_expect_tx(full + s, TC_B_BYTES);          // one contiguous 32 KB piece of xh
                    skd::bulk_g2s(smem + s * TC_STAGE_BYTES + TC_A_BYTES, xh + ((size_t) tile_n * nst + it) * (TC_B_BYTES / 2), TC_B_BYTES, full + s);
                    if (++s == TC_STAGES) { s = 0; ++round; }
                }
                if (!ok) break;
                if (kb >= 2) ok = skd::mbar_wait_bounded(acc_empty + set, ((kb >> 1) - 1) & 1, timeout_flag);
                if (!ok) break;
                uint8_t* s2 = smem + TC_OFF_S2 + set * TC_S2_BYTES;
                fence_async_smem();                    // order the copies below after the generic-proxy reads just observed
                skd::mbar_expect_tx(s2_full + set, TC_S2B_BYTES + TC_N * 4);
                skd::bulk_g2s(s2 + TC_S2A_BYTES, hs + ((size_t) tile_n * bpr + kb) * (TC_S2B_BYTES / 2), TC_S2B_BYTES, s2_full + set);
                // the slot of super-block kb-2: every epilogue warp arrived on acc_empty after reading it
                skd::bulk_g2s(smem + TC_OFF_DX + (kb % TC_DX_SLOTS) * TC_N * 4, dxt + (size_t) kb * m_pad + col0, TC_N * 4, s2_full + set);
            }
        }
        __syncwarp();
    } else if (warp < TC_PROD_WARPS) {
        // ------------------------------------------- producers of the A operand -------------------------------------------
        // Never touch TMEM: they run ahead of the MMAs by the depth of the stage ring while the epilogue warps fold.
        const int r = tid & 127, half = tid >> 7;       // weight row of the tile; which 16 bytes of each 32-byte group
        const int grow = min(row0 + r, rows - 1);
        bool ok = true;
        // this thread's 16 bytes of each 32-byte group of the row's super-block, and the header; one block ahead
        uint4 q[4], qn[4];
        uint4 hd, hdn;
        {
            const size_t blk = (size_t) grow * bpr;
#pragma unroll
            for (int i = 0; i < 4; ++i) qn[i] = ld_nc_v4(qs + blk * 128 + i * 32 + half * 16);
            hdn = ld_nc_v4(hdr + blk * 16);
        }
        int s = 0, round = 0;
        for (int kb = 0; kb < bpr && ok; ++kb) {
            const int set = kb & 1;
#pragma unroll
            for (int i = 0; i < 4; ++i) q[i] = qn[i];
            hd = hdn;
            if (kb + 1 < bpr) {
                const size_t blk = (size_t) grow * bpr + kb + 1;
#pragma unroll
                for (int i = 0; i < 4; ++i) qn[i] = ld_nc_v4(qs + blk * 128 + i * 32 + half * 16);
                hdn = ld_nc_v4(hdr + blk * 16);
            }
            uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
            skd::k4_unpack(hd.y, hd.z, hd.w, sc_lo, sc_hi, mn_lo, mn_hi);

#pragma unroll
            for (int j = 0; j < 2; ++j) {              // stage = groups 2j, 2j+1 of the super-block
                if (round > 0 && !__all_sync(0xffffffffu, wait_backoff(empty + s, (round - 1) & 1, timeout_flag))) { ok = false; break; }
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int gq = 2 * j + h;
                    // 64-k half: k 0..31 = low nibbles x sc[2gq], k 32..63 = high nibbles x sc[2gq+1]; this thread's four
                    // words are bytes 16*half.. of the group: chunks 2*half, 2*half+1 of each nibble half. High nibbles
                    // stay in place (f16 1024 + 16 n) and take scale/16, so only the odd bytes need a shift.
                    const uint32_t scw = gq < 2 ? sc_lo : sc_hi;
                    const int i_lo = (int) ((scw >> (16 * (gq & 1))) & 0xff), i_hi = (int) ((scw >> (16 * (gq & 1) + 8)) & 0xff);
                    const __half2 ml = __half2half2(__int2half_rn(i_lo)), mh = __half2half2(__hmul(__int2half_rn(i_hi), __float2half_rn(0.0625f)));
                    const __half2 nl = __hmul2(ml, __float2half2_rn(-1024.0f)), nh = __hmul2(mh, __float2half2_rn(-1024.0f));
                    const uint32_t wv[4] = {q[gq].x, q[gq].y, q[gq].z, q[gq].w};
                    // 128-byte rows, chunk index XOR row (128B swizzle)
                    uint8_t* arow = smem + s * TC_STAGE_BYTES + h * (TC_A_BYTES / 2) + (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
                    for (int p2 = 0; p2 < 2; ++p2) {
                        const int part = 2 * half + p2;
                        uint32_t lo4[4], hi4[4];
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const uint32_t w = wv[2 * p2 + e], w8 = w >> 8;
                            const uint32_t x02 = (w & 0x000f000fu) | 0x64006400u, x13 = (w8 & 0x000f000fu) | 0x64006400u;
                            const uint32_t y02 = (w & 0x00f000f0u) | 0x64006400u, y13 = (w8 & 0x00f000f0u) | 0x64006400u;
                            __half2 v;
                            v = __hfma2(*reinterpret_cast<const __half2*>(&x02), ml, nl); lo4[2 * e] = *reinterpret_cast<uint32_t*>(&v);
                            v = __hfma2(*reinterpret_cast<const __half2*>(&x13), ml, nl); lo4[2 * e + 1] = *reinterpret_cast<uint32_t*>(&v);
                            v = __hfma2(*reinterpret_cast<const __half2*>(&y02), mh, nh); hi4[2 * e] = *reinterpret_cast<uint32_t*>(&v);
                            v = __hfma2(*reinterpret_cast<const __half2*>(&y13), mh, nh); hi4[2 * e + 1] = *reinterpret_cast<uint32_t*>(&v);
                        }
                        *reinterpret_cast<uint4*>(arow + ((part ^ (r & 7)) << 4)) = make_uint4(lo4[0], lo4[1], lo4[2], lo4[3]);
                        *reinterpret_cast<uint4*>(arow + (((4 + part) ^ (r & 7)) << 4)) = make_uint4(hi4[0], hi4[1], hi4[2], hi4[3]);
                    }
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive1(full + s);
                if (++s == TC_STAGES) { s = 0; ++round; }
            }
            if (!ok) break;
            // S2 operand of this super-block: mins (each twice) against the sums of 16 codes. Its buffer was last read by
            // the S2 MMA of super-block kb-2, whose completion acc_full[set] reported (observed here, not consumed).
            {
                if (kb >= 2 && !__all_sync(0xffffffffu, wait_backoff(acc_full + set, ((kb >> 1) - 1) & 1, timeout_flag))) { ok = false; break; }
                uint8_t* s2 = smem + TC_OFF_S2 + set * TC_S2_BYTES;
                const uint32_t mnw = half ? mn_hi : mn_lo;           // half 0 / 1 writes the chunks of sub-blocks 0..3 / 4..7
                uint32_t mm[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const __half2 vv = __half2half2(__int2half_rn((int) ((mnw >> (8 * i)) & 0xff)));
                    mm[i] = *reinterpret_cast<const uint32_t*>(&vv);
                }
                *reinterpret_cast<uint4*>(s2 + (r >> 3) * 256 + half * 128 + (r & 7) * 16) = make_uint4(mm[0], mm[1], mm[2], mm[3]);
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive1(s2_full + set);
            }
        }
        if (!ok) {                                      // give copies in flight time to land before the CTA leaves
            for (int i = 0; i < 64; ++i) __nanosleep(1000);
        }
    } else {
        // ------------------------------- epilogue: fold every super-block out of TMEM -------------------------------
        const int e = tid - TC_PROD_WARPS * 32;
        const int r = e & 127, part = e >> 7;           // TMEM lane = weight row (warp % 4 is its 32-lane quarter); which share of the columns
        const int grow = min(row0 + r, rows - 1);
        constexpr int NC = TC_N / (TC_EPI_WARPS / 4);
        float yacc[NC];
#pragma unroll
        for (int i = 0; i < NC; ++i) yacc[i] = 0.0f;
        bool ok = true;
        uint32_t ddn = *reinterpret_cast<const uint32_t*>(hdr + (size_t) grow * bpr * 16);      // (d, dmin) of the row's block, one ahead
        for (int kb = 0; kb < bpr && ok; ++kb) {
            const int set = kb & 1;
            const uint32_t dd = ddn;
            if (kb + 1 < bpr) ddn = *reinterpret_cast<const uint32_t*>(hdr + ((size_t) grow * bpr + kb + 1) * 16);
            const float dw = __half2float(__ushort_as_half((unsigned short) (dd & 0xffff)));
            const float dminw = __half2float(__ushort_as_half((unsigned short) (dd >> 16)));
            // the verdict of a wait is made warp-uniform: the lanes meet again at the __syncwarp before the arrive
            if (!__all_sync(0xffffffffu, wait_backoff(acc_full + set, (kb >> 1) & 1, timeout_flag))) { ok = false; break; }
            // the block scales below were written by a bulk copy: observe the barrier that tracked it (long complete)
            if (!__all_sync(0xffffffffu, wait_backoff(s2_full + set, (kb >> 1) & 1, timeout_flag))) { ok = false; break; }
            tc_fence_after();
            const float* dx = (const float*) (smem + TC_OFF_DX) + (kb % TC_DX_SLOTS) * TC_N + part * NC;
            const uint32_t t0 = tmem + ((uint32_t) ((warp & 3) * 32) << 16) + set * 256 + part * NC;
#pragma unroll
            for (int c = 0; c < NC; c += 16) {
                float s1[16], s2[16];
                tmem_ld16x2(t0 + c, t0 + 128 + c, s1, s2);
#pragma unroll
                for (int i = 0; i < 16; i += 4) {
                    const float4 x4 = *reinterpret_cast<const float4*>(dx + c + i);
                    yacc[c + i] = fmaf(x4.x, fmaf(-dminw, s2[i], dw * s1[i]), yacc[c + i]);
                    yacc[c + i + 1] = fmaf(x4.y, fmaf(-dminw, s2[i + 1], dw * s1[i + 1]), yacc[c + i + 1]);
                    yacc[c + i + 2] = fmaf(x4.z, fmaf(-dminw, s2[i + 2], dw * s1[i + 2]), yacc[c + i + 2]);
                    yacc[c + i + 3] = fmaf(x4.w, fmaf(-dminw, s2[i + 3], dw * s1[i + 3]), yacc[c + i + 3]);
                }
            }
            tc_fence_before();
            fence_async_smem();                        // the scales just read will be overwritten through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive1(acc_empty + set);
        }
        skd::pdl_wait();                               // y and resid may still be in use by kernels launched before this one
        if (ok && row0 + r < rows) {
#pragma unroll
            for (int c = 0; c < NC; ++c)
                if (col0 + part * NC + c < m) {
                    const size_t o = (size_t) (col0 + part * NC + c) * rows + row0 + r;
                    y[o] = resid ? resid[o] + yacc[c] : yacc[c];
                }
        }
        if (!ok) {
            for (int i = 0; i < 64; ++i) __nanosleep(1000);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

}  // namespace

// y[m][w.rows] (= resid +) for m >= TC_MIN_ROWS quantized activation rows. Returns 1 when not taken (the caller
// falls back to the mma.sync tile kernel): other encodings, few rows, or scratch that would have to grow
// while the stream is being captured.
int32_t launch_gemm_tc(const Weight& w, ActQ8K a, int m, float* y, const float* resid, cudaStream_t s) {
    if (w.enc != SKAINET_ENC_Q4_K || m < TC_MIN_ROWS || w.bpr < 1) return 1;
    const int m_pad = (m + TC_N - 1) / TC_N * TC_N;
    const size_t xh_bytes = (size_t) m_pad * w.cols * 2, hs_bytes = (size_t) m_pad * (w.cols / 16) * 2, dx_bytes = (size_t) w.bpr * m_pad * 4;
    const size_t need = xh_bytes + hs_bytes + dx_bytes + 3 * 256;
    // the operand tiles live in the calling stream's own scratch (calls on different streams do not share them)
    if (scratch_capacity(s, SCRATCH_GEMM) < need) {
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(s, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) { cudaGetLastError(); return 1; }
    }
    void* base = nullptr;
    SK_TRY(scratch_get(s, SCRATCH_GEMM, need, &base));
    auto up = [](size_t v) { return (v + 255) & ~(size_t) 255; };
    __half* xh = (__half*) base;
    __half* hs = (__half*) ((uint8_t*) base + up(xh_bytes));
    float* dxt = (float*) ((uint8_t*) base + up(xh_bytes) + up(hs_bytes));
    SK_TRY(ensure_dynamic_smem((const void*) q4k_gemm_tc_kernel, TC_SMEM));
    const int64_t n16 = (int64_t) m_pad * (w.cols / 16);
    SK_CUDA(launch_pdl(act_f16_tiles_kernel, dim3((unsigned) ((n16 + 255) / 256)), dim3(256), 0, s, a, m, m_pad, w.cols, xh, hs, dxt));
    dim3 grid((w.rows + TC_M - 1) / TC_M, m_pad / TC_N);
    SK_CUDA(launch_pdl(q4k_gemm_tc_kernel, grid, dim3(TC_WORKERS + 64), (size_t) TC_SMEM, s, (const uint8_t*) w.qs, (const uint8_t*) w.hdr, w.rows, w.bpr,
                       (const __half*) xh, (const __half*) hs, (const float*) dxt, m, m_pad, y, resid, device_timeout_flag()));
    return SKAINET_CUDA_OK;
}

}  // namespace sk
