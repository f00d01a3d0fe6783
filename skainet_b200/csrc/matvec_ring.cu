// Persistent ring matvec for LARGE weights (m = 1): a ring of shared-memory stages is kept filled by a producer
// warp (cp.async.bulk / TMA, one "full" mbarrier per stage counted in bytes) while NC consumer warps — one output
// row of the stage each — drain it and hand stages back through "empty" mbarriers. The rings are the SM's bytes in
// flight (up to ~190 KB), so HBM stays busy for the whole launch. The one-tile kernel (matvec_fused.cu) remains
// the choice for small weights, where a CTA's prologue would not amortise.
//
// Stage = NC rows x one column group (16 Q4_K super-blocks / 2048 Q8_0 codes). Consumers read stages
// bank-conflict free with the same lane mapping and arithmetic as matvec_fused.cu. Every mbarrier wait
// is bounded and reports through the device flag. Reference arithmetic: native/src/q4k_matmul.c:143-251,
// native/src/q8_0_matmul.c:68-118.
//
// Shape of the Q4_K kernel, from measurement on B200 (57344 x 8192 and 8192 x 28672 weights, launches timed in a
// CUDA graph over distinct weights): four independent groups of 1 producer + 4 consumer warps per SM is the
// fastest arrangement (0.92 of the measured copy bandwidth on the first weight); 8, 12 or 16 consumer warps
// behind one producer reach 0.49-0.54, and rings private to each warp, refilled by the warp itself (no producer,
// no "empty" barriers), 0.65-0.79. As four CTAs per SM the groups each stage their own copy of the activation,
// which for a 28672-column row leaves three CTAs of three stages; as four groups of ONE CTA they share one copy
// (this kernel): 28.0 -> 25.3 us on that weight, and a fused norm + quantize prologue runs once per SM instead of
// four times, which is what makes it pay up to 8192 columns. Asking L2 for the head of the next weight from the
// producers' tails (prefetch.global.L2 or cp.async.bulk.prefetch.L2) made the decode step slower at every
// budget tried and is not done.
#include "common.cuh"
#include "actquant.cuh"
#include "tma.cuh"
#include "matvec_fused.cuh"
#include "actprep.cuh"

#include <cstdlib>

namespace sk {

constexpr int RG_MAX_STAGES = 8;
constexpr size_t RG_SMEM_MAX = 200 * 1024;
// shared memory per SM given to the rings of its resident CTAs
#ifndef SK_RING_BUDGET_KB
#define SK_RING_BUDGET_KB 190
#endif
static size_t ring_budget() { return (size_t) SK_RING_BUDGET_KB << 10; }

template <int NC>
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(NC * 32) : "memory"); }
// named barriers: 1 = the consumer warps of all groups (activation staging), 2..NG+1 = the NC consumer warps of one
// group (written as immediates: a register operand makes the compiler reserve all sixteen)
constexpr int RG_BAR_ALL = 1;
template <int NC, int NG>
__device__ __forceinline__ void group_sync(int grp) {
    if (NG == 1 || grp == 0) asm volatile("bar.sync 2, %0;" ::"n"(NC * 32) : "memory");
    else if (grp == 1) asm volatile("bar.sync 3, %0;" ::"n"(NC * 32) : "memory");
    else if (grp == 2) asm volatile("bar.sync 4, %0;" ::"n"(NC * 32) : "memory");
    else asm volatile("bar.sync 5, %0;" ::"n"(NC * 32) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(skd::smem_u32(bar)) : "memory");
}

// Work distribution: row group g belongs to CTA g mod grid. Handing groups out through a device counter instead
// (CTAs that finish early take more) was measured and dropped: the consumers are latency-bound, and learning
// the group's index from shared memory after each stage barrier cost them more (48.5 against 42.2 us on the
// 57344 x 8192 weight) than the evener finish gained.

// ================================================================================================
// Q4_K. Stage: qs part [NC][16][128] then hdr part [NC][16][16].
// ================================================================================================
template <int NC, int NG, int PREP, int EPI>
__global__ void __launch_bounds__(NG * (NC + 1) * 32)
q4k_matvec_ring_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ hdr, int rows, int bpr, MatvecIn in,
                       int cols, float* __restrict__ y, const float* __restrict__ resid, int nstages, int* __restrict__ timeout_flag, PeerOut peer) {
    constexpr int S_QS = NC * 16 * 128, S_HDR = NC * 16 * 16, S_BYTES = S_QS + S_HDR;
    extern __shared__ __align__(128) uint8_t smem[];
    // NG independent groups (one producer warp + NC consumer warps, own ring and barriers each) share one copy of
    // the activation: what NG CTAs per SM would do, without NG copies of a long row.
    // layout: rings [NG] | q8 (swizzled) | split sub-block sums | d | reduce scratch | barriers [NG] | peer gather [NG]
    const int lane = threadIdx.x & 31;
    const int grp = NG == 1 ? 0 : (int) (threadIdx.x >> 5) / (NC + 1);
    const int warp = (int) (threadIdx.x >> 5) - grp * (NC + 1);          // 0..NC-1 consumers, NC the producer
    uint8_t* s_ring = smem + (size_t) grp * nstages * S_BYTES;
    int8_t* s_q8 = (int8_t*) (smem + (size_t) NG * nstages * S_BYTES);
    uint8_t* s_bs = (uint8_t*) (s_q8 + cols);                      // 16 bytes per block
    float* s_d = (float*) (s_bs + cols / 16);
    float* s_red = (float*) ((uint8_t*) s_d + ((bpr * 4 + 15) & ~15));      // NG * NC floats (at most 16)
    uint64_t* full = (uint64_t*) (s_red + 16) + grp * 2 * RG_MAX_STAGES;
    uint64_t* empty = full + RG_MAX_STAGES;
    float* s_out = (float*) ((uint64_t*) (s_red + 16) + NG * 2 * RG_MAX_STAGES) + grp * 2 * NC;   // [2][NC]: a row group's results, gathered for the peer stores

    const int vcta = (int) blockIdx.x * NG + grp, vgrid = (int) gridDim.x * NG;   // row group g belongs to group g mod vgrid
    const int nrg = (rows + NC - 1) / NC;                     // row groups in the matrix
    const int ncg = (bpr + 15) >> 4;                          // column groups per row
    const int my_rgs = vcta < nrg ? (nrg - 1 - vcta) / vgrid + 1 : 0;

    if (warp == NC && lane == 0) {
        for (int s = 0; s < nstages; ++s) { skd::mbar_init(full + s, 1); skd::mbar_init(empty + s, NC); }
        skd::mbar_fence_init();
    }
    __syncthreads();
    skd::pdl_launch_dependents();

    if (warp == NC) {
        // ---------------- producer: the weights depend on no predecessor ----------------
        int stage = 0, round = 0;
        for (int rgi = 0; rgi < my_rgs; ++rgi) {
            const int row0 = (vcta + rgi * vgrid) * NC, nr = min(NC, rows - row0);
            for (int cg = 0; cg < ncg; ++cg) {
                if (round > 0 && !skd::mbar_wait_bounded(empty + stage, (round - 1) & 1, timeout_flag)) return;
                const int b0 = cg * 16, nb = min(16, bpr - b0);
                uint8_t* dst = s_ring + (size_t) stage * S_BYTES;
                if (lane == 0) skd::mbar_expect_tx(full + stage, (uint32_t) nr * nb * 144);
                __syncwarp();
                if (bpr == 16) {               // rows are contiguous: two copies move the whole stage
                    if (lane == 0) skd::bulk_g2s(dst, qs + (size_t) row0 * 16 * 128, (uint32_t) nr * 16 * 128, full + stage);
                    if (lane == 1) skd::bulk_g2s(dst + S_QS, hdr + (size_t) row0 * 16 * 16, (uint32_t) nr * 16 * 16, full + stage);
                } else if (lane < 2 * nr) {    // one row segment per lane: qs by lanes 0..nr-1, hdr by the next nr
                    const int r = lane < nr ? lane : lane - nr;
                    const size_t blk = (size_t) (row0 + r) * bpr + b0;
                    if (lane < nr) skd::bulk_g2s(dst + (size_t) r * 16 * 128, qs + blk * 128, (uint32_t) nb * 128, full + stage);
                    else skd::bulk_g2s(dst + S_QS + (size_t) r * 16 * 16, hdr + blk * 16, (uint32_t) nb * 16, full + stage);
                }
                if (++stage == nstages) { stage = 0; ++round; }
            }
        }
        skd::pdl_wait();
        return;
    }

    // ---------------- consumers ----------------
    skd::pdl_wait();                                   // the activation is the predecessor's output
    // taken as already quantized, or quantized here (optionally RMS-normalised first) while the ring fills
    q8k_prep_to_smem<PREP, NG * NC, RG_BAR_ALL>(in, cols, bpr, s_q8, s_bs, s_d, s_red, grp * NC + warp, lane, (grp * NC + warp) * 32 + lane);
    prep_sync<NG * NC, RG_BAR_ALL>();

    const int h = lane & 1, slot = lane >> 1, s1 = (slot >> 1) & 1;
    const int off_lo = (h ^ (s1 << 1)) * 16, off_hi = ((2 + h) ^ (s1 << 1)) * 16;
    int woff[4], aoff[4];
    uint32_t ssel[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int g = (k + slot) & 3;
        woff[k] = 32 * g; aoff[k] = 64 * g;
        ssel[k] = (uint32_t) (2 * g) | ((uint32_t) (2 * g + 1) << 4);
    }
    uint4 a_lo[4], a_hi[4];
    uint2 bs = make_uint2(0, 0);
    float di = 0.0f;
    int stage = 0, phase = 0;
    const int par = EPI == EPI_PEER ? (*reinterpret_cast<const volatile int*>(peer.round) & 1) : 0;
    int obuf = 0;

    // Rows past the end of the matrix (last group only) are computed on whatever the stage holds and never written.
    for (int rgi = 0; rgi < my_rgs; ++rgi) {
        const bool first = rgi == 0;
        const int rg = vcta + rgi * vgrid;
        float acc = 0.0f;
        for (int cg = 0; cg < ncg; ++cg) {
            const int b = cg * 16 + slot;
            const bool live = b < bpr;
            if ((ncg > 1 || first) && live) {          // this lane's activation slice of column group cg
                const int8_t* qa = s_q8 + (size_t) b * 256;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    a_lo[k] = skd::lds128(qa + aoff[k] + off_lo);
                    a_hi[k] = skd::lds128(qa + aoff[k] + off_hi);
                }
                bs = *reinterpret_cast<const uint2*>(s_bs + (size_t) b * 16 + 8 * h);
                di = s_d[b];
            }
            if (!skd::mbar_wait_bounded(full + stage, phase, timeout_flag)) return;
            if (live) {
                const uint8_t* st = s_ring + (size_t) stage * S_BYTES;
                const uint8_t* qp = st + ((size_t) warp * 16 + slot) * 128 + h * 16;
                const uint4 hd = skd::lds128(st + S_QS + ((size_t) warp * 16 + slot) * 16);
                const float d = __half2float(__ushort_as_half((unsigned short) (hd.x & 0xffff)));
                const float dmin = __half2float(__ushort_as_half((unsigned short) (hd.x >> 16)));
                uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
                skd::k4_unpack(hd.y, hd.z, hd.w, sc_lo, sc_hi, mn_lo, mn_hi);
                int sdot = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint4 w = skd::lds128(qp + woff[k]);
                    const uint32_t scw = __byte_perm(sc_lo, sc_hi, ssel[k]);
                    int dl = 0, dh = 0;   // dh carries the high nibbles in place: 16 x the dot
                    dl = __dp4a((int) (w.x & 0x0f0f0f0fu), (int) a_lo[k].x, dl);
                    dl = __dp4a((int) (w.y & 0x0f0f0f0fu), (int) a_lo[k].y, dl);
                    dl = __dp4a((int) (w.z & 0x0f0f0f0fu), (int) a_lo[k].z, dl);
                    dl = __dp4a((int) (w.w & 0x0f0f0f0fu), (int) a_lo[k].w, dl);
                    dh = skd::dp4a_us(w.x & 0xf0f0f0f0u, a_hi[k].x, dh);
                    dh = skd::dp4a_us(w.y & 0xf0f0f0f0u, a_hi[k].y, dh);
                    dh = skd::dp4a_us(w.z & 0xf0f0f0f0u, a_hi[k].z, dh);
                    dh = skd::dp4a_us(w.w & 0xf0f0f0f0u, a_hi[k].w, dh);
                    sdot = __dp2a_lo((int) __byte_perm((uint32_t) dl, (uint32_t) (dh >> 4), 0x5410), (int) scw, sdot);
                }
                const uint32_t mn = h ? mn_hi : mn_lo;   // lane h accounts the mins of sub-blocks 4h..4h+3
                const int msum = (__dp4a((int) mn, (int) bs.x, 0) << 7) + __dp4a((int) mn, (int) bs.y, 0);
                acc += di * (d * (float) sdot - dmin * (float) msum);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty + stage);   // this warp is done reading the stage
            if (++stage == nstages) { stage = 0; phase ^= 1; }
        }
        const float v = skd::warp_sum(acc);
        const int row = rg * NC + warp;
        if (EPI == EPI_PEER) {
            // the group's NC rows, four at a time, into this rank's slot of every rank's inbox: the exchange of the
            // group sum rides on the matvec instead of following it (two result buffers: one barrier per group)
            if (lane == 0) s_out[obuf * NC + warp] = row < rows ? (resid ? resid[row] + v : v) : 0.0f;
            group_sync<NC, NG>(grp);
            if (warp == 0 && lane < (NC / 4) * peer.world) {
                const int g = lane % (NC / 4), p = lane / (NC / 4), base = rg * NC + 4 * g;
                const float* o = s_out + obuf * NC + 4 * g;
                if (base + 3 < rows) peer_store4(peer, par, p, base, o[0], o[1], o[2], o[3]);
                else for (int k = 0; k < 4 && base + k < rows; ++k) peer_store1(peer, par, p, base + k, o[k]);
            }
            obuf ^= 1;
        } else if (lane == 0 && row < rows) y[row] = EPI == EPI_ADD ? resid[row] + v : v;
    }
}

// ================================================================================================
// Q8_0. Stage: codes [NC][2048] then scales [NC][64] f16.
// ================================================================================================
constexpr int RG8_COLS = 2048;

template <int NC, int NG, int PREP, int EPI>
__global__ void __launch_bounds__(NG * (NC + 1) * 32)
q8_0_matvec_ring_kernel(const int8_t* __restrict__ codes, const __half* __restrict__ scales, int rows, int cols, MatvecIn in,
                        float* __restrict__ y, const float* __restrict__ resid, int nstages, int* __restrict__ timeout_flag) {
    constexpr int S_CODES = NC * RG8_COLS, S_SC = NC * (RG8_COLS / 32) * 2, S_BYTES = S_CODES + S_SC;
    extern __shared__ __align__(128) uint8_t smem[];
    // NG groups (producer warp + NC consumer warps, own ring and barriers) around one staged activation, as in the Q4_K kernel
    const int bpr = cols >> 5;
    const int lane = threadIdx.x & 31;
    const int grp = NG == 1 ? 0 : (int) (threadIdx.x >> 5) / (NC + 1);
    const int warp = (int) (threadIdx.x >> 5) - grp * (NC + 1);
    uint8_t* s_ring = smem + (size_t) grp * nstages * S_BYTES;
    int8_t* s_hi = (int8_t*) (smem + (size_t) NG * nstages * S_BYTES);
    int8_t* s_lo = s_hi + cols;
    float* s_dx = (float*) (s_lo + cols);
    float* s_red = (float*) ((uint8_t*) s_dx + ((bpr * 4 + 15) & ~15));     // NG * NC floats (at most 16)
    uint64_t* full = (uint64_t*) (s_red + 16) + grp * 2 * RG_MAX_STAGES;
    uint64_t* empty = full + RG_MAX_STAGES;

    const int vcta = (int) blockIdx.x * NG + grp, vgrid = (int) gridDim.x * NG;
    const int nrg = (rows + NC - 1) / NC;
    const int ncg = (cols + RG8_COLS - 1) / RG8_COLS;
    const int my_rgs = vcta < nrg ? (nrg - 1 - vcta) / vgrid + 1 : 0;

    if (warp == NC && lane == 0) {
        for (int s = 0; s < nstages; ++s) { skd::mbar_init(full + s, 1); skd::mbar_init(empty + s, NC); }
        skd::mbar_fence_init();
    }
    __syncthreads();
    skd::pdl_launch_dependents();

    if (warp == NC) {
        int stage = 0, round = 0;
        for (int rgi = 0; rgi < my_rgs; ++rgi) {
            const int row0 = (vcta + rgi * vgrid) * NC, nr = min(NC, rows - row0);
            for (int cg = 0; cg < ncg; ++cg) {
                if (round > 0 && !skd::mbar_wait_bounded(empty + stage, (round - 1) & 1, timeout_flag)) return;
                const int c0 = cg * RG8_COLS, nc = min(RG8_COLS, cols - c0);
                uint8_t* dst = s_ring + (size_t) stage * S_BYTES;
                if (lane == 0) skd::mbar_expect_tx(full + stage, (uint32_t) nr * (nc + nc / 16));
                __syncwarp();
                if (lane < 2 * nr) {
                    const int r = lane < nr ? lane : lane - nr;
                    if (lane < nr) skd::bulk_g2s(dst + (size_t) r * RG8_COLS, codes + (size_t) (row0 + r) * cols + c0, (uint32_t) nc, full + stage);
                    else skd::bulk_g2s(dst + S_CODES + (size_t) r * (RG8_COLS / 16), scales + (size_t) (row0 + r) * bpr + (c0 >> 5), (uint32_t) nc / 16, full + stage);
                }
                if (++stage == nstages) { stage = 0; ++round; }
            }
        }
        skd::pdl_wait();
        return;
    }

    skd::pdl_wait();
    split_prep_to_smem<PREP, NG * NC, RG_BAR_ALL>(in, cols, bpr, s_hi, s_lo, s_dx, s_red, grp * NC + warp, lane, (grp * NC + warp) * 32 + lane);
    prep_sync<NG * NC, RG_BAR_ALL>();

    uint4 ah[4], al[4];
    float dx[4];
    int stage = 0, phase = 0;
    for (int rgi = 0; rgi < my_rgs; ++rgi) {
        const bool first = rgi == 0;
        const int rg = vcta + rgi * vgrid;
        float acc = 0.0f;
        for (int cg = 0; cg < ncg; ++cg) {
            const int c0 = cg * RG8_COLS, nc = min(RG8_COLS, cols - c0);
            if (ncg > 1 || first) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int c = j * 512 + lane * 16;            // code offset inside the column group
                    if (c < nc) {
                        ah[j] = skd::lds128(s_hi + c0 + c); al[j] = skd::lds128(s_lo + c0 + c);
                        dx[j] = s_dx[(c0 + c) >> 5];
                    } else { ah[j] = make_uint4(0, 0, 0, 0); al[j] = ah[j]; dx[j] = 0.0f; }
                }
            }
            if (!skd::mbar_wait_bounded(full + stage, phase, timeout_flag)) return;
            {
                const uint8_t* st = s_ring + (size_t) stage * S_BYTES;
                const int8_t* wr = (const int8_t*) st + (size_t) warp * RG8_COLS;
                const __half* sr = (const __half*) (st + S_CODES) + (size_t) warp * (RG8_COLS / 32);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int c = j * 512 + lane * 16;
                    if (c < nc) {
                        const uint4 w = skd::lds128(wr + c);
                        int dh = 0, dl = 0;
                        dh = __dp4a((int) w.x, (int) ah[j].x, dh); dh = __dp4a((int) w.y, (int) ah[j].y, dh);
                        dh = __dp4a((int) w.z, (int) ah[j].z, dh); dh = __dp4a((int) w.w, (int) ah[j].w, dh);
                        dl = __dp4a((int) w.x, (int) al[j].x, dl); dl = __dp4a((int) w.y, (int) al[j].y, dl);
                        dl = __dp4a((int) w.z, (int) al[j].z, dl); dl = __dp4a((int) w.w, (int) al[j].w, dl);
                        acc += (__half2float(sr[c >> 5]) * dx[j]) * (float) (dh * 128 + dl);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty + stage);
            if (++stage == nstages) { stage = 0; phase ^= 1; }
        }
        const float v = skd::warp_sum(acc);
        const int row = rg * NC + warp;
        if (lane == 0 && row < rows) y[row] = EPI == EPI_ADD ? resid[row] + v : v;
    }
}

// ================================================================================================
// dispatch (m = 1). Returns 1 when the shape is outside what these take.
// ================================================================================================
// One CTA per SM of RG_GROUPS groups; the ring depth is what the activation leaves of the budget.
constexpr int RG_GROUPS = 4, RG_GROUP_ROWS = 4;
template <int PREP, int EPI>
static int32_t launch_q4k_ring(const Weight& w, const MatvecIn& in, float* y, const float* resid, int* flag, cudaStream_t s,
                               const PeerOut& peer = PeerOut()) {
    constexpr size_t STAGE = (size_t) RG_GROUPS * RG_GROUP_ROWS * 16 * 144;
    const size_t fixed = (size_t) w.cols + w.cols / 16 + ((w.bpr * 4 + 15) & ~15) + 64 + RG_GROUPS * (2 * RG_MAX_STAGES * 8 + 2 * RG_GROUP_ROWS * 4) + 256;
    if (ring_budget() <= fixed) return 1;
    const int ns = (int) std::min<size_t>(RG_MAX_STAGES, (ring_budget() - fixed) / STAGE);
    if (ns < 3) return 1;
    auto kernel = q4k_matvec_ring_kernel<RG_GROUP_ROWS, RG_GROUPS, PREP, EPI>;
    SK_TRY(ensure_dynamic_smem((const void*) kernel, (int) RG_SMEM_MAX + 1024));
    const int nrg = (w.rows + RG_GROUP_ROWS - 1) / RG_GROUP_ROWS, grid = std::min(sm_count(), (nrg + RG_GROUPS - 1) / RG_GROUPS);
    SK_CUDA(launch_pdl(kernel, dim3(grid), dim3(RG_GROUPS * (RG_GROUP_ROWS + 1) * 32), fixed + ns * STAGE, s, (const uint8_t*) w.qs,
                       (const uint8_t*) w.hdr, w.rows, w.bpr, in, w.cols, y, resid, ns, flag, peer));
    return SKAINET_CUDA_OK;
}
template <int PREP, int EPI>
static int32_t launch_q8_ring(const Weight& w, const MatvecIn& in, float* y, const float* resid, int* flag, cudaStream_t s) {
    constexpr size_t STAGE = (size_t) RG_GROUPS * RG_GROUP_ROWS * (RG8_COLS + RG8_COLS / 16);
    const size_t fixed = (size_t) 2 * w.cols + ((w.bpr * 4 + 15) & ~15) + 64 + RG_GROUPS * 2 * RG_MAX_STAGES * 8 + 256;
    if (ring_budget() <= fixed) return 1;
    const int ns = (int) std::min<size_t>(RG_MAX_STAGES, (ring_budget() - fixed) / STAGE);
    if (ns < 3) return 1;
    auto kernel = q8_0_matvec_ring_kernel<RG_GROUP_ROWS, RG_GROUPS, PREP, EPI>;
    SK_TRY(ensure_dynamic_smem((const void*) kernel, (int) RG_SMEM_MAX + 1024));
    const int nrg = (w.rows + RG_GROUP_ROWS - 1) / RG_GROUP_ROWS, grid = std::min(sm_count(), (nrg + RG_GROUPS - 1) / RG_GROUPS);
    SK_CUDA(launch_pdl(kernel, dim3(grid), dim3(RG_GROUPS * (RG_GROUP_ROWS + 1) * 32), fixed + ns * STAGE, s, (const int8_t*) w.qs,
                       (const __half*) w.hdr, w.rows, w.cols, in, y, resid, ns, flag));
    return SKAINET_CUDA_OK;
}

int32_t launch_matvec_ring(const Weight& w, const MatvecIn& in, int prep, float* y, const float* resid, cudaStream_t s, const PeerOut* peer) {
    int* flag = device_timeout_flag();
    if (w.rows <= 0) return 1;
    if (peer && (w.enc != SKAINET_ENC_Q4_K || (prep != PREP_QUANTIZED && prep != PREP_SWIGLU_F32))) return 1;
    if (prep == PREP_SWIGLU_F32 && w.enc != SKAINET_ENC_Q4_K) return 1;
    if (w.enc == SKAINET_ENC_Q4_K) {
        if (peer) return prep == PREP_SWIGLU_F32 ? launch_q4k_ring<PREP_SWIGLU_F32, EPI_PEER>(w, in, y, resid, flag, s, *peer)
                                                 : launch_q4k_ring<PREP_QUANTIZED, EPI_PEER>(w, in, y, resid, flag, s, *peer);
        switch (prep * 2 + (resid ? EPI_ADD : EPI_STORE)) {
            case PREP_SWIGLU_F32 * 2 + EPI_STORE: return launch_q4k_ring<PREP_SWIGLU_F32, EPI_STORE>(w, in, y, resid, flag, s);
            case PREP_SWIGLU_F32 * 2 + EPI_ADD:   return launch_q4k_ring<PREP_SWIGLU_F32, EPI_ADD>(w, in, y, resid, flag, s);
            case PREP_QUANTIZED * 2 + EPI_STORE: return launch_q4k_ring<PREP_QUANTIZED, EPI_STORE>(w, in, y, resid, flag, s);
            case PREP_QUANTIZED * 2 + EPI_ADD:   return launch_q4k_ring<PREP_QUANTIZED, EPI_ADD>(w, in, y, resid, flag, s);
            case PREP_F32 * 2 + EPI_STORE:       return launch_q4k_ring<PREP_F32, EPI_STORE>(w, in, y, resid, flag, s);
            case PREP_F32 * 2 + EPI_ADD:         return launch_q4k_ring<PREP_F32, EPI_ADD>(w, in, y, resid, flag, s);
            case PREP_NORM_F32 * 2 + EPI_STORE:  return launch_q4k_ring<PREP_NORM_F32, EPI_STORE>(w, in, y, resid, flag, s);
            default:                             return launch_q4k_ring<PREP_NORM_F32, EPI_ADD>(w, in, y, resid, flag, s);
        }
    }
    if (w.enc == SKAINET_ENC_Q8_0) {
        if (w.cols % 256 != 0) return 1;
        switch (prep * 2 + (resid ? EPI_ADD : EPI_STORE)) {
            case PREP_QUANTIZED * 2 + EPI_STORE: return launch_q8_ring<PREP_QUANTIZED, EPI_STORE>(w, in, y, resid, flag, s);
            case PREP_QUANTIZED * 2 + EPI_ADD:   return launch_q8_ring<PREP_QUANTIZED, EPI_ADD>(w, in, y, resid, flag, s);
            case PREP_F32 * 2 + EPI_STORE:       return launch_q8_ring<PREP_F32, EPI_STORE>(w, in, y, resid, flag, s);
            case PREP_F32 * 2 + EPI_ADD:         return launch_q8_ring<PREP_F32, EPI_ADD>(w, in, y, resid, flag, s);
            case PREP_NORM_F32 * 2 + EPI_STORE:  return launch_q8_ring<PREP_NORM_F32, EPI_STORE>(w, in, y, resid, flag, s);
            default:                             return launch_q8_ring<PREP_NORM_F32, EPI_ADD>(w, in, y, resid, flag, s);
        }
    }
    return 1;
}

}  // namespace sk
