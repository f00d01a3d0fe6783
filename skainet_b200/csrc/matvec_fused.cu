// Fused single-row matvec for decode (m = 1): activation prep + dequant-fused dot + epilogue in one
// launch, with the CTA's weight tile fetched by TMA.
//
// Each CTA owns a tile of 4*RW consecutive output rows. Thread 0 issues the whole tile as RW
// sub-tiles of four rows (cp.async.bulk, one mbarrier per sub-tile) before anything else, so under
// programmatic dependent launch the weights are already on their way while the kernel that produces
// the activation is still running. The four warps then prepare the activation once per CTA — taken as
// already quantized, or quantized from fp32, or RMS-normalised and quantized, with every global load
// of the row issued before the first use (one L2 round trip) — and walk the sub-tiles in arrival
// order: warp w owns row 4r+w of sub-tile r, so compute on the first rows overlaps the arrival of the
// rest. Shared-memory reads are bank-conflict free (rotated group order for the 128-byte code blocks,
// XOR-swizzled activation chunks). The epilogue stores the row result or adds it to a residual.
// Every mbarrier wait is bounded and reports through a device flag.
//
// HBM-bound: algorithmic bytes = rows*(cols/256)*144 (Q4_K) or rows*(cols/32)*34 (Q8_0) + 4*(rows+cols).
// Arithmetic as in matvec.cu (reference: native/src/q4k_matmul.c:74-92,143-251,
// native/src/q8_0_matmul.c:68-118, native/src/f32_fused.c:255-271 for the norm).
#include "common.cuh"
#include "actquant.cuh"
#include "tma.cuh"
#include "matvec_fused.cuh"
#include "actprep.cuh"

#include <cstdlib>

namespace sk {

constexpr int MF_WARPS = 4;
constexpr int MF_THREADS = MF_WARPS * 32;
constexpr int MF_MAX_RW = 4;
constexpr size_t MF_SMEM_MAX = 100 * 1024;
// Measured crossover between the one-tile and the ring kernel. With the activation already quantized (the decoder's o
// and down projections, everything under tensor parallelism) the two trade places shape by shape below 20 MB. When the
// kernel itself quantizes an fp32 row, the ring kernel does so once per SM and the one-tile kernel once per CTA, and the
// ring kernel wins down to a few MB (Q4_K 4096 x 4096: 3.3 against 5.2 us; 8192 x 1024: 4.1 against 4.6-5.7 us).
// matvec_uses_ring() holds the rule.
constexpr size_t RING_MIN_BYTES = (size_t) 20 << 20, RING_MIN_BYTES_F32_ROW = (size_t) 4 << 20;

// ================================================================================================
// Q4_K (activation preparation: actprep.cuh)
// ================================================================================================
template <int RW, int PREP, int EPI>
__global__ void __launch_bounds__(MF_THREADS)
q4k_matvec_fused_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ hdr, int rows, int bpr,
                        MatvecIn in, int cols, float* __restrict__ y, const float* __restrict__ resid,
                        int* __restrict__ timeout_flag, PeerOut peer) {
    constexpr int R = MF_WARPS * RW;
    extern __shared__ __align__(128) uint8_t smem[];
    // layout: qs tile | hdr tile | q8 (swizzled) | bsums | d | reduce scratch | barriers
    uint8_t* s_qs = smem;
    uint8_t* s_hdr = s_qs + (size_t) R * bpr * 128;
    int8_t* s_q8 = (int8_t*) (s_hdr + (size_t) R * bpr * 16);
    int16_t* s_bs = (int16_t*) (s_q8 + cols);   // 16 bytes per block
    float* s_d = (float*) ((uint8_t*) s_bs + cols / 16);
    float* s_red = (float*) ((uint8_t*) s_d + ((bpr * 4 + 15) & ~15));
    uint64_t* bars = (uint64_t*) (s_red + 4);
    float* s_out = (float*) (bars + MF_MAX_RW);          // the tile's results, gathered for the peer stores

    const int row0 = blockIdx.x * R;
    const int nrows = min(R, rows - row0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    if (threadIdx.x == 0) {
#pragma unroll
        for (int r = 0; r < RW; ++r) skd::mbar_init(bars + r, 1);
        skd::mbar_fence_init();
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            const int nr = min(MF_WARPS, nrows - MF_WARPS * r);
            if (nr > 0) {
                const uint32_t bq = (uint32_t) nr * bpr * 128, bh = (uint32_t) nr * bpr * 16;
                const size_t first = (size_t) (row0 + MF_WARPS * r) * bpr;
                skd::mbar_expect_tx(bars + r, bq + bh);
                skd::bulk_g2s(s_qs + (size_t) MF_WARPS * r * bpr * 128, qs + first * 128, bq, bars + r);
                skd::bulk_g2s(s_hdr + (size_t) MF_WARPS * r * bpr * 16, hdr + first * 16, bh, bars + r);
            }
        }
    }
    skd::pdl_launch_dependents();
    skd::pdl_wait();                       // the activation is the predecessor's output
    q8k_prep_to_smem<PREP, MF_WARPS, 0>(in, cols, bpr, s_q8, s_bs, s_d, s_red, warp, lane, threadIdx.x);
    __syncthreads();                       // also orders thread 0's barrier init before everyone's wait

    const int h = lane & 1, slot = lane >> 1, sw1 = (slot >> 1) & 1;
    const int off_lo = (h ^ (sw1 << 1)) * 16, off_hi = ((2 + h) ^ (sw1 << 1)) * 16;
    const int ncg = (bpr + 15) >> 4;
    uint4 a_lo[4], a_hi[4];
    uint2 bs = make_uint2(0, 0);
    float di = 0.0f;
    // lane-constant per rotated group k: byte offsets of the group and the selector that fetches its
    // (even, odd) sub-block scales from the eight unpacked scale bytes
    int woff[4], aoff[4];
    uint32_t ssel[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int g = (k + slot) & 3;
        woff[k] = 32 * g; aoff[k] = 64 * g;
        ssel[k] = (uint32_t) (2 * g) | ((uint32_t) (2 * g + 1) << 4);
    }

#pragma unroll
    for (int r = 0; r < RW; ++r) {
        const int rl = MF_WARPS * r + warp;
        if (MF_WARPS * r >= nrows) break;                                  // CTA-uniform
        if (!skd::mbar_wait_bounded(bars + r, 0, timeout_flag)) return;
        float acc = 0.0f;
        for (int cg = 0; cg < ncg; ++cg) {
            const int b = cg * 16 + slot;
            const bool live = b < bpr;
            if ((ncg > 1 || r == 0) && live) {             // this lane's activation slice of column group cg
                const int8_t* qa = s_q8 + (size_t) b * 256;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    a_lo[k] = skd::lds128(qa + aoff[k] + off_lo);
                    a_hi[k] = skd::lds128(qa + aoff[k] + off_hi);
                }
                bs = *reinterpret_cast<const uint2*>((const uint8_t*) s_bs + (size_t) b * 16 + 8 * h);
                di = s_d[b];
            }
            if (live && rl < nrows) {
                const size_t blk = (size_t) rl * bpr + b;
                const uint8_t* qp = s_qs + blk * 128 + h * 16;
                const uint4 hd = skd::lds128(s_hdr + blk * 16);
                const float d = __half2float(__ushort_as_half((unsigned short) (hd.x & 0xffff)));
                const float dmin = __half2float(__ushort_as_half((unsigned short) (hd.x >> 16)));
                uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
                skd::k4_unpack(hd.y, hd.z, hd.w, sc_lo, sc_hi, mn_lo, mn_hi);
                int sdot = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint4 w = skd::lds128(qp + woff[k]);
                    const uint32_t scw = __byte_perm(sc_lo, sc_hi, ssel[k]);   // low bytes: scales of sub-blocks 2g, 2g+1
                    int dl = 0, dh = 0;   // dh carries the high nibbles in place: 16 x the dot
                    dl = __dp4a((int) (w.x & 0x0f0f0f0fu), (int) a_lo[k].x, dl);
                    dl = __dp4a((int) (w.y & 0x0f0f0f0fu), (int) a_lo[k].y, dl);
                    dl = __dp4a((int) (w.z & 0x0f0f0f0fu), (int) a_lo[k].z, dl);
                    dl = __dp4a((int) (w.w & 0x0f0f0f0fu), (int) a_lo[k].w, dl);
                    dh = skd::dp4a_us(w.x & 0xf0f0f0f0u, a_hi[k].x, dh);
                    dh = skd::dp4a_us(w.y & 0xf0f0f0f0u, a_hi[k].y, dh);
                    dh = skd::dp4a_us(w.z & 0xf0f0f0f0u, a_hi[k].z, dh);
                    dh = skd::dp4a_us(w.w & 0xf0f0f0f0u, a_hi[k].w, dh);
                    // |dl|, |dh/16| <= 16*15*127 fit int16: both products in one dp2a
                    sdot = __dp2a_lo((int) __byte_perm((uint32_t) dl, (uint32_t) (dh >> 4), 0x5410), (int) scw, sdot);
                }
                const uint32_t mn = h ? mn_hi : mn_lo;   // lane h accounts the mins of sub-blocks 4h..4h+3
                const int msum = (__dp4a((int) mn, (int) bs.x, 0) << 7) + __dp4a((int) mn, (int) bs.y, 0);
                acc += di * (d * (float) sdot - dmin * (float) msum);
            }
        }
        const float v = skd::warp_sum(acc);
        if (EPI == EPI_PEER) { if (lane == 0) s_out[rl] = rl < nrows ? (resid ? resid[row0 + rl] + v : v) : 0.0f; }
        else if (lane == 0 && rl < nrows) y[row0 + rl] = EPI == EPI_ADD ? resid[row0 + rl] + v : v;
    }
    if (EPI == EPI_PEER) {
        // the tile's rows, four at a time, into this rank's slot of every rank's inbox: the exchange of the group sum
        // rides on the matvec instead of following it
        __syncthreads();
        const int par = *reinterpret_cast<const volatile int*>(peer.round) & 1;
        constexpr int G4 = R / 4;
        for (int t = threadIdx.x; t < G4 * peer.world; t += MF_THREADS) {
            const int g = t % G4, p = t / G4, base = row0 + 4 * g;
            if (base + 3 < rows) peer_store4(peer, par, p, base, s_out[4 * g], s_out[4 * g + 1], s_out[4 * g + 2], s_out[4 * g + 3]);
            else for (int k = 0; k < 4 && base + k < rows; ++k) peer_store1(peer, par, p, base + k, s_out[4 * g + k]);
        }
    }
}

// ================================================================================================
// Q8_0
// ================================================================================================
template <int RW, int PREP, int EPI>
__global__ void __launch_bounds__(MF_THREADS)
q8_0_matvec_fused_kernel(const int8_t* __restrict__ codes, const __half* __restrict__ scales, int rows, int cols,
                         MatvecIn in, float* __restrict__ y, const float* __restrict__ resid, int* __restrict__ timeout_flag) {
    constexpr int R = MF_WARPS * RW;
    extern __shared__ __align__(128) uint8_t smem[];
    const int bpr = cols >> 5;
    int8_t* s_codes = (int8_t*) smem;
    __half* s_scales = (__half*) (s_codes + (size_t) R * cols);
    int8_t* s_hi = (int8_t*) (s_scales + (size_t) R * bpr);
    int8_t* s_lo = s_hi + cols;
    float* s_dx = (float*) (s_lo + cols);
    float* s_red = (float*) ((uint8_t*) s_dx + ((bpr * 4 + 15) & ~15));
    uint64_t* bars = (uint64_t*) (s_red + 4);

    const int row0 = blockIdx.x * R;
    const int nrows = min(R, rows - row0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    if (threadIdx.x == 0) {
#pragma unroll
        for (int r = 0; r < RW; ++r) skd::mbar_init(bars + r, 1);
        skd::mbar_fence_init();
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            const int nr = min(MF_WARPS, nrows - MF_WARPS * r);
            if (nr > 0) {
                const uint32_t bc = (uint32_t) nr * cols, bsz = (uint32_t) nr * bpr * 2;
                const size_t first = (size_t) (row0 + MF_WARPS * r);
                skd::mbar_expect_tx(bars + r, bc + bsz);
                skd::bulk_g2s(s_codes + (size_t) MF_WARPS * r * cols, codes + first * cols, bc, bars + r);
                skd::bulk_g2s(s_scales + (size_t) MF_WARPS * r * bpr, scales + first * bpr, bsz, bars + r);
            }
        }
    }
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    split_prep_to_smem<PREP, MF_WARPS, 0>(in, cols, bpr, s_hi, s_lo, s_dx, s_red, warp, lane, threadIdx.x);
    __syncthreads();

    const int nchunks = cols >> 4;
#pragma unroll
    for (int r = 0; r < RW; ++r) {
        const int rl = MF_WARPS * r + warp;
        if (MF_WARPS * r >= nrows) break;
        if (!skd::mbar_wait_bounded(bars + r, 0, timeout_flag)) return;
        float acc = 0.0f;
        if (rl < nrows) {
            const int8_t* wr = s_codes + (size_t) rl * cols;
            const __half* sr = s_scales + (size_t) rl * bpr;
#pragma unroll 4
            for (int c = lane; c < nchunks; c += 32) {
                const uint4 w = skd::lds128(wr + c * 16);
                const uint4 ah = skd::lds128(s_hi + c * 16), al = skd::lds128(s_lo + c * 16);
                int dh = 0, dl = 0;
                dh = __dp4a((int) w.x, (int) ah.x, dh); dh = __dp4a((int) w.y, (int) ah.y, dh);
                dh = __dp4a((int) w.z, (int) ah.z, dh); dh = __dp4a((int) w.w, (int) ah.w, dh);
                dl = __dp4a((int) w.x, (int) al.x, dl); dl = __dp4a((int) w.y, (int) al.y, dl);
                dl = __dp4a((int) w.z, (int) al.z, dl); dl = __dp4a((int) w.w, (int) al.w, dl);
                acc += (__half2float(sr[c >> 1]) * s_dx[c >> 1]) * (float) (dh * 128 + dl);
            }
        }
        const float v = skd::warp_sum(acc);
        if (lane == 0 && rl < nrows) y[row0 + rl] = EPI == EPI_ADD ? resid[row0 + rl] + v : v;
    }
}

// ================================================================================================
// dispatch (m = 1 only). Returns 1 when the shape is outside what these kernels take.
// ================================================================================================
// rows per warp: the largest tile under the budget, then halved while the grid would leave SMs short
static int pick_rw(size_t fixed, size_t row_bytes, int rows) {
    int rw = MF_MAX_RW;
    while (rw >= 1 && fixed + (size_t) MF_WARPS * rw * row_bytes > MF_SMEM_MAX) rw >>= 1;
    if (rw < 1) return 0;
    while (rw > 1 && (fixed + (size_t) MF_WARPS * rw * row_bytes > 48 * 1024 ||
                      (rows + MF_WARPS * rw - 1) / (MF_WARPS * rw) < 3 * sm_count())) rw >>= 1;
    return rw;
}

template <int RW, int PREP, int EPI>
static int32_t launch_q4k_f(const Weight& w, const MatvecIn& in, float* y, const float* resid, size_t smem, int* flag, cudaStream_t s,
                            const PeerOut& peer = PeerOut()) {
    SK_TRY(ensure_dynamic_smem((const void*) q4k_matvec_fused_kernel<RW, PREP, EPI>, (int) MF_SMEM_MAX + 1024));
    const int R = MF_WARPS * RW;
    SK_CUDA(launch_pdl(q4k_matvec_fused_kernel<RW, PREP, EPI>, dim3((w.rows + R - 1) / R), dim3(MF_THREADS), smem, s,
                       (const uint8_t*) w.qs, (const uint8_t*) w.hdr, w.rows, w.bpr, in, w.cols, y, resid, flag, peer));
    return SKAINET_CUDA_OK;
}
template <int RW, int PREP, int EPI>
static int32_t launch_q8_f(const Weight& w, const MatvecIn& in, float* y, const float* resid, size_t smem, int* flag, cudaStream_t s) {
    SK_TRY(ensure_dynamic_smem((const void*) q8_0_matvec_fused_kernel<RW, PREP, EPI>, (int) MF_SMEM_MAX + 1024));
    const int R = MF_WARPS * RW;
    SK_CUDA(launch_pdl(q8_0_matvec_fused_kernel<RW, PREP, EPI>, dim3((w.rows + R - 1) / R), dim3(MF_THREADS), smem, s,
                       (const int8_t*) w.qs, (const __half*) w.hdr, w.rows, w.cols, in, y, resid, flag));
    return SKAINET_CUDA_OK;
}

#define SK_MF_PE(FN, RWV)                                                                              \
    switch (prep * 2 + epi) {                                                                          \
        case PREP_QUANTIZED * 2 + EPI_STORE: return FN<RWV, PREP_QUANTIZED, EPI_STORE>(w, in, y, resid, smem, flag, s); \
        case PREP_QUANTIZED * 2 + EPI_ADD:   return FN<RWV, PREP_QUANTIZED, EPI_ADD>(w, in, y, resid, smem, flag, s);   \
        case PREP_F32 * 2 + EPI_STORE:       return FN<RWV, PREP_F32, EPI_STORE>(w, in, y, resid, smem, flag, s);       \
        case PREP_F32 * 2 + EPI_ADD:         return FN<RWV, PREP_F32, EPI_ADD>(w, in, y, resid, smem, flag, s);         \
        case PREP_NORM_F32 * 2 + EPI_STORE:  return FN<RWV, PREP_NORM_F32, EPI_STORE>(w, in, y, resid, smem, flag, s);  \
        default:                             return FN<RWV, PREP_NORM_F32, EPI_ADD>(w, in, y, resid, smem, flag, s);    \
    }
#define SK_MF_RW(FN)                          \
    switch (rw) {                             \
        case 4: SK_MF_PE(FN, 4)               \
        case 2: SK_MF_PE(FN, 2)               \
        default: SK_MF_PE(FN, 1)              \
    }

bool matvec_uses_ring(const Weight& w, int prep) {
    if (w.enc != SKAINET_ENC_Q4_K && w.enc != SKAINET_ENC_Q8_0) return false;
    if (w.packed_bytes >= (int64_t) RING_MIN_BYTES) return true;
    if (w.enc != SKAINET_ENC_Q4_K || w.packed_bytes < (int64_t) RING_MIN_BYTES_F32_ROW) return false;
    if (prep != PREP_QUANTIZED) return true;
    // An already quantized row: the ring kernel where its static schedule fills the machine. Row groups of four go round
    // robin over four groups per SM; when the last round is mostly empty (2560 rows: 640 groups over 592 slots) the
    // one-tile kernel is faster (5.3 against 6.1 us), otherwise the ring kernel is (1280 x 8192: 4.5 against 4.9 us;
    // 8192 x 2048: 5.6 against 6.0; 4096 x 4096: 4.8 against 5.4).
    const int nrg = (w.rows + 3) / 4, slots = 4 * std::min(sm_count(), (nrg + 3) / 4);
    const int rounds = (nrg + slots - 1) / slots;
    return (int64_t) rounds * slots * 4 <= (int64_t) nrg * 5;          // at most a quarter of the slots idle
}

int32_t launch_matvec_fused(const Weight& w, const MatvecIn& in, int prep, float* y, const float* resid, cudaStream_t s,
                            const PeerOut* peer) {
    int* flag = device_timeout_flag();
    if (w.rows <= 0) return 1;
    if (peer && (w.enc != SKAINET_ENC_Q4_K || (prep != PREP_QUANTIZED && prep != PREP_SWIGLU_F32))) return 1;
    // Large weights go to the persistent ring kernel.
    if (matvec_uses_ring(w, prep)) {
        const int32_t st = launch_matvec_ring(w, in, prep, y, resid, s, peer);
        if (st != 1) return st;
    }
    if (prep == PREP_SWIGLU_F32) return 1;              // only the ring kernel takes the gate | up form
    const int epi = resid ? EPI_ADD : EPI_STORE;
    if (w.enc == SKAINET_ENC_Q4_K) {
        const size_t fixed = (size_t) w.cols + w.cols / 16 + ((w.bpr * 4 + 15) & ~15) + 16 + MF_MAX_RW * 8 + 64 + 64;
        const int rw = pick_rw(fixed, (size_t) w.bpr * 144, w.rows);
        if (rw == 0) return 1;
        const size_t smem = fixed + (size_t) MF_WARPS * rw * w.bpr * 144;
        if (peer) {
            switch (rw) {
                case 4: return launch_q4k_f<4, PREP_QUANTIZED, EPI_PEER>(w, in, y, resid, smem, flag, s, *peer);
                case 2: return launch_q4k_f<2, PREP_QUANTIZED, EPI_PEER>(w, in, y, resid, smem, flag, s, *peer);
                default: return launch_q4k_f<1, PREP_QUANTIZED, EPI_PEER>(w, in, y, resid, smem, flag, s, *peer);
            }
        }
        SK_MF_RW(launch_q4k_f)
    }
    if (w.enc == SKAINET_ENC_Q8_0) {
        if (w.cols % 256 != 0) return 1;     // scale rows must be whole 16-byte units for the bulk copy
        const size_t fixed = (size_t) 2 * w.cols + ((w.bpr * 4 + 15) & ~15) + 16 + MF_MAX_RW * 8 + 64;
        const int rw = pick_rw(fixed, (size_t) w.cols + w.bpr * 2, w.rows);
        if (rw == 0) return 1;
        const size_t smem = fixed + (size_t) MF_WARPS * rw * (w.cols + w.bpr * 2);
        SK_MF_RW(launch_q8_f)
    }
    return 1;
}

}  // namespace sk
