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

#include <cstdlib>

namespace sk {

constexpr int MF_WARPS = 4;
constexpr int MF_THREADS = MF_WARPS * 32;
constexpr int MF_MAX_RW = 4;
constexpr size_t MF_SMEM_MAX = 100 * 1024;

__device__ __forceinline__ float cta_sum(float v, float* red, int warp, int lane) {
    v = skd::warp_sum(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    const float t = (red[0] + red[1]) + (red[2] + red[3]);
    __syncthreads();
    return t;
}

// ================================================================================================
// Q4_K
// ================================================================================================
// Activation prep for K-quant weights, into shared memory: int8 codes (16-byte chunks XOR-swizzled
// per block pair), per-32 sums, per-256 scales. Warp w takes blocks w, w+4, ...; a lane holds
// elements 4l..4l+3 and 128+4l..128+4l+3 of a block, and all loads of a batch of blocks are issued
// before the first is used.
template <int PREP>
__device__ __forceinline__ void q8k_prep_to_smem(const MatvecIn& in, int cols, int bpr, int8_t* s_q8, int16_t* s_bs,
                                                 float* s_d, float* s_red, int warp, int lane) {
    if (PREP == PREP_QUANTIZED) {
        for (int c = threadIdx.x; c < (cols >> 4); c += MF_THREADS) {
            const int blk = c >> 4, ch = c & 15;
            *reinterpret_cast<uint4*>(s_q8 + (size_t) blk * 256 + (ch ^ (((blk >> 1) & 1) << 1)) * 16) = skd::ld_ro(in.q8.q + (size_t) c * 16);
        }
        // sub-block sums as two int8 planes (sum = 128*hi + lo) so the mins term is two dp4a per lane:
        // per block 16 bytes = [hi of sub-blocks 0..3 | lo 0..3 | hi 4..7 | lo 4..7]
        for (int c = threadIdx.x; c < (cols >> 5); c += MF_THREADS) {
            const int sum = (int) __ldg(in.q8.bsums + c), hi = (sum + 64) >> 7, lo = sum - (hi << 7);
            int8_t* dst = (int8_t*) s_bs + (size_t) (c >> 3) * 16 + ((c >> 2) & 1) * 8 + (c & 3);
            dst[0] = (int8_t) hi; dst[4] = (int8_t) lo;
        }
        for (int c = threadIdx.x; c < bpr; c += MF_THREADS) s_d[c] = __ldg(in.q8.d + c);
        return;
    }
    constexpr int B = 4;     // blocks per warp per batch: 8 float4 loads in flight per lane
    float nscale = 1.0f;
    if (PREP == PREP_NORM_F32) {
        float ss = 0.0f;
        for (int b0 = warp; b0 < bpr; b0 += MF_WARPS * B) {
            float4 v[2 * B];
#pragma unroll
            for (int j = 0; j < B; ++j) {
                const int blk = b0 + j * MF_WARPS;
                if (blk < bpr) {
                    v[2 * j] = __ldg(reinterpret_cast<const float4*>(in.x + (size_t) blk * 256) + lane);
                    v[2 * j + 1] = __ldg(reinterpret_cast<const float4*>(in.x + (size_t) blk * 256) + 32 + lane);
                } else { v[2 * j] = make_float4(0, 0, 0, 0); v[2 * j + 1] = v[2 * j]; }
            }
#pragma unroll
            for (int j = 0; j < 2 * B; ++j) ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
        }
        ss = cta_sum(ss, s_red, warp, lane);
        nscale = 1.0f / sqrtf(ss * (1.0f / (float) cols) + in.eps);
    }
    for (int b0 = warp; b0 < bpr; b0 += MF_WARPS * B) {
        float4 v[2 * B], g[2 * B];
#pragma unroll
        for (int j = 0; j < B; ++j) {
            const int blk = b0 + j * MF_WARPS;
            if (blk < bpr) {
                v[2 * j] = __ldg(reinterpret_cast<const float4*>(in.x + (size_t) blk * 256) + lane);
                v[2 * j + 1] = __ldg(reinterpret_cast<const float4*>(in.x + (size_t) blk * 256) + 32 + lane);
                if (PREP == PREP_NORM_F32) {
                    g[2 * j] = __ldg(reinterpret_cast<const float4*>(in.gamma + (size_t) blk * 256) + lane);
                    g[2 * j + 1] = __ldg(reinterpret_cast<const float4*>(in.gamma + (size_t) blk * 256) + 32 + lane);
                }
            } else { v[2 * j] = make_float4(0, 0, 0, 0); v[2 * j + 1] = v[2 * j]; g[2 * j] = v[2 * j]; g[2 * j + 1] = v[2 * j]; }
        }
#pragma unroll
        for (int j = 0; j < B; ++j) {
            const int blk = b0 + j * MF_WARPS;
            if (blk >= bpr) continue;                         // warp-uniform
            float e[8] = {v[2 * j].x, v[2 * j].y, v[2 * j].z, v[2 * j].w, v[2 * j + 1].x, v[2 * j + 1].y, v[2 * j + 1].z, v[2 * j + 1].w};
            if (PREP == PREP_NORM_F32) {
                const float ge[8] = {g[2 * j].x, g[2 * j].y, g[2 * j].z, g[2 * j].w, g[2 * j + 1].x, g[2 * j + 1].y, g[2 * j + 1].z, g[2 * j + 1].w};
#pragma unroll
                for (int i = 0; i < 8; ++i) e[i] = (e[i] * nscale) * ge[i];
            }
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(e[i]));
            amax = skd::warp_max(amax);
            const float inv = amax > 0.0f ? 127.0f / amax : 0.0f;
            int q[8], s0 = 0, s1 = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) q[i] = max(-127, min(127, __float2int_rn(e[i] * inv)));
#pragma unroll
            for (int i = 0; i < 4; ++i) { s0 += q[i]; s1 += q[4 + i]; }
            const uint32_t p0 = (uint32_t) (q[0] & 0xff) | ((uint32_t) (q[1] & 0xff) << 8) | ((uint32_t) (q[2] & 0xff) << 16) | ((uint32_t) (q[3] & 0xff) << 24);
            const uint32_t p1 = (uint32_t) (q[4] & 0xff) | ((uint32_t) (q[5] & 0xff) << 8) | ((uint32_t) (q[6] & 0xff) << 16) | ((uint32_t) (q[7] & 0xff) << 24);
            const int swz = ((blk >> 1) & 1) << 1;
            int8_t* dst = s_q8 + (size_t) blk * 256 + (lane & 3) * 4;
            *reinterpret_cast<uint32_t*>(dst + ((lane >> 2) ^ swz) * 16) = p0;          // elements 4l..4l+3: chunk l/4
            *reinterpret_cast<uint32_t*>(dst + ((8 + (lane >> 2)) ^ swz) * 16) = p1;    // elements 128+4l..: chunk 8+l/4
            // sub-block sums: eight lanes per 32 elements
            s0 += __shfl_xor_sync(0xffffffffu, s0, 1); s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
            s0 += __shfl_xor_sync(0xffffffffu, s0, 2); s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
            s0 += __shfl_xor_sync(0xffffffffu, s0, 4); s1 += __shfl_xor_sync(0xffffffffu, s1, 4);
            if ((lane & 7) == 0) {       // sub-blocks lane/8 (first half) and 4 + lane/8 (second half)
                int8_t* dst = (int8_t*) s_bs + (size_t) blk * 16 + (lane >> 3);
                const int h0 = (s0 + 64) >> 7, h1 = (s1 + 64) >> 7;
                dst[0] = (int8_t) h0; dst[4] = (int8_t) (s0 - (h0 << 7));
                dst[8] = (int8_t) h1; dst[12] = (int8_t) (s1 - (h1 << 7));
            }
            if (lane == 0) s_d[blk] = amax > 0.0f ? amax / 127.0f : 0.0f;
        }
    }
}

template <int RW, int PREP, int EPI>
__global__ void __launch_bounds__(MF_THREADS)
q4k_matvec_fused_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ hdr, int rows, int bpr,
                        MatvecIn in, int cols, float* __restrict__ y, const float* __restrict__ resid,
                        int* __restrict__ timeout_flag) {
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
    q8k_prep_to_smem<PREP>(in, cols, bpr, s_q8, s_bs, s_d, s_red, warp, lane);
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
        if (lane == 0 && rl < nrows) y[row0 + rl] = EPI == EPI_ADD ? resid[row0 + rl] + v : v;
    }
}

// ================================================================================================
// Q8_0
// ================================================================================================
// Activation prep for Q8_0 weights: the fp32 row as hi*128+lo int8 planes with one scale per 32.
template <int PREP>
__device__ __forceinline__ void split_prep_to_smem(const MatvecIn& in, int cols, int bpr, int8_t* s_hi, int8_t* s_lo,
                                                   float* s_dx, float* s_red, int warp, int lane) {
    if (PREP == PREP_QUANTIZED) {
        for (int c = threadIdx.x; c < (cols >> 4); c += MF_THREADS) {
            *reinterpret_cast<uint4*>(s_hi + (size_t) c * 16) = skd::ld_ro(in.split.hi + (size_t) c * 16);
            *reinterpret_cast<uint4*>(s_lo + (size_t) c * 16) = skd::ld_ro(in.split.lo + (size_t) c * 16);
        }
        for (int c = threadIdx.x; c < bpr; c += MF_THREADS) s_dx[c] = __ldg(in.split.d + c);
        return;
    }
    constexpr int B = 8;     // float4 loads in flight per thread
    const int n4 = cols >> 2;
    float nscale = 1.0f;
    if (PREP == PREP_NORM_F32) {
        float ss = 0.0f;
        for (int i0 = threadIdx.x; i0 < n4; i0 += MF_THREADS * B) {
            float4 v[B];
#pragma unroll
            for (int j = 0; j < B; ++j) {
                const int i = i0 + j * MF_THREADS;
                v[j] = i < n4 ? __ldg(reinterpret_cast<const float4*>(in.x) + i) : make_float4(0, 0, 0, 0);
            }
#pragma unroll
            for (int j = 0; j < B; ++j) ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
        }
        ss = cta_sum(ss, s_red, warp, lane);
        nscale = 1.0f / sqrtf(ss * (1.0f / (float) cols) + in.eps);
    }
    // thread t holds float4 chunk i = t + 128*j; a 32-block is eight consecutive chunks = eight lanes
    const int n4_pad = (n4 + MF_THREADS - 1) / MF_THREADS * MF_THREADS;   // keep whole warps in the shuffles
    for (int i0 = threadIdx.x; i0 < n4_pad; i0 += MF_THREADS * B) {
        float4 v[B], g[B];
#pragma unroll
        for (int j = 0; j < B; ++j) {
            const int i = i0 + j * MF_THREADS;
            const bool ok = i < n4;
            v[j] = ok ? __ldg(reinterpret_cast<const float4*>(in.x) + i) : make_float4(0, 0, 0, 0);
            if (PREP == PREP_NORM_F32) g[j] = ok ? __ldg(reinterpret_cast<const float4*>(in.gamma) + i) : make_float4(0, 0, 0, 0);
        }
#pragma unroll
        for (int j = 0; j < B; ++j) {
            const int i = i0 + j * MF_THREADS;
            if (i - (int) threadIdx.x >= n4_pad) continue;                // warp-uniform
            float e[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
            if (PREP == PREP_NORM_F32) {
                e[0] = (e[0] * nscale) * g[j].x; e[1] = (e[1] * nscale) * g[j].y;
                e[2] = (e[2] * nscale) * g[j].z; e[3] = (e[3] * nscale) * g[j].w;
            }
            float amax = fmaxf(fmaxf(fabsf(e[0]), fabsf(e[1])), fmaxf(fabsf(e[2]), fabsf(e[3])));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
            const float inv = amax > 0.0f ? 16256.0f / amax : 0.0f;
            uint32_t ph = 0, pl = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                int q = max(-16256, min(16256, __float2int_rn(e[k] * inv)));
                const int hi = (q + 64) >> 7, lo = q - (hi << 7);
                ph |= (uint32_t) (hi & 0xff) << (8 * k); pl |= (uint32_t) (lo & 0xff) << (8 * k);
            }
            if (i < n4) {
                *reinterpret_cast<uint32_t*>(s_hi + (size_t) i * 4) = ph;
                *reinterpret_cast<uint32_t*>(s_lo + (size_t) i * 4) = pl;
                if ((i & 7) == 0) s_dx[i >> 3] = amax > 0.0f ? amax / 16256.0f : 0.0f;
            }
        }
    }
}

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
    split_prep_to_smem<PREP>(in, cols, bpr, s_hi, s_lo, s_dx, s_red, warp, lane);
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
template <typename K>
static int32_t set_smem_once(K kernel, bool* done) {
    if (!*done) {
        SK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) MF_SMEM_MAX + 1024));
        *done = true;
    }
    return SKAINET_CUDA_OK;
}

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
static int32_t launch_q4k_f(const Weight& w, const MatvecIn& in, float* y, const float* resid, size_t smem, int* flag, cudaStream_t s) {
    static bool done = false;
    SK_TRY(set_smem_once(q4k_matvec_fused_kernel<RW, PREP, EPI>, &done));
    const int R = MF_WARPS * RW;
    SK_CUDA(launch_pdl(q4k_matvec_fused_kernel<RW, PREP, EPI>, dim3((w.rows + R - 1) / R), dim3(MF_THREADS), smem, s,
                       (const uint8_t*) w.qs, (const uint8_t*) w.hdr, w.rows, w.bpr, in, w.cols, y, resid, flag));
    return SKAINET_CUDA_OK;
}
template <int RW, int PREP, int EPI>
static int32_t launch_q8_f(const Weight& w, const MatvecIn& in, float* y, const float* resid, size_t smem, int* flag, cudaStream_t s) {
    static bool done = false;
    SK_TRY(set_smem_once(q8_0_matvec_fused_kernel<RW, PREP, EPI>, &done));
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

int32_t launch_matvec_fused(const Weight& w, const MatvecIn& in, int prep, float* y, const float* resid, cudaStream_t s) {
    int* flag = device_timeout_flag();
    if (w.rows <= 0) return 1;
    // Large weights go to the persistent ring kernel (SKAINET_RING_MIN_MB overrides the size threshold).
    static const int64_t ring_min = []() { const char* e = getenv("SKAINET_RING_MIN_MB"); return (int64_t) (e ? atoi(e) : 20) << 20; }();
    if (prep == PREP_QUANTIZED && w.packed_bytes >= ring_min) {
        const int32_t st = launch_matvec_ring(w, in, y, resid, s);
        if (st != 1) return st;
    }
    const int epi = resid ? EPI_ADD : EPI_STORE;
    if (w.enc == SKAINET_ENC_Q4_K) {
        const size_t fixed = (size_t) w.cols + w.cols / 16 + ((w.bpr * 4 + 15) & ~15) + 16 + MF_MAX_RW * 8 + 64;
        const int rw = pick_rw(fixed, (size_t) w.bpr * 144, w.rows);
        if (rw == 0) return 1;
        const size_t smem = fixed + (size_t) MF_WARPS * rw * w.bpr * 144;
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
