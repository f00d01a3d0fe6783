// Activation preparation inside a matvec kernel's prologue: the fp32 row (optionally RMS-normalised) is
// quantized straight into the CTA's shared memory, so a decode-step linear is one launch instead of a
// quantizer launch plus a matvec launch. Shared by the one-tile kernels (matvec_fused.cu, all warps of the
// CTA prepare) and the ring kernels (matvec_ring.cu, the consumer warps prepare while the producer warp
// already streams weights). Arithmetic: skainet_q8_quantize_block, native/src/q4k_matmul.c:74-92;
// RMSNorm as native/src/f32_fused.c:255-271.
#pragma once
#include "common.cuh"
#include "actquant.cuh"
#include "matvec_fused.cuh"

#ifdef __CUDACC__
namespace sk {

// Barrier over the NW warps that prepare the activation: the whole CTA (BAR == 0) or named barrier BAR.
template <int NW, int BAR>
__device__ __forceinline__ void prep_sync() {
    if (BAR == 0) __syncthreads();
    else asm volatile("bar.sync %0, %1;" ::"n"(BAR), "n"(NW * 32) : "memory");
}

// Sum over the NW preparing warps in a fixed order; red holds at least NW floats.
template <int NW, int BAR>
__device__ __forceinline__ float prep_sum(float v, float* red, int warp, int lane) {
    v = skd::warp_sum(v);
    if (lane == 0) red[warp] = v;
    prep_sync<NW, BAR>();
    float t = (red[0] + red[1]) + (red[2] + red[3]);
#pragma unroll
    for (int i = 4; i < NW; i += 4) t += (red[i] + red[i + 1]) + (red[i + 2] + red[i + 3]);
    prep_sync<NW, BAR>();
    return t;
}

// K-quant weights: int8 codes (16-byte chunks XOR-swizzled per block pair), per-32 sums as two int8 planes
// (sum = 128*hi + lo; per block 16 bytes = [hi of sub-blocks 0..3 | lo 0..3 | hi 4..7 | lo 4..7]) and per-256
// scales, into shared memory. Warp w takes blocks w, w+NW, ...; a lane holds elements 4l..4l+3 and
// 128+4l..128+4l+3 of a block, and all loads of a batch of blocks are issued before the first is used.
// tid = index of the thread among the NW*32 preparing threads.
template <int PREP, int NW, int BAR>
__device__ __forceinline__ void q8k_prep_to_smem(const MatvecIn& in, int cols, int bpr, int8_t* s_q8, void* s_bs_v,
                                                 float* s_d, float* s_red, int warp, int lane, int tid) {
    int8_t* s_bs = (int8_t*) s_bs_v;
    constexpr int NT = NW * 32;
    if (PREP == PREP_QUANTIZED) {
        for (int c = tid; c < (cols >> 4); c += NT) {
            const int blk = c >> 4, ch = c & 15;
            *reinterpret_cast<uint4*>(s_q8 + (size_t) blk * 256 + (ch ^ (((blk >> 1) & 1) << 1)) * 16) = skd::ld_ro(in.q8.q + (size_t) c * 16);
        }
        for (int c = tid; c < (cols >> 5); c += NT) {
            const int sum = (int) __ldg(in.q8.bsums + c), hi = (sum + 64) >> 7, lo = sum - (hi << 7);
            int8_t* dst = s_bs + (size_t) (c >> 3) * 16 + ((c >> 2) & 1) * 8 + (c & 3);
            dst[0] = (int8_t) hi; dst[4] = (int8_t) lo;
        }
        for (int c = tid; c < bpr; c += NT) s_d[c] = __ldg(in.q8.d + c);
        return;
    }
    constexpr int B = 4;     // blocks per warp per batch: 8 float4 loads in flight per lane
    float nscale = 1.0f;
    if (PREP == PREP_NORM_F32) {
        float ss = 0.0f;
        for (int b0 = warp; b0 < bpr; b0 += NW * B) {
            float4 v[2 * B];
#pragma unroll
            for (int j = 0; j < B; ++j) {
                const int blk = b0 + j * NW;
                if (blk < bpr) {
                    v[2 * j] = __ldg(reinterpret_cast<const float4*>(in.x + (size_t) blk * 256) + lane);
                    v[2 * j + 1] = __ldg(reinterpret_cast<const float4*>(in.x + (size_t) blk * 256) + 32 + lane);
                } else { v[2 * j] = make_float4(0, 0, 0, 0); v[2 * j + 1] = v[2 * j]; }
            }
#pragma unroll
            for (int j = 0; j < 2 * B; ++j) ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
        }
        ss = prep_sum<NW, BAR>(ss, s_red, warp, lane);
        nscale = 1.0f / sqrtf(ss * (1.0f / (float) cols) + in.eps);
    }
    for (int b0 = warp; b0 < bpr; b0 += NW * B) {
        float4 v[2 * B], g[2 * B];
#pragma unroll
        for (int j = 0; j < B; ++j) {
            const int blk = b0 + j * NW;
            if (blk < bpr) {
                v[2 * j] = __ldg(reinterpret_cast<const float4*>(in.x + (size_t) blk * 256) + lane);
                v[2 * j + 1] = __ldg(reinterpret_cast<const float4*>(in.x + (size_t) blk * 256) + 32 + lane);
                if (PREP == PREP_NORM_F32) {
                    g[2 * j] = __ldg(reinterpret_cast<const float4*>(in.gamma + (size_t) blk * 256) + lane);
                    g[2 * j + 1] = __ldg(reinterpret_cast<const float4*>(in.gamma + (size_t) blk * 256) + 32 + lane);
                }
                if (PREP == PREP_SWIGLU_F32) {       // the "up" half follows the "gate" half of the row
                    g[2 * j] = __ldg(reinterpret_cast<const float4*>(in.x + cols + (size_t) blk * 256) + lane);
                    g[2 * j + 1] = __ldg(reinterpret_cast<const float4*>(in.x + cols + (size_t) blk * 256) + 32 + lane);
                }
            } else { v[2 * j] = make_float4(0, 0, 0, 0); v[2 * j + 1] = v[2 * j]; g[2 * j] = v[2 * j]; g[2 * j + 1] = v[2 * j]; }
        }
#pragma unroll
        for (int j = 0; j < B; ++j) {
            const int blk = b0 + j * NW;
            if (blk >= bpr) continue;                         // warp-uniform
            float e[8] = {v[2 * j].x, v[2 * j].y, v[2 * j].z, v[2 * j].w, v[2 * j + 1].x, v[2 * j + 1].y, v[2 * j + 1].z, v[2 * j + 1].w};
            if (PREP == PREP_NORM_F32) {
                const float ge[8] = {g[2 * j].x, g[2 * j].y, g[2 * j].z, g[2 * j].w, g[2 * j + 1].x, g[2 * j + 1].y, g[2 * j + 1].z, g[2 * j + 1].w};
#pragma unroll
                for (int i = 0; i < 8; ++i) e[i] = (e[i] * nscale) * ge[i];
            }
            if (PREP == PREP_SWIGLU_F32) {       // the arithmetic of prep_kernel<PK_SWIGLU> (stepops.cu), bit for bit
                const float ue[8] = {g[2 * j].x, g[2 * j].y, g[2 * j].z, g[2 * j].w, g[2 * j + 1].x, g[2 * j + 1].y, g[2 * j + 1].z, g[2 * j + 1].w};
#pragma unroll
                for (int i = 0; i < 8; ++i) e[i] = (e[i] * (1.0f / (1.0f + expf(-e[i])))) * ue[i];
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
                int8_t* bd = s_bs + (size_t) blk * 16 + (lane >> 3);
                const int h0 = (s0 + 64) >> 7, h1 = (s1 + 64) >> 7;
                bd[0] = (int8_t) h0; bd[4] = (int8_t) (s0 - (h0 << 7));
                bd[8] = (int8_t) h1; bd[12] = (int8_t) (s1 - (h1 << 7));
            }
            if (lane == 0) s_d[blk] = amax > 0.0f ? amax / 127.0f : 0.0f;
        }
    }
}

// Q8_0 weights: the fp32 row as hi*128+lo int8 planes with one scale per 32 elements.
template <int PREP, int NW, int BAR>
__device__ __forceinline__ void split_prep_to_smem(const MatvecIn& in, int cols, int bpr, int8_t* s_hi, int8_t* s_lo,
                                                   float* s_dx, float* s_red, int warp, int lane, int tid) {
    constexpr int NT = NW * 32;
    if (PREP == PREP_QUANTIZED) {
        for (int c = tid; c < (cols >> 4); c += NT) {
            *reinterpret_cast<uint4*>(s_hi + (size_t) c * 16) = skd::ld_ro(in.split.hi + (size_t) c * 16);
            *reinterpret_cast<uint4*>(s_lo + (size_t) c * 16) = skd::ld_ro(in.split.lo + (size_t) c * 16);
        }
        for (int c = tid; c < bpr; c += NT) s_dx[c] = __ldg(in.split.d + c);
        return;
    }
    constexpr int B = 8;     // float4 loads in flight per thread
    const int n4 = cols >> 2;
    float nscale = 1.0f;
    if (PREP == PREP_NORM_F32) {
        float ss = 0.0f;
        for (int i0 = tid; i0 < n4; i0 += NT * B) {
            float4 v[B];
#pragma unroll
            for (int j = 0; j < B; ++j) {
                const int i = i0 + j * NT;
                v[j] = i < n4 ? __ldg(reinterpret_cast<const float4*>(in.x) + i) : make_float4(0, 0, 0, 0);
            }
#pragma unroll
            for (int j = 0; j < B; ++j) ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
        }
        ss = prep_sum<NW, BAR>(ss, s_red, warp, lane);
        nscale = 1.0f / sqrtf(ss * (1.0f / (float) cols) + in.eps);
    }
    // thread t holds float4 chunk i = t + NT*j; a 32-block is eight consecutive chunks = eight lanes
    const int n4_pad = (n4 + NT - 1) / NT * NT;   // keep whole warps in the shuffles
    for (int i0 = tid; i0 < n4_pad; i0 += NT * B) {
        float4 v[B], g[B];
#pragma unroll
        for (int j = 0; j < B; ++j) {
            const int i = i0 + j * NT;
            const bool ok = i < n4;
            v[j] = ok ? __ldg(reinterpret_cast<const float4*>(in.x) + i) : make_float4(0, 0, 0, 0);
            if (PREP == PREP_NORM_F32) g[j] = ok ? __ldg(reinterpret_cast<const float4*>(in.gamma) + i) : make_float4(0, 0, 0, 0);
        }
#pragma unroll
        for (int j = 0; j < B; ++j) {
            const int i = i0 + j * NT;
            if (i - tid >= n4_pad) continue;                // uniform over the preparing threads
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

}  // namespace sk
#endif
