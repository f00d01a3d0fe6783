// Activation quantizers shared by the stand-alone quantize kernels and by kernels that fuse the
// quantization into their epilogue (RMSNorm, SwiGLU, attention merge).
#pragma once
#include "common.cuh"

namespace sk {

// int8 activation, one scale per 256 elements, plus per-32 sums of the codes (for the mins term).
// Follows skainet_q8_quantize_block, native/src/q4k_matmul.c:74-92.
struct ActQ8K {
    int8_t* q;        // [m][cols]
    float* d;         // [m][cols/256]   d_in = maxabs / 127
    int16_t* bsums;   // [m][cols/32]    sum of the 32 codes of each sub-block
};
// fp32 activation carried as hi*128 + lo with one scale per 32 elements (15-bit two-term split).
struct ActSplit {
    int8_t* hi;       // [m][cols]
    int8_t* lo;       // [m][cols]
    float* d;         // [m][cols/32]    amax / 16256
};
ActQ8K act_q8k_layout(void* scratch, int m, int cols);
// attention.cu
int32_t launch_attn_decode_quant(const float* q, int64_t q_row_stride, const __half* k, const __half* v, float* out, int batch,
                                 int heads, int kv_heads, int d, int64_t cache_stride, const int32_t* kv_len, int max_kv_len,
                                 float scale, int window, void* scratch, bool split, ActQ8K oq, ActSplit os, cudaStream_t s);
ActSplit act_split_layout(void* scratch, int m, int cols);
// attention.cu: the attention of one decode step (rope and cache append inside the split-K kernel, then merge + quantizer)
int32_t launch_attn_step(const float* qkv, __half* k, __half* v, float* out, int batch, int heads, int kv_heads, int d,
                         int64_t cache_stride, const int32_t* kv_len, int max_kv_len, float scale, int window, const float* cos_t,
                         const float* sin_t, int rope_mode, void* scratch, bool split, ActQ8K oq, ActSplit os, cudaStream_t s);

}  // namespace sk

#ifdef __CUDACC__
namespace skd {

// One warp quantizes eight values per lane (lane L holds elements 8L..8L+7 of the 256-block).
// d_in = maxabs/127, q = clamp(rint(x * (127/maxabs)), +-127); an all-zero block gives d_in = 0.
__device__ __forceinline__ void quant_q8k_regs(const float (&v)[8], int8_t* q_out, float* d_out, int16_t* bsums_out, int lane) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = warp_max(amax);
    const float inv = amax > 0.0f ? 127.0f / amax : 0.0f;
    int sum = 0;
    uint32_t p0 = 0, p1 = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int q = __float2int_rn(v[i] * inv);
        q = max(-127, min(127, q));
        sum += q;
        if (i < 4) p0 |= (uint32_t) (q & 0xff) << (8 * i); else p1 |= (uint32_t) (q & 0xff) << (8 * (i - 4));
    }
    *reinterpret_cast<uint2*>(q_out + lane * 8) = make_uint2(p0, p1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if ((lane & 3) == 0) bsums_out[lane >> 2] = (int16_t) sum;
    if (lane == 0) *d_out = amax > 0.0f ? amax / 127.0f : 0.0f;
}
__device__ __forceinline__ void quant_q8k_block(const float* x, int8_t* q_out, float* d_out, int16_t* bsums_out, int lane) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(x) + lane * 2);
    const float4 b = __ldg(reinterpret_cast<const float4*>(x) + lane * 2 + 1);
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    quant_q8k_regs(v, q_out, d_out, bsums_out, lane);
}

// Four lanes quantize one 32-element block (lane part p holds elements 8p..8p+7).
// q = rint(x * 16256/amax) in [-16256, 16256]; hi = floor((q+64)/128) in [-127,127]; lo = q-128*hi in [-64,63].
__device__ __forceinline__ void quant_split_regs(const float (&v)[8], sk::ActSplit a, int64_t blk, int part, bool live) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const float inv = amax > 0.0f ? 16256.0f / amax : 0.0f;
    uint32_t h0 = 0, h1 = 0, l0 = 0, l1 = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int q = __float2int_rn(v[i] * inv);
        q = max(-16256, min(16256, q));
        const int hi = (q + 64) >> 7;
        const int lo = q - (hi << 7);
        if (i < 4) { h0 |= (uint32_t) (hi & 0xff) << (8 * i); l0 |= (uint32_t) (lo & 0xff) << (8 * i); }
        else { h1 |= (uint32_t) (hi & 0xff) << (8 * (i - 4)); l1 |= (uint32_t) (lo & 0xff) << (8 * (i - 4)); }
    }
    if (live) {
        *reinterpret_cast<uint2*>(a.hi + blk * 32 + part * 8) = make_uint2(h0, h1);
        *reinterpret_cast<uint2*>(a.lo + blk * 32 + part * 8) = make_uint2(l0, l1);
        if (part == 0) a.d[blk] = amax > 0.0f ? amax / 16256.0f : 0.0f;
    }
}
__device__ __forceinline__ void quant_split_block(const float* x, sk::ActSplit a, int64_t blk, int part, bool live) {
    const float4 p = __ldg(reinterpret_cast<const float4*>(x + blk * 32 + part * 8));
    const float4 q = __ldg(reinterpret_cast<const float4*>(x + blk * 32 + part * 8) + 1);
    const float v[8] = {p.x, p.y, p.z, p.w, q.x, q.y, q.z, q.w};
    quant_split_regs(v, a, blk, part, live);
}

}  // namespace skd
#endif
