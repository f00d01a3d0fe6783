// Attention kernels.
//
//  * attn_decode: GQA decode attention (one query row per head) streaming an f16 KV cache, split over
//    the key axis (flash-decoding): each CTA reads its keys once for all query heads of a KV head,
//    keeps an fp32 online softmax, and a second small kernel merges the splits in a fixed order.
//    HBM-bound: bytes = 2 * kv_len * head_dim * 2 per (batch, kv head).
//  * sdpa_rows: the general contract of the reference kernel — any seq_q, causal / sliding window /
//    right context / key lengths / dense additive mask — one CTA per query row, K/V in fp32 or f16.
//
// Semantics follow native/src/f32_fused.c:304-360 (key range :313-324, masked score -1e30 :92,
// max-subtracted exp and divide-by-sum :194-218, fully masked row -> uniform :347-351) and
// skainet-lang/skainet-lang-core/src/commonMain/kotlin/sk/ainet/lang/tensor/ops/AttentionMask.kt:57-78.
#include "common.cuh"
#include "actquant.cuh"
#include "tma.cuh"

#include <mutex>

namespace sk {

constexpr float MASKED = -1.0e30f;

// =================================================================================================
// Decode attention, split-K.
// =================================================================================================
constexpr int AD_THREADS = 128;          // 4 warps = 8 half-warp workers
constexpr int AD_WORKERS = AD_THREADS / 16;
constexpr int AD_TK = 4;                 // keys per worker per step (loads in flight: 2*AD_TK x 16 B per lane)

__device__ __forceinline__ float half16_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 8);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v;
}
__device__ __forceinline__ void unpack8(const uint4& r, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}

// partial record per (batch, head, split): [m, l, acc[D]]
template <int D, int G>
__global__ void __launch_bounds__(AD_THREADS)
attn_decode_kernel(const float* __restrict__ q, const __half* __restrict__ kc, const __half* __restrict__ vc,
                   float* __restrict__ out, float* __restrict__ part, int heads, int kv_heads, int64_t cache_stride,
                   const int32_t* __restrict__ kv_len, float scale, int window, int chunk, int splits,
                   int64_t q_row_stride, int always_partials) {
    static_assert(D == 128 || D == 64, "head_dim");
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    constexpr int LPK = D / 8;            // lanes per key (16 B = 8 halves per lane)
    constexpr int KPW = 32 / LPK;         // keys per warp-load
    constexpr int NW = AD_THREADS / LPK;  // workers in the CTA
    __shared__ float sm_m[NW][G], sm_l[NW][G];
    __shared__ float sm_acc[NW][G][D];

    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int worker = threadIdx.x / LPK, wl = threadIdx.x % LPK;
    const int len = kv_len[b];
    int first = 0, end = len;
    if (window > 0 && len - window > first) first = len - window;
    const int begin = max(first, split * chunk), stop = min(end, (split + 1) * chunk);

    float qr[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const float* qp = q + (int64_t) b * q_row_stride + (int64_t) (kvh * G + g) * D + wl * 8;
        const float4 a = __ldg((const float4*) qp), c = __ldg((const float4*) qp + 1);
        qr[g][0] = a.x; qr[g][1] = a.y; qr[g][2] = a.z; qr[g][3] = a.w;
        qr[g][4] = c.x; qr[g][5] = c.y; qr[g][6] = c.z; qr[g][7] = c.w;
    }
    float m[G], l[G], acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = MASKED; l[g] = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] = 0.0f;
    }
    const __half* kb = kc + ((int64_t) b * kv_heads + kvh) * cache_stride * D + wl * 8;
    const __half* vb = vc + ((int64_t) b * kv_heads + kvh) * cache_stride * D + wl * 8;

    // Workers of one warp walk in lock-step (shuffles are warp-wide), so the loop bound is per warp.
    const int warp_first_worker = (threadIdx.x >> 5) * KPW;
    for (int k0 = begin + warp_first_worker * AD_TK; k0 < stop; k0 += NW * AD_TK) {
        const int kmine = k0 + (worker - warp_first_worker) * AD_TK;
        uint4 kr[AD_TK], vr[AD_TK];
#pragma unroll
        for (int t = 0; t < AD_TK; ++t) {
            const int key = kmine + t;
            if (key < stop) {
                kr[t] = skd::ld_stream(kb + (int64_t) key * D);
                vr[t] = skd::ld_stream(vb + (int64_t) key * D);
            } else { kr[t] = make_uint4(0, 0, 0, 0); vr[t] = make_uint4(0, 0, 0, 0); }
        }
        float s[AD_TK][G];
#pragma unroll
        for (int t = 0; t < AD_TK; ++t) {
            float kf[8]; unpack8(kr[t], kf);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float p = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) p += qr[g][i] * kf[i];
                if (LPK == 16) p = half16_sum(p);
                else { p += __shfl_xor_sync(~0u, p, 4); p += __shfl_xor_sync(~0u, p, 2); p += __shfl_xor_sync(~0u, p, 1); }
                s[t][g] = (kmine + t < stop) ? p * scale : MASKED;
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float mx = m[g];
#pragma unroll
            for (int t = 0; t < AD_TK; ++t) mx = fmaxf(mx, s[t][g]);
            const float corr = expf(m[g] - mx);
            m[g] = mx;
            l[g] *= corr;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[g][i] *= corr;
#pragma unroll
            for (int t = 0; t < AD_TK; ++t) s[t][g] = (kmine + t < stop) ? expf(s[t][g] - mx) : 0.0f;
        }
#pragma unroll
        for (int t = 0; t < AD_TK; ++t) {
            float vf[8]; unpack8(vr[t], vf);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                l[g] += s[t][g];
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[g][i] += s[t][g] * vf[i];
            }
        }
    }
    // merge the CTA's workers (fixed order)
#pragma unroll
    for (int g = 0; g < G; ++g) {
        if (wl == 0) { sm_m[worker][g] = m[g]; sm_l[worker][g] = l[g]; }
#pragma unroll
        for (int i = 0; i < 8; ++i) sm_acc[worker][g][wl * 8 + i] = acc[g][i];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * D; idx += AD_THREADS) {
        const int g = idx / D, dd = idx % D;
        float mx = MASKED;
        for (int w = 0; w < NW; ++w) mx = fmaxf(mx, sm_m[w][g]);
        float lt = 0.0f, at = 0.0f;
        for (int w = 0; w < NW; ++w) {
            const float c = expf(sm_m[w][g] - mx);
            lt += c * sm_l[w][g];
            at += c * sm_acc[w][g][dd];
        }
        const int head = kvh * G + g;
        if (splits == 1 && !always_partials) {
            out[((int64_t) b * heads + head) * D + dd] = lt > 0.0f ? at / lt : 0.0f;
        } else {
            float* rec = part + (((int64_t) b * heads + head) * splits + split) * (D + 2);
            rec[2 + dd] = at;
            if (dd == 0) { rec[0] = mx; rec[1] = lt; }
        }
    }
}

template <int D>
__global__ void attn_merge_kernel(const float* __restrict__ part, float* __restrict__ out, int splits) {
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    const int64_t bh = blockIdx.x;
    const float* rec = part + bh * splits * (D + 2);
    float mx = MASKED;
    for (int s = 0; s < splits; ++s) mx = fmaxf(mx, rec[s * (D + 2)]);
    for (int dd = threadIdx.x; dd < D; dd += blockDim.x) {
        float lt = 0.0f, at = 0.0f;
        for (int s = 0; s < splits; ++s) {
            const float c = expf(rec[s * (D + 2)] - mx);
            lt += c * rec[s * (D + 2) + 1];
            at += c * rec[s * (D + 2) + 2 + dd];
        }
        out[bh * D + dd] = lt > 0.0f ? at / lt : 0.0f;
    }
}

static int decode_splits(int batch, int kv_heads, int max_kv_len) {
    const int ctas = batch * kv_heads;
    int want = (sm_count() * 4 + ctas - 1) / ctas;            // ~4 CTAs of 128 threads per SM
    const int by_len = (max_kv_len + 127) / 128;              // at least 128 keys per split
    want = std::max(1, std::min(want, by_len));
    return std::min(want, 256);
}

size_t attn_scratch_bytes(int batch, int heads, int head_dim, int max_kv_len) {
    // kv_heads is not known here; the bound below holds for any grouping (splits <= 256).
    const int splits = std::min(256, std::max(1, (max_kv_len + 127) / 128));
    return (size_t) batch * heads * splits * (head_dim + 2) * sizeof(float);
}

// Merge of the key splits fused with the activation quantizer of the projection that follows: one CTA
// per 256 consecutive outputs of a row (two 128-wide heads or four 64-wide ones), fp32 result kept as
// well. grid (heads*D/256, batch), 256 threads.
template <int D, bool SPLIT>
__global__ void __launch_bounds__(256)
attn_merge_quant_kernel(const float* __restrict__ part, float* __restrict__ out, int splits, int heads, ActQ8K oq, ActSplit os) {
    __shared__ float red[8];
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    const int b = blockIdx.y, e = blockIdx.x * 256 + threadIdx.x, n = heads * D;
    const int head = e / D, dd = e % D, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* rec = part + ((int64_t) b * heads + head) * splits * (D + 2);
    float mx = MASKED;
    for (int s = 0; s < splits; ++s) mx = fmaxf(mx, rec[s * (D + 2)]);
    float lt = 0.0f, at = 0.0f;
    for (int s = 0; s < splits; ++s) {
        const float c = expf(rec[s * (D + 2)] - mx);
        lt += c * rec[s * (D + 2) + 1];
        at += c * rec[s * (D + 2) + 2 + dd];
    }
    const float v = lt > 0.0f ? at / lt : 0.0f;
    out[(int64_t) b * n + e] = v;
    if (SPLIT) {                 // one scale per 32 values = per warp
        const float amax = skd::warp_max(fabsf(v));
        const float inv = amax > 0.0f ? 16256.0f / amax : 0.0f;
        const int q = max(-16256, min(16256, __float2int_rn(v * inv)));
        const int hi = (q + 64) >> 7, lo = q - (hi << 7);
        os.hi[(int64_t) b * n + e] = (int8_t) hi; os.lo[(int64_t) b * n + e] = (int8_t) lo;
        if (lane == 0) os.d[((int64_t) b * n + e) >> 5] = amax > 0.0f ? amax / 16256.0f : 0.0f;
    } else {                     // one scale per 256 values = per CTA, code sums per warp
        float amax = skd::warp_max(fabsf(v));
        if (lane == 0) red[warp] = amax;
        __syncthreads();
        amax = fmaxf(fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3])), fmaxf(fmaxf(red[4], red[5]), fmaxf(red[6], red[7])));
        const float inv = amax > 0.0f ? 127.0f / amax : 0.0f;
        const int q = max(-127, min(127, __float2int_rn(v * inv)));
        oq.q[(int64_t) b * n + e] = (int8_t) q;
        int sum = q;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) oq.bsums[((int64_t) b * n + e) >> 5] = (int16_t) sum;
        if (threadIdx.x == 0) oq.d[((int64_t) b * n + e) >> 8] = amax > 0.0f ? amax / 127.0f : 0.0f;
    }
}

template <int D, int G>
static void launch_decode_dg(const float* q, const __half* k, const __half* v, float* out, float* part, int batch,
                             int heads, int kv_heads, int64_t cache_stride, const int32_t* kv_len, float scale,
                             int window, int chunk, int splits, int64_t q_row_stride, int always_partials, cudaStream_t s) {
    dim3 grid(splits, kv_heads, batch);
    launch_pdl(attn_decode_kernel<D, G>, grid, dim3(AD_THREADS), 0, s, q, k, v, out, part, heads, kv_heads, cache_stride, kv_len,
               scale, window, chunk, splits, q_row_stride, always_partials);
    if (splits > 1 && !always_partials) launch_pdl(attn_merge_kernel<D>, dim3(batch * heads), dim3(D), 0, s, (const float*) part, out, splits);
}

static int32_t attn_decode_impl(const float* q, int64_t q_row_stride, const __half* k, const __half* v, float* out, int batch, int heads,
                                int kv_heads, int d, int64_t cache_stride, const int32_t* kv_len, int max_kv_len,
                                float scale, int window, void* scratch, int always_partials, int* splits_out, cudaStream_t s);

int32_t launch_attn_decode(const float* q, const __half* k, const __half* v, float* out, int batch, int heads,
                           int kv_heads, int d, int64_t cache_stride, const int32_t* kv_len, int max_kv_len,
                           float scale, int window, void* scratch, cudaStream_t s) {
    return attn_decode_impl(q, (int64_t) heads * d, k, v, out, batch, heads, kv_heads, d, cache_stride, kv_len, max_kv_len, scale, window,
                            scratch, 0, nullptr, s);
}

// Decode attention whose result is also quantized for the projection that follows (q8 per 256 for
// K-quant weights, two-term split for Q8_0): split-K kernel, then one merge+quantize kernel. q rows may
// be strided (read straight out of a merged q|k|v buffer). heads*d must be a multiple of 256.
int32_t launch_attn_decode_quant(const float* q, int64_t q_row_stride, const __half* k, const __half* v, float* out, int batch,
                                 int heads, int kv_heads, int d, int64_t cache_stride, const int32_t* kv_len, int max_kv_len,
                                 float scale, int window, void* scratch, bool split, ActQ8K oq, ActSplit os, cudaStream_t s) {
    if (batch <= 0 || heads <= 0) return SKAINET_CUDA_OK;
    if ((heads * d) % 256 != 0) { set_error("attn_decode_quant: heads*head_dim %d is not a multiple of 256", heads * d); return SKAINET_CUDA_ERR_INVALID; }
    int splits = 1;
    SK_TRY(attn_decode_impl(q, q_row_stride, k, v, out, batch, heads, kv_heads, d, cache_stride, kv_len, max_kv_len, scale, window, scratch, 1, &splits, s));
    dim3 grid(heads * d / 256, batch);
    if (d == 128) {
        if (split) SK_CUDA(launch_pdl(attn_merge_quant_kernel<128, true>, grid, dim3(256), 0, s, (const float*) scratch, out, splits, heads, oq, os));
        else SK_CUDA(launch_pdl(attn_merge_quant_kernel<128, false>, grid, dim3(256), 0, s, (const float*) scratch, out, splits, heads, oq, os));
    } else {
        if (split) SK_CUDA(launch_pdl(attn_merge_quant_kernel<64, true>, grid, dim3(256), 0, s, (const float*) scratch, out, splits, heads, oq, os));
        else SK_CUDA(launch_pdl(attn_merge_quant_kernel<64, false>, grid, dim3(256), 0, s, (const float*) scratch, out, splits, heads, oq, os));
    }
    return SKAINET_CUDA_OK;
}

static int32_t attn_decode_impl(const float* q, int64_t q_row_stride, const __half* k, const __half* v, float* out, int batch, int heads,
                                int kv_heads, int d, int64_t cache_stride, const int32_t* kv_len, int max_kv_len,
                                float scale, int window, void* scratch, int always_partials, int* splits_out, cudaStream_t s) {
    if (batch <= 0 || heads <= 0) return SKAINET_CUDA_OK;
    const int G = heads / kv_heads;
    const int splits = decode_splits(batch, kv_heads, std::max(1, max_kv_len));
    int chunk = (std::max(1, max_kv_len) + splits - 1) / splits;
    chunk = (chunk + 31) & ~31;
    float* part = (float*) scratch;
    if (splits_out) *splits_out = splits;
#define SK_AD(DD, GG) launch_decode_dg<DD, GG>(q, k, v, out, part, batch, heads, kv_heads, cache_stride, kv_len, scale, window, chunk, splits, q_row_stride, always_partials, s)
    if (d == 128) {
        switch (G) { case 1: SK_AD(128, 1); break; case 2: SK_AD(128, 2); break; case 4: SK_AD(128, 4); break; case 8: SK_AD(128, 8); break;
            default: set_error("attn_decode: heads/kv_heads = %d not in {1,2,4,8}", G); return SKAINET_CUDA_ERR_INVALID; }
    } else if (d == 64) {
        switch (G) { case 1: SK_AD(64, 1); break; case 2: SK_AD(64, 2); break; case 4: SK_AD(64, 4); break; case 8: SK_AD(64, 8); break;
            default: set_error("attn_decode: heads/kv_heads = %d not in {1,2,4,8}", G); return SKAINET_CUDA_ERR_INVALID; }
    } else { set_error("attn_decode: head_dim %d not in {64,128}", d); return SKAINET_CUDA_ERR_INVALID; }
#undef SK_AD
    SK_CUDA(cudaGetLastError());
    return SKAINET_CUDA_OK;
}

// =================================================================================================
// General SDPA: one CTA (4 warps) per query row; warps take keys round-robin, lanes split head_dim.
// =================================================================================================
__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__half v) { return __half2float(v); }

template <typename KV, int E>   // E = head_dim / 32 elements per lane
__global__ void __launch_bounds__(128)
sdpa_rows_kernel(const float* __restrict__ q, const KV* __restrict__ k, const KV* __restrict__ v, float* __restrict__ out,
                 int heads, int kv_heads, int seq_q, int seq_kv, int64_t kv_stride, float scale, int causal, int window,
                 int right_context, const int32_t* __restrict__ lengths, const int32_t* __restrict__ q_abs_base,
                 const float* __restrict__ mask, int mb, int mh, int mq, int mk, int token_major) {
    constexpr int D = E * 32;
    __shared__ float sm_m[4], sm_l[4], sm_acc[4][D];
    const int64_t row = blockIdx.x;
    const int qi = (int) (row % seq_q);
    const int h = (int) ((row / seq_q) % heads);
    const int b = (int) (row / ((int64_t) seq_q * heads));
    const int kvh = h / (heads / kv_heads);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // q/out are [batch, heads, seq_q, D] (the reference contract) or, token-major, [batch, seq_q, heads, D]
    const int64_t qrow = token_major ? ((int64_t) b * seq_q + qi) * heads + h : row;

    // key range under the structural rules
    const int abs_q = q_abs_base ? q_abs_base[b] + qi : seq_kv - seq_q + qi;
    int first = 0, end = seq_kv;
    if (window > 0) { first = max(first, abs_q - window + 1); end = min(end, abs_q + right_context + 1); }
    if (causal && abs_q + 1 < end) end = abs_q + 1;
    if (lengths && lengths[b] < end) end = lengths[b];
    if (end < 0) end = 0;
    if (first > end) first = end;
    int pf = first, pe = end;
    if (mask != nullptr || first >= end) { pf = 0; pe = seq_kv; }
    const float* mrow = nullptr;
    if (mask) {
        const int bi = mb == 1 ? 0 : b;
        const int hi = mh == 1 ? 0 : (mh == heads ? h : kvh);
        mrow = mask + (((int64_t) bi * mh + hi) * mq + (mq == 1 ? 0 : qi)) * mk;
    }
    float qr[E];
#pragma unroll
    for (int e = 0; e < E; ++e) qr[e] = q[qrow * D + lane + 32 * e];
    const KV* kb = k + ((int64_t) b * kv_heads + kvh) * kv_stride * D;
    const KV* vb = v + ((int64_t) b * kv_heads + kvh) * kv_stride * D;

    float m = MASKED * 2.0f, l = 0.0f, acc[E];
#pragma unroll
    for (int e = 0; e < E; ++e) acc[e] = 0.0f;
    for (int ki = pf + warp; ki < pe; ki += 4) {
        float s;
        if (ki >= first && ki < end) {
            float p = 0.0f;
#pragma unroll
            for (int e = 0; e < E; ++e) p += qr[e] * to_f(kb[(int64_t) ki * D + lane + 32 * e]);
            s = skd::warp_sum(p) * scale;
        } else s = MASKED;
        if (mrow) s += mk == 1 ? mrow[0] : mrow[ki];
        const float mx = fmaxf(m, s);
        const float corr = expf(m - mx), p = expf(s - mx);
        m = mx;
        l = l * corr + p;
#pragma unroll
        for (int e = 0; e < E; ++e) acc[e] = acc[e] * corr + p * to_f(vb[(int64_t) ki * D + lane + 32 * e]);
    }
    if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
    for (int e = 0; e < E; ++e) sm_acc[warp][lane + 32 * e] = acc[e];
    __syncthreads();
    for (int dd = threadIdx.x; dd < D; dd += 128) {
        float mx = sm_m[0];
        for (int w = 1; w < 4; ++w) mx = fmaxf(mx, sm_m[w]);
        float lt = 0.0f, at = 0.0f;
        for (int w = 0; w < 4; ++w) { const float c = expf(sm_m[w] - mx); lt += c * sm_l[w]; at += c * sm_acc[w][dd]; }
        out[qrow * D + dd] = lt > 0.0f ? at / lt : 0.0f;
    }
}

template <typename KV>
static int32_t launch_sdpa_t(const float* q, const KV* k, const KV* v, float* out, int batch, int heads, int kv_heads,
                             int seq_q, int seq_kv, int64_t kv_stride, int d, float scale, int causal, int window,
                             int right_context, const int32_t* lengths, const int32_t* q_abs_base, const float* mask,
                             int mb, int mh, int mq, int mk, int token_major, cudaStream_t s) {
    const int64_t rows = (int64_t) batch * heads * seq_q;
    if (rows <= 0) return SKAINET_CUDA_OK;
    if (rows > 0x7fffffff) { set_error("sdpa: too many query rows"); return SKAINET_CUDA_ERR_INVALID; }
#define SK_SD(E) sdpa_rows_kernel<KV, E><<<(unsigned) rows, 128, 0, s>>>(q, k, v, out, heads, kv_heads, seq_q, seq_kv, kv_stride, scale, causal, window, right_context, lengths, q_abs_base, mask, mb, mh, mq, mk, token_major)
    switch (d) {
        case 32: SK_SD(1); break;
        case 64: SK_SD(2); break;
        case 128: SK_SD(4); break;
        case 256: SK_SD(8); break;
        default: set_error("sdpa: head_dim %d not in {32,64,128,256}", d); return SKAINET_CUDA_ERR_INVALID;
    }
#undef SK_SD
    SK_CUDA(cudaGetLastError());
    return SKAINET_CUDA_OK;
}

int32_t launch_sdpa_f32(const float* q, const float* k, const float* v, float* out, int batch, int heads, int kv_heads,
                        int seq_q, int seq_kv, int d, float scale, int causal, int window, int right_context,
                        const int32_t* lengths, const float* mask, int mb, int mh, int mq, int mk, cudaStream_t s) {
    return launch_sdpa_t<float>(q, k, v, out, batch, heads, kv_heads, seq_q, seq_kv, seq_kv, d, scale, causal, window,
                                right_context, lengths, nullptr, mask, mb, mh, mq, mk, 0, s);
}

// Causal attention of a block of new queries over an f16 cache (prefill): query qi of batch b sits at
// absolute position q_abs_base[b] + qi and sees keys [0, that position]. q/out are token-major
// [batch, seq_q, heads, D], the layout the projections produce.
int32_t launch_sdpa_cache(const float* q, const __half* k, const __half* v, float* out, int batch, int heads,
                          int kv_heads, int seq_q, int seq_kv, int64_t cache_stride, int d, float scale, int window,
                          const int32_t* q_abs_base, cudaStream_t s) {
    return launch_sdpa_t<__half>(q, k, v, out, batch, heads, kv_heads, seq_q, seq_kv, cache_stride, d, scale, 1, window,
                                 0, nullptr, q_abs_base, nullptr, 0, 0, 0, 0, 1, s);
}

// =================================================================================================
// Decode attention without any allocation: the split-K partials live in a fixed device array.
// =================================================================================================
// Capacity of the built-in partials area, in floats (4 MiB). Every GPU that loads the library holds it
// until the process exits.
constexpr size_t ATTN_STATIC_FLOATS = (size_t) 1 << 20;
static __device__ __align__(256) float g_attn_static_partials[ATTN_STATIC_FLOATS];

// The array's name is only a host-side stand-in; the address kernels may use comes from the runtime,
// once per device, with that device current.
static float* g_attn_static_ptr[64] = {nullptr};
static std::mutex g_attn_static_mu;

static int32_t attn_static_partials(float** out) {
    int dev = 0;
    SK_CUDA(cudaGetDevice(&dev));
    SK_REQUIRE(dev >= 0 && dev < 64, "attn_decode_noalloc: device ordinal %d not supported", dev);
    std::lock_guard<std::mutex> lk(g_attn_static_mu);
    if (!g_attn_static_ptr[dev]) {
        float* p = nullptr;
        SK_CUDA(cudaGetSymbolAddress((void**) &p, g_attn_static_partials));
        g_attn_static_ptr[dev] = p;
    }
    *out = g_attn_static_ptr[dev];
    return SKAINET_CUDA_OK;
}

}  // namespace sk

extern "C" int32_t skainet_cuda_attn_decode_noalloc_dev(const float* q, const uint16_t* k_cache, const uint16_t* v_cache, float* out,
                                                        int32_t batch, int32_t heads, int32_t kv_heads, int32_t head_dim,
                                                        int64_t cache_stride, const int32_t* kv_len_dev, int32_t max_kv_len,
                                                        float scale, int32_t window, skainet_stream_t stream) {
    using namespace sk;
    if (batch <= 0 || heads <= 0) return SKAINET_CUDA_OK;
    SK_REQUIRE(kv_heads > 0 && heads % kv_heads == 0, "attn_decode_noalloc: heads %d not a multiple of kv_heads %d", heads, kv_heads);
    SK_REQUIRE(head_dim == 64 || head_dim == 128, "attn_decode_noalloc: head_dim %d not in {64,128}", head_dim);
    SK_REQUIRE(max_kv_len >= 0 && cache_stride >= max_kv_len, "attn_decode_noalloc: cache_stride %lld < max_kv_len %d", (long long) cache_stride, max_kv_len);
    SK_REQUIRE(q && k_cache && v_cache && out && kv_len_dev, "attn_decode_noalloc: null pointer");
    SK_REQUIRE((((uintptr_t) q | (uintptr_t) k_cache | (uintptr_t) v_cache) & 15) == 0, "attn_decode_noalloc: q/k/v must be 16-byte aligned");
    SK_TRY(ensure_device());
    const int splits = decode_splits(batch, kv_heads, std::max(1, max_kv_len));
    const size_t need = (size_t) batch * heads * splits * (head_dim + 2);
    SK_REQUIRE(need <= ATTN_STATIC_FLOATS,
               "attn_decode_noalloc: batch %d x heads %d x %d key splits needs %zu floats of partials, the built-in area holds %zu; "
               "use skainet_cuda_attn_decode_dev for this size", batch, heads, splits, need, (size_t) ATTN_STATIC_FLOATS);
    float* partials = nullptr;
    SK_TRY(attn_static_partials(&partials));
    return launch_attn_decode(q, (const __half*) k_cache, (const __half*) v_cache, out, batch, heads, kv_heads, head_dim, cache_stride,
                              kv_len_dev, max_kv_len, scale, window, partials, as_stream(stream));
}
