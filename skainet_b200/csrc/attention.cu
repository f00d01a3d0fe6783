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

#include <cstdlib>
#include <cstring>
#include <mutex>

namespace sk {

constexpr float MASKED = -1.0e30f;

// =================================================================================================
// Decode attention, split-K: merge of the partial records.
// =================================================================================================
// Merge of split-K partial records {max, sum, acc[D]}: thread (group, element) folds the splits
// group, group+MG, .. in chunks of eight whose loads are all issued before the first use (one memory
// round trip per chunk), then the MG groups are folded in a fixed order through shared memory. Returns
// the merged output element to the threads of group 0; the other groups get 0.
constexpr int MG = 4;          // split groups per CTA
template <int D, int E>        // E = elements per CTA
__device__ __forceinline__ float merge_splits(const float* __restrict__ rec, int splits, int dd, int e, int grp, float (*sm)[MG][E]) {
    float mx = MASKED, lt = 0.0f, at = 0.0f;
    for (int s0 = grp * 8; s0 < splits; s0 += MG * 8) {
        float mm[8], ll[8], aa[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const bool live = s0 + i < splits;
            const float* r = rec + (int64_t) (s0 + i) * (D + 2);
            mm[i] = live ? __ldg(r) : MASKED;
            ll[i] = live ? __ldg(r + 1) : 0.0f;
            aa[i] = live ? __ldg(r + 2 + dd) : 0.0f;
        }
        float cm = mx;
#pragma unroll
        for (int i = 0; i < 8; ++i) cm = fmaxf(cm, mm[i]);
        const float c0 = expf(mx - cm);
        lt *= c0; at *= c0; mx = cm;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float c = expf(mm[i] - cm);
            lt += c * ll[i];
            at += c * aa[i];
        }
    }
    sm[0][grp][e] = mx; sm[1][grp][e] = lt; sm[2][grp][e] = at;
    __syncthreads();
    if (grp != 0) return 0.0f;
    float m2 = mx;
#pragma unroll
    for (int g2 = 1; g2 < MG; ++g2) m2 = fmaxf(m2, sm[0][g2][e]);
    float l2 = 0.0f, a2 = 0.0f;
#pragma unroll
    for (int g2 = 0; g2 < MG; ++g2) {
        const float c = expf(sm[0][g2][e] - m2);
        l2 += c * sm[1][g2][e];
        a2 += c * sm[2][g2][e];
    }
    return l2 > 0.0f ? a2 / l2 : 0.0f;
}

// grid batch*heads, D*MG threads
template <int D>
__global__ void __launch_bounds__(D * MG) attn_merge_kernel(const float* __restrict__ part, float* __restrict__ out, int splits) {
    __shared__ float sm[3][MG][D];
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    const int64_t bh = blockIdx.x;
    const int dd = threadIdx.x % D, grp = threadIdx.x / D;
    const float v = merge_splits<D, D>(part + bh * splits * (D + 2), splits, dd, dd, grp, sm);
    if (grp == 0) out[bh * D + dd] = v;
}

// =================================================================================================
// Decode attention on the tensor cores (mma.sync m16n8k16, f16 x f16 -> f32): the kernel used for every
// group size. Scores and P.V are small contractions (heads x dims x keys) whose operands are the f16
// cache rows themselves, so the CUDA cores only do the softmax. Rows of the 16-row MMA tile hold the
// group's query heads twice: rows 0..7 the f16 high part of q (resp. of the probabilities), rows 8..15
// the f16 low part, so one MMA yields both halves of a two-term product and fp32 accuracy is kept
// although the cache is f16 (exact) and q / p are split hi + lo.
//
// Lane (g = lane/4, t = lane%4). K tile as B operand (dims x 8 keys): the lane loads 16-byte chunks
// t, t+4, .. of key g straight from HBM; the four half2 of a chunk are the B registers of two k-steps
// (the order of dims inside the contraction is free as long as q uses the same order). The scores come
// out as C[head g][keys 2t, 2t+1] — exactly the A layout P.V needs. V tile as B operand (keys x 8 dims):
// the lane loads chunk g (+8) of keys 2t, 2t+1, 2t+8, 2t+9 and pairs equal dims of adjacent keys with
// one prmt each. Each warp walks its own keys with an online softmax; warps, then key splits, are merged
// in a fixed order.
// =================================================================================================
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// (x, y) -> f16 high parts packed, f16 low parts (x - hi(x)) packed
__device__ __forceinline__ void split_pack(float x, float y, uint32_t& hi, uint32_t& lo) {
    const __half hx = __float2half_rn(x), hy = __float2half_rn(y);
    const __half lx = __float2half_rn(x - __half2float(hx)), ly = __float2half_rn(y - __half2float(hy));
    hi = (uint32_t) __half_as_ushort(hx) | ((uint32_t) __half_as_ushort(hy) << 16);
    lo = (uint32_t) __half_as_ushort(lx) | ((uint32_t) __half_as_ushort(ly) << 16);
}

constexpr int AM_WARPS = 8;
constexpr float LOG2E = 1.4426950408889634f;
// exp(x) for x <= 0 through the ex2 unit (relative error ~1e-7 after the fp32 pre-scale)
__device__ __forceinline__ float fast_exp(float x) { return exp2f(x * LOG2E); }

// What the decode step folds into the attention kernel (FUSE): the rotary embedding of q and of the token's new key,
// and the append of that key and value to the f16 cache. q, k, v of the token arrive unrotated in one merged row
// [q heads | k heads | v heads]. (Folding the key splits inside the kernel as well, by the CTA of a kv head that
// finishes last, was measured and dropped: that one CTA's serial pass over the records cost more than the merge
// kernel's launch, 9.34 against 8.97 ms per step on the 70B shape.)
struct AttnStep {
    const float* qkv;            // [batch][(heads + 2 kv_heads) * D], unrotated
    const float* cos_t;          // rotation factors [max_seq][D/2]
    const float* sin_t;
    __half* kc_w;                // the caches, writable: the key / value of position kv_len - 1 are written here
    __half* vc_w;
    int rope_mode;               // 0: pairs (2i, 2i+1), 1: pairs (i, i + D/2)
};

// (x, y) of one rotation pair -> rotated, each product and sum rounded on its own (the restatement's order)
__device__ __forceinline__ void rope_pair(float& x, float& y, float c, float sn) {
    const float rx = __fsub_rn(__fmul_rn(x, c), __fmul_rn(y, sn)), ry = __fadd_rn(__fmul_rn(x, sn), __fmul_rn(y, c));
    x = rx; y = ry;
}
// Four consecutive elements [e0, e0+4) of a head row at `base`, rotated for position p.
template <int D>
__device__ __forceinline__ float4 rope_load4(const float* __restrict__ base, int e0, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                             int p, int mode) {
    float4 f = __ldg((const float4*) (base + e0));
    const float* cr = cos_t + (size_t) p * (D / 2);
    const float* sr = sin_t + (size_t) p * (D / 2);
    if (mode == 0) {
        const int i = e0 >> 1;
        rope_pair(f.x, f.y, __ldg(cr + i), __ldg(sr + i));
        rope_pair(f.z, f.w, __ldg(cr + i + 1), __ldg(sr + i + 1));
    } else {
        const bool lower = e0 < D / 2;
        const int i = lower ? e0 : e0 - D / 2;
        float4 o = __ldg((const float4*) (base + (lower ? e0 + D / 2 : e0 - D / 2)));
        float* fa = &f.x; float* oa = &o.x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float x = lower ? fa[k] : oa[k], y = lower ? oa[k] : fa[k];
            rope_pair(x, y, __ldg(cr + i + k), __ldg(sr + i + k));
            fa[k] = lower ? x : y;
        }
    }
    return f;
}

template <int D, bool FUSE>
__global__ void __launch_bounds__(AM_WARPS * 32)
attn_decode_mma_kernel(const float* __restrict__ q, int64_t q_row_stride, const __half* __restrict__ kc, const __half* __restrict__ vc,
                       float* __restrict__ part, int heads, int kv_heads, int G, int64_t cache_stride,
                       const int32_t* __restrict__ kv_len, float scale, int window, int chunk, int splits, float* __restrict__ out_direct,
                       int max_len, int ring_start, int ring_cap, AttnStep step) {
    constexpr int S4 = D / 32;     // chunks of a K row per lane
    constexpr int KS = D / 16;     // k-steps of the score contraction
    constexpr int U = D / 64;      // chunks of a V row per lane
    constexpr int NT = D / 8;      // 8-dim output tiles
    constexpr int NP = AM_WARPS + (FUSE ? 1 : 0);      // partial records merged per CTA: one per warp (+ the token's own key)
    __shared__ float sm_m[NP][8], sm_l[NP][8], sm_c[NP][8];
    __shared__ uint32_t sm_q[KS][4][32];
    __shared__ float sm_acc[NP][8][D + 4];
    __shared__ float sm_knew[FUSE ? D : 1];
    skd::pdl_launch_dependents();
    skd::pdl_wait();

    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int len = min(__ldg(kv_len + b), max_len);      // never past what the launch was sized (and the cache allocated) for
    int first = 0;
    if (window > 0 && len - window > first) first = len - window;
    // FUSE: the newest key (index len - 1) is not in the cache yet; the CTA whose split would hold it appends it and
    // accounts for it as one more partial record, so nobody reads that cache slot in this launch.
    const int keys = FUSE ? len - 1 : len;
    const bool owner = FUSE && len > 0 && split == min((len - 1) / chunk, splits - 1);
    const int begin = max(first, split * chunk), stop = min(keys, (split + 1) * chunk);

    const __half* kb = kc + ((int64_t) b * kv_heads + kvh) * cache_stride * D;
    const __half* vb = vc + ((int64_t) b * kv_heads + kvh) * cache_stride * D;
    const uint4 zero4 = make_uint4(0, 0, 0, 0);
    // Key i of the visible run sits in cache slot i, or, when the cache is a ring of ring_cap slots whose oldest
    // visible key is in slot ring_start, in slot (ring_start + i) mod ring_cap: a wrapped window is read as the two
    // runs it occupies, in place. The softmax is a sum over keys, so the slot order needs no gather.
    auto slot_of = [&](int key) -> int64_t {
        int sl = key + ring_start;
        if (ring_cap > 0 && sl >= ring_cap) sl -= ring_cap;
        return (int64_t) sl;
    };

    // loads of a 16-key tile: K as (key g | g+8, chunks t+4s), V as (keys 2t,2t+1,2t+8,2t+9, chunks g+8u).
    // Two tiles (A, B) are kept in flight per warp: with one CTA of eight warps per SM that is 128 KB of
    // loads outstanding per SM, enough to cover the HBM latency at full bandwidth.
    uint4 krA[2][S4], vrA[4][U], krB[2][S4], vrB[4][U];
    auto load_tile = [&](uint4 (&kr)[2][S4], uint4 (&vr)[4][U], int k0) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const int key = k0 + 8 * nt + g;
#pragma unroll
            for (int s = 0; s < S4; ++s) kr[nt][s] = key < stop ? skd::ld_stream(kb + slot_of(key) * D + (t + 4 * s) * 8) : zero4;
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            const int key = k0 + 2 * t + (kk & 1) + 8 * (kk >> 1);
#pragma unroll
            for (int u = 0; u < U; ++u) vr[kk][u] = key < stop ? skd::ld_stream(vb + slot_of(key) * D + (g + 8 * u) * 8) : zero4;
        }
    };
    constexpr int STEP = AM_WARPS * 16;
    int k0 = begin + warp * 16;
    if (k0 < stop) load_tile(krA, vrA, k0);          // in flight while q is fetched and split below
    if (k0 + STEP < stop) load_tile(krB, vrB, k0 + STEP);

    // q of head g as A fragments, per k-step {hi(k 2t..), lo(k 2t..), hi(k 2t+8..), lo(k 2t+8..)}: warp w
    // converts k-step w (k-step 2s+j covers floats 4j..4j+3 of chunk t+4s) and all warps read the result.
    const int pos_new = len - 1;                       // FUSE: the position being decoded
    for (int ks = warp; ks < KS; ks += AM_WARPS) {
        float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
        if (g < G) {
            const float* qrow = q + (int64_t) b * q_row_stride + (int64_t) (kvh * G + g) * D;
            const int e0 = (t + 4 * (ks >> 1)) * 8 + 4 * (ks & 1);
            f = FUSE ? rope_load4<D>(qrow, e0, step.cos_t, step.sin_t, pos_new, step.rope_mode) : __ldg((const float4*) (qrow + e0));
        }
        uint32_t h0, l0, h1, l1;
        split_pack(f.x, f.y, h0, l0);
        split_pack(f.z, f.w, h1, l1);
        sm_q[ks][0][lane] = h0; sm_q[ks][1][lane] = l0; sm_q[ks][2][lane] = h1; sm_q[ks][3][lane] = l1;
    }
    if (FUSE) {
        // the token's own key and value: rotated / rounded to binary16 exactly as the cache will hold them, appended by
        // the owner CTA, and entered as partial record AM_WARPS (score of head hg against the new key, weight 1, its value)
        if (owner) {
            const float* krow = step.qkv + (int64_t) b * q_row_stride + (int64_t) (heads + kvh) * D;
            const float* vrow = step.qkv + (int64_t) b * q_row_stride + (int64_t) (heads + kv_heads + kvh) * D;
            int sl = pos_new + ring_start;
            if (ring_cap > 0 && sl >= ring_cap) sl -= ring_cap;
            __half* kdst = step.kc_w + (((int64_t) b * kv_heads + kvh) * cache_stride + sl) * D;
            __half* vdst = step.vc_w + (((int64_t) b * kv_heads + kvh) * cache_stride + sl) * D;
            if (threadIdx.x < D / 4) {
                const int e0 = threadIdx.x * 4;
                const float4 kf = rope_load4<D>(krow, e0, step.cos_t, step.sin_t, pos_new, step.rope_mode);
                const __half2 k01 = __floats2half2_rn(kf.x, kf.y), k23 = __floats2half2_rn(kf.z, kf.w);
                *reinterpret_cast<__half2*>(kdst + e0) = k01; *reinterpret_cast<__half2*>(kdst + e0 + 2) = k23;
                const float2 a = __half22float2(k01), c2 = __half22float2(k23);
                sm_knew[e0] = a.x; sm_knew[e0 + 1] = a.y; sm_knew[e0 + 2] = c2.x; sm_knew[e0 + 3] = c2.y;
            } else if (threadIdx.x < D / 2) {
                const int e0 = (threadIdx.x - D / 4) * 4;
                const float4 vf = __ldg((const float4*) (vrow + e0));
                const __half2 v01 = __floats2half2_rn(vf.x, vf.y), v23 = __floats2half2_rn(vf.z, vf.w);
                *reinterpret_cast<__half2*>(vdst + e0) = v01; *reinterpret_cast<__half2*>(vdst + e0 + 2) = v23;
                const float2 a = __half22float2(v01), c2 = __half22float2(v23);
#pragma unroll
                for (int hg = 0; hg < 8; ++hg) { sm_acc[AM_WARPS][hg][e0] = a.x; sm_acc[AM_WARPS][hg][e0 + 1] = a.y; sm_acc[AM_WARPS][hg][e0 + 2] = c2.x; sm_acc[AM_WARPS][hg][e0 + 3] = c2.y; }
            }
        } else {
            for (int i = threadIdx.x; i < 8 * (D + 4); i += AM_WARPS * 32) (&sm_acc[AM_WARPS][0][0])[i] = 0.0f;
        }
    }
    __syncthreads();
    if (FUSE) {
        // warp hg: score of head hg against the new key (fp32 rotated q, the cache's binary16 key)
        const int hg = warp;
        float sc_new = MASKED;
        if (owner && hg < G) {
            const float* qrow = q + (int64_t) b * q_row_stride + (int64_t) (kvh * G + hg) * D;
            float p = 0.0f;
#pragma unroll
            for (int e0 = lane * 4; e0 < D; e0 += 128) {
                const float4 f = rope_load4<D>(qrow, e0, step.cos_t, step.sin_t, pos_new, step.rope_mode);
                p += f.x * sm_knew[e0] + f.y * sm_knew[e0 + 1] + f.z * sm_knew[e0 + 2] + f.w * sm_knew[e0 + 3];
            }
            sc_new = skd::warp_sum(p) * scale;
        }
        if (lane == 0) { sm_m[AM_WARPS][hg] = sc_new; sm_l[AM_WARPS][hg] = (owner && hg < G) ? 1.0f : 0.0f; }
    }
    uint32_t qa[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks)
#pragma unroll
        for (int j = 0; j < 4; ++j) qa[ks][j] = sm_q[ks][j][lane];

    float m = MASKED, l = 0.0f;
    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) { o[i][0] = 0.f; o[i][1] = 0.f; o[i][2] = 0.f; o[i][3] = 0.f; }

    auto tile = [&](const uint4 (&kr)[2][S4], const uint4 (&vr)[4][U], int k0) {
        // ---- scores of head g for keys k0 + {2t, 2t+1, 8+2t, 8+2t+1}
        float sc[4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int s = 0; s < S4; ++s) {
                mma_f16(c, qa[2 * s], kr[nt][s].x, kr[nt][s].y);
                mma_f16(c, qa[2 * s + 1], kr[nt][s].z, kr[nt][s].w);
            }
            const int key = k0 + 8 * nt + 2 * t;
            sc[2 * nt] = key < stop ? (c[0] + c[2]) * scale : MASKED;
            sc[2 * nt + 1] = key + 1 < stop ? (c[1] + c[3]) * scale : MASKED;
        }
        float mx = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float mnew = fmaxf(m, mx);
        const float corr = fast_exp(m - mnew);
        const bool rescale = m != mnew && l != 0.0f;      // nothing to rescale before the first key or when the max holds
        m = mnew;
        float p[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] = sc[i] > 0.5f * MASKED ? fast_exp(sc[i] - mnew) : 0.0f;
        l = l * corr + (p[0] + p[1]) + (p[2] + p[3]);
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
            for (int i = 0; i < NT; ++i) { o[i][0] *= corr; o[i][1] *= corr; o[i][2] *= corr; o[i][3] *= corr; }
        }
        uint32_t pa[4];
        split_pack(p[0], p[1], pa[0], pa[1]);
        split_pack(p[2], p[3], pa[2], pa[3]);
        // ---- out[head g][dims] += P . V ; tile (u, i): column n <-> dim 8*(n + 8u) + i
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t v0[4] = {vr[0][u].x, vr[0][u].y, vr[0][u].z, vr[0][u].w}, v1[4] = {vr[1][u].x, vr[1][u].y, vr[1][u].z, vr[1][u].w};
            const uint32_t v8[4] = {vr[2][u].x, vr[2][u].y, vr[2][u].z, vr[2][u].w}, v9[4] = {vr[3][u].x, vr[3][u].y, vr[3][u].z, vr[3][u].w};
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                mma_f16(o[u * 8 + 2 * r], pa, __byte_perm(v0[r], v1[r], 0x5410), __byte_perm(v8[r], v9[r], 0x5410));
                mma_f16(o[u * 8 + 2 * r + 1], pa, __byte_perm(v0[r], v1[r], 0x7632), __byte_perm(v8[r], v9[r], 0x7632));
            }
        }
    };
    while (k0 < stop) {
        tile(krA, vrA, k0);
        if (k0 + 2 * STEP < stop) load_tile(krA, vrA, k0 + 2 * STEP);
        k0 += STEP;
        if (k0 >= stop) break;
        tile(krB, vrB, k0);
        if (k0 + 2 * STEP < stop) load_tile(krB, vrB, k0 + 2 * STEP);
        k0 += STEP;
    }
    // the per-lane sums of l cover different keys; m is already uniform over the four lanes of a head
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    // ---- merge the warps (fixed order), one partial record per (batch, head, split)
    if (t == 0) { sm_m[warp][g] = m; sm_l[warp][g] = l; }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            sm_acc[warp][g][8 * (2 * t + 8 * u) + i] = o[u * 8 + i][0] + o[u * 8 + i][2];
            sm_acc[warp][g][8 * (2 * t + 1 + 8 * u) + i] = o[u * 8 + i][1] + o[u * 8 + i][3];
        }
    __syncthreads();
    if (threadIdx.x < 8 * NP) {             // weight of (record w, head hg) in the merged record
        const int w = threadIdx.x >> 3, hg = threadIdx.x & 7;
        float mxx = MASKED;
#pragma unroll
        for (int w2 = 0; w2 < NP; ++w2) mxx = fmaxf(mxx, sm_m[w2][hg]);
        sm_c[w][hg] = sm_m[w][hg] > 0.5f * MASKED ? fast_exp(sm_m[w][hg] - mxx) : 0.0f;
    }
    __syncthreads();
    const bool direct = out_direct != nullptr;
    for (int idx = threadIdx.x; idx < G * D; idx += AM_WARPS * 32) {
        const int hg = idx / D, dd = idx % D;
        float at = 0.0f;
#pragma unroll
        for (int w = 0; w < NP; ++w) at += sm_c[w][hg] * sm_acc[w][hg][dd];
        if (direct) {                // a single key split: this is the final result, no records and no merge launch
            float lt = 0.0f;
#pragma unroll
            for (int w = 0; w < NP; ++w) lt += sm_c[w][hg] * sm_l[w][hg];
            out_direct[((int64_t) b * heads + kvh * G + hg) * D + dd] = lt > 0.0f ? at / lt : 0.0f;
            continue;
        }
        float* rec = part + (((int64_t) b * heads + kvh * G + hg) * splits + split) * (D + 2);
        rec[2 + dd] = at;
        if (dd == 0) {
            float mxx = MASKED, lt = 0.0f;
#pragma unroll
            for (int w = 0; w < NP; ++w) { mxx = fmaxf(mxx, sm_m[w][hg]); lt += sm_c[w][hg] * sm_l[w][hg]; }
            rec[0] = mxx; rec[1] = lt;
        }
    }
}

// Fewest keys a split is given: one 16-key tile per warp of the split-K kernel.
static int attn_min_keys() { return 128; }
static int decode_splits(int batch, int kv_heads, int max_kv_len) {
    // One wave: the split-K kernel holds one CTA of eight warps per SM (register-bound), and a second wave
    // would double its time. Each split gets at least min_keys keys (one 16-key tile per warp at 128).
    const int ctas = batch * kv_heads;
    int want = std::max(1, sm_count() / ctas);
    const int min_keys = attn_min_keys();
    const int by_len = (max_kv_len + min_keys - 1) / min_keys;
    want = std::max(1, std::min(want, by_len));
    return std::min(want, 256);
}

size_t attn_scratch_bytes(int batch, int heads, int head_dim, int max_kv_len) {
    // kv_heads is not known here; the bound below holds for any grouping (splits <= 256).
    const int splits = std::min(256, std::max(1, (max_kv_len + attn_min_keys() - 1) / attn_min_keys()));
    return (size_t) batch * heads * splits * (head_dim + 2) * sizeof(float);
}

// Merge of the key splits fused with the activation quantizer of the projection that follows: one CTA
// per 256 consecutive outputs of a row (two 128-wide heads or four 64-wide ones), fp32 result kept as
// well. grid (heads*D/256, batch), 256*MG threads (MG split groups, see merge_splits).
template <int D, bool SPLIT>
__global__ void __launch_bounds__(256 * MG)
attn_merge_quant_kernel(const float* __restrict__ part, float* __restrict__ out, int splits, int heads, ActQ8K oq, ActSplit os) {
    __shared__ float red[8];
    __shared__ float sm[3][MG][256];
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    const int el = threadIdx.x & 255, grp = threadIdx.x >> 8;
    const int b = blockIdx.y, e = blockIdx.x * 256 + el, n = heads * D;
    const int head = e / D, dd = e % D, lane = threadIdx.x & 31, warp = el >> 5;
    const float v = merge_splits<D, 256>(part + ((int64_t) b * heads + head) * splits * (D + 2), splits, dd, el, grp, sm);
    if (grp != 0) return;        // the quantizer below runs on the first 256 threads and synchronises them by a named barrier
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
        asm volatile("bar.sync 1, 256;" ::: "memory");
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
                             int window, int chunk, int splits, int64_t q_row_stride, int always_partials, int max_len, int ring_start,
                             int ring_cap, cudaStream_t s) {
    dim3 grid(splits, kv_heads, batch);
    const bool direct = splits == 1 && !always_partials;
    launch_pdl(attn_decode_mma_kernel<D, false>, grid, dim3(AM_WARPS * 32), 0, s, q, q_row_stride, k, v, part, heads, kv_heads, G, cache_stride, kv_len,
               scale, window, chunk, splits, direct ? out : (float*) nullptr, max_len, ring_start, ring_cap, AttnStep());
    if (!always_partials && !direct) launch_pdl(attn_merge_kernel<D>, dim3(batch * heads), dim3(D * MG), 0, s, (const float*) part, out, splits);
}

static int32_t attn_decode_impl(const float* q, int64_t q_row_stride, const __half* k, const __half* v, float* out, int batch, int heads,
                                int kv_heads, int d, int64_t cache_stride, const int32_t* kv_len, int max_kv_len,
                                float scale, int window, void* scratch, int always_partials, int* splits_out, cudaStream_t s,
                                int ring_start = 0, int ring_cap = 0);

int32_t launch_attn_decode(const float* q, const __half* k, const __half* v, float* out, int batch, int heads,
                           int kv_heads, int d, int64_t cache_stride, const int32_t* kv_len, int max_kv_len,
                           float scale, int window, void* scratch, cudaStream_t s) {
    return attn_decode_impl(q, (int64_t) heads * d, k, v, out, batch, heads, kv_heads, d, cache_stride, kv_len, max_kv_len, scale, window,
                            scratch, 0, nullptr, s);
}

// One sequence over a cache that may be a ring: the visible keys are the `len` slots starting at ring_start,
// wrapping at ring_cap (0 = a plain cache). kv_len_dev holds len.
int32_t launch_attn_decode_ring(const float* q, const __half* k, const __half* v, float* out, int heads, int kv_heads, int d,
                                int64_t cache_stride, const int32_t* kv_len_dev, int len, float scale, int ring_start, int ring_cap,
                                void* scratch, cudaStream_t s) {
    return attn_decode_impl(q, (int64_t) heads * d, k, v, out, 1, heads, kv_heads, d, cache_stride, kv_len_dev, len, scale, 0,
                            scratch, 0, nullptr, s, ring_start, ring_cap);
}

// The attention of one decode step: q | k | v of the new token arrive unrotated in qkv [batch][(heads + 2 kv_heads) * d];
// the split-K kernel rotates q and the new key, appends key and value to the f16 caches at position kv_len - 1 and attends
// over the kv_len visible keys; the merge kernel folds the key splits and leaves out [batch][heads * d] together with its
// quantized form for the projection that follows. Two launches (the separate rope + append kernel is gone). Needs
// heads * d to be a multiple of 256; returns 1 when it is not (the caller then runs the separate kernels).
int32_t launch_attn_step(const float* qkv, __half* k, __half* v, float* out, int batch, int heads, int kv_heads, int d,
                         int64_t cache_stride, const int32_t* kv_len, int max_kv_len, float scale, int window, const float* cos_t,
                         const float* sin_t, int rope_mode, void* scratch, bool split, ActQ8K oq, ActSplit os, cudaStream_t s) {
    if (batch <= 0 || heads <= 0) return SKAINET_CUDA_OK;
    const int G = heads / kv_heads;
    if ((heads * d) % 256 != 0 || G > 8 || (G & (G - 1)) != 0 || (d != 64 && d != 128)) return 1;
    const int splits = decode_splits(batch, kv_heads, std::max(1, max_kv_len));
    int chunk = (std::max(1, max_kv_len) + splits - 1) / splits;
    chunk = (chunk + 31) & ~31;
    AttnStep st;
    st.qkv = qkv; st.cos_t = cos_t; st.sin_t = sin_t; st.kc_w = k; st.vc_w = v; st.rope_mode = rope_mode;
    const int64_t stride = (int64_t) (heads + 2 * kv_heads) * d;
    dim3 grid(splits, kv_heads, batch);
    if (d == 128)
        SK_CUDA(launch_pdl(attn_decode_mma_kernel<128, true>, grid, dim3(AM_WARPS * 32), 0, s, qkv, stride, (const __half*) k, (const __half*) v, (float*) scratch,
                           heads, kv_heads, G, cache_stride, kv_len, scale, window, chunk, splits, (float*) nullptr, std::max(1, max_kv_len), 0, 0, st));
    else
        SK_CUDA(launch_pdl(attn_decode_mma_kernel<64, true>, grid, dim3(AM_WARPS * 32), 0, s, qkv, stride, (const __half*) k, (const __half*) v, (float*) scratch,
                           heads, kv_heads, G, cache_stride, kv_len, scale, window, chunk, splits, (float*) nullptr, std::max(1, max_kv_len), 0, 0, st));
    dim3 mgrid(heads * d / 256, batch);
    if (d == 128) {
        if (split) SK_CUDA(launch_pdl(attn_merge_quant_kernel<128, true>, mgrid, dim3(256 * MG), 0, s, (const float*) scratch, out, splits, heads, oq, os));
        else SK_CUDA(launch_pdl(attn_merge_quant_kernel<128, false>, mgrid, dim3(256 * MG), 0, s, (const float*) scratch, out, splits, heads, oq, os));
    } else {
        if (split) SK_CUDA(launch_pdl(attn_merge_quant_kernel<64, true>, mgrid, dim3(256 * MG), 0, s, (const float*) scratch, out, splits, heads, oq, os));
        else SK_CUDA(launch_pdl(attn_merge_quant_kernel<64, false>, mgrid, dim3(256 * MG), 0, s, (const float*) scratch, out, splits, heads, oq, os));
    }
    return SKAINET_CUDA_OK;
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
        if (split) SK_CUDA(launch_pdl(attn_merge_quant_kernel<128, true>, grid, dim3(256 * MG), 0, s, (const float*) scratch, out, splits, heads, oq, os));
        else SK_CUDA(launch_pdl(attn_merge_quant_kernel<128, false>, grid, dim3(256 * MG), 0, s, (const float*) scratch, out, splits, heads, oq, os));
    } else {
        if (split) SK_CUDA(launch_pdl(attn_merge_quant_kernel<64, true>, grid, dim3(256 * MG), 0, s, (const float*) scratch, out, splits, heads, oq, os));
        else SK_CUDA(launch_pdl(attn_merge_quant_kernel<64, false>, grid, dim3(256 * MG), 0, s, (const float*) scratch, out, splits, heads, oq, os));
    }
    return SKAINET_CUDA_OK;
}

static int32_t attn_decode_impl(const float* q, int64_t q_row_stride, const __half* k, const __half* v, float* out, int batch, int heads,
                                int kv_heads, int d, int64_t cache_stride, const int32_t* kv_len, int max_kv_len,
                                float scale, int window, void* scratch, int always_partials, int* splits_out, cudaStream_t s,
                                int ring_start, int ring_cap) {
    if (batch <= 0 || heads <= 0) return SKAINET_CUDA_OK;
    const int G = heads / kv_heads;
    const int splits = decode_splits(batch, kv_heads, std::max(1, max_kv_len));
    int chunk = (std::max(1, max_kv_len) + splits - 1) / splits;
    chunk = (chunk + 31) & ~31;
    float* part = (float*) scratch;
    if (splits_out) *splits_out = splits;
#define SK_AD(DD, GG) launch_decode_dg<DD, GG>(q, k, v, out, part, batch, heads, kv_heads, cache_stride, kv_len, scale, window, chunk, splits, q_row_stride, always_partials, std::max(1, max_kv_len), ring_start, ring_cap, s)
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

// =================================================================================================
// Prefill attention on the tensor cores: the same fragment scheme as attn_decode_mma_kernel with the roles of
// the MMA rows changed: rows 0..7 are eight CONSECUTIVE QUERY POSITIONS of one head (f16 high parts; rows
// 8..15 the low parts), so a K/V tile read once serves eight queries. Each row has its own causal (and
// window) limit; one CTA sees the whole key range of its queries, so the result is final (no split records).
// grid (ceil(seq_q/8), heads, batch), eight warps taking 16-key tiles round-robin, two tiles in flight per warp.
// q / out are token-major [batch, seq_q, heads, D]; query qi of batch b sits at q_abs_base[b] + qi.
// =================================================================================================
template <int D>
__global__ void __launch_bounds__(AM_WARPS * 32)
attn_prefill_mma_kernel(const float* __restrict__ q, const __half* __restrict__ kc, const __half* __restrict__ vc, float* __restrict__ out,
                        int heads, int kv_heads, int seq_q, int64_t cache_stride, const int32_t* __restrict__ q_abs_base,
                        float scale, int window) {
    constexpr int S4 = D / 32, KS = D / 16, U = D / 64, NT = D / 8;
    __shared__ float sm_m[AM_WARPS][8], sm_l[AM_WARPS][8], sm_c[AM_WARPS][8];
    __shared__ uint32_t sm_q[KS][4][32];
    __shared__ float sm_acc[AM_WARPS][8][D + 4];
    skd::pdl_launch_dependents();
    skd::pdl_wait();

    const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int kvh = h / (heads / kv_heads);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int base = __ldg(q_abs_base + b);
    const int nq = min(8, seq_q - qt * 8);                        // live query rows of this tile
    // row g: keys [first_g, end_g); the CTA walks [begin, stop)
    const int qi = qt * 8 + g;
    const int end_g = g < nq ? base + qi + 1 : 0;
    const int first_g = window > 0 ? max(0, end_g - window) : 0;
    const int stop = base + qt * 8 + nq;
    const int begin = window > 0 ? max(0, base + qt * 8 + 1 - window) : 0;

    const __half* kb = kc + ((int64_t) b * kv_heads + kvh) * cache_stride * D;
    const __half* vb = vc + ((int64_t) b * kv_heads + kvh) * cache_stride * D;
    const uint4 zero4 = make_uint4(0, 0, 0, 0);
    uint4 krA[2][S4], vrA[4][U], krB[2][S4], vrB[4][U];
    auto load_tile = [&](uint4 (&kr)[2][S4], uint4 (&vr)[4][U], int k0) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const int key = k0 + 8 * nt + g;
#pragma unroll
            for (int s = 0; s < S4; ++s) kr[nt][s] = key < stop ? skd::ld_ro(kb + (int64_t) key * D + (t + 4 * s) * 8) : zero4;
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            const int key = k0 + 2 * t + (kk & 1) + 8 * (kk >> 1);
#pragma unroll
            for (int u = 0; u < U; ++u) vr[kk][u] = key < stop ? skd::ld_ro(vb + (int64_t) key * D + (g + 8 * u) * 8) : zero4;
        }
    };
    constexpr int STEP = AM_WARPS * 16;
    int k0 = (begin & ~15) + warp * 16;
    if (k0 < stop) load_tile(krA, vrA, k0);
    if (k0 + STEP < stop) load_tile(krB, vrB, k0 + STEP);

    for (int ks = warp; ks < KS; ks += AM_WARPS) {
        float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
        if (g < nq) f = __ldg((const float4*) (q + (((int64_t) b * seq_q + qi) * heads + h) * D + (t + 4 * (ks >> 1)) * 8 + 4 * (ks & 1)));
        uint32_t h0, l0, h1, l1;
        split_pack(f.x, f.y, h0, l0);
        split_pack(f.z, f.w, h1, l1);
        sm_q[ks][0][lane] = h0; sm_q[ks][1][lane] = l0; sm_q[ks][2][lane] = h1; sm_q[ks][3][lane] = l1;
    }
    __syncthreads();
    uint32_t qa[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks)
#pragma unroll
        for (int j = 0; j < 4; ++j) qa[ks][j] = sm_q[ks][j][lane];

    float m = MASKED, l = 0.0f;
    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) { o[i][0] = 0.f; o[i][1] = 0.f; o[i][2] = 0.f; o[i][3] = 0.f; }

    auto tile = [&](const uint4 (&kr)[2][S4], const uint4 (&vr)[4][U], int k0) {
        float sc[4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int s = 0; s < S4; ++s) {
                mma_f16(c, qa[2 * s], kr[nt][s].x, kr[nt][s].y);
                mma_f16(c, qa[2 * s + 1], kr[nt][s].z, kr[nt][s].w);
            }
            const int key = k0 + 8 * nt + 2 * t;
            sc[2 * nt] = (key >= first_g && key < end_g) ? (c[0] + c[2]) * scale : MASKED;
            sc[2 * nt + 1] = (key + 1 >= first_g && key + 1 < end_g) ? (c[1] + c[3]) * scale : MASKED;
        }
        float mx = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float mnew = fmaxf(m, mx);
        const float corr = fast_exp(m - mnew);
        const bool rescale = m != mnew && l != 0.0f;
        m = mnew;
        float p[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] = sc[i] > 0.5f * MASKED ? fast_exp(sc[i] - mnew) : 0.0f;
        l = l * corr + (p[0] + p[1]) + (p[2] + p[3]);
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
            for (int i = 0; i < NT; ++i) { o[i][0] *= corr; o[i][1] *= corr; o[i][2] *= corr; o[i][3] *= corr; }
        }
        uint32_t pa[4];
        split_pack(p[0], p[1], pa[0], pa[1]);
        split_pack(p[2], p[3], pa[2], pa[3]);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t v0[4] = {vr[0][u].x, vr[0][u].y, vr[0][u].z, vr[0][u].w}, v1[4] = {vr[1][u].x, vr[1][u].y, vr[1][u].z, vr[1][u].w};
            const uint32_t v8[4] = {vr[2][u].x, vr[2][u].y, vr[2][u].z, vr[2][u].w}, v9[4] = {vr[3][u].x, vr[3][u].y, vr[3][u].z, vr[3][u].w};
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                mma_f16(o[u * 8 + 2 * r], pa, __byte_perm(v0[r], v1[r], 0x5410), __byte_perm(v8[r], v9[r], 0x5410));
                mma_f16(o[u * 8 + 2 * r + 1], pa, __byte_perm(v0[r], v1[r], 0x7632), __byte_perm(v8[r], v9[r], 0x7632));
            }
        }
    };
    while (k0 < stop) {
        tile(krA, vrA, k0);
        if (k0 + 2 * STEP < stop) load_tile(krA, vrA, k0 + 2 * STEP);
        k0 += STEP;
        if (k0 >= stop) break;
        tile(krB, vrB, k0);
        if (k0 + 2 * STEP < stop) load_tile(krB, vrB, k0 + 2 * STEP);
        k0 += STEP;
    }
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (t == 0) { sm_m[warp][g] = m; sm_l[warp][g] = l; }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            sm_acc[warp][g][8 * (2 * t + 8 * u) + i] = o[u * 8 + i][0] + o[u * 8 + i][2];
            sm_acc[warp][g][8 * (2 * t + 1 + 8 * u) + i] = o[u * 8 + i][1] + o[u * 8 + i][3];
        }
    __syncthreads();
    if (threadIdx.x < 8 * AM_WARPS) {
        const int w = threadIdx.x >> 3, hg = threadIdx.x & 7;
        float mxx = MASKED;
#pragma unroll
        for (int w2 = 0; w2 < AM_WARPS; ++w2) mxx = fmaxf(mxx, sm_m[w2][hg]);
        sm_c[w][hg] = fast_exp(sm_m[w][hg] - mxx);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nq * D; idx += AM_WARPS * 32) {
        const int hg = idx / D, dd = idx % D;
        float at = 0.0f, lt = 0.0f;
#pragma unroll
        for (int w = 0; w < AM_WARPS; ++w) { at += sm_c[w][hg] * sm_acc[w][hg][dd]; lt += sm_c[w][hg] * sm_l[w][hg]; }
        out[(((int64_t) b * seq_q + qt * 8 + hg) * heads + h) * D + dd] = lt > 0.0f ? at / lt : 0.0f;
    }
}

// Causal attention of a block of new queries over an f16 cache (prefill): query qi of batch b sits at
// absolute position q_abs_base[b] + qi and sees keys [0, that position]. q/out are token-major
// [batch, seq_q, heads, D], the layout the projections produce.
int32_t launch_sdpa_cache(const float* q, const __half* k, const __half* v, float* out, int batch, int heads,
                          int kv_heads, int seq_q, int seq_kv, int64_t cache_stride, int d, float scale, int window,
                          const int32_t* q_abs_base, cudaStream_t s) {
    if ((d == 128 || d == 64) && batch > 0 && seq_q > 0 && heads % kv_heads == 0 && batch <= 65535 && heads <= 65535) {
        dim3 grid((seq_q + 7) / 8, heads, batch);
        if (d == 128) SK_CUDA(launch_pdl(attn_prefill_mma_kernel<128>, grid, dim3(AM_WARPS * 32), 0, s, q, k, v, out, heads, kv_heads, seq_q, cache_stride, q_abs_base, scale, window));
        else SK_CUDA(launch_pdl(attn_prefill_mma_kernel<64>, grid, dim3(AM_WARPS * 32), 0, s, q, k, v, out, heads, kv_heads, seq_q, cache_stride, q_abs_base, scale, window));
        return SKAINET_CUDA_OK;
    }
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
