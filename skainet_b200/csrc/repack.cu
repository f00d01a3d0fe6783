// Upload-time plane split of packed GGUF blocks, its exact inverse, the bit-exact decoders, the
// packed-table row gather, and the seeded on-device weight generator used by the bench harness.
//
// Decoders follow skainet-io/skainet-io-gguf/src/commonMain/kotlin/sk/ainet/io/gguf/dequant/DequantOps.kt
// (Q8_0 :338-355, get_scale_min_k4 :585-598, Q4_K :600-644, Q5_K and Q6_K after that) with every
// product and difference individually rounded (__fmul_rn/__fsub_rn: no FMA contraction), which is
// what makes the output bit-identical to the JVM's strict binary32 arithmetic.
#include "common.cuh"

namespace sk {

// A weight as device code sees it.
struct WView {
    int enc, rows, cols, bpr;
    const uint8_t* qs; const uint8_t* hdr; const uint8_t* extra; const uint8_t* aux;
};
static WView view_of(const Weight& w) { return WView{w.enc, w.rows, w.cols, w.bpr, w.qs, w.hdr, w.extra, w.aux}; }

// -------------------------------------------------------------------------------------------------
// canonical <-> planes. `to_planes` true: canonical -> planes, false: planes -> canonical.
// One thread moves one 2-byte unit (every block size and every field offset of the four formats is
// even, and that is the only alignment a canonical Q8_0/Q6_K block guarantees).
// -------------------------------------------------------------------------------------------------
__global__ void plane_permute_kernel(uint16_t* canon, uint16_t* qs, uint16_t* hdr, uint16_t* extra, uint16_t* aux,
                                     int enc, int rows, int bpr, int order, int bb2, bool to_planes) {
    const int64_t total = (int64_t) rows * bpr * bb2;
    for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < total; i += (int64_t) gridDim.x * blockDim.x) {
        const int64_t cblk = i / bb2;          // block index in canonical order
        const int u = (int) (i - cblk * bb2);  // 2-byte unit inside the block
        int64_t o, b;
        if (order == SKAINET_ORDER_ROW_MAJOR) { o = cblk / bpr; b = cblk - o * bpr; }
        else { b = cblk / rows; o = cblk - b * rows; }
        const int64_t pblk = o * bpr + b;      // planes are always row-major
        uint16_t* dst;
        switch (enc) {
            case SKAINET_ENC_Q8_0:   // [d:1][codes:16]
                dst = u < 1 ? hdr + pblk : qs + pblk * 16 + (u - 1);
                break;
            case SKAINET_ENC_Q4_K:   // [hdr:8][qs:64]
                dst = u < 8 ? hdr + pblk * 8 + u : qs + pblk * 64 + (u - 8);
                break;
            case SKAINET_ENC_Q5_K:   // [hdr:8][qh:16][qs:64]
                dst = u < 8 ? hdr + pblk * 8 + u : (u < 24 ? extra + pblk * 16 + (u - 8) : qs + pblk * 64 + (u - 24));
                break;
            default:                 // Q6_K [ql:64][qh:32][scales:8][d:1]
                dst = u < 64 ? qs + pblk * 64 + u
                    : (u < 96 ? extra + pblk * 32 + (u - 64) : (u < 104 ? hdr + pblk * 8 + (u - 96) : aux + pblk));
                break;
        }
        if (to_planes) *dst = canon[i]; else canon[i] = *dst;
    }
}

int32_t launch_split_planes(const uint8_t* canon_dev, Weight& w, int order, cudaStream_t s) {
    const int bb2 = block_bytes(w.enc) / 2;
    const int64_t total = (int64_t) w.rows * w.bpr * bb2;
    if (total == 0) return SKAINET_CUDA_OK;
    const int grid = (int) std::min<int64_t>((total + 255) / 256, 148 * 32);
    plane_permute_kernel<<<grid, 256, 0, s>>>((uint16_t*) canon_dev, (uint16_t*) w.qs, (uint16_t*) w.hdr,
        (uint16_t*) w.extra, (uint16_t*) w.aux, w.enc, w.rows, w.bpr, order, bb2, true);
    SK_CUDA(cudaGetLastError());
    return SKAINET_CUDA_OK;
}

int32_t launch_join_planes(const Weight& w, uint8_t* canon_dev, cudaStream_t s) {
    const int bb2 = block_bytes(w.enc) / 2;
    const int64_t total = (int64_t) w.rows * w.bpr * bb2;
    if (total == 0) return SKAINET_CUDA_OK;
    const int grid = (int) std::min<int64_t>((total + 255) / 256, 148 * 32);
    plane_permute_kernel<<<grid, 256, 0, s>>>((uint16_t*) canon_dev, (uint16_t*) w.qs, (uint16_t*) w.hdr,
        (uint16_t*) w.extra, (uint16_t*) w.aux, w.enc, w.rows, w.bpr, SKAINET_ORDER_ROW_MAJOR, bb2, false);
    SK_CUDA(cudaGetLastError());
    return SKAINET_CUDA_OK;
}

// -------------------------------------------------------------------------------------------------
// Decoders. One element per thread: these run at load/test time, not in the decode loop.
// `blk` points at the block's bytes per plane; e is the element index inside the block.
// -------------------------------------------------------------------------------------------------
__device__ __forceinline__ float half_bits_to_float(uint16_t h) { return __half2float(__ushort_as_half(h)); }

__device__ __forceinline__ void k4_scale_min(const uint8_t* s, int j, int& sc, int& mn) {
    if (j < 4) { sc = s[j] & 0x3F; mn = s[j + 4] & 0x3F; }
    else {
        sc = (s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4);
        mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

__device__ float decode_elem(int enc, const uint8_t* qs, const uint8_t* hdr, const uint8_t* extra, const uint8_t* aux, int e) {
    switch (enc) {
        case SKAINET_ENC_Q8_0: {
            const float d = half_bits_to_float(*(const uint16_t*) hdr);
            return __fmul_rn(d, (float) (int) (int8_t) qs[e]);
        }
        case SKAINET_ENC_Q4_K:
        case SKAINET_ENC_Q5_K: {
            const float d = half_bits_to_float(*(const uint16_t*) hdr);
            const float dmin = half_bits_to_float(*(const uint16_t*) (hdr + 2));
            const int sb = e >> 5, g = e >> 6, l = e & 31;
            int sc, mn; k4_scale_min(hdr + 4, sb, sc, mn);
            const uint8_t pb = qs[32 * g + l];
            int q = (sb & 1) ? (pb >> 4) : (pb & 0x0F);
            if (enc == SKAINET_ENC_Q5_K) q |= ((extra[l] >> sb) & 1) << 4;
            return __fsub_rn(__fmul_rn(__fmul_rn(d, (float) sc), (float) q), __fmul_rn(dmin, (float) mn));
        }
        default: {  // Q6_K: element e = 128*n + 32*quarter + l
            const float d = half_bits_to_float(*(const uint16_t*) aux);
            const int n = e >> 7, r = e & 127, quarter = r >> 5, l = r & 31;
            const uint8_t* ql = qs + 64 * n; const uint8_t* qh = extra + 32 * n; const int8_t* sc = (const int8_t*) hdr + 8 * n;
            const uint8_t lb = ql[l + ((quarter & 1) ? 32 : 0)];
            const int low = (quarter & 2) ? (lb >> 4) : (lb & 0x0F);
            const int q = (low | (((qh[l] >> (2 * quarter)) & 3) << 4)) - 32;
            return __fmul_rn(__fmul_rn(d, (float) (int) sc[(l >> 4) + 2 * quarter]), (float) q);
        }
    }
}

__device__ __forceinline__ float decode_at(const WView& w, int64_t pblk, int e) {
    switch (w.enc) {
        case SKAINET_ENC_Q8_0: return decode_elem(w.enc, w.qs + pblk * 32, w.hdr + pblk * 2, nullptr, nullptr, e);
        case SKAINET_ENC_Q4_K: return decode_elem(w.enc, w.qs + pblk * 128, w.hdr + pblk * 16, nullptr, nullptr, e);
        case SKAINET_ENC_Q5_K: return decode_elem(w.enc, w.qs + pblk * 128, w.hdr + pblk * 16, w.extra + pblk * 32, nullptr, e);
        default:               return decode_elem(w.enc, w.qs + pblk * 128, w.hdr + pblk * 16, w.extra + pblk * 64, w.aux + pblk * 2, e);
    }
}

__global__ void dequant_weight_kernel(WView w, float* out) {
    const int be = w.enc == SKAINET_ENC_Q8_0 ? 32 : 256;
    const int64_t total = (int64_t) w.rows * w.cols;
    for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < total; i += (int64_t) gridDim.x * blockDim.x)
        out[i] = decode_at(w, i / be, (int) (i % be));
}

int32_t launch_dequant_weight(const Weight& w, float* out, cudaStream_t s) {
    const int64_t total = (int64_t) w.rows * w.cols;
    if (total == 0) return SKAINET_CUDA_OK;
    const int grid = (int) std::min<int64_t>((total + 255) / 256, 148 * 32);
    dequant_weight_kernel<<<grid, 256, 0, s>>>(view_of(w), out);
    SK_CUDA(cudaGetLastError());
    return SKAINET_CUDA_OK;
}

// Canonical (un-split) blocks straight to floats: the twin of DequantOps.dequant*FromBytes.
__global__ void dequant_canonical_kernel(int enc, const uint8_t* canon, int64_t nblocks, float* out) {
    const int be = enc == SKAINET_ENC_Q8_0 ? 32 : 256;
    const int64_t total = nblocks * be;
    for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < total; i += (int64_t) gridDim.x * blockDim.x) {
        const int64_t blk = i / be; const int e = (int) (i % be);
        const uint8_t* p;
        float v;
        switch (enc) {
            case SKAINET_ENC_Q8_0: p = canon + blk * 34;  v = decode_elem(enc, p + 2, p, nullptr, nullptr, e); break;
            case SKAINET_ENC_Q4_K: p = canon + blk * 144; v = decode_elem(enc, p + 16, p, nullptr, nullptr, e); break;
            case SKAINET_ENC_Q5_K: p = canon + blk * 176; v = decode_elem(enc, p + 48, p, p + 16, nullptr, e); break;
            default:               p = canon + blk * 210; v = decode_elem(enc, p, p + 192, p + 128, p + 208, e); break;
        }
        out[i] = v;
    }
}

int32_t launch_dequant_canonical(int enc, const uint8_t* canon_dev, int64_t nblocks, float* out, cudaStream_t s) {
    if (nblocks == 0) return SKAINET_CUDA_OK;
    const int64_t total = nblocks * block_elems(enc);
    const int grid = (int) std::min<int64_t>((total + 255) / 256, 148 * 32);
    dequant_canonical_kernel<<<grid, 256, 0, s>>>(enc, canon_dev, nblocks, out);
    SK_CUDA(cudaGetLastError());
    return SKAINET_CUDA_OK;
}

// out[i, :] = dequant(W[ids[i], :]); ids outside [0, rows) give a zero row.
__global__ void embed_kernel(WView w, const int32_t* ids, int n, float* out) {
    const int i = blockIdx.x;
    const int row = ids[i];
    const int be = w.enc == SKAINET_ENC_Q8_0 ? 32 : 256;
    for (int c = threadIdx.x; c < w.cols; c += blockDim.x) {
        float v = 0.0f;
        if (row >= 0 && row < w.rows) v = decode_at(w, (int64_t) row * w.bpr + c / be, c % be);
        out[(int64_t) i * w.cols + c] = v;
    }
}

int32_t launch_embed(const Weight& w, const int32_t* ids, int n, float* out, cudaStream_t s) {
    if (n == 0) return SKAINET_CUDA_OK;
    embed_kernel<<<n, 256, 0, s>>>(view_of(w), ids, n, out);
    SK_CUDA(cudaGetLastError());
    return SKAINET_CUDA_OK;
}

// -------------------------------------------------------------------------------------------------
// Seeded synthetic weights, generated and packed on the device (bench/test harness).
// -------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
// Standard normal from a (seed, index) counter: Box-Muller on two 24-bit uniforms.
__device__ __forceinline__ float normal_at(uint64_t seed, uint64_t idx) {
    const uint64_t r = mix64(seed * 0xD1342543DE82EF95ull + idx);
    const float u1 = ((float) ((r >> 40) & 0xFFFFFF) + 1.0f) * (1.0f / 16777216.0f);   // (0, 1]
    const float u2 = (float) ((r >> 16) & 0xFFFFFF) * (1.0f / 16777216.0f);
    return sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
}

// One warp per Q4_K super-block; lane L owns elements 8L..8L+7 (sub-block L/4).
// The value of element (r, c) of the FULL tensor depends only on (seed, r * full_cols + c), so a shard
// generated with its (row0, col0) offsets holds exactly the corresponding slice of the full tensor.
__global__ void synth_q4k_kernel(uint8_t* qs, uint8_t* hdr, int64_t nblocks, uint64_t seed, float std, int mode,
                                 int bpr, int64_t row0, int64_t col0, int64_t full_cols) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (blockIdx.x * (int64_t) blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t) gridDim.x * blockDim.x) >> 5;
    for (int64_t blk = warp; blk < nblocks; blk += nwarps) {
        if (mode == 1) {  // random valid block: random codes/scales, sane f16 fields
            const uint64_t r0 = mix64(seed ^ (uint64_t) (blk * 64 + lane)), r1 = mix64(r0);
            if (lane < 16) {
                *(uint2*) (qs + blk * 128 + lane * 8) = make_uint2((uint32_t) r0, (uint32_t) (r0 >> 32));
            }
            if (lane == 16) {
                const float d = 0.0002f + 0.0004f * (float) ((r1 >> 8) & 0xFF) / 255.0f;
                const float dm = 0.0002f + 0.0004f * (float) ((r1 >> 16) & 0xFF) / 255.0f;
                uint4 h;
                h.x = (uint32_t) __half_as_ushort(__float2half_rn(d)) | ((uint32_t) __half_as_ushort(__float2half_rn(dm)) << 16);
                h.y = (uint32_t) r0; h.z = (uint32_t) (r0 >> 32); h.w = (uint32_t) (r1 >> 32);
                *(uint4*) (hdr + blk * 16) = h;
            }
            continue;
        }
        float v[8];
        float lo = 0.0f, hi = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[i] = std * normal_at(seed, (uint64_t) ((row0 + blk / bpr) * full_cols + col0 + (blk % bpr) * 256 + lane * 8 + i));
            lo = fminf(lo, v[i]); hi = fmaxf(hi, v[i]);
        }
        lo = fminf(lo, __shfl_xor_sync(~0u, lo, 1)); lo = fminf(lo, __shfl_xor_sync(~0u, lo, 2));
        hi = fmaxf(hi, __shfl_xor_sync(~0u, hi, 1)); hi = fmaxf(hi, __shfl_xor_sync(~0u, hi, 2));
        hi = fmaxf(hi, lo);
        const float scale = (hi - lo) / 15.0f, mneg = -lo;
        const float smax = skd::warp_max(scale), mmax = skd::warp_max(mneg);
        const __half dh = __float2half_rn(smax / 63.0f), dmh = __float2half_rn(mmax / 63.0f);
        const float d = __half2float(dh), dm = __half2float(dmh);
        int sc = d > 0.0f ? min(63, max(0, __float2int_rn(scale / d))) : 0;
        int mn = dm > 0.0f ? min(63, max(0, __float2int_rn(mneg / dm))) : 0;
        const float eff = d * (float) sc, off = dm * (float) mn;
        uint32_t codes = 0;  // eight 4-bit codes
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            int q = eff > 0.0f ? __float2int_rn((v[i] + off) / eff) : 0;
            q = min(15, max(0, q));
            codes |= (uint32_t) q << (4 * i);
        }
        // byte i of group g = code[64g + i] | code[64g + 32 + i] << 4: lanes of an even sub-block pair with lane+4.
        const uint32_t other = __shfl_down_sync(~0u, codes, 4);
        const int sb = lane >> 2;
        if ((sb & 1) == 0) {
            uint32_t w0 = 0, w1 = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                w0 |= (((codes >> (4 * i)) & 15u) | (((other >> (4 * i)) & 15u) << 4)) << (8 * i);
                w1 |= (((codes >> (4 * (i + 4))) & 15u) | (((other >> (4 * (i + 4))) & 15u) << 4)) << (8 * i);
            }
            *(uint2*) (qs + blk * 128 + (sb >> 1) * 32 + (lane & 3) * 8) = make_uint2(w0, w1);
        }
        // header: gather the eight (sc, mn) pairs (lane 4j holds sub-block j's).
        int scs[8], mns[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) { scs[j] = __shfl_sync(~0u, sc, 4 * j); mns[j] = __shfl_sync(~0u, mn, 4 * j); }
        if (lane == 0) {
            uint8_t s[12];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                s[j] = (uint8_t) ((scs[j] & 0x3F) | ((scs[j + 4] >> 4) << 6));
                s[j + 4] = (uint8_t) ((mns[j] & 0x3F) | ((mns[j + 4] >> 4) << 6));
                s[j + 8] = (uint8_t) ((scs[j + 4] & 0x0F) | ((mns[j + 4] & 0x0F) << 4));
            }
            uint4 h;
            h.x = (uint32_t) __half_as_ushort(dh) | ((uint32_t) __half_as_ushort(dmh) << 16);
            h.y = s[0] | (s[1] << 8) | (s[2] << 16) | ((uint32_t) s[3] << 24);
            h.z = s[4] | (s[5] << 8) | (s[6] << 16) | ((uint32_t) s[7] << 24);
            h.w = s[8] | (s[9] << 8) | (s[10] << 16) | ((uint32_t) s[11] << 24);
            *(uint4*) (hdr + blk * 16) = h;
        }
    }
}

// One lane per element, one warp per Q8_0 block (rule of Q8_0Quantizer.kt:28-53).
__global__ void synth_q8_0_kernel(int8_t* codes, __half* scales, int64_t nblocks, uint64_t seed, float std, int mode,
                                  int bpr, int64_t row0, int64_t col0, int64_t full_cols) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (blockIdx.x * (int64_t) blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t) gridDim.x * blockDim.x) >> 5;
    for (int64_t blk = warp; blk < nblocks; blk += nwarps) {
        if (mode == 1) {
            const uint64_t r = mix64(seed ^ (uint64_t) (blk * 32 + lane));
            codes[blk * 32 + lane] = (int8_t) (r & 0xFF);
            if (lane == 0) scales[blk] = __float2half_rn(0.0001f + 0.0003f * (float) ((r >> 8) & 0xFF) / 255.0f);
            continue;
        }
        const float v = std * normal_at(seed, (uint64_t) ((row0 + blk / bpr) * full_cols + col0 + (blk % bpr) * 32 + lane));
        const float amax = skd::warp_max(fabsf(v));
        const float d = amax / 127.0f;
        const float id = d != 0.0f ? 1.0f / d : 0.0f;
        int q = __float2int_rd(v * id + 0.5f);
        q = min(127, max(-127, q));
        codes[blk * 32 + lane] = (int8_t) q;
        if (lane == 0) scales[blk] = __float2half_rn(d);
    }
}

int32_t launch_synth(Weight& w, uint64_t seed, float std, int mode, int64_t row0, int64_t col0, int64_t full_cols, cudaStream_t s) {
    const int64_t nblocks = (int64_t) w.rows * w.bpr;
    if (nblocks == 0) return SKAINET_CUDA_OK;
    const int grid = (int) std::min<int64_t>((nblocks + 7) / 8, 148 * 16);
    if (full_cols <= 0) full_cols = w.cols;
    if (w.enc == SKAINET_ENC_Q4_K) synth_q4k_kernel<<<grid, 256, 0, s>>>(w.qs, w.hdr, nblocks, seed, std, mode, w.bpr, row0, col0, full_cols);
    else if (w.enc == SKAINET_ENC_Q8_0) synth_q8_0_kernel<<<grid, 256, 0, s>>>((int8_t*) w.qs, (__half*) w.hdr, nblocks, seed, std, mode, w.bpr, row0, col0, full_cols);
    else { set_error("weight_synth: encoding %d not supported", w.enc); return SKAINET_CUDA_ERR_INVALID; }
    SK_CUDA(cudaGetLastError());
    return SKAINET_CUDA_OK;
}

}  // namespace sk
