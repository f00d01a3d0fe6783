// TurboQuant KV-cache compression on the device: the codec of the reference's TurboQuantKvCacheStore
// (skainet-lang/skainet-lang-core/src/commonMain/kotlin/sk/ainet/lang/tensor/storage/TurboQuantKvCacheStore.kt:62-199),
// one block per (layer, position, head) for keys and for values:
//   RandomRotation.kt:38-131   seeded sign flips (kotlin.random.Random = xorwow) + normalised Walsh-Hadamard transform
//   ScalarQuantizer.kt:35-73   symmetric per-32 quantizer, fp32 scale = absmax / (2^(bits-1) - 1), codes rounded to even
//   BitPacker.kt:23-181        2 / 3 / 4 / 8-bit codes with bias 2^(bits-1), a little-endian bit stream
//   QjlResidual.kt:24-97       optional residual: 1 bit (sign against a second seeded sign sequence, rms scale) or 2-4 bits
//   TurboQuantCodec.kt:33-99   encode = rotate, quantize, pack (, residual); decode = the inverse chain
// Every fp32 operation is written with the round-to-nearest intrinsics so that none is fused, and in the reference's
// order: encoded bytes, scales and decoded values are bit-identical to the reference's (its golden digests,
// Goldens.kt:62-71, are reproduced through this file by tests/test_kv_turboquant.py).
// Encode: one CTA of head_dim threads per vector (a token's vectors are few). Decode: one warp per vector, transform by lane
// shuffles. head_dim a power of two from 32 to 256 (the transform then covers the whole vector; the reference's handling of
// other sizes is not built).
#include "common.cuh"
#include "turboquant.cuh"

namespace sk {

namespace {

// kotlin.random.Random(seed: Int): xorwow (Marsaglia), 64 draws discarded at construction
struct KotlinRandom {
    uint32_t x, y, z, w, v, addend;
    __device__ explicit KotlinRandom(int32_t seed) {
        const uint32_t s1 = (uint32_t) seed, s2 = (uint32_t) (seed >> 31);
        x = s1; y = s2; z = 0; w = 0; v = ~s1; addend = (s1 << 10) ^ (s2 >> 4);
        for (int i = 0; i < 64; ++i) next();
    }
    __device__ uint32_t next() {
        uint32_t t = x;
        t ^= t >> 2;
        x = y; y = z; z = w;
        const uint32_t v0 = v;
        w = v0;
        t = (t ^ (t << 1)) ^ v0 ^ (v0 << 4);
        v = t;
        addend += 362437u;
        return t + addend;
    }
};

// RandomRotation.seedFor
__device__ __forceinline__ int32_t tq_seed_for(int layer, int head, int pos) {
    uint32_t h = (uint32_t) layer;
    h = h * 31u + (uint32_t) head;
    h = h * 31u + (uint32_t) pos;
    h ^= h >> 16; h *= 0x85ebca6bu; h ^= h >> 13; h *= 0xc2b2ae35u; h ^= h >> 16;
    return (int32_t) h;
}

// nextBoolean() for elements 0..n-1 as bit masks (one thread; bit i of word i/32)
__device__ void tq_sign_words(int32_t seed, int n, uint32_t* words) {
    KotlinRandom rng(seed);
    for (int w0 = 0; w0 < n; w0 += 32) {
        uint32_t m = 0;
        for (int i = 0; i < 32 && w0 + i < n; ++i) m |= (rng.next() >> 31) << i;
        words[w0 >> 5] = m;
    }
}

// in-place normalised Walsh-Hadamard transform of x[D] in shared memory, D = blockDim.x a power of two
__device__ void tq_wht(float* x, int D, int t) {
    for (int h = 1; h < D; h <<= 1) {
        __syncthreads();
        if ((t & h) == 0) {
            const float a = x[t], b = x[t + h];
            x[t] = __fadd_rn(a, b); x[t + h] = __fsub_rn(a, b);
        }
    }
    __syncthreads();
    x[t] = __fmul_rn(x[t], __fdiv_rn(1.0f, __fsqrt_rn((float) D)));
    __syncthreads();
}

// ScalarQuantizer.quantize for this thread's element; one warp = one group of 32. Returns the code, *scale the group's.
__device__ __forceinline__ int tq_quantize(float v, int bits, float* scale) {
    const int max_code = (1 << (bits - 1)) - 1;
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float sc = amax > 0.0f ? __fdiv_rn(amax, (float) max_code) : 0.0f;
    *scale = sc;
    if (!(sc > 0.0f)) return 0;
    const int q = __float2int_rn(__fmul_rn(v, __fdiv_rn(1.0f, sc)));       // round half to even, as kotlin.math.round
    return max(-max_code, min(max_code, q));
}

// BitPacker.pack: byte b of the little-endian stream of (code + bias) fields of `bits` bits
__device__ __forceinline__ uint8_t tq_pack_byte(const int8_t* codes, int n, int bits, int b) {
    if (bits == 8) return (uint8_t) codes[b];           // 8-bit codes are stored as they are, without a bias (BitPacker.kt:174)
    const int bias = 1 << (bits - 1), mask = (1 << bits) - 1, bit0 = 8 * b;
    uint32_t acc = 0;
    for (int i = bit0 / bits; i < n && i * bits < bit0 + 8; ++i) {
        const uint32_t u = (uint32_t) ((int) codes[i] + bias) & mask;
        const int sh = i * bits - bit0;
        acc |= sh >= 0 ? (u << sh) : (u >> (-sh));
    }
    return (uint8_t) (acc & 0xff);
}
__device__ __forceinline__ int tq_unpack(const uint8_t* packed, int nbytes, int bits, int i) {
    if (bits == 8) return (int) (int8_t) packed[i];
    const int bias = 1 << (bits - 1), mask = (1 << bits) - 1, bp = i * bits, b = bp >> 3, off = bp & 7;
    uint32_t two = packed[b];
    if (b + 1 < nbytes) two |= (uint32_t) packed[b + 1] << 8;
    return (int) ((two >> off) & mask) - bias;
}

constexpr int TQ_MAX_D = 256;
__device__ __forceinline__ void tq_store(float* p, float v) { *p = v; }
__device__ __forceinline__ void tq_store(__half* p, float v) { *p = __float2half_rn(v); }

// grid (heads), block D. rows [heads][D] fp32 of one token of one layer.
__global__ void __launch_bounds__(TQ_MAX_D)
tq_encode_kernel(const float* __restrict__ rows, TqPlane pl, int layer, int pos, int heads, int D, int max_seq, int32_t seed_xor, int fixed_seed) {
    __shared__ float x[TQ_MAX_D];
    __shared__ float r[TQ_MAX_D];
    __shared__ int8_t codes[TQ_MAX_D];
    __shared__ float gsc[TQ_MAX_D / 32];
    __shared__ uint32_t sg[TQ_MAX_D / 32], rsg[TQ_MAX_D / 32];
    const int t = threadIdx.x, head = blockIdx.x, lane = t & 31, warp = t >> 5;
    const int32_t seed = fixed_seed ? seed_xor : (tq_seed_for(layer, head, pos) ^ seed_xor);      // fixed_seed: seed_xor IS the seed (codec entries)
    const size_t vec = ((size_t) layer * max_seq + pos) * heads + head;
    const int cps = tq_packed_size(D, pl.bits), ng = D / 32;
    if (t == 0) tq_sign_words(seed, D, sg);
    if (t == (D > 32 ? 32 : 0) && pl.rbits == 1) tq_sign_words((int32_t) ((uint32_t) seed + 1u), D, rsg);       // a second warp, side by side
    float v = rows[(size_t) head * D + t];
    __syncthreads();
    if (pl.signs && t < ng) pl.signs[vec * ng + t] = sg[t];
    if (pl.rsigns && pl.rbits == 1 && t < ng) pl.rsigns[vec * ng + t] = rsg[t];
    if ((sg[t >> 5] >> lane) & 1) v = -v;
    x[t] = v;
    tq_wht(x, D, t);
    v = x[t];
    float sc;
    const int q = tq_quantize(v, pl.bits, &sc);
    codes[t] = (int8_t) q;
    if (lane == 0) pl.scales[vec * ng + warp] = sc;
    __syncthreads();
    for (int b = t; b < cps; b += D) pl.codes[vec * cps + b] = tq_pack_byte(codes, D, pl.bits, b);
    if (pl.rbits == 0) return;
    // residual of the rotated vector against its dequantised codes
    const float res = __fsub_rn(v, __fmul_rn((float) q, sc));
    const int rps = tq_packed_size(D, pl.rbits);
    if (pl.rbits == 1) {
        r[t] = res;
        __syncthreads();
        if (t == 0) {
            float s = 0.0f;
            for (int i = 0; i < D; ++i) s = __fadd_rn(s, __fmul_rn(r[i], r[i]));
            pl.rscale[vec] = __fsqrt_rn(__fdiv_rn(s, (float) D));
        }
        const float sgn = ((rsg[t >> 5] >> lane) & 1) ? 1.0f : -1.0f;
        const uint32_t word = __ballot_sync(0xffffffffu, __fmul_rn(res, sgn) >= 0.0f);
        if (lane < 4) pl.resid[vec * rps + warp * 4 + lane] = (uint8_t) (word >> (8 * lane));
    } else {
        __syncthreads();                       // every thread has packed from codes[]
        float rsc;
        const int rq = tq_quantize(res, pl.rbits, &rsc);
        codes[t] = (int8_t) rq;
        if (lane == 0) gsc[warp] = rsc;
        __syncthreads();
        for (int b = t; b < rps; b += D) pl.resid[vec * rps + b] = tq_pack_byte(codes, D, pl.rbits, b);
        if (t == 0) {
            float m = 0.0f;
            for (int g = 0; g < ng; ++g) m = __fadd_rn(m, gsc[g]);
            pl.rscale[vec] = __fdiv_rn(m, (float) ng);
        }
    }
}

// One WARP per vector, EPL = head_dim / 32 elements per lane (element e = 32 i + lane): the butterflies between elements
// less than 32 apart are lane shuffles, the others stay inside a lane, so a decode has no barrier at all. The pairs and the
// order of the stages are the reference's, each result one fp32 add or subtract: bit-identical to the shared-memory form.
// Vectors are numbered position-major: vector = p * heads + head of the window [start_pos, start_pos + n).
// out [heads][n][D], fp32 (exactly the reference's decode) or rounded to binary16.
template <typename OUT, int EPL>
__global__ void __launch_bounds__(256)
tq_decode_kernel(TqPlane pl, int layer, int start_pos, int n, int heads, int32_t seed_xor, int fixed_seed, int max_seq, OUT* __restrict__ out) {
    constexpr int D = EPL * 32;
    const int lane = threadIdx.x & 31;
    const int64_t widx = (int64_t) blockIdx.x * 8 + (threadIdx.x >> 5);
    if (widx >= (int64_t) n * heads) return;
    const int p = (int) (widx / heads), head = (int) (widx % heads), pos = start_pos + p;
    const int32_t seed = fixed_seed ? seed_xor : (tq_seed_for(layer, head, pos) ^ seed_xor);
    const size_t vec = ((size_t) layer * max_seq + pos) * heads + head;
    const int cps = tq_packed_size(D, pl.bits);
    uint32_t sg[EPL], rsg[EPL];
    if (pl.signs) {
#pragma unroll
        for (int i = 0; i < EPL; ++i) sg[i] = pl.signs[vec * EPL + i];
    } else {                                   // one-vector codec calls: lane 0 runs the generator
        uint32_t wds[EPL];
        if (lane == 0) tq_sign_words(seed, D, wds);
#pragma unroll
        for (int i = 0; i < EPL; ++i) sg[i] = __shfl_sync(0xffffffffu, wds[i], 0);
    }
    if (pl.rbits == 1) {
        if (pl.rsigns) {
#pragma unroll
            for (int i = 0; i < EPL; ++i) rsg[i] = pl.rsigns[vec * EPL + i];
        } else {
            uint32_t wds[EPL];
            if (lane == 0) tq_sign_words((int32_t) ((uint32_t) seed + 1u), D, wds);
#pragma unroll
            for (int i = 0; i < EPL; ++i) rsg[i] = __shfl_sync(0xffffffffu, wds[i], 0);
        }
    }
    float v[EPL];
    const uint8_t* codes = pl.codes + vec * cps;
#pragma unroll
    for (int i = 0; i < EPL; ++i) v[i] = __fmul_rn((float) tq_unpack(codes, cps, pl.bits, 32 * i + lane), pl.scales[vec * EPL + i]);
    if (pl.rbits == 1) {
        const float rs = pl.rscale[vec];
        const uint8_t* rb = pl.resid + vec * (size_t) (D / 8);
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const int e = 32 * i + lane, bit = (rb[e >> 3] >> (e & 7)) & 1;
            const float sgn = ((rsg[i] >> lane) & 1) ? 1.0f : -1.0f;
            v[i] = __fadd_rn(v[i], __fmul_rn(bit ? rs : -rs, sgn));
        }
    } else if (pl.rbits > 1) {
        const int rps = tq_packed_size(D, pl.rbits);
        const float rs = pl.rscale[vec];
#pragma unroll
        for (int i = 0; i < EPL; ++i) v[i] = __fadd_rn(v[i], __fmul_rn((float) tq_unpack(pl.resid + vec * rps, rps, pl.rbits, 32 * i + lane), rs));
    }
    // Walsh-Hadamard: stages h = 1 .. 16 across lanes, h = 32 .. D/2 inside the lane
#pragma unroll
    for (int h = 1; h < 32; h <<= 1) {
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const float o = __shfl_xor_sync(0xffffffffu, v[i], h);
            v[i] = (lane & h) ? __fsub_rn(o, v[i]) : __fadd_rn(v[i], o);
        }
    }
#pragma unroll
    for (int hi = 1; hi < EPL; hi <<= 1) {
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            if ((i & hi) == 0) {
                const float a = v[i], bb = v[i + hi];
                v[i] = __fadd_rn(a, bb); v[i + hi] = __fsub_rn(a, bb);
            }
        }
    }
    const float norm = __fdiv_rn(1.0f, __fsqrt_rn((float) D));
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        float r = __fmul_rn(v[i], norm);
        if ((sg[i] >> lane) & 1) r = -r;
        tq_store(out + ((size_t) head * n + p) * D + 32 * i + lane, r);
    }
}

template <typename OUT>
int32_t tq_decode_dispatch(const TqPlane& pl, int layer, int start_pos, int n, int heads, int D, int max_seq, int32_t seed_xor, bool fixed_seed, OUT* out, cudaStream_t s) {
    if (n <= 0) return SKAINET_CUDA_OK;
    const unsigned grid = (unsigned) (((int64_t) n * heads + 7) / 8);
    const int fs = fixed_seed ? 1 : 0;
    switch (D) {
        case 32: tq_decode_kernel<OUT, 1><<<grid, 256, 0, s>>>(pl, layer, start_pos, n, heads, seed_xor, fs, max_seq, out); break;
        case 64: tq_decode_kernel<OUT, 2><<<grid, 256, 0, s>>>(pl, layer, start_pos, n, heads, seed_xor, fs, max_seq, out); break;
        case 128: tq_decode_kernel<OUT, 4><<<grid, 256, 0, s>>>(pl, layer, start_pos, n, heads, seed_xor, fs, max_seq, out); break;
        case 256: tq_decode_kernel<OUT, 8><<<grid, 256, 0, s>>>(pl, layer, start_pos, n, heads, seed_xor, fs, max_seq, out); break;
        default: set_error("turboquant decode: head_dim %d not in {32,64,128,256}", D); return SKAINET_CUDA_ERR_INVALID;
    }
    SK_CUDA(cudaGetLastError());
    return SKAINET_CUDA_OK;
}

}  // namespace

int32_t launch_tq_encode(const float* rows, const TqPlane& pl, int layer, int pos, int heads, int D, int max_seq, int32_t seed_xor, cudaStream_t s, bool fixed_seed) {
    tq_encode_kernel<<<heads, D, 0, s>>>(rows, pl, layer, pos, heads, D, max_seq, seed_xor, fixed_seed ? 1 : 0);
    SK_CUDA(cudaGetLastError());
    return SKAINET_CUDA_OK;
}

int32_t launch_tq_decode(const TqPlane& pl, int layer, int start_pos, int n, int heads, int D, int max_seq, int32_t seed_xor, float* out, cudaStream_t s, bool fixed_seed) {
    return tq_decode_dispatch<float>(pl, layer, start_pos, n, heads, D, max_seq, seed_xor, fixed_seed, out, s);
}

int32_t launch_tq_decode_f16(const TqPlane& pl, int layer, int start_pos, int n, int heads, int D, int max_seq, int32_t seed_xor, __half* out, cudaStream_t s) {
    return tq_decode_dispatch<__half>(pl, layer, start_pos, n, heads, D, max_seq, seed_xor, false, out, s);
}

}  // namespace sk

using namespace sk;

extern "C" {

// Host twins of TurboQuantCodec.encode / decode for ONE vector with an explicit seed.
int32_t skainet_cuda_turboquant_encode(const float* input, int32_t n, int32_t bits, int32_t residual_bits, int32_t seed, uint8_t* codes_out,
                                       float* scales_out, uint8_t* residual_out, float* residual_scale_out) {
    SK_REQUIRE(n == 32 || n == 64 || n == 128 || n == 256, "turboquant_encode: %d elements not in {32,64,128,256}", n);
    SK_REQUIRE(bits == 2 || bits == 3 || bits == 4 || bits == 8, "bits must be 2, 3, 4, or 8, got %d", bits);
    SK_REQUIRE(residual_bits >= 0 && residual_bits <= 4, "residualBits must be 1-4 (0: no residual stage), got %d", residual_bits);
    SK_REQUIRE(input && codes_out && scales_out && (residual_bits == 0 || (residual_out && residual_scale_out)), "turboquant_encode: null pointer");
    SK_TRY(ensure_device());
    std::lock_guard<std::mutex> lk(twin_mutex());
    const size_t cps = tq_packed_size(n, bits), rps = residual_bits ? tq_packed_size(n, residual_bits) : 0;
    const size_t o_x = 0, o_sc = 1024, o_rs = 1280, o_codes = 1536, o_res = 2048, total = 2560;
    void* base = nullptr;
    SK_TRY(scratch_get(nullptr, SCRATCH_TWIN_A, total, &base));
    uint8_t* b = (uint8_t*) base;
    TqPlane pl;
    pl.codes = b + o_codes; pl.scales = (float*) (b + o_sc); pl.resid = b + o_res; pl.rscale = (float*) (b + o_rs); pl.bits = bits; pl.rbits = residual_bits;
    SK_CUDA(cudaMemcpyAsync(b + o_x, input, sizeof(float) * n, cudaMemcpyHostToDevice, nullptr));
    SK_TRY(launch_tq_encode((const float*) (b + o_x), pl, 0, 0, 1, n, 1, seed, nullptr, true));
    SK_CUDA(cudaMemcpyAsync(codes_out, pl.codes, cps, cudaMemcpyDeviceToHost, nullptr));
    SK_CUDA(cudaMemcpyAsync(scales_out, pl.scales, sizeof(float) * (n / 32), cudaMemcpyDeviceToHost, nullptr));
    if (residual_bits) {
        SK_CUDA(cudaMemcpyAsync(residual_out, pl.resid, rps, cudaMemcpyDeviceToHost, nullptr));
        SK_CUDA(cudaMemcpyAsync(residual_scale_out, pl.rscale, sizeof(float), cudaMemcpyDeviceToHost, nullptr));
    }
    SK_CUDA(cudaStreamSynchronize(nullptr));
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_turboquant_decode(const uint8_t* codes, const float* scales, const uint8_t* residual, float residual_scale, int32_t n,
                                       int32_t bits, int32_t residual_bits, int32_t seed, float* output) {
    SK_REQUIRE(n == 32 || n == 64 || n == 128 || n == 256, "turboquant_decode: %d elements not in {32,64,128,256}", n);
    SK_REQUIRE(bits == 2 || bits == 3 || bits == 4 || bits == 8, "bits must be 2, 3, 4, or 8, got %d", bits);
    SK_REQUIRE(residual_bits >= 0 && residual_bits <= 4, "residualBits must be 1-4 (0: no residual stage), got %d", residual_bits);
    SK_REQUIRE(codes && scales && output && (residual_bits == 0 || residual), "turboquant_decode: null pointer");
    SK_TRY(ensure_device());
    std::lock_guard<std::mutex> lk(twin_mutex());
    const size_t cps = tq_packed_size(n, bits), rps = residual_bits ? tq_packed_size(n, residual_bits) : 0;
    const size_t o_x = 0, o_sc = 1024, o_rs = 1280, o_codes = 1536, o_res = 2048, total = 2560;
    void* base = nullptr;
    SK_TRY(scratch_get(nullptr, SCRATCH_TWIN_A, total, &base));
    uint8_t* b = (uint8_t*) base;
    TqPlane pl;
    pl.codes = b + o_codes; pl.scales = (float*) (b + o_sc); pl.resid = b + o_res; pl.rscale = (float*) (b + o_rs); pl.bits = bits; pl.rbits = residual_bits;
    SK_CUDA(cudaMemcpyAsync(pl.codes, codes, cps, cudaMemcpyHostToDevice, nullptr));
    SK_CUDA(cudaMemcpyAsync(pl.scales, scales, sizeof(float) * (n / 32), cudaMemcpyHostToDevice, nullptr));
    if (residual_bits) {
        SK_CUDA(cudaMemcpyAsync(pl.resid, residual, rps, cudaMemcpyHostToDevice, nullptr));
        SK_CUDA(cudaMemcpyAsync(pl.rscale, &residual_scale, sizeof(float), cudaMemcpyHostToDevice, nullptr));
    }
    SK_TRY(launch_tq_decode(pl, 0, 0, 1, 1, n, 1, seed, (float*) (b + o_x), nullptr, true));
    SK_CUDA(cudaMemcpyAsync(output, b + o_x, sizeof(float) * n, cudaMemcpyDeviceToHost, nullptr));
    SK_CUDA(cudaStreamSynchronize(nullptr));
    return SKAINET_CUDA_OK;
}

}  // extern "C"
