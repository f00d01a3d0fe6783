// fp32 row and elementwise kernels of the decode path: RMSNorm, RoPE, SiLU/SwiGLU, add/mul,
// arg-max, fp32->fp16 and the availability probe. All are latency/HBM-bound; rows are handled by one
// CTA each with 128-bit loads where the row is 16-byte aligned.
//
// Contracts: native/src/f32_fused.c:255-286 (rms norm), native/src/f32_ops.c:107-114,198-211
// (binary), :222-273 (unary), native/src/skainet_smoke.c (probe),
// skainet-backends/skainet-backend-cpu/src/commonMain/kotlin/sk/ainet/exec/tensor/ops/DefaultCpuOps.kt:3042-3078 (arg max).
#include "common.cuh"

namespace sk {

// ---- block reductions ---------------------------------------------------------------------------------
__device__ __forceinline__ float block_sum(float v, float* sh) {
    v = skd::warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    float t = 0.0f;
    for (int i = 0; i < nw; ++i) t += sh[i];   // fixed order: every thread gets the same bits
    __syncthreads();
    return t;
}

// ---- RMSNorm ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rms_norm_kernel(const float* __restrict__ in, const float* __restrict__ gamma,
                                                       float* __restrict__ out, int cols, float eps) {
    __shared__ float sh[32];
    const float* x = in + (int64_t) blockIdx.x * cols;
    float* o = out + (int64_t) blockIdx.x * cols;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) { const float v = x[i]; ss += v * v; }
    ss = block_sum(ss, sh);
    const float scale = 1.0f / sqrtf(ss * (1.0f / (float) cols) + eps);
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        float v = x[i] * scale;
        if (gamma) v *= gamma[i];
        o[i] = v;
    }
}
int32_t launch_rms_norm(const float* in, const float* gamma, float* out, int rows, int cols, float eps, cudaStream_t s) {
    if (rows <= 0 || cols <= 0) return SKAINET_CUDA_OK;
    rms_norm_kernel<<<rows, 256, 0, s>>>(in, gamma, out, cols, eps);
    SK_CUDA(cudaGetLastError());
    return SKAINET_CUDA_OK;
}

// ---- elementwise -------------------------------------------------------------------------------------------
__device__ __forceinline__ float sigmoid_ref(float x) { return 1.0f / (1.0f + expf(-x)); }

__global__ void unary_kernel(int op, const float* __restrict__ in, float* __restrict__ out, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) {
        const float x = in[i];
        float r;
        switch (op) {
            case 0: r = x < 0.0f ? 0.0f : x; break;
            case 1: r = sigmoid_ref(x); break;
            case 2: r = x * sigmoid_ref(x); break;
            case 3: { const float inner = x + 0.044715f * (x * x * x); r = 0.5f * x * (1.0f + tanhf(0.7978845608f * inner)); break; }
            case 4: { const double xd = (double) x; r = (float) (0.5 * xd * (1.0 + erf(xd * 0.70710678118654752440))); break; }
            case 5: r = (float) erf((double) x); break;
            default: r = tanhf(x); break;
        }
        out[i] = r;
    }
}
int32_t launch_unary(int op, const float* in, float* out, int64_t n, cudaStream_t s) {
    if (n <= 0) return SKAINET_CUDA_OK;
    unary_kernel<<<(int) std::min<int64_t>((n + 255) / 256, 148 * 16), 256, 0, s>>>(op, in, out, n);
    SK_CUDA(cudaGetLastError());
    return SKAINET_CUDA_OK;
}

__global__ void binary_kernel(int op, const float* __restrict__ a, int am, const float* __restrict__ b, int bm,
                              float* __restrict__ out, int64_t n, int inner) {
    for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) {
        const float x = a[am == 0 ? i : (am == 1 ? 0 : i % inner)];
        const float y = b[bm == 0 ? i : (bm == 1 ? 0 : i % inner)];
        out[i] = op == 0 ? x + y : (op == 1 ? x - y : (op == 2 ? x * y : x / y));
    }
}
int32_t launch_binary(int op, const float* a, int am, const float* b, int bm, float* out, int64_t n, int inner, cudaStream_t s) {
    if (n <= 0) return SKAINET_CUDA_OK;
    binary_kernel<<<(int) std::min<int64_t>((n + 255) / 256, 148 * 16), 256, 0, s>>>(op, a, am, b, bm, out, n, inner > 0 ? inner : 1);
    SK_CUDA(cudaGetLastError());
    return SKAINET_CUDA_OK;
}

__global__ void swiglu_kernel(const float* __restrict__ g, const float* __restrict__ u, float* __restrict__ out, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x)
        out[i] = (g[i] * sigmoid_ref(g[i])) * u[i];
}
int32_t launch_swiglu(const float* g, const float* u, float* out, int64_t n, cudaStream_t s) {
    if (n <= 0) return SKAINET_CUDA_OK;
    swiglu_kernel<<<(int) std::min<int64_t>((n + 255) / 256, 148 * 16), 256, 0, s>>>(g, u, out, n);
    SK_CUDA(cudaGetLastError());
    return SKAINET_CUDA_OK;
}

// ---- RoPE ------------------------------------------------------------------------------------------------------
// One thread per (row, head, pair). The angle is evaluated in double and rounded once, so host-side
// tables built the same way give identical factors.
__global__ void rope_kernel(float* x, const int32_t* __restrict__ pos, int rows, int heads, int d, float theta, int mode) {
    const int half = d >> 1;
    const int64_t total = (int64_t) rows * heads * half;
    for (int64_t t = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; t < total; t += (int64_t) gridDim.x * blockDim.x) {
        const int i = (int) (t % half);
        const int64_t rh = t / half;
        const int r = (int) (rh / heads);
        const double ang = (double) pos[r] * pow((double) theta, -2.0 * (double) i / (double) d);
        const float c = (float) cos(ang), s = (float) sin(ang);
        float* base = x + rh * d;
        float* px = base + (mode == 0 ? 2 * i : i);
        float* py = base + (mode == 0 ? 2 * i + 1 : i + half);
        const float a = *px, b = *py;
        *px = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
        *py = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
    }
}
int32_t launch_rope(float* x, const int32_t* pos, int rows, int heads, int d, float theta, int mode, cudaStream_t s) {
    const int64_t total = (int64_t) rows * heads * (d / 2);
    if (total <= 0) return SKAINET_CUDA_OK;
    rope_kernel<<<(int) std::min<int64_t>((total + 127) / 128, 148 * 16), 128, 0, s>>>(x, pos, rows, heads, d, theta, mode);
    SK_CUDA(cudaGetLastError());
    return SKAINET_CUDA_OK;
}

// ---- arg max (lowest index on ties) ---------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ x, int cols, int32_t* __restrict__ out) {
    __shared__ float sv[32];
    __shared__ int si[32];
    const float* r = x + (int64_t) blockIdx.x * cols;
    float best = -INFINITY; int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        const float v = r[i];
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(~0u, best, o); const int oi = __shfl_xor_sync(~0u, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        best = lane < nw ? sv[lane] : -INFINITY; bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(~0u, best, o); const int oi = __shfl_xor_sync(~0u, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
    }
}
int32_t launch_argmax(const float* x, int rows, int cols, int32_t* out, cudaStream_t s) {
    if (rows <= 0) return SKAINET_CUDA_OK;
    argmax_kernel<<<rows, 1024, 0, s>>>(x, cols, out);
    SK_CUDA(cudaGetLastError());
    return SKAINET_CUDA_OK;
}

// ---- conversions, probe ------------------------------------------------------------------------------------------
__global__ void f32_to_f16_kernel(const float* __restrict__ in, __half* __restrict__ out, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x)
        out[i] = __float2half_rn(in[i]);
}
int32_t launch_f32_to_f16(const float* in, uint16_t* out, int64_t n, cudaStream_t s) {
    if (n <= 0) return SKAINET_CUDA_OK;
    f32_to_f16_kernel<<<(int) std::min<int64_t>((n + 255) / 256, 148 * 32), 256, 0, s>>>(in, (__half*) out, n);
    SK_CUDA(cudaGetLastError());
    return SKAINET_CUDA_OK;
}

__global__ void smoke_kernel(const float* __restrict__ in, float* __restrict__ out, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = 2.0f * in[i];
}
int32_t launch_smoke(const float* in, float* out, int n, cudaStream_t s) {
    if (n <= 0) return SKAINET_CUDA_OK;
    smoke_kernel<<<(n + 255) / 256, 256, 0, s>>>(in, out, n);
    SK_CUDA(cudaGetLastError());
    return SKAINET_CUDA_OK;
}

}  // namespace sk
