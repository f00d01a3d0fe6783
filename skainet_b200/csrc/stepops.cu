// Step operators shared by the decoder runtime and the fused-op entry points (see stepops.cuh), and the C entries
// a graph executor's fused-op handlers call: fused_qkv_proj and fused_swiglu_ffn
// (skainet-compile/skainet-compile-opt/src/commonMain/kotlin/sk/ainet/compile/opt/passes/LLMFusionPass.kt:17-23,86,117;
// CPU decompositions in skainet-compile/skainet-compile-dag/src/commonMain/kotlin/sk/ainet/lang/graph/exec/LLMFusedOpHandlers.kt:27-68,86-196).
#include "stepops.cuh"
#include "tma.cuh"
#include "matvec_fused.cuh"

namespace sk {


// Activation prep between two matvecs: (optional RMSNorm | SwiGLU) then quantization for the next
// matvec, q8 per 256 (K-quant weights) or the two-term split per 32 (Q8_0 weights).
// grid (ceil(n/2048), rows), 256 threads: a CTA quantizes 2048 consecutive elements of one row (eight
// per thread; a warp = one 256-block, four lanes = one 32-block). For RMSNorm every CTA of the row sums
// the whole row's squares itself (n fp32 values out of L2) instead of synchronising across CTAs.
// in: [rows][n] (PK_SWIGLU: [rows][2n] = gate | up).
template <int MODE, bool SPLIT>
__global__ void __launch_bounds__(256)
prep_kernel(const float* __restrict__ in, const float* __restrict__ gamma, float eps, int n, ActQ8K oq, ActSplit os) {
    __shared__ float red[8];
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    const int row = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* x = in + (size_t) row * (MODE == PK_SWIGLU ? 2 * n : n);
    float nscale = 1.0f;
    if (MODE == PK_NORM) {
        float ss = 0.0f;
        for (int i0 = threadIdx.x; i0 < (n >> 2); i0 += 256 * 4) {      // four loads in flight per thread
            float4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int i = i0 + j * 256;
                v[j] = i < (n >> 2) ? __ldg(reinterpret_cast<const float4*>(x) + i) : make_float4(0, 0, 0, 0);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
        }
        ss = skd::warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float t = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) t += red[i];
        nscale = 1.0f / sqrtf(t * (1.0f / (float) n) + eps);
    }
    const int n8 = n >> 3;
    const int c = blockIdx.x * 256 + threadIdx.x;          // this thread's 8-element chunk of the row
    const bool ok = c < n8;
    const int cc = ok ? c : 0;
    float v[8];
    {
        const float4 a = __ldg(reinterpret_cast<const float4*>(x) + 2 * cc), b = __ldg(reinterpret_cast<const float4*>(x) + 2 * cc + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    if (MODE == PK_NORM) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * cc), b = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * cc + 1);
        const float g[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = (v[i] * nscale) * g[i];
    }
    if (MODE == PK_SWIGLU) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(x + n) + 2 * cc), b = __ldg(reinterpret_cast<const float4*>(x + n) + 2 * cc + 1);
        const float u[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = (v[i] * (1.0f / (1.0f + expf(-v[i])))) * u[i];
    }
    if (!ok) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.0f;
    }
    if (SPLIT) {
        ActSplit o = os;
        o.hi += (size_t) row * n; o.lo += (size_t) row * n; o.d += (size_t) row * (n >> 5);
        skd::quant_split_regs(v, o, cc >> 2, cc & 3, ok);
    } else if (c - lane < n8) {       // warp-uniform: the warp's 256-block lies inside the row
        const int blk = cc >> 5;
        skd::quant_q8k_regs(v, oq.q + (size_t) row * n + (size_t) blk * 256, oq.d + (size_t) row * (n >> 8) + blk,
                            oq.bsums + (size_t) row * (n >> 5) + (size_t) blk * 8, lane);
    }
}


template <int MODE>
static int32_t launch_prep_mode(const float* in, const float* gamma, float eps, int rows, int n, bool split, void* act, cudaStream_t s) {
    ActQ8K oq = {nullptr, nullptr, nullptr}; ActSplit os = {nullptr, nullptr, nullptr};
    if (split) {
        os = act_split_layout(act, rows, n);
        SK_CUDA(launch_pdl(prep_kernel<MODE, true>, dim3((n + 2047) / 2048, rows), dim3(256), 0, s, in, gamma, eps, n, oq, os));
    } else {
        oq = act_q8k_layout(act, rows, n);
        SK_CUDA(launch_pdl(prep_kernel<MODE, false>, dim3((n + 2047) / 2048, rows), dim3(256), 0, s, in, gamma, eps, n, oq, os));
    }
    return SKAINET_CUDA_OK;
}

int32_t launch_prep(int mode, const float* in, const float* gamma, float eps, int rows, int n, bool split, void* act, cudaStream_t s) {
    switch (mode) {
        case PK_NORM: return launch_prep_mode<PK_NORM>(in, gamma, eps, rows, n, split, act, s);
        case PK_SWIGLU: return launch_prep_mode<PK_SWIGLU>(in, gamma, eps, rows, n, split, act, s);
        default: return launch_prep_mode<PK_QUANT>(in, gamma, eps, rows, n, split, act, s);
    }
}

__global__ void add_rows_kernel(float* __restrict__ x, const float* __restrict__ y, int64_t n) {
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) x[i] += y[i];
}


int32_t launch_linear_q(const Weight& w, void* act, int rows, float* y, float* resid_inplace, float* tmp, cudaStream_t s) {
    if (rows == 1) {
        MatvecIn in;
        if (w.enc == SKAINET_ENC_Q8_0) in.split = act_split_layout(act, 1, w.cols); else in.q8 = act_q8k_layout(act, 1, w.cols);
        const int32_t st = launch_matvec_fused(w, in, PREP_QUANTIZED, resid_inplace ? resid_inplace : y, resid_inplace, s);
        if (st != 1) return st;
    }
    if (rows >= 2) {
        const int32_t st = w.enc == SKAINET_ENC_Q8_0
            ? launch_gemm_mma_q8(w, act_split_layout(act, rows, w.cols), rows, resid_inplace ? resid_inplace : y, resid_inplace, s)
            : launch_gemm_mma(w, act_q8k_layout(act, rows, w.cols), rows, resid_inplace ? resid_inplace : y, resid_inplace, s);
        if (st != 1) return st;
    }
    if (w.enc == SKAINET_ENC_Q6_K)            // a Q6_K tensor inside a K-quant model: its kernels add the residual themselves
        return launch_matvec_kq(w, nullptr, act_q8k_layout(act, rows, w.cols), rows, resid_inplace ? resid_inplace : y, SKAINET_ACT_NATIVE, s, resid_inplace);
    float* out = resid_inplace ? tmp : y;
    SK_TRY(launch_matvec(w, nullptr, act, rows, out, SKAINET_ACT_NATIVE, s));
    if (resid_inplace) {
        const int64_t n = (int64_t) rows * w.rows;
        SK_CUDA(launch_pdl(add_rows_kernel, dim3((unsigned) std::min<int64_t>((n + 255) / 256, 1184)), dim3(256), 0, s, resid_inplace, (const float*) out, n));
    }
    return SKAINET_CUDA_OK;
}

// rows of `a` then rows of `b` (then `c`) in one resident weight; the parts must share cols and encoding.
int32_t weight_concat_rows(const Weight* a, const Weight* b, const Weight* c, Weight** out) {
    const int rows = a->rows + b->rows + (c ? c->rows : 0);
    SK_TRY(weight_alloc(a->enc, rows, a->cols, out));
    Weight* w = *out;
    const Weight* parts[3] = {a, b, c};
    // bytes per block of each plane (see the Weight record): main codes, header / scales, extra bit plane, aux scale plane
    size_t pb[4] = {128, 16, 0, 0};
    if (a->enc == SKAINET_ENC_Q8_0) { pb[0] = 32; pb[1] = 2; }
    else if (a->enc == SKAINET_ENC_Q5_K) pb[2] = 32;
    else if (a->enc == SKAINET_ENC_Q6_K) { pb[2] = 64; pb[3] = 2; }
    size_t row_off = 0;
    for (int i = 0; i < 3; ++i) {
        const Weight* p = parts[i];
        if (!p) continue;
        const size_t nb = (size_t) p->rows * p->bpr, off = row_off * a->bpr;
        uint8_t* dst[4] = {w->qs, w->hdr, w->extra, w->aux};
        const uint8_t* src[4] = {p->qs, p->hdr, p->extra, p->aux};
        for (int k = 0; k < 4; ++k)
            if (pb[k]) SK_CUDA(cudaMemcpy(dst[k] + off * pb[k], src[k], nb * pb[k], cudaMemcpyDeviceToDevice));
        row_off += p->rows;
    }
    return SKAINET_CUDA_OK;
}

// rows [r0, r0 + n) of src[m][stride] -> dst[m][n]
__global__ void slice_rows_kernel(const float* __restrict__ src, float* __restrict__ dst, int m, int stride, int r0, int n) {
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < (int64_t) m * n; i += (int64_t) gridDim.x * blockDim.x)
        dst[i] = src[(i / n) * stride + r0 + (i % n)];
}

// src[m][n] -> columns [r0, r0 + n) of dst[m][stride]
__global__ void scatter_rows_kernel(const float* __restrict__ src, float* __restrict__ dst, int m, int stride, int r0, int n) {
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < (int64_t) m * n; i += (int64_t) gridDim.x * blockDim.x)
        dst[(i / n) * stride + r0 + (i % n)] = src[i];
}
int32_t launch_scatter_rows(const float* src, float* dst, int m, int stride, int r0, int n, cudaStream_t s) {
    const int64_t total = (int64_t) m * n;
    SK_CUDA(launch_pdl(scatter_rows_kernel, dim3((unsigned) std::min<int64_t>((total + 255) / 256, 2368)), dim3(256), 0, s, src, dst, m, stride, r0, n));
    return SKAINET_CUDA_OK;
}

// Quantized (optionally RMS-normalised) activation rows of x into the stream's activation scratch.
static int32_t prepare_rows(const Weight& w, const float* x, const float* gamma, float eps, int m, cudaStream_t s, void** act) {
    const size_t need = act_scratch_bytes(w.enc, SKAINET_ACT_NATIVE, m, w.cols);
    SK_TRY(scratch_get(s, SCRATCH_ACT, need, act));
    return launch_prep(gamma ? PK_NORM : PK_QUANT, x, gamma, eps, m, w.cols, w.enc == SKAINET_ENC_Q8_0, *act, s);
}

}  // namespace sk

using namespace sk;

extern "C" {

int32_t skainet_cuda_weight_concat_rows(skainet_weight_t a, skainet_weight_t b, skainet_weight_t c, skainet_weight_t* out) {
    SK_REQUIRE(out != nullptr, "weight_concat_rows: null output");
    *out = 0;
    Weight *wa = weight_from_handle(a), *wb = wa ? weight_from_handle(b) : nullptr, *wc = nullptr;
    if (!wa || !wb) return SKAINET_CUDA_ERR_HANDLE;
    if (c != 0 && !(wc = weight_from_handle(c))) return SKAINET_CUDA_ERR_HANDLE;
    for (const Weight* p : {wb, wc})
        if (p) SK_REQUIRE(p->enc == wa->enc && p->cols == wa->cols, "weight_concat_rows: parts differ in encoding or input dimension");
    SK_TRY(ensure_device());
    Weight* w = nullptr;
    SK_TRY(weight_concat_rows(wa, wb, wc, &w));
    SK_CUDA(cudaDeviceSynchronize());
    *out = weight_to_handle(w);
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_fused_qkv_proj_dev(skainet_weight_t wqkv, int32_t q_rows, int32_t k_rows, int32_t v_rows, const float* x_dev,
                                        const float* gamma_dev, float eps, int32_t m, float* q_dev, float* k_dev, float* v_dev,
                                        skainet_stream_t stream) {
    Weight* w = weight_from_handle(wqkv);
    if (!w) return SKAINET_CUDA_ERR_HANDLE;
    SK_REQUIRE(w->enc == SKAINET_ENC_Q4_K || w->enc == SKAINET_ENC_Q8_0 || w->enc == SKAINET_ENC_Q6_K, "fused_qkv_proj: encoding %d not supported", w->enc);
    SK_REQUIRE(q_rows > 0 && k_rows > 0 && v_rows > 0 && q_rows + k_rows + v_rows == w->rows,
               "fused_qkv_proj: %d + %d + %d output rows, the merged weight has %d", q_rows, k_rows, v_rows, w->rows);
    SK_REQUIRE(m >= 0, "fused_qkv_proj: negative row count %d", m);
    if (m == 0) return SKAINET_CUDA_OK;
    SK_REQUIRE(x_dev && q_dev && k_dev && v_dev, "fused_qkv_proj: null pointer");
    SK_REQUIRE((((uintptr_t) x_dev | (uintptr_t) gamma_dev) & 15) == 0, "fused_qkv_proj: x and gamma must be 16-byte aligned");
    SK_TRY(ensure_device());
    cudaStream_t s = as_stream(stream);
    // one row whose three outputs already lie back to back: the matvec writes them directly
    const bool contiguous = m == 1 && k_dev == q_dev + q_rows && v_dev == k_dev + k_rows;
    float* y = q_dev;
    if (!contiguous) {
        void* tmp = nullptr;
        SK_TRY(scratch_get(s, SCRATCH_FFN, sizeof(float) * (size_t) m * w->rows, &tmp));
        y = (float*) tmp;
    }
    void* act = nullptr;
    SK_TRY(prepare_rows(*w, x_dev, gamma_dev, eps, m, s, &act));
    SK_TRY(launch_linear_q(*w, act, m, y, nullptr, nullptr, s));
    if (!contiguous) {
        const int offs[3] = {0, q_rows, q_rows + k_rows}, ns[3] = {q_rows, k_rows, v_rows};
        float* outs[3] = {q_dev, k_dev, v_dev};
        for (int i = 0; i < 3; ++i) {
            const int64_t n = (int64_t) m * ns[i];
            SK_CUDA(launch_pdl(slice_rows_kernel, dim3((unsigned) std::min<int64_t>((n + 255) / 256, 2368)), dim3(256), 0, s, (const float*) y, outs[i], m,
                               w->rows, offs[i], ns[i]));
        }
    }
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_fused_swiglu_ffn_dev(skainet_weight_t w_gate_up, skainet_weight_t w_down, const float* x_dev, const float* gamma_dev,
                                          float eps, int32_t m, const float* resid_dev, float* out_dev, skainet_stream_t stream) {
    Weight* wgu = weight_from_handle(w_gate_up);
    Weight* wd = wgu ? weight_from_handle(w_down) : nullptr;
    if (!wgu || !wd) return SKAINET_CUDA_ERR_HANDLE;
    for (const Weight* w : {wgu, wd})
        SK_REQUIRE(w->enc == SKAINET_ENC_Q4_K || w->enc == SKAINET_ENC_Q8_0 || w->enc == SKAINET_ENC_Q6_K, "fused_swiglu_ffn: encoding %d not supported", w->enc);
    // gate|up and down may differ in encoding (a Q6_K ffn_down behind Q4_K gate and up, as K-quant files carry them), as long
    // as both take the same activation form
    SK_REQUIRE((wgu->enc == SKAINET_ENC_Q8_0) == (wd->enc == SKAINET_ENC_Q8_0), "fused_swiglu_ffn: Q8_0 and K-quant weights cannot be mixed");
    SK_REQUIRE(wgu->rows % 2 == 0 && wgu->rows / 2 == wd->cols, "fused_swiglu_ffn: gate|up has %d rows, down takes %d inputs", wgu->rows, wd->cols);
    SK_REQUIRE(m >= 0, "fused_swiglu_ffn: negative row count %d", m);
    if (m == 0) return SKAINET_CUDA_OK;
    SK_REQUIRE(x_dev && out_dev, "fused_swiglu_ffn: null pointer");
    SK_REQUIRE((((uintptr_t) x_dev | (uintptr_t) gamma_dev) & 15) == 0, "fused_swiglu_ffn: x and gamma must be 16-byte aligned");
    SK_TRY(ensure_device());
    cudaStream_t s = as_stream(stream);
    const int F = wd->cols;
    // scratch: gate|up rows, and (shapes without a residual epilogue) one output-sized row block
    void* tmp = nullptr;
    const size_t gu_bytes = (sizeof(float) * (size_t) m * 2 * F + 255) & ~(size_t) 255;
    SK_TRY(scratch_get(s, SCRATCH_FFN, gu_bytes + sizeof(float) * (size_t) m * wd->rows, &tmp));
    float* gu = (float*) tmp;
    float* spare = (float*) ((uint8_t*) tmp + gu_bytes);
    // the activation scratch is sized once for both quantized forms it will hold
    void* act = nullptr;
    const size_t need = std::max(act_scratch_bytes(wgu->enc, SKAINET_ACT_NATIVE, m, wgu->cols), act_scratch_bytes(wd->enc, SKAINET_ACT_NATIVE, m, F));
    SK_TRY(scratch_get(s, SCRATCH_ACT, need, &act));
    SK_TRY(launch_prep(gamma_dev ? PK_NORM : PK_QUANT, x_dev, gamma_dev, eps, m, wgu->cols, wgu->enc == SKAINET_ENC_Q8_0, act, s));
    SK_TRY(launch_linear_q(*wgu, act, m, gu, nullptr, nullptr, s));
    if (resid_dev && resid_dev != out_dev) SK_CUDA(cudaMemcpyAsync(out_dev, resid_dev, sizeof(float) * (size_t) m * wd->rows, cudaMemcpyDeviceToDevice, s));
    // One row into a ring-sized Q4_K down projection of at most 8192 inputs: the ring kernel computes silu(gate) * up and
    // quantizes it in its own prologue, as the decoder's step does.
    if (m == 1 && wd->enc == SKAINET_ENC_Q4_K && F <= 8192 && matvec_uses_ring(*wd, PREP_SWIGLU_F32)) {
        MatvecIn in; in.x = gu;
        const int32_t st = launch_matvec_fused(*wd, in, PREP_SWIGLU_F32, out_dev, resid_dev ? out_dev : nullptr, s);
        if (st != 1) return st;
    }
    SK_TRY(launch_prep(PK_SWIGLU, gu, nullptr, 0.0f, m, F, wd->enc == SKAINET_ENC_Q8_0, act, s));       // silu(gate) * up, quantized for down
    if (resid_dev == nullptr) return launch_linear_q(*wd, act, m, out_dev, nullptr, nullptr, s);
    return launch_linear_q(*wd, act, m, nullptr, out_dev, spare, s);
}

}  // extern "C"
