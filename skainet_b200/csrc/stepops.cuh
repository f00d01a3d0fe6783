// The operators a decode step strings between its matvecs, shared by the decoder runtime (llama.cu) and by
// the graph-level fused-op entry points (stepops.cu): activation prep kernels (RMSNorm | SwiGLU fused with the
// activation quantizer), the linear over an already quantized activation, and row concatenation of weights.
#pragma once
#include "common.cuh"
#include "actquant.cuh"
#include "matvec_fused.cuh"

namespace sk {

enum { PK_QUANT = 0, PK_NORM = 1, PK_SWIGLU = 2 };

// act <- quantize(mode(in)) for `rows` rows of n elements (PK_SWIGLU: in is [rows][2n] = gate | up). split selects the
// two-term form Q8_0 weights take; otherwise int8 per 256 (K-quant weights). act is laid out by act_*_layout(act, rows, n).
int32_t launch_prep(int mode, const float* in, const float* gamma, float eps, int rows, int n, bool split, void* act, cudaStream_t s);

// y[rows][w.rows] (= resid_inplace +) W . act for activation rows already quantized into act. With a residual the
// result is added in place into resid_inplace (y is ignored); tmp must hold rows * w.rows floats for the shapes whose
// kernels have no residual epilogue.
int32_t launch_linear_q(const Weight& w, void* act, int rows, float* y, float* resid_inplace, float* tmp, cudaStream_t s);

// src[m][n] into columns [r0, r0 + n) of dst[m][stride]
int32_t launch_scatter_rows(const float* src, float* dst, int m, int stride, int r0, int n, cudaStream_t s);

// rows of a, then b (then c, may be null) in one new resident weight; the parts must share cols and encoding.
int32_t weight_concat_rows(const Weight* a, const Weight* b, const Weight* c, Weight** out);

}  // namespace sk
