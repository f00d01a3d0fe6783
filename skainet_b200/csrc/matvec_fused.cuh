// Interface of the fused single-row matvec (matvec_fused.cu).
#pragma once
#include "common.cuh"
#include "actquant.cuh"
#include "comm.cuh"

namespace sk {

// How the activation reaches the kernel.
enum { PREP_QUANTIZED = 0,   // already quantized in global memory (q8 for K-quants, split for Q8_0)
       PREP_F32 = 1,         // fp32 row, quantized inside the kernel
       PREP_NORM_F32 = 2,    // fp32 row, RMS-normalised with gamma and eps, then quantized
       PREP_SWIGLU_F32 = 3 };  // x = gate | up (2 * cols floats): silu(gate) * up, then quantized (ring kernel, K-quant weights)
enum { EPI_STORE = 0, EPI_ADD = 1,     // y = W x   |   y = resid + W x
       EPI_PEER = 2 };                 // (resid +) W x stored into every tensor-parallel rank's inbox instead of y

struct MatvecIn {
    const float* x = nullptr;       // PREP_F32 / PREP_NORM_F32
    const float* gamma = nullptr;   // PREP_NORM_F32
    float eps = 0.0f;
    ActQ8K q8 = {nullptr, nullptr, nullptr};       // PREP_QUANTIZED, K-quant weights
    ActSplit split = {nullptr, nullptr, nullptr};  // PREP_QUANTIZED, Q8_0 weights
};

// y[rows] (= resid +) W . prep(x). Returns SKAINET_CUDA_OK, an error status, or 1 when the shape is
// outside what the kernel takes (the caller then uses the general kernels).
// With a peer-output descriptor (tensor parallelism, Q4_K, activation already quantized) the result rows go to the
// group's inboxes from the kernel's own epilogue and y is not written.
int32_t launch_matvec_fused(const Weight& w, const MatvecIn& in, int prep, float* y, const float* resid, cudaStream_t s,
                            const PeerOut* peer = nullptr);

// Whether launch_matvec_fused hands this weight to the ring kernel (by size and by the form the activation arrives in).
bool matvec_uses_ring(const Weight& w, int prep);

// matvec_ring.cu: the persistent ring kernel for large weights, same activation forms and return convention.
int32_t launch_matvec_ring(const Weight& w, const MatvecIn& in, int prep, float* y, const float* resid, cudaStream_t s,
                           const PeerOut* peer = nullptr);
// gemm_mma.cu: y[m][w.rows] (= resid +) for m >= 2 quantized activation rows on the tensor cores; 1 = not taken
int32_t launch_gemm_mma(const Weight& w, ActQ8K a, int m, float* y, const float* resid, cudaStream_t s);
int32_t launch_gemm_mma_q8(const Weight& w, ActSplit a, int m, float* y, const float* resid, cudaStream_t s);
// Fewest activation rows sent to the tcgen05 kernel. Its call has a floor (activation tile preparation + one wave of
// 128 x 128 tiles): measured per call on the 25 MB shapes, tcgen05 / mma.sync: 128 rows 86 / 64 us, 256 rows 108 / 95,
// 384 rows 111 / 131, 512 rows 132 / 176.
constexpr int TC_MIN_ROWS = 288;
// gemm_ring.cu: 2..8 activation rows over a Q4_K weight through the persistent ring; 1 = not taken
int32_t launch_rows_ring(const Weight& w, ActQ8K a, int m, float* y, const float* resid, cudaStream_t s);
// gemm_tc.cu: the same for m >= 128 on tcgen05 with TMEM accumulators; 1 = not taken
int32_t launch_gemm_tc(const Weight& w, ActQ8K a, int m, float* y, const float* resid, cudaStream_t s);

}  // namespace sk
