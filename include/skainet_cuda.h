/*
 * skainet_cuda.h — C ABI of libskainet_cuda.so, the sm_100a (B200) kernel library behind SKaiNET's
 * kernel SPI (skainet-backends/skainet-backend-api). Plain pointers and sizes only.
 *
 * Two groups of entry points:
 *
 *  1. DROP-IN TWINS of the reference's native C ABI
 *     (skainet-backends/skainet-backend-native-cpu/native/include/skainet_kernels.h). Same argument
 *     lists, HOST pointers, caller owns all memory, nothing is retained past return. The one
 *     difference: they return an int32_t status instead of void (the reference has no error
 *     channel; a GPU backend needs one). These are what a JNI shim in the style of
 *     skainet-backends/skainet-backend-jni-cpu/native/skainet_jni.c binds 1:1.
 *
 *  2. The RESIDENT API: weights uploaded once to HBM (-> opaque handle), activations and the KV
 *     cache kept on the device, every call taking an optional CUDA stream. This is what a decode
 *     loop uses; the twins above are built on it.
 *
 * Conventions: every function returns SKAINET_CUDA_OK (0) or a negative status and never aborts the
 * process; skainet_cuda_last_error() gives the calling thread's last message. There is no CPU
 * fallback anywhere: without a usable GPU every compute entry returns SKAINET_CUDA_ERR_NODEVICE.
 * Thread safety: entry points may be called from several threads; calls that share a stream are
 * ordered on it, calls on different streams use separate scratch.
 */
#ifndef SKAINET_CUDA_H
#define SKAINET_CUDA_H

#include <stdint.h>

#if defined(__GNUC__) || defined(__clang__)
#  define SKAINET_CUDA_API __attribute__((visibility("default")))
#else
#  define SKAINET_CUDA_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes --------------------------------------------------------------------------- */
#define SKAINET_CUDA_OK             0
#define SKAINET_CUDA_ERR_INVALID   (-1)  /* bad argument; the Kotlin side raises IllegalArgumentException */
#define SKAINET_CUDA_ERR_CUDA      (-2)  /* a CUDA runtime call failed (message in last_error)        */
#define SKAINET_CUDA_ERR_NODEVICE  (-3)  /* no usable GPU: provider.isAvailable() == false            */
#define SKAINET_CUDA_ERR_OOM       (-4)  /* device or host allocation failed                          */
#define SKAINET_CUDA_ERR_HANDLE    (-5)  /* unknown / freed weight, cache or model handle             */
#define SKAINET_CUDA_ERR_TIMEOUT   (-6)  /* a bounded device-side wait gave up                        */
#define SKAINET_CUDA_ERR_COMM      (-7)  /* collective library unavailable or failed                  */

/* ---- encodings, weight orders, activation modes ---------------------------------------------- */
#define SKAINET_ENC_Q8_0  8    /* ggml Q8_0: 34-byte blocks of 32 (f16 d, 32 int8)                    */
#define SKAINET_ENC_Q4_K  12   /* ggml Q4_K: 144-byte super-blocks of 256                             */
#define SKAINET_ENC_Q5_K  13   /* ggml Q5_K: 176-byte super-blocks of 256                             */
#define SKAINET_ENC_Q6_K  14   /* ggml Q6_K: 210-byte super-blocks of 256                             */

/* Byte order of a packed [out, in] weight handed to upload (KernelKey layout classes,
 * skainet-backends/skainet-backend-api/src/commonMain/kotlin/sk/ainet/backend/api/kernel/KernelKey.kt:77-90). */
#define SKAINET_ORDER_ROW_MAJOR   0   /* BLOCKED_ROW_MAJOR: (o * blocks_per_row + b), GGUF file order  */
#define SKAINET_ORDER_INPUT_MAJOR 1   /* BLOCKED_INPUT_MAJOR ("feed order"): (b * out + o)             */

/* How the activation enters the integer dot.
 * NATIVE follows the reference kernel of the weight's format: Q4_K / Q6_K quantize each
 * 256-element activation block to int8 with one scale (native/src/q4k_matmul.c:74-92,
 * native/src/q6k_matmul.c:53-67); Q8_0 keeps fp32 activations (native/src/q8_0_matmul.c:61-67), which this
 * library carries as an exact two-term int8 split (hi*128+lo, 15 bits) per 32-element block; Q5_K keeps
 * fp32 activations as they are (native/src/q5k_matmul.c:93-215).
 * F32 is the exact-float arithmetic of the scalar Kotlin kernels
 * (skainet-backends/skainet-backend-cpu/src/commonMain/kotlin/sk/ainet/exec/kernel/ScalarQ4_KMatmulKernel.kt:15-82). */
#define SKAINET_ACT_NATIVE 0
#define SKAINET_ACT_F32    1

typedef int64_t skainet_weight_t;   /* opaque handle of a device-resident packed weight */
typedef int64_t skainet_kv_t;       /* opaque handle of a device-resident KV-cache store    */
typedef void*   skainet_stream_t;   /* a cudaStream_t, or NULL for the default stream   */

/* ---- library / device ------------------------------------------------------------------------ */
SKAINET_CUDA_API const char* skainet_cuda_last_error(void);
SKAINET_CUDA_API const char* skainet_cuda_version(void);
SKAINET_CUDA_API int32_t skainet_cuda_device_count(void);
/* Select the device this thread's later calls run on (default 0). */
SKAINET_CUDA_API int32_t skainet_cuda_set_device(int32_t device);
/* Device facts a host needs for sizing: [0]=SM count, [1]=L2 bytes, [2]=total HBM bytes, [3]=cc major*10+minor. */
SKAINET_CUDA_API int32_t skainet_cuda_device_info(int64_t* out4);

/* Synchronises the device and reports SKAINET_CUDA_ERR_TIMEOUT if any kernel since the last call gave
 * up a bounded wait (its outputs are then invalid); clears the condition. The reference has no
 * counterpart: its kernels cannot time out. */
SKAINET_CUDA_API int32_t skainet_cuda_device_status(void);

/* ---- 1. drop-in twins (HOST pointers) -------------------------------------------------------- */

/* Availability probe, out[i] = 2*in[i] computed on the GPU.
 * Replaces skainet_smoke_double, native/include/skainet_kernels.h:37 (used by
 * skainet-backends/skainet-backend-jni-cpu/src/main/kotlin/sk/ainet/exec/kernel/jni/JniKernelProvider.kt:36-45). */
SKAINET_CUDA_API int32_t skainet_cuda_smoke_double(const float* input, float* output, int32_t length);

/* Q4_K matvec, feed-order weight. Replaces skainet_q4k_matmul, skainet_kernels.h:57-66
 * (SPI Q4KMatmulKernel.kt:54-59). input_dim % 256 != 0 -> ERR_INVALID; input_dim <= 0 or
 * output_dim <= 0 -> OK with the output untouched (native/src/q4k_matmul.c:326). */
SKAINET_CUDA_API int32_t skainet_cuda_q4k_matmul(const float* input, int32_t input_offset,
    const uint8_t* weight, int32_t weight_byte_offset, int32_t input_dim, int32_t output_dim,
    float* output, int32_t output_offset);
/* Row-major (GGUF file order) weight. Replaces skainet_q4k_matmul_rm, skainet_kernels.h:80-89. */
SKAINET_CUDA_API int32_t skainet_cuda_q4k_matmul_rm(const float* input, int32_t input_offset,
    const uint8_t* weight, int32_t weight_byte_offset, int32_t input_dim, int32_t output_dim,
    float* output, int32_t output_offset);
/* Q8_0 matvec, feed order. Replaces skainet_q8_0_matmul, skainet_kernels.h:327-336
 * (SPI Q8_0MatmulKernel.kt:42-47). input_dim % 32 != 0 -> ERR_INVALID; input_dim <= 0 zeroes the
 * output (native/src/q8_0_matmul.c:175-179). */
SKAINET_CUDA_API int32_t skainet_cuda_q8_0_matmul(const float* input, int32_t input_offset,
    const uint8_t* weight, int32_t weight_byte_offset, int32_t input_dim, int32_t output_dim,
    float* output, int32_t output_offset);
/* Row-major. Replaces skainet_q8_0_matmul_rm, skainet_kernels.h:179-188. */
SKAINET_CUDA_API int32_t skainet_cuda_q8_0_matmul_rm(const float* input, int32_t input_offset,
    const uint8_t* weight, int32_t weight_byte_offset, int32_t input_dim, int32_t output_dim,
    float* output, int32_t output_offset);

/* Q6_K matvec (int8 activations per 256, integer group dots), feed order and row-major. Replace skainet_q6k_matmul and
 * skainet_q6k_matmul_rm, skainet_kernels.h:135-166 (SPI Q6KMatmulKernel.kt, KernelProvider.kt:86). Contract as the Q4_K
 * twins: input_dim % 256 != 0 -> ERR_INVALID; input_dim <= 0 or output_dim <= 0 -> OK with the output untouched
 * (native/src/q6k_matmul.c:284). */
SKAINET_CUDA_API int32_t skainet_cuda_q6k_matmul(const float* input, int32_t input_offset,
    const uint8_t* weight, int32_t weight_byte_offset, int32_t input_dim, int32_t output_dim,
    float* output, int32_t output_offset);
SKAINET_CUDA_API int32_t skainet_cuda_q6k_matmul_rm(const float* input, int32_t input_offset,
    const uint8_t* weight, int32_t weight_byte_offset, int32_t input_dim, int32_t output_dim,
    float* output, int32_t output_offset);
/* Q5_K matvec (fp32 activations), feed order and row-major. Replace skainet_q5k_matmul and skainet_q5k_matmul_rm,
 * skainet_kernels.h:105-114,251-260 (SPI Q5KMatmulKernel.kt, KernelProvider.kt:92); same contract
 * (native/src/q5k_matmul.c:264). */
SKAINET_CUDA_API int32_t skainet_cuda_q5k_matmul(const float* input, int32_t input_offset,
    const uint8_t* weight, int32_t weight_byte_offset, int32_t input_dim, int32_t output_dim,
    float* output, int32_t output_offset);
SKAINET_CUDA_API int32_t skainet_cuda_q5k_matmul_rm(const float* input, int32_t input_offset,
    const uint8_t* weight, int32_t weight_byte_offset, int32_t input_dim, int32_t output_dim,
    float* output, int32_t output_offset);

/* out[r,c] = in[r,c] / sqrt(mean(in[r,:]^2) + eps) * gamma[c]; gamma may be NULL.
 * Replaces skainet_f32_rms_norm, skainet_kernels.h:574-576 (SPI Fp32FusedKernels.kt:46-52). */
SKAINET_CUDA_API int32_t skainet_cuda_f32_rms_norm(const float* in, const float* gamma, float* out,
    int32_t rows, int32_t cols, float eps);

/* softmax(q k^T scale + rules + mask) v with grouped-query heads; q/out [batch,heads,seq_q,head_dim],
 * k/v [batch,kv_heads,seq_kv,head_dim], all fp32 on the host. Rules: causal, sliding window with
 * right_context, per-batch key lengths (NULL = none), dense additive mask broadcast over mask_* dims
 * (NULL = none). Replaces skainet_f32_sdpa, skainet_kernels.h:578-585 (SPI Fp32FusedKernels.kt:75-84).
 * head_dim must be 64 or 128 (ERR_INVALID otherwise). K and V are carried on the device in fp32 by
 * this entry, so it is value-compatible with the reference; the f16-cache kernel is the resident one. */
SKAINET_CUDA_API int32_t skainet_cuda_f32_sdpa(const float* q, const float* k, const float* v, float* out,
    int32_t batch, int32_t heads, int32_t kv_heads, int32_t seq_q, int32_t seq_kv, int32_t head_dim,
    float scale, int32_t causal, int32_t window, int32_t right_context, const int32_t* lengths,
    const float* mask, int32_t mask_b, int32_t mask_h, int32_t mask_q, int32_t mask_k);

/* Elementwise. op/mode numbering as the reference: unary {0 relu,1 sigmoid,2 silu,3 gelu(tanh),
 * 4 gelu(erf),5 erf,6 tanh}; binary {0 add,1 sub,2 mul,3 div} with modes {0 full,1 scalar,2 bias}.
 * Replace skainet_f32_unary / skainet_f32_binary, skainet_kernels.h:530-537. */
SKAINET_CUDA_API int32_t skainet_cuda_f32_unary(int32_t op, const float* in, float* out, int32_t n);
SKAINET_CUDA_API int32_t skainet_cuda_f32_binary(int32_t op, const float* a, int32_t a_mode,
    const float* b, int32_t b_mode, float* out, int32_t n, int32_t inner);

/* Packed blocks (canonical byte order) -> fp32, bit-exact with the reference decoders
 * (skainet-io/skainet-io-gguf/src/commonMain/kotlin/sk/ainet/io/gguf/dequant/DequantOps.kt:338-355,600-644
 * and the Q5_K / Q6_K routines after them). nblocks blocks in, nblocks*block_elems floats out. */
SKAINET_CUDA_API int32_t skainet_cuda_dequant(int32_t encoding, const uint8_t* packed, int64_t nblocks, float* out);

/* ---- 2. resident API (DEVICE pointers unless a name says host) ------------------------------- */
SKAINET_CUDA_API int32_t skainet_cuda_malloc(void** dev_ptr, int64_t nbytes);
SKAINET_CUDA_API int32_t skainet_cuda_free(void* dev_ptr);
SKAINET_CUDA_API int32_t skainet_cuda_memcpy_h2d(void* dev_dst, const void* host_src, int64_t nbytes, skainet_stream_t stream);
SKAINET_CUDA_API int32_t skainet_cuda_memcpy_d2h(void* host_dst, const void* dev_src, int64_t nbytes, skainet_stream_t stream);
SKAINET_CUDA_API int32_t skainet_cuda_stream_create(skainet_stream_t* out);
SKAINET_CUDA_API int32_t skainet_cuda_stream_destroy(skainet_stream_t stream);
SKAINET_CUDA_API int32_t skainet_cuda_stream_sync(skainet_stream_t stream);

/* Upload a packed [rows = out, cols = in] weight once; the bytes are re-laid out for the kernels on
 * the device (both SPI byte orders accepted, the counterpart of PackedWeights.toKernelOrder,
 * skainet-backends/skainet-backend-api/src/commonMain/kotlin/sk/ainet/backend/api/kernel/PackedWeights.kt:63-95).
 * cols must be a multiple of the block size and nbytes == rows*(cols/block)*block_bytes. */
SKAINET_CUDA_API int32_t skainet_cuda_weight_upload(const uint8_t* host_bytes, int64_t nbytes, int32_t encoding,
    int32_t rows, int32_t cols, int32_t order, skainet_weight_t* out);
/* Same, from canonical bytes that already sit in device memory (e.g. a GGUF tensor read straight to HBM). */
SKAINET_CUDA_API int32_t skainet_cuda_weight_from_device(const uint8_t* dev_bytes, int64_t nbytes, int32_t encoding,
    int32_t rows, int32_t cols, int32_t order, skainet_weight_t* out);
/* Bench/test harness: a seeded weight generated and packed on the device. mode 0: values
 * std*N(0,1) (counter-based generator) quantized by the library's own packer (Q8_0 rule:
 * Q8_0Quantizer.kt:28-53; Q4_K: min/max packer); mode 1: random valid blocks (random codes and
 * scales, f16 fields forced to sane values) in the manner of the reference's microbench fixture
 * (skainet-backends/skainet-backend-native-cpu/src/jvmTest/kotlin/sk/ainet/exec/kernel/Q8_0MatmulMicrobenchTest.kt:21-32). */
SKAINET_CUDA_API int32_t skainet_cuda_weight_synth(int32_t encoding, int32_t rows, int32_t cols, uint64_t seed,
    float std, int32_t mode, skainet_weight_t* out);
/* Canonical row-major packed bytes of a resident weight back to the host (so the same bytes can be
 * handed to the CPU reference). nbytes must match. */
SKAINET_CUDA_API int32_t skainet_cuda_weight_export(skainet_weight_t w, uint8_t* host_bytes, int64_t nbytes);
SKAINET_CUDA_API int32_t skainet_cuda_weight_info(skainet_weight_t w, int64_t* out4 /* enc, rows, cols, packed bytes */);
SKAINET_CUDA_API int32_t skainet_cuda_weight_free(skainet_weight_t w);
/* Whole weight -> fp32 [rows, cols] on the device, bit-exact with the reference decoders. */
SKAINET_CUDA_API int32_t skainet_cuda_weight_dequant(skainet_weight_t w, float* dev_out, skainet_stream_t stream);

/* y[m, rows] = x[m, cols] . W^T on the device. Q4_K / Q8_0: the dequant-fused matvec for m = 1 (and Q4_K up to
 * 2 rows), tensor-core tile kernels above that (mma.sync; tcgen05 with TMEM accumulators for Q4_K from 288 rows).
 * Q6_K (native mode = int8 activations per 256 like skainet_q6k_matmul_rm, native/src/q6k_matmul.c:344-357): one warp
 * per output row and up to eight activation rows per pass over the weight, an mma.sync tile kernel from nine rows,
 * every row bit-identical to the single-row result. Q5_K (fp32 activations in both modes, native/src/q5k_matmul.c):
 * one warp per output row, up to four activation rows per pass; from five rows (native mode) an mma.sync tile kernel
 * with the activation carried as two f16 terms.
 * Counterpart of PackedViewMatmulKernel.runWith
 * (skainet-backends/skainet-backend-api/src/commonMain/kotlin/sk/ainet/backend/api/kernel/PackedViewMatmulKernel.kt:69-107),
 * which issues m matvec calls. act_mode: SKAINET_ACT_*. */
SKAINET_CUDA_API int32_t skainet_cuda_matmul_dev(skainet_weight_t w, const float* x_dev, int32_t m, float* y_dev,
    int32_t act_mode, skainet_stream_t stream);

/* One decode-step linear in a single launch: y[rows] = (resid +) W . quantize(norm(x)) for one
 * activation row. gamma_dev != NULL applies RMSNorm (x / sqrt(mean(x^2)+eps) * gamma, the arithmetic
 * of skainet_f32_rms_norm, skainet_kernels.h:574-576) before the reference's activation
 * quantization; resid_dev != NULL adds the result to a residual (y may alias resid). This is the
 * CUDA handler for the graph-level fused ops `fused_rms_norm` + matmul (+ add) that
 * skainet-compile/skainet-compile-opt/src/commonMain/kotlin/sk/ainet/compile/opt/passes/LLMFusionPass.kt:12-22 emits. */
SKAINET_CUDA_API int32_t skainet_cuda_matvec_fused_dev(skainet_weight_t w, const float* x_dev, const float* gamma_dev,
    float eps, const float* resid_dev, float* y_dev, skainet_stream_t stream);

/* Graph-level fused ops (skainet-compile/skainet-compile-opt/src/commonMain/kotlin/sk/ainet/compile/opt/passes/LLMFusionPass.kt:17-23):
 * the entries a CUDA FusedOpHandler calls in place of the CPU decompositions of
 * skainet-compile/skainet-compile-dag/src/commonMain/kotlin/sk/ainet/lang/graph/exec/LLMFusedOpHandlers.kt. Both take an optional
 * RMSNorm in front (gamma_dev != NULL: the fused_rms_norm node that feeds them, LLMFusedOpHandlers.kt:44-68), so a decoder
 * block is norm+qkv and norm+ffn. Q4_K / Q8_0 weights; m activation rows. */
/* Rows of a, then b, then c (0 = none) as one new resident weight: what a handler does once when it first sees the three
 * projections of a fused_qkv_proj node (LLMFusedOpHandlers.kt:143-196 "concatenate the weight matrices and do a single
 * matmul + split") or gate and up of a fused_swiglu_ffn node. The parts stay valid and owned by the caller. */
SKAINET_CUDA_API int32_t skainet_cuda_weight_concat_rows(skainet_weight_t a, skainet_weight_t b, skainet_weight_t c, skainet_weight_t* out);
/* fused_qkv_proj (LLMFusionPass.kt:117, LLMFusedOpHandlers.kt:143-196): q[m, q_rows], k[m, k_rows], v[m, v_rows] = x[m, cols] . W^T
 * for the merged weight's three row ranges, one pass over the activation. Encodings: Q4_K, Q8_0, Q6_K. */
SKAINET_CUDA_API int32_t skainet_cuda_fused_qkv_proj_dev(skainet_weight_t w_qkv, int32_t q_rows, int32_t k_rows, int32_t v_rows,
    const float* x_dev, const float* gamma_dev, float eps, int32_t m, float* q_dev, float* k_dev, float* v_dev, skainet_stream_t stream);
/* fused_swiglu_ffn (LLMFusionPass.kt:86, LLMFusedOpHandlers.kt:86-127): out[m, d] = (resid +) W_down . (silu(W_gate x) * (W_up x)),
 * gate and up as one merged weight (gate rows first); the intermediate never leaves the device and is quantized for the
 * down projection inside the SwiGLU kernel. resid_dev may be NULL or equal out_dev. Encodings: Q4_K, Q8_0, Q6_K; the
 * down projection may be Q6_K behind Q4_K gate and up (the mix K-quant files carry), Q8_0 goes with Q8_0 only. */
SKAINET_CUDA_API int32_t skainet_cuda_fused_swiglu_ffn_dev(skainet_weight_t w_gate_up, skainet_weight_t w_down, const float* x_dev,
    const float* gamma_dev, float eps, int32_t m, const float* resid_dev, float* out_dev, skainet_stream_t stream);

/* Row kernels on the device (contracts as the twins above). */
SKAINET_CUDA_API int32_t skainet_cuda_rms_norm_dev(const float* in, const float* gamma, float* out,
    int32_t rows, int32_t cols, float eps, skainet_stream_t stream);
SKAINET_CUDA_API int32_t skainet_cuda_unary_dev(int32_t op, const float* in, float* out, int64_t n, skainet_stream_t stream);
SKAINET_CUDA_API int32_t skainet_cuda_binary_dev(int32_t op, const float* a, int32_t a_mode, const float* b, int32_t b_mode,
    float* out, int64_t n, int32_t inner, skainet_stream_t stream);
/* out = silu(gate) * up (the fused_swiglu_ffn gate of
 * skainet-compile/skainet-compile-opt/src/commonMain/kotlin/sk/ainet/compile/opt/passes/LLMFusionPass.kt:12-22). */
SKAINET_CUDA_API int32_t skainet_cuda_swiglu_dev(const float* gate, const float* up, float* out, int64_t n, skainet_stream_t stream);
/* Rotary embedding in place on x[rows, heads, head_dim] with one position per row (positions[rows],
 * device int32). The reference has no RoPE code; convention: angle = pos * theta^(-2i/d), computed in
 * double and rounded once; mode 0 rotates (2i, 2i+1), mode 1 rotates (i, i+d/2). */
SKAINET_CUDA_API int32_t skainet_cuda_rope_dev(float* x, const int32_t* positions, int32_t rows, int32_t heads,
    int32_t head_dim, float theta, int32_t mode, skainet_stream_t stream);
/* index of the maximum of each row, lowest index on ties
 * (skainet-backends/skainet-backend-cpu/src/commonMain/kotlin/sk/ainet/exec/tensor/ops/DefaultCpuOps.kt:3042-3078). */
SKAINET_CUDA_API int32_t skainet_cuda_argmax_dev(const float* x, int32_t rows, int32_t cols, int32_t* out_idx, skainet_stream_t stream);
/* Rows of a packed table decoded on demand: out[i, :] = dequant(W[ids[i], :]) — the gather over a
 * RowDequantSource (DefaultCpuOps.kt:3746-3793). */
SKAINET_CUDA_API int32_t skainet_cuda_embed_dev(skainet_weight_t table, const int32_t* ids_dev, int32_t n, float* out,
    skainet_stream_t stream);

/* The full attention contract of skainet_cuda_f32_sdpa (skainet_kernels.h:578-585) on device-resident fp32 tensors: what a
 * resident-activation ops class calls for ops.scaledDotProductAttention (TensorOps.kt:410-458) so that q, k, v and the
 * result never cross to the host. lengths_dev / mask_dev are device pointers (NULL = none). */
SKAINET_CUDA_API int32_t skainet_cuda_sdpa_dev(const float* q, const float* k, const float* v, float* out,
    int32_t batch, int32_t heads, int32_t kv_heads, int32_t seq_q, int32_t seq_kv, int32_t head_dim,
    float scale, int32_t causal, int32_t window, int32_t right_context, const int32_t* lengths_dev,
    const float* mask_dev, int32_t mask_b, int32_t mask_h, int32_t mask_q, int32_t mask_k, skainet_stream_t stream);

/* GQA decode attention over an f16 KV cache resident in HBM: one query row per (batch, head),
 * split over the key axis with an fp32 softmax merge. k_cache / v_cache are binary16
 * [batch, kv_heads, cache_stride(keys), head_dim]; kv_len[b] keys are visible to batch b's query
 * (the decode case of f32_fused.c:313-324: causal with seq_q = 1 sees every cached key); window > 0
 * keeps only the last `window` keys. q/out fp32 [batch, heads, head_dim]. head_dim 64 or 128. */
SKAINET_CUDA_API int32_t skainet_cuda_attn_decode_dev(const float* q, const uint16_t* k_cache, const uint16_t* v_cache,
    float* out, int32_t batch, int32_t heads, int32_t kv_heads, int32_t head_dim, int64_t cache_stride,
    const int32_t* kv_len_dev, int32_t max_kv_len, float scale, int32_t window, skainet_stream_t stream);
/* The same decode attention for callers that must not allocate. It has no counterpart in the
 * reference. skainet_cuda_attn_decode_dev keeps its split-K partial results in per-stream scratch that
 * it grows with cudaMalloc when a larger problem arrives; some hosts cannot have that happen: a decode
 * loop that runs under a fixed memory plan and asserts zero allocations per step (the reference's own
 * acceptance harness does, DecodeAcceptanceTest.kt:24-90), a latency-critical thread for which the
 * device-wide synchronisation inside cudaMalloc is a stall, or a process whose allocator hooks forbid
 * device allocation after start-up. This entry takes the same arguments and computes the same result
 * with the same kernels, but its partials live in an array built into the library image: 2^20 floats
 * (4 MiB) per GPU, held from library load to process exit. It calls no cudaMalloc, cudaFree or other
 * allocating routine.
 *   Limit: batch * heads * key_splits * (head_dim + 2) <= 2^20 floats, where key_splits is what the
 *   launcher picks for (batch, kv_heads, max_kv_len) — at most 256. Larger problems are refused with
 *   SKAINET_CUDA_ERR_INVALID and a message naming the size; nothing is launched.
 *   First call on a device: resolves the array's device address (cudaGetSymbolAddress, with that device
 *   current). Make that first call before any stream capture begins.
 *   Sharing: every call on a device uses the one array. The kernels overwrite every partial record they
 *   later read, so nothing has to be cleared between calls; but two calls whose kernels overlap on the
 *   GPU (different streams, no ordering between them) race on it and both results are undefined. */
SKAINET_CUDA_API int32_t skainet_cuda_attn_decode_noalloc_dev(const float* q, const uint16_t* k_cache, const uint16_t* v_cache,
    float* out, int32_t batch, int32_t heads, int32_t kv_heads, int32_t head_dim, int64_t cache_stride,
    const int32_t* kv_len_dev, int32_t max_kv_len, float scale, int32_t window, skainet_stream_t stream);
/* fp32 [n] -> binary16 [n], round to nearest even (filling the cache from host-prepared K/V). */
SKAINET_CUDA_API int32_t skainet_cuda_f32_to_f16_dev(const float* in, uint16_t* out, int64_t n, skainet_stream_t stream);

/* ---- 3. KV-cache store resident in HBM -------------------------------------------------------- */
/* The device counterpart of the reference's KvCacheStore
 * (skainet-lang/skainet-lang-core/src/commonMain/kotlin/sk/ainet/lang/tensor/storage/KvCacheStore.kt:125-157) as
 * DefaultKvCacheStore implements it (DefaultKvCacheStore.kt:76-131,170-177,235-263): one sequence, per layer keys and
 * values [heads, max_seq, head_dim], here in binary16 (the store's configurable element type, KvCacheStore.kt:58-74;
 * reads convert back exactly). Positions are absolute. sliding_window != 0 makes the buffer a ring that keeps the
 * newest max_seq positions (appending past max_seq overwrites the oldest); otherwise a full cache refuses the append.
 * The sequence length advances when the last layer has been appended. head_dim 64 or 128. */
SKAINET_CUDA_API int32_t skainet_cuda_kv_create(int32_t n_layers, int32_t n_heads, int32_t head_dim, int32_t max_seq,
    int32_t sliding_window, skainet_kv_t* out);
/* The same store holding TurboQuant blocks instead of binary16 rows: the device counterpart of TurboQuantKvCacheStore
 * (skainet-lang/skainet-lang-core/src/commonMain/kotlin/sk/ainet/lang/tensor/storage/TurboQuantKvCacheStore.kt:62-199), one block per
 * (layer, position, head) with the rotation seed RandomRotation.seedFor(layer, head, position) for keys and that seed xor 0x5A5A5A5A
 * for values. key_bits / value_bits in {2,3,4,8}; *_residual_bits 0 = rotation + scalar quantizer only (PolarOnly), 1..4 = with the
 * residual stage (PolarPlusQjl). Dense only (a full cache refuses the append); head_dim in {32,64,128,256}. Encoded bytes, scales and
 * the values a read returns are bit-identical to the reference's. kv_info reports ring = 2 and, as physical bytes, what the
 * reference's memoryReport counts (the blocks of the positions held); beside every block the device also keeps the rotation's sign
 * sequence (head_dim / 8 bytes), so that a read does not re-run the sequential generator. kv_attn_decode_dev decodes the window's blocks
 * and attends them: through binary16 rows and the split-K kernel for head_dim 64 / 128 with 1, 2, 4 or 8 query heads per cache head, in
 * fp32 otherwise; the window must end at or before currentSeqLen. */
SKAINET_CUDA_API int32_t skainet_cuda_kv_create_turboquant(int32_t n_layers, int32_t n_heads, int32_t head_dim, int32_t max_seq,
    int32_t key_bits, int32_t key_residual_bits, int32_t value_bits, int32_t value_residual_bits, skainet_kv_t* out);
/* TurboQuantCodec.encode / decode for one vector of n in {32,64,128,256} floats with an explicit seed
 * (skainet-lang/skainet-lang-core/src/commonMain/kotlin/sk/ainet/lang/tensor/ops/turboquant/TurboQuantCodec.kt:33-85); HOST pointers.
 * codes_out: packedSize(n, bits) bytes (BitPacker.kt:46-54); scales_out: n / 32 floats; residual_out / residual_scale_out only when
 * residual_bits > 0 (packedSize(n, residual_bits) bytes, one float). The same bytes the reference's golden test digests. */
SKAINET_CUDA_API int32_t skainet_cuda_turboquant_encode(const float* input, int32_t n, int32_t bits, int32_t residual_bits, int32_t seed,
    uint8_t* codes_out, float* scales_out, uint8_t* residual_out, float* residual_scale_out);
SKAINET_CUDA_API int32_t skainet_cuda_turboquant_decode(const uint8_t* codes, const float* scales, const uint8_t* residual, float residual_scale,
    int32_t n, int32_t bits, int32_t residual_bits, int32_t seed, float* output);
SKAINET_CUDA_API int32_t skainet_cuda_kv_free(skainet_kv_t kv);
/* appendToken(layer, key, value): key / value are [heads, head_dim] fp32; host pointers, or device pointers with a stream.
 * A full non-ring cache -> SKAINET_CUDA_ERR_INVALID ("KV cache is full", IllegalStateException in the reference). */
SKAINET_CUDA_API int32_t skainet_cuda_kv_append(skainet_kv_t kv, int32_t layer, const float* key_host, const float* value_host);
SKAINET_CUDA_API int32_t skainet_cuda_kv_append_dev(skainet_kv_t kv, int32_t layer, const float* key_dev, const float* value_dev,
    skainet_stream_t stream);
/* readKeys / readValues (which = 0 / 1): positions [start_pos, end_pos) as fp32 [heads, end_pos - start_pos, head_dim] on the
 * host, oldest first also when the range crosses the end of the ring. start_pos before the oldest held position or end_pos
 * beyond the sequence -> SKAINET_CUDA_ERR_INVALID. */
SKAINET_CUDA_API int32_t skainet_cuda_kv_read(skainet_kv_t kv, int32_t layer, int32_t which, int32_t start_pos, int32_t end_pos,
    float* host_out);
/* evict(fromPos): the sequence length becomes from_pos (truncation, speculative-decoding rollback). On a cache that has not
 * wrapped the evicted slots are zeroed like the reference does; positions a wrapped ring had already overwritten stay
 * unavailable afterwards (reads and windows before them are refused). */
SKAINET_CUDA_API int32_t skainet_cuda_kv_evict(skainet_kv_t kv, int32_t from_pos);
SKAINET_CUDA_API int32_t skainet_cuda_kv_clear(skainet_kv_t kv);
/* out8 = {currentSeqLen, windowStart, maxSeqLen, layers, heads, head_dim, ring (0/1), physical bytes of keys + values}. */
SKAINET_CUDA_API int32_t skainet_cuda_kv_info(skainet_kv_t kv, int64_t* out8);
/* One decode step of attention over positions [from_pos, to_pos) of a layer: out[h] = softmax(q[h] . K^T * scale) V for
 * q_heads query heads (a multiple 1, 2, 4 or 8 of the cache's heads; query head h reads cache head h / group), q / out
 * device fp32 [q_heads, head_dim]; scale 0 means 1/sqrt(head_dim). The window is read in place, as the one or two runs it
 * occupies in the ring: the device form of WindowedAttention.decodeStep over keyWindow / valueWindow
 * (skainet-lang/skainet-lang-core/src/commonMain/kotlin/sk/ainet/lang/memory/WindowedAttention.kt:32-80). to_pos may be
 * currentSeqLen + 1 while a token's layers are being appended (the sequence length advances only with the last layer). */
SKAINET_CUDA_API int32_t skainet_cuda_kv_attn_decode_dev(skainet_kv_t kv, int32_t layer, const float* q_dev, float* out_dev,
    int32_t q_heads, int32_t from_pos, int32_t to_pos, float scale, skainet_stream_t stream);

/* ---- 4. diagnostics (no counterpart in the reference; nothing on the product path calls these) ---- */

/* Exercises the bounded-wait failure path (skainet_cuda_device_status) without any fault: launches a kernel whose only wait is on a barrier nothing completes.
 * outcome = 2 when the kernel gave up after its poll limit and still ran to its end (the expected result; the next
 * skainet_cuda_device_status() then returns SKAINET_CUDA_ERR_TIMEOUT once), 1 if the wait unexpectedly succeeded,
 * 0 if the kernel did not finish. Takes a second or so. The reference has no counterpart. */
SKAINET_CUDA_API int32_t skainet_cuda_selftest_bounded_wait(int32_t* outcome);

/* Measurement aid with no counterpart in the reference: reads every byte of a resident weight once
 * with plain vector loads and computes nothing. The bench times it over the same weights as the matvec
 * to report the floor a launch of that many bytes can reach on this GPU. */
SKAINET_CUDA_API int32_t skainet_cuda_probe_read_dev(skainet_weight_t w, skainet_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* SKAINET_CUDA_H */
