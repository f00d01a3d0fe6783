// Shared host/device helpers of libskainet_cuda: status + error plumbing, the resident weight
// record, per-stream scratch, and small device utilities used by every kernel file.
#pragma once
#include <mutex>

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <string>

#include "../../include/skainet_cuda.h"

namespace sk {

// ---- error plumbing ----------------------------------------------------------------------------
void set_error(const char* fmt, ...);
int32_t cuda_fail(cudaError_t e, const char* what, const char* file, int line);
int32_t ensure_device();   // SKAINET_CUDA_OK once a usable sm_100 device is current on this thread

#define SK_CUDA(call)                                                        \
    do {                                                                     \
        cudaError_t _e = (call);                                             \
        if (_e != cudaSuccess) return ::sk::cuda_fail(_e, #call, __FILE__, __LINE__); \
    } while (0)

#define SK_TRY(expr)                              \
    do {                                          \
        int32_t _s = (expr);                      \
        if (_s != SKAINET_CUDA_OK) return _s;     \
    } while (0)

#define SK_REQUIRE(cond, ...)                     \
    do {                                          \
        if (!(cond)) {                            \
            ::sk::set_error(__VA_ARGS__);         \
            return SKAINET_CUDA_ERR_INVALID;      \
        }                                         \
    } while (0)

inline cudaStream_t as_stream(skainet_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

// ---- block geometry ----------------------------------------------------------------------------
inline int block_elems(int enc) { return enc == SKAINET_ENC_Q8_0 ? 32 : 256; }
inline int block_bytes(int enc) {
    switch (enc) {
        case SKAINET_ENC_Q8_0: return 34;
        case SKAINET_ENC_Q4_K: return 144;
        case SKAINET_ENC_Q5_K: return 176;
        case SKAINET_ENC_Q6_K: return 210;
        default: return 0;
    }
}

// ---- a weight resident in HBM -------------------------------------------------------------------
// The canonical GGUF blocks are split into planes at upload so that every plane is 16-byte
// addressable per lane and (for the batched GEMM) a plain 2-D tensor for TMA:
//   Q8_0: codes  int8 [rows][cols]                 scales f16 [rows][cols/32]
//   Q4_K: qs     u8   [rows][cols/256][128]        hdr 16 B   [rows][cols/256]  (d, dmin, 12 scale bytes)
//   Q5_K: qs as Q4_K, hdr as Q4_K,                 extra qh   [rows][cols/256][32]
//   Q6_K: ql     u8   [rows][cols/256][128]        hdr 16 B = 16 int8 scales; extra: qh [..][64] ; d f16 plane in aux
// The split is a pure byte permutation: export() restores the canonical bytes exactly.
struct Weight {
    int32_t enc = 0, rows = 0, cols = 0, bpr = 0;  // bpr = blocks per row
    uint8_t* qs = nullptr;     // main code plane
    uint8_t* hdr = nullptr;    // per-block header / scale plane
    uint8_t* extra = nullptr;  // Q5_K qh / Q6_K qh
    uint8_t* aux = nullptr;    // Q6_K d plane (f16)
    void* base = nullptr;      // the single allocation holding all planes
    int64_t packed_bytes = 0;  // canonical size
    int device = 0;
    uint64_t magic = 0;
};
Weight* weight_from_handle(skainet_weight_t h);   // nullptr (+ error set) when unknown


// ---- per-stream scratch --------------------------------------------------------------------------
// Device scratch reused across calls on one stream (quantized activations, split-K partials).
// Grown on demand outside stream capture; never shrinks.
int32_t scratch_get(cudaStream_t stream, int slot, size_t nbytes, void** out);
size_t scratch_capacity(cudaStream_t stream, int slot);   // bytes the slot holds now (0 if never used)
void scratch_release(cudaStream_t stream);                // frees every slot of a stream about to be destroyed
// Entry points that take HOST pointers stage through the default stream's scratch slots: one such call at a time per process.
std::mutex& twin_mutex();
enum { SCRATCH_ACT = 0, SCRATCH_ATTN = 1, SCRATCH_TWIN_A = 2, SCRATCH_TWIN_B = 3, SCRATCH_TWIN_C = 4,
       SCRATCH_TWIN_D = 5, SCRATCH_TWIN_E = 6, SCRATCH_TWIN_F = 7, SCRATCH_FUSED = 8, SCRATCH_FUSED2 = 9, SCRATCH_GEMM = 10,
       SCRATCH_FFN = 11, SCRATCH_SLOTS = 12 };

int sm_count();
// Raises a kernel's dynamic shared-memory limit to at least `bytes` on the CURRENT device, once per (kernel, device):
// the attribute belongs to each device's copy of the function, so a process that drives several GPUs sets it on each.
int32_t ensure_dynamic_smem(const void* kernel, int bytes);
int32_t launch_bounded_wait_selftest(int* reached_end, cudaStream_t s);   // probe.cu
int* device_timeout_flag();   // current device's int, set by a kernel whose bounded wait ran out (nullptr if unavailable)
int32_t timeout_status(int flag_value);       // OK for 0, else ERR_TIMEOUT with a message naming the kind of wait
int32_t set_thread_device(int device);        // cudaSetDevice + the thread's device bookkeeping

// ---- launchers implemented in the kernel files ------------------------------------------------------
// repack.cu
int32_t launch_split_planes(const uint8_t* canon_dev, Weight& w, int order, cudaStream_t s);
int32_t launch_join_planes(const Weight& w, uint8_t* canon_dev, cudaStream_t s);
int32_t launch_dequant_weight(const Weight& w, float* out, cudaStream_t s);
int32_t launch_dequant_canonical(int enc, const uint8_t* canon_dev, int64_t nblocks, float* out, cudaStream_t s);
int32_t launch_synth(Weight& w, uint64_t seed, float std, int mode, int64_t row0, int64_t col0, int64_t full_cols, cudaStream_t s);
// api.cu: weight records for other translation units
int32_t weight_alloc(int enc, int rows, int cols, Weight** out);
void weight_release(Weight* w);
skainet_weight_t weight_to_handle(Weight* w);
// attention.cu: causal attention of a block of new queries over an f16 cache (prefill)
int32_t launch_sdpa_cache(const float* q, const __half* k, const __half* v, float* out, int batch, int heads,
                          int kv_heads, int seq_q, int seq_kv, int64_t cache_stride, int d, float scale, int window,
                          const int32_t* q_abs_base, cudaStream_t s);
int32_t launch_embed(const Weight& w, const int32_t* ids, int n, float* out, cudaStream_t s);
// matvec.cu
size_t act_scratch_bytes(int enc, int act_mode, int m, int cols);
int32_t launch_act_quant(int enc, int act_mode, const float* x, int m, int cols, void* scratch, cudaStream_t s);
struct ActQ8K;
// matvec_kq.cu: Q6_K (int8-per-256 or fp32 activations) and Q5_K (fp32 activations) over resident planes
int32_t launch_matvec_kq(const Weight& w, const float* x, ActQ8K a, int m, float* y, int act_mode, cudaStream_t s, const float* resid = nullptr);
// gemm_kq.cu: Q6_K weights x m quantized activation rows on the tensor cores (mma.sync); 1 = not taken
int32_t launch_gemm_q6k(const Weight& w, ActQ8K a, int m, float* y, const float* resid, cudaStream_t s);
// gemm_kq.cu: Q5_K weights x m fp32 activation rows carried as two f16 terms (hi + lo) plus per-32 sums, on the tensor cores.
// Activation rows from which a Q5_K product takes this path (fewer rows: the row kernel of matvec_kq.cu, four per pass).
// 11008 x 4096: 47 us here for up to 32 rows against 42 us for four rows and 83 us for eight through the row kernel.
constexpr int Q5K_GEMM_MIN_ROWS = 5;
size_t act_f16split_bytes(int m, int cols);
int32_t launch_act_f16split(const float* x, int m, int cols, void* scratch, cudaStream_t s);
int32_t launch_gemm_q5k(const Weight& w, const void* act_scratch, int m, float* y, cudaStream_t s);
int32_t launch_matvec(const Weight& w, const float* x, const void* act_scratch, int m, float* y, int act_mode,
                      cudaStream_t s);
// matvec_stream.cu: rows m0..m0+mm of the quantized activation; returns 1 when the shape is not taken
int32_t launch_matvec_stream(const Weight& w, const void* act_scratch, int m_total, int m0, int mm, float* y, cudaStream_t s);
// probe.cu
int32_t launch_probe_read(const Weight& w, uint32_t* sink, cudaStream_t s);
// rowops.cu
int32_t launch_rms_norm(const float* in, const float* gamma, float* out, int rows, int cols, float eps, cudaStream_t s);
int32_t launch_unary(int op, const float* in, float* out, int64_t n, cudaStream_t s);
int32_t launch_binary(int op, const float* a, int am, const float* b, int bm, float* out, int64_t n, int inner, cudaStream_t s);
int32_t launch_swiglu(const float* g, const float* u, float* out, int64_t n, cudaStream_t s);
int32_t launch_rope(float* x, const int32_t* pos, int rows, int heads, int d, float theta, int mode, cudaStream_t s);
int32_t launch_argmax(const float* x, int rows, int cols, int32_t* out, cudaStream_t s);
int32_t launch_f32_to_f16(const float* in, uint16_t* out, int64_t n, cudaStream_t s);
int32_t launch_smoke(const float* in, float* out, int n, cudaStream_t s);
// attention.cu
size_t attn_scratch_bytes(int batch, int heads, int head_dim, int max_kv_len);
int32_t launch_attn_decode(const float* q, const __half* k, const __half* v, float* out, int batch, int heads,
                           int kv_heads, int d, int64_t cache_stride, const int32_t* kv_len, int max_kv_len,
                           float scale, int window, void* scratch, cudaStream_t s);
int32_t launch_attn_decode_ring(const float* q, const __half* k, const __half* v, float* out, int heads, int kv_heads, int d,
                                int64_t cache_stride, const int32_t* kv_len_dev, int len, float scale, int ring_start, int ring_cap,
                                void* scratch, cudaStream_t s);
int32_t launch_sdpa_f32(const float* q, const float* k, const float* v, float* out, int batch, int heads, int kv_heads,
                        int seq_q, int seq_kv, int d, float scale, int causal, int window, int right_context,
                        const int32_t* lengths, const float* mask, int mb, int mh, int mq, int mk, cudaStream_t s);

}  // namespace sk

// ---- device utilities ----------------------------------------------------------------------------
#ifdef __CUDACC__
namespace skd {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// 16-byte read-only load that does not linger in L1 (weights are streamed exactly once).
__device__ __forceinline__ uint4 ld_stream(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
__device__ __forceinline__ uint4 ld_ro(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

// ggml get_scale_min_k4 on the three scale words of a Q4_K/Q5_K header:
// sc[0..3] | sc[4..7] | mn[0..3] | mn[4..7], one value per byte.
__device__ __forceinline__ void k4_unpack(uint32_t u0, uint32_t u1, uint32_t u2, uint32_t& sc_lo, uint32_t& sc_hi,
                                          uint32_t& mn_lo, uint32_t& mn_hi) {
    sc_lo = u0 & 0x3f3f3f3fu;
    mn_lo = u1 & 0x3f3f3f3fu;
    sc_hi = (u2 & 0x0f0f0f0fu) | (((u0 >> 6) & 0x03030303u) << 4);
    mn_hi = ((u2 >> 4) & 0x0f0f0f0fu) | (((u1 >> 6) & 0x03030303u) << 4);
}
__device__ __forceinline__ int byte_of(uint32_t w, int i) { return (w >> (8 * i)) & 0xff; }

}  // namespace skd
#endif
