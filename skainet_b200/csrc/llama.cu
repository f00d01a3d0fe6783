// Llama-style decoder runtime (include/skainet_cuda_llama.h): resident weights, f16 KV cache, one
// CUDA graph per decode step and context-length bucket, greedy sampling on the device, optional
// tensor parallelism. The step is a chain of PDL-launched kernels:
//
//   embed -> [ norm+quant -> qkv matvec -> rope + cache append -> split-K attention -> quant
//              -> o matvec (+residual) -> norm+quant -> gate|up matvec -> swiglu+quant
//              -> down matvec (+residual) ] x layers -> norm+quant -> head matvec -> arg max (+advance)
//
// Every matvec weight prefetch (TMA) starts while its predecessor still runs; the small "prep"
// kernels between them turn an fp32 row into the quantized activation the next matvec consumes, which
// is where RMSNorm and SwiGLU live. Operator contracts: see the header.
#include "common.cuh"
#include <cstdlib>
#include "actquant.cuh"
#include "matvec_fused.cuh"
#include "tma.cuh"
#include "comm.cuh"
#include "stepops.cuh"
#include "../../include/skainet_cuda_llama.h"

#include <cmath>
#include <map>
#include <mutex>
#include <unordered_set>
#include <vector>

namespace sk {

// ================================================================================================
// small kernels of the step
// ================================================================================================
constexpr int PROLOGUE_PREP_MAX_COLS = 4096, PROLOGUE_PREP_MAX_COLS_RING = 8192;
// Prompt rows per pass of the body: the tcgen05 GEMM takes 132 us for 512 rows of a 25 MB weight against 2 x 95 us for two
// passes of 256 through the mma.sync kernel (and 2 x 108 us through itself).
constexpr int PREFILL_CHUNK_ROWS = 512;
#ifndef SK_SWIGLU_PROLOGUE_MAX_COLS
#define SK_SWIGLU_PROLOGUE_MAX_COLS 8192
#endif
// Widest down-projection input whose SwiGLU the ring kernel computes itself. 11008 inputs (the 7B shape) measured slower that
// way although the step has 32 launches fewer: 1.471 against 1.451 ms.
constexpr int SWIGLU_PROLOGUE_MAX_COLS = SK_SWIGLU_PROLOGUE_MAX_COLS;

// After the merged q|k|v matvec: rotate q in place, rotate k and append it with v to the f16 cache at
// each sequence's position. grid (rows, heads + 2*kv_heads), head_dim/2 threads. The rotation factors
// come from a table built on the host in double precision.
__global__ void rope_append_kernel(float* __restrict__ qkv, int heads, int kv_heads, int d, const float* __restrict__ cos_t,
                                   const float* __restrict__ sin_t, const int32_t* __restrict__ pos, const int32_t* __restrict__ seq_of_row,
                                   int pos_step, __half* __restrict__ kc, __half* __restrict__ vc, int64_t cache_stride, int mode) {
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    const int row = blockIdx.x, hh = blockIdx.y, i = threadIdx.x, half = d >> 1;
    const int seq = seq_of_row ? seq_of_row[row] : row;
    const int p = pos[seq] + (pos_step ? row : 0);       // prefill: consecutive rows of one sequence
    float* base = qkv + (size_t) row * (heads + 2 * kv_heads) * d + (size_t) hh * d;
    if (hh < heads + kv_heads) {
        const float c = cos_t[(size_t) p * half + i], s = sin_t[(size_t) p * half + i];
        const int ix = mode == 0 ? 2 * i : i, iy = mode == 0 ? 2 * i + 1 : i + half;
        const float a = base[ix], b = base[iy];
        const float ra = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)), rb = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
        if (hh < heads) { base[ix] = ra; base[iy] = rb; }
        else {
            __half* dst = kc + (((size_t) seq * kv_heads + (hh - heads)) * cache_stride + p) * d;
            dst[ix] = __float2half_rn(ra); dst[iy] = __float2half_rn(rb);
        }
    } else {
        __half* dst = vc + (((size_t) seq * kv_heads + (hh - heads - kv_heads)) * cache_stride + p) * d;
        dst[2 * i] = __float2half_rn(base[2 * i]); dst[2 * i + 1] = __float2half_rn(base[2 * i + 1]);
    }
}

// q rows out of the merged q|k|v buffer into a dense [rows][heads*d] buffer (attention input).
__global__ void gather_q_kernel(const float* __restrict__ qkv, float* __restrict__ q, int qdim, int stride) {
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    for (int c = threadIdx.x; c < qdim; c += blockDim.x) q[(size_t) blockIdx.x * qdim + c] = qkv[(size_t) blockIdx.x * stride + c];
}

// Arg max per row (lowest index on ties) + bookkeeping of the step: the token becomes the next
// step's input, is recorded in the output log, and the sequence position advances.
__global__ void __launch_bounds__(1024)
argmax_advance_kernel(const float* __restrict__ logits, int cols, int32_t* __restrict__ cur_token, int32_t* __restrict__ pos,
                      int32_t* __restrict__ log, int32_t* __restrict__ log_cursor, int batch) {
    __shared__ float sv[32];
    __shared__ int si[32];
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    const float* r = logits + (size_t) blockIdx.x * cols;
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
        if (lane == 0) {
            const int tok = bi == 0x7fffffff ? 0 : bi;
            cur_token[blockIdx.x] = tok;
            pos[blockIdx.x] += 1;
            if (log) log[(size_t) log_cursor[0] * batch + blockIdx.x] = tok;
        }
    }
}
__global__ void bump_cursor_kernel(int32_t* cursor) { skd::pdl_launch_dependents(); skd::pdl_wait(); cursor[0] += 1; }

// Seeded f16 noise into the cache (fake_prefill). The value of an element depends only on the seed and on its
// place in the unsharded cache (global kv head, position, dim), so every tensor-parallel size decodes the same context.
__global__ void fill_cache_kernel(__half* kc, __half* vc, int64_t n, int64_t per_head, int head0, uint64_t seed) {
    for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) {
        const int64_t gi = i + (int64_t) head0 * per_head;      // index in the full [kv_heads][max_seq][head_dim] cache of the sequence
        uint64_t z = (seed + (uint64_t) gi) * 0x9E3779B97F4A7C15ull;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull; z ^= z >> 27;
        kc[i] = __float2half_rn(((float) (z & 0xFFFF) / 32768.0f - 1.0f) * 1.7f);
        vc[i] = __float2half_rn(((float) ((z >> 16) & 0xFFFF) / 32768.0f - 1.0f) * 1.7f);
    }
}

// ================================================================================================
// the model
// ================================================================================================
struct Layer {
    Weight *wq = nullptr, *wk = nullptr, *wv = nullptr, *wo = nullptr, *wgate = nullptr, *wup = nullptr, *wdown = nullptr;
    Weight *wqkv = nullptr, *wgu = nullptr;     // merged at finalize
    float *g_attn = nullptr, *g_ffn = nullptr;
    __half *kc = nullptr, *vc = nullptr;        // [max_batch][kv_heads_local][max_seq][head_dim]
};

struct Model {
    skainet_llama_config cfg;
    int heads_l, kv_heads_l, ffn_l, vocab_l;   // this rank's shard sizes
    std::vector<Layer> layers;
    Weight *embed = nullptr, *head = nullptr;
    float* g_out = nullptr;
    float *cos_t = nullptr, *sin_t = nullptr;
    // activations ([rows] = max(max_batch, prefill chunk))
    int max_rows = 0;
    float *x = nullptr, *qkv = nullptr, *q = nullptr, *attn = nullptr, *gu = nullptr, *tmp = nullptr, *logits = nullptr, *logits_full = nullptr;
    void *act = nullptr; size_t act_bytes = 0;
    void *attn_scratch = nullptr; size_t attn_scratch_bytes = 0;
    int32_t *cur_token = nullptr, *pos = nullptr, *kv_len = nullptr, *log = nullptr, *log_cursor = nullptr, *row_seq = nullptr;
    int log_cap = 0;
    std::vector<int> host_pos;
    cudaStream_t stream = nullptr;
    std::map<std::pair<int, int>, cudaGraphExec_t> graphs;   // (batch, bucket) -> step graph
    bool finalized = false;
    Comm* comm = nullptr;
    bool comm_broken = false;      // a peer wait ran out: the group's inboxes are out of step, the model refuses further steps
    int device = 0;
    int* d_flag = nullptr;         // the device's bounded-wait flag (owned by the library, not by the model)
    int* h_flag = nullptr;         // pinned host copy read after every synchronising call
    uint64_t magic = 0;
};

static const uint64_t MODEL_MAGIC = 0x534b4d4f44454cull;
static std::mutex g_model_mu;
static std::unordered_set<Model*> g_models;

static Model* model_from_handle(skainet_model_t h) {
    Model* m = reinterpret_cast<Model*>(h);
    std::lock_guard<std::mutex> lk(g_model_mu);
    if (!m || g_models.find(m) == g_models.end() || m->magic != MODEL_MAGIC) {
        set_error("unknown or freed model handle %lld", (long long) h);
        return nullptr;
    }
    return m;
}

template <typename T>
static int32_t dalloc(T** p, size_t count) {
    *p = nullptr;
    if (count == 0) return SKAINET_CUDA_OK;
    SK_CUDA(cudaMalloc((void**) p, count * sizeof(T)));
    return SKAINET_CUDA_OK;
}

// A K-quant model takes Q6_K tensors beside its Q4_K ones (real Q4_K_M files carry ffn_down, attn_v and the output
// head that way): both consume the same int8-per-256 activation (native/src/q6k_matmul.c:53-67 is the Q4_K quantizer).
static int32_t check_weight_shape(const Weight* w, int enc, int rows, int cols, const char* what) {
    SK_REQUIRE(w->enc == enc || (enc == SKAINET_ENC_Q4_K && w->enc == SKAINET_ENC_Q6_K), "%s: encoding %d, model expects %d", what, w->enc, enc);
    SK_REQUIRE(w->rows == rows && w->cols == cols, "%s: shape [%d, %d], model expects [%d, %d]", what, w->rows, w->cols, rows, cols);
    return SKAINET_CUDA_OK;
}

static int bucket_of(const Model& m, int len) {
    int b = 256;
    while (b < len) b <<= 1;
    return std::min(b, m.cfg.max_seq);
}

// y[rows][w.rows] (= resid +) W . act   for activation rows already quantized into m.act.
static int32_t linear(Model& m, const Weight& w, int rows, float* y, float* resid_inplace, cudaStream_t s) {
    return launch_linear_q(w, m.act, rows, y, resid_inplace, m.tmp, s);
}

template <int MODE>
static int32_t prep(Model& m, const float* in, const float* gamma, int rows, int n, bool split, cudaStream_t s) {
    return launch_prep(MODE, in, gamma, m.cfg.rms_eps, rows, n, split, m.act, s);
}

// y[rows][w.rows] = W . quantize(rmsnorm(x, gamma)). One activation row takes a single launch where the matvec
// kernel can normalise and quantize the row in its own prologue while its first weight tiles are in flight: up to
// 4096 elements in the one-tile kernel (one prologue per CTA, several CTAs per SM), up to 8192 in the ring kernel
// (one prologue per SM; 70B shape, 8192 columns: 8.26 against 8.47 ms per step). Wider rows keep the separate
// prep kernel: every CTA would re-read the fp32 row and the gains, 12 bytes per element out of L2 against one for
// the quantized row.
static int32_t linear_normed(Model& m, const Weight& w, const float* x, const float* gamma, int rows, float* y, cudaStream_t s) {
    if (rows == 1 && w.cols <= (matvec_uses_ring(w, PREP_NORM_F32) ? PROLOGUE_PREP_MAX_COLS_RING : PROLOGUE_PREP_MAX_COLS)) {
        MatvecIn in; in.x = x; in.gamma = gamma; in.eps = m.cfg.rms_eps;
        const int32_t st = launch_matvec_fused(w, in, PREP_NORM_F32, y, nullptr, s);
        if (st != 1) return st;
    }
    SK_TRY(prep<PK_NORM>(m, x, gamma, rows, w.cols, w.enc == SKAINET_ENC_Q8_0, s));
    return linear(m, w, rows, y, nullptr, s);
}

// Sum over the TP group, in place (no-op on one GPU).
static int32_t tp_sum(Model& m, float* buf, int64_t n, cudaStream_t s) {
    if (m.cfg.tp_world <= 1) return SKAINET_CUDA_OK;
    return comm_all_reduce_sum(m.comm, buf, n, s);
}

// The transformer body over `rows` activation rows in m.x. decode: row b = sequence b, one token each;
// prefill: rows = consecutive tokens of sequence `seq`. kv_bound bounds the keys attention visits.
// final_gamma != nullptr asks for the output norm to be folded into the last group sum where that is possible;
// *final_prepared then says whether m.act already holds the quantized, normalised rows for the output head.
static int32_t body(Model& m, int rows, bool prefill, int seq, int kv_bound, cudaStream_t s, const float* final_gamma = nullptr,
                    bool* final_prepared = nullptr) {
    const auto& c = m.cfg;
    const int D = c.head_dim, H = m.heads_l, HK = m.kv_heads_l, qkv_dim = (H + 2 * HK) * D;
    const bool lin_split = c.linear_enc == SKAINET_ENC_Q8_0;      // Q8_0 linears take the two-term activation, K-quants int8 per 256
    const float scale = 1.0f / sqrtf((float) D);
    // Projections that share one input and write side by side into out[rows][stride]: one merged weight when their
    // encodings agree (finalize merged them), else one linear per part over the same prepared activation.
    auto projections = [&](Weight* merged, std::initializer_list<Weight*> parts, bool prepared, const float* gamma, float* out, int stride) -> int32_t {
        if (merged) return prepared ? linear(m, *merged, rows, out, nullptr, s) : linear_normed(m, *merged, m.x, gamma, rows, out, s);
        if (!prepared) SK_TRY(prep<PK_NORM>(m, m.x, gamma, rows, c.d_model, lin_split, s));
        int off = 0;
        for (Weight* w : parts) {
            if (rows == 1) SK_TRY(linear(m, *w, 1, out + off, nullptr, s));
            else { SK_TRY(linear(m, *w, rows, m.q, nullptr, s)); SK_TRY(launch_scatter_rows(m.q, out, rows, stride, off, w->rows, s)); }
            off += w->rows;
        }
        return SKAINET_CUDA_OK;
    };
    const bool tp = c.tp_world > 1, rank0 = c.tp_rank == 0;
    // Under TP the group sum of a row-parallel projection is fused with the RMSNorm + quantizer that follows it
    // when the peer-memory kernel applies; `normed` says the next layer's input is already prepared.
    // Returns with `prepared` saying whether the quantized normalised row is already in m.act.
    auto sum_then_norm = [&](const float* gamma, bool* prepared) -> int32_t {
        *prepared = false;
        if (tp && !lin_split) {
            const int32_t st = comm_all_reduce_norm_quant(m.comm, m.x, rows, c.d_model, gamma, c.rms_eps, act_q8k_layout(m.act, rows, c.d_model), s);
            if (st == SKAINET_CUDA_OK) *prepared = true;
            if (st != 1) return st;
        }
        return tp_sum(m, m.x, (int64_t) rows * c.d_model, s);
    };
    // A row-parallel projection (o, down) and what follows it. Under TP with one activation row the matvec's own
    // epilogue stores its partial rows into every rank's inbox (rank 0 carries the residual), and the kernel that
    // follows only gathers, sums, normalises with gamma_next and quantizes. Otherwise: the projection into the
    // residual stream, then the group sum (fused with norm + quantizer where the peer-memory kernel applies).
    // gate_up != nullptr (the down projection of one row): the activation is silu(gate) * up of that fp32 row; where the
    // ring kernel can compute and quantize it in its own prologue the SwiGLU launch is skipped, else it runs first.
    auto row_parallel = [&](const Weight& w, const float* gamma_next, bool* prepared, const float* gate_up = nullptr) -> int32_t {
        *prepared = false;
        bool swiglu_inside = gate_up && rows == 1 && w.enc == SKAINET_ENC_Q4_K && w.cols <= SWIGLU_PROLOGUE_MAX_COLS && matvec_uses_ring(w, PREP_SWIGLU_F32);
        for (;;) {
            MatvecIn in;
            int prep_mode = PREP_QUANTIZED;
            if (swiglu_inside) { in.x = gate_up; prep_mode = PREP_SWIGLU_F32; }
            else {
                if (gate_up) SK_TRY(prep<PK_SWIGLU>(m, gate_up, nullptr, rows, w.cols, w.enc == SKAINET_ENC_Q8_0, s));
                if (w.enc == SKAINET_ENC_Q8_0) in.split = act_split_layout(m.act, 1, w.cols); else in.q8 = act_q8k_layout(m.act, 1, w.cols);
            }
            PeerOut po;
            int32_t st = 1;
            if (tp && !lin_split && gamma_next && comm_peer_out(m.comm, rows, c.d_model, &po)) {
                st = launch_matvec_fused(w, in, prep_mode, nullptr, rank0 ? m.x : nullptr, s, &po);
                if (st == SKAINET_CUDA_OK) {
                    SK_TRY(comm_gather_norm_quant(m.comm, m.x, rows, c.d_model, gamma_next, c.rms_eps, act_q8k_layout(m.act, rows, c.d_model), s));
                    *prepared = true;
                    return SKAINET_CUDA_OK;
                }
                if (st != 1) return st;
            }
            if (swiglu_inside) {
                st = (tp && !rank0) ? launch_matvec_fused(w, in, prep_mode, m.x, nullptr, s) : launch_matvec_fused(w, in, prep_mode, m.x, m.x, s);
                if (st == 1) { swiglu_inside = false; continue; }       // the ring kernel declined: SwiGLU as its own launch
                if (st != SKAINET_CUDA_OK) return st;
            } else if (tp && !rank0) SK_TRY(linear(m, w, rows, m.x, nullptr, s)); else SK_TRY(linear(m, w, rows, nullptr, m.x, s));
            break;
        }
        if (tp && gamma_next) return sum_then_norm(gamma_next, prepared);
        return tp_sum(m, m.x, (int64_t) rows * c.d_model, s);
    };
    bool normed = false;
    for (int l = 0; l < c.n_layers; ++l) {
        Layer& L = m.layers[l];
        SK_TRY(projections(L.wqkv, {L.wq, L.wk, L.wv}, normed, L.g_attn, m.qkv, qkv_dim));    // normed: the group sum already left the quantized row
        normed = false;
        const bool o_split = L.wo->enc == SKAINET_ENC_Q8_0;
        if (!prefill) {          // rope of q and of the new key and the cache append ride inside the split-K attention kernel
            ActQ8K oq = {nullptr, nullptr, nullptr}; ActSplit os = {nullptr, nullptr, nullptr};
            if (o_split) os = act_split_layout(m.act, rows, H * D); else oq = act_q8k_layout(m.act, rows, H * D);
            const int32_t st = launch_attn_step(m.qkv, L.kc, L.vc, m.attn, rows, H, HK, D, c.max_seq, m.kv_len, kv_bound, scale, 0, m.cos_t, m.sin_t,
                                                c.rope_mode, m.attn_scratch, o_split, oq, os, s);
            if (st != 1 && st != SKAINET_CUDA_OK) return st;
            if (st == SKAINET_CUDA_OK) {
                bool ffn_ready = false;
                SK_TRY(row_parallel(*L.wo, L.g_ffn, &ffn_ready));
                SK_TRY(projections(L.wgu, {L.wgate, L.wup}, ffn_ready, L.g_ffn, m.gu, 2 * m.ffn_l));
                SK_TRY(row_parallel(*L.wdown, l + 1 < c.n_layers ? m.layers[l + 1].g_attn : final_gamma, &normed, m.gu));
                continue;
            }
        }
        SK_CUDA(launch_pdl(rope_append_kernel, dim3(rows, H + 2 * HK), dim3(D / 2), 0, s, m.qkv, H, HK, D, (const float*) m.cos_t,
                           (const float*) m.sin_t, (const int32_t*) m.pos, (const int32_t*) (prefill ? m.row_seq : nullptr), prefill ? 1 : 0,
                           L.kc, L.vc, (int64_t) c.max_seq, c.rope_mode));
        const bool fused_attn = !prefill && (H * D) % 256 == 0;
        if (!fused_attn) SK_CUDA(launch_pdl(gather_q_kernel, dim3(rows), dim3(256), 0, s, (const float*) m.qkv, m.q, H * D, qkv_dim));
        if (prefill) {
            const __half* kc = L.kc + (size_t) seq * HK * c.max_seq * D;
            const __half* vc = L.vc + (size_t) seq * HK * c.max_seq * D;
            SK_TRY(launch_sdpa_cache(m.q, kc, vc, m.attn, 1, H, HK, rows, kv_bound, c.max_seq, D, scale, 0, m.pos + seq, s));
        } else if (fused_attn) {   // q read in place from the merged buffer; merge of the key splits quantizes for o_proj
            ActQ8K oq = {nullptr, nullptr, nullptr}; ActSplit os = {nullptr, nullptr, nullptr};
            if (o_split) os = act_split_layout(m.act, rows, H * D); else oq = act_q8k_layout(m.act, rows, H * D);
            SK_TRY(launch_attn_decode_quant(m.qkv, qkv_dim, L.kc, L.vc, m.attn, rows, H, HK, D, c.max_seq, m.kv_len, kv_bound, scale, 0,
                                            m.attn_scratch, o_split, oq, os, s));
        } else {
            SK_TRY(launch_attn_decode(m.q, L.kc, L.vc, m.attn, rows, H, HK, D, c.max_seq, m.kv_len, kv_bound, scale, 0, m.attn_scratch, s));
        }
        if (!fused_attn) SK_TRY(prep<PK_QUANT>(m, m.attn, nullptr, rows, H * D, o_split, s));
        bool ffn_ready = false;
        SK_TRY(row_parallel(*L.wo, L.g_ffn, &ffn_ready));
        SK_TRY(projections(L.wgu, {L.wgate, L.wup}, ffn_ready, L.g_ffn, m.gu, 2 * m.ffn_l));
        SK_TRY(prep<PK_SWIGLU>(m, m.gu, nullptr, rows, m.ffn_l, L.wdown->enc == SKAINET_ENC_Q8_0, s));
        SK_TRY(row_parallel(*L.wdown, l + 1 < c.n_layers ? m.layers[l + 1].g_attn : final_gamma, &normed));
    }
    if (final_prepared) *final_prepared = normed;
    return SKAINET_CUDA_OK;
}

__global__ void begin_step_kernel(const int32_t* __restrict__ pos, int32_t* __restrict__ kv_len, int batch) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < batch) kv_len[b] = pos[b] + 1;
}

// Row-wise arg max of a vocabulary shard -> (value, global index) pairs, for the TP merge.
__global__ void __launch_bounds__(1024)
argmax_pairs_kernel(const float* __restrict__ logits, int cols, int idx_offset, float* __restrict__ vals, int32_t* __restrict__ idxs) {
    __shared__ float sv[32];
    __shared__ int si[32];
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    const float* r = logits + (size_t) blockIdx.x * cols;
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
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int) (blockDim.x >> 5); ++w)
            if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
        vals[blockIdx.x] = best; idxs[blockIdx.x] = (bi == 0x7fffffff ? 0 : bi) + idx_offset;
    }
}
// Arg max of one chunk of a row's logits -> out[chunk][row] as a (value, index) record: with a vocabulary of 128256 one
// CTA per row would scan for tens of microseconds at the end of every step; the chunks of all rows run side by side and
// finish_step_kernel picks among them (lowest index on ties, as the reference's arg max does).
constexpr int ARGMAX_CHUNKS = 32;
__global__ void __launch_bounds__(256)
argmax_chunks_kernel(const float* __restrict__ logits, int cols, int chunk_cols, float2* __restrict__ out, int batch) {
    __shared__ float sv[8];
    __shared__ int si[8];
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    const int row = blockIdx.x, c0 = blockIdx.y * chunk_cols, c1 = min(cols, c0 + chunk_cols);
    const float* r = logits + (size_t) row * cols;
    float best = -INFINITY; int bi = 0x7fffffff;
    for (int i = c0 + threadIdx.x; i < c1; i += 256) {
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
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
        out[(size_t) blockIdx.y * batch + row] = make_float2(best, __int_as_float(bi));
    }
}
// pairs[world][batch] as (float, int) interleaved 8-byte records -> token per row, then the step's bookkeeping
__global__ void finish_step_kernel(const float2* __restrict__ pairs, int world, int batch, int32_t* __restrict__ cur_token,
                                   int32_t* __restrict__ pos, int32_t* __restrict__ log, const int32_t* __restrict__ log_cursor) {
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= batch) return;
    float best = -INFINITY; int bi = 0x7fffffff;
    for (int r = 0; r < world; ++r) {
        const float2 p = pairs[(size_t) r * batch + b];
        const int idx = __float_as_int(p.y);
        if (p.x > best || (p.x == best && idx < bi)) { best = p.x; bi = idx; }
    }
    if (bi == 0x7fffffff) bi = 0;               // no finite logit in the row
    cur_token[b] = bi; pos[b] += 1;
    if (log) log[(size_t) log_cursor[0] * batch + b] = bi;
}
__global__ void pack_pairs_kernel(const float* vals, const int32_t* idxs, float2* out, int n) {
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = make_float2(vals[i], __int_as_float(idxs[i]));
}

// Enqueues one greedy decode step for sequences 0..batch-1 on s.
static int32_t enqueue_step(Model& m, int batch, int kv_bound, cudaStream_t s) {
    const auto& c = m.cfg;
    begin_step_kernel<<<(batch + 255) / 256, 256, 0, s>>>(m.pos, m.kv_len, batch);
    SK_TRY(launch_embed(*m.embed, m.cur_token, batch, m.x, s));
    bool head_ready = false;
    const bool fold_out_norm = c.tp_world > 1 && c.table_enc != SKAINET_ENC_Q8_0;      // the fused sum quantizes for K-quant weights
    SK_TRY(body(m, batch, false, 0, kv_bound, s, fold_out_norm ? m.g_out : nullptr, &head_ready));
    if (head_ready) SK_TRY(linear(m, *m.head, batch, m.logits, nullptr, s));
    else SK_TRY(linear_normed(m, *m.head, m.x, m.g_out, batch, m.logits, s));
    if (c.tp_world > 1) {
        float* vals = m.tmp; int32_t* idxs = (int32_t*) (m.tmp + batch);
        float2* mine = (float2*) (m.tmp + 2 * batch); float2* all = mine + batch;
        SK_CUDA(launch_pdl(argmax_pairs_kernel, dim3(batch), dim3(1024), 0, s, (const float*) m.logits, m.vocab_l, c.tp_rank * m.vocab_l, vals, idxs));
        SK_CUDA(launch_pdl(pack_pairs_kernel, dim3((batch + 255) / 256), dim3(256), 0, s, (const float*) vals, (const int32_t*) idxs, mine, batch));
        SK_TRY(comm_all_gather(m.comm, mine, all, (int64_t) batch * 8, s));
        SK_CUDA(launch_pdl(finish_step_kernel, dim3((batch + 255) / 256), dim3(256), 0, s, (const float2*) all, c.tp_world, batch, m.cur_token, m.pos, m.log, (const int32_t*) m.log_cursor));
    } else if (c.vocab >= 8192 && (size_t) 2 * ARGMAX_CHUNKS * batch <= (size_t) m.max_rows * std::max(c.d_model, 64)) {
        float2* pairs = (float2*) m.tmp;          // free again once the head has run
        const int chunk_cols = (c.vocab + ARGMAX_CHUNKS - 1) / ARGMAX_CHUNKS;
        SK_CUDA(launch_pdl(argmax_chunks_kernel, dim3(batch, ARGMAX_CHUNKS), dim3(256), 0, s, (const float*) m.logits, c.vocab, chunk_cols, pairs, batch));
        SK_CUDA(launch_pdl(finish_step_kernel, dim3((batch + 255) / 256), dim3(256), 0, s, (const float2*) pairs, ARGMAX_CHUNKS, batch, m.cur_token, m.pos, m.log, (const int32_t*) m.log_cursor));
    } else {
        SK_CUDA(launch_pdl(argmax_advance_kernel, dim3(batch), dim3(1024), 0, s, (const float*) m.logits, c.vocab, m.cur_token, m.pos, m.log, m.log_cursor, batch));
    }
    SK_CUDA(launch_pdl(bump_cursor_kernel, dim3(1), dim3(1), 0, s, m.log_cursor));
    SK_CUDA(cudaGetLastError());
    return SKAINET_CUDA_OK;
}

static int32_t step_graph(Model& m, int batch, int bucket, cudaGraphExec_t* out) {
    auto key = std::make_pair(batch, bucket);
    auto it = m.graphs.find(key);
    if (it != m.graphs.end()) { *out = it->second; return SKAINET_CUDA_OK; }
    cudaGraph_t g = nullptr;
    SK_CUDA(cudaStreamBeginCapture(m.stream, cudaStreamCaptureModeThreadLocal));
    const int32_t st = enqueue_step(m, batch, bucket, m.stream);
    cudaError_t e = cudaStreamEndCapture(m.stream, &g);
    if (st != SKAINET_CUDA_OK) { if (g) cudaGraphDestroy(g); return st; }
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamEndCapture(step)", __FILE__, __LINE__);
    cudaGraphExec_t ge = nullptr;
    e = cudaGraphInstantiate(&ge, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGraphInstantiate(step)", __FILE__, __LINE__);
    m.graphs[key] = ge;
    *out = ge;
    return SKAINET_CUDA_OK;
}

static int max_host_pos(const Model& m, int batch) {
    int p = 0;
    for (int b = 0; b < batch; ++b) p = std::max(p, m.host_pos[b]);
    return p;
}

static int32_t run_steps(Model& m, int batch, int n_steps) {
    for (int i = 0; i < n_steps; ++i) {
        const int need = max_host_pos(m, batch) + 1;
        SK_REQUIRE(need <= m.cfg.max_seq, "decode: sequence would exceed max_seq %d", m.cfg.max_seq);
        cudaGraphExec_t ge;
        SK_TRY(step_graph(m, batch, bucket_of(m, need), &ge));
        SK_CUDA(cudaGraphLaunch(ge, m.stream));
        for (int b = 0; b < batch; ++b) m.host_pos[b] += 1;
    }
    return SKAINET_CUDA_OK;
}

// The model's device becomes the calling thread's device (flag, SM count and scratch follow it).
static int32_t set_device_of(Model& m) { return set_thread_device(m.device); }

// Copies the bounded-wait flag next to the results a call is about to wait for ...
static int32_t flag_fetch(Model& m, cudaStream_t s) {
    if (m.d_flag && m.h_flag) SK_CUDA(cudaMemcpyAsync(m.h_flag, m.d_flag, sizeof(int), cudaMemcpyDeviceToHost, s));
    return SKAINET_CUDA_OK;
}
// ... and, after the stream has been synchronised, turns a raised flag into SKAINET_CUDA_ERR_TIMEOUT (clearing it).
// A peer wait that ran out leaves the group's inboxes out of step, so the model refuses further steps.
static int32_t flag_check(Model& m) {
    if (!m.d_flag || !m.h_flag) return SKAINET_CUDA_OK;
    const int v = *m.h_flag;
    if (v == 0) return SKAINET_CUDA_OK;
    *m.h_flag = 0;
    cudaMemsetAsync(m.d_flag, 0, sizeof(int), m.stream);
    if (v == 2) m.comm_broken = true;
    return timeout_status(v);
}

static void free_model(Model* m) {
    for (auto& kv : m->graphs) cudaGraphExecDestroy(kv.second);
    for (auto& L : m->layers) {
        for (Weight* w : {L.wq, L.wk, L.wv, L.wo, L.wgate, L.wup, L.wdown, L.wqkv, L.wgu}) if (w) weight_release(w);
        cudaFree(L.g_attn); cudaFree(L.g_ffn); cudaFree(L.kc); cudaFree(L.vc);
    }
    if (m->embed) weight_release(m->embed);
    if (m->head && m->head != m->embed) weight_release(m->head);
    for (void* p : {(void*) m->g_out, (void*) m->cos_t, (void*) m->sin_t, (void*) m->x, (void*) m->qkv, (void*) m->q, (void*) m->attn,
                    (void*) m->gu, (void*) m->tmp, (void*) m->logits, (void*) m->logits_full, m->act, m->attn_scratch, (void*) m->cur_token,
                    (void*) m->pos, (void*) m->kv_len, (void*) m->log, (void*) m->log_cursor, (void*) m->row_seq})
        if (p) cudaFree(p);
    comm_destroy(m->comm);
    if (m->h_flag) cudaFreeHost(m->h_flag);
    if (m->stream) { scratch_release(m->stream); cudaStreamDestroy(m->stream); }
    m->magic = 0;
    delete m;
}

}  // namespace sk

using namespace sk;

extern "C" {

int32_t skainet_cuda_llama_create(const skainet_llama_config* cfg, skainet_model_t* out) {
    SK_REQUIRE(cfg && out, "llama_create: null argument");
    *out = 0;
    const auto& c = *cfg;
    SK_REQUIRE(c.n_layers > 0 && c.d_model > 0 && c.n_heads > 0 && c.n_kv_heads > 0 && c.ffn_dim > 0 && c.vocab > 0, "llama_create: non-positive dimension");
    SK_REQUIRE(c.head_dim == 64 || c.head_dim == 128, "llama_create: head_dim %d not in {64,128}", c.head_dim);
    SK_REQUIRE(c.n_heads % c.n_kv_heads == 0, "llama_create: n_heads %d not a multiple of n_kv_heads %d", c.n_heads, c.n_kv_heads);
    const int G = c.n_heads / c.n_kv_heads;
    SK_REQUIRE(G == 1 || G == 2 || G == 4 || G == 8, "llama_create: heads per kv head %d not in {1,2,4,8}", G);
    SK_REQUIRE(c.tp_world >= 1 && c.tp_rank >= 0 && c.tp_rank < c.tp_world, "llama_create: bad tensor-parallel position %d/%d", c.tp_rank, c.tp_world);
    SK_REQUIRE(c.n_kv_heads % c.tp_world == 0 && c.ffn_dim % c.tp_world == 0 && c.vocab % c.tp_world == 0,
               "llama_create: kv heads, ffn_dim and vocab must divide by the tensor-parallel size %d", c.tp_world);
    SK_REQUIRE(block_bytes(c.linear_enc) && block_bytes(c.table_enc), "llama_create: unknown encoding");
    SK_REQUIRE(c.linear_enc == SKAINET_ENC_Q4_K || c.linear_enc == SKAINET_ENC_Q8_0, "llama_create: linear encoding %d has no matvec kernel", c.linear_enc);
    SK_REQUIRE(c.table_enc == SKAINET_ENC_Q4_K || c.table_enc == SKAINET_ENC_Q8_0, "llama_create: table encoding %d has no matvec kernel", c.table_enc);
    const int be = block_elems(c.linear_enc);
    SK_REQUIRE(c.d_model % 256 == 0 && (c.ffn_dim / c.tp_world) % be == 0 && (c.n_heads / c.tp_world * c.head_dim) % be == 0,
               "llama_create: d_model, ffn_dim/tp and heads*head_dim/tp must be multiples of the block size");
    SK_REQUIRE(c.max_seq >= 1 && c.max_batch >= 1, "llama_create: max_seq and max_batch must be positive");
    SK_REQUIRE(c.max_batch <= 4096, "llama_create: max_batch %d above 4096", c.max_batch);
    SK_TRY(ensure_device());
    Model* m = new Model();
    m->cfg = c;
    cudaGetDevice(&m->device);
    m->d_flag = device_timeout_flag();          // allocate the per-device flag now: not allowed later inside stream capture
    if (cudaMallocHost((void**) &m->h_flag, sizeof(int)) == cudaSuccess) *m->h_flag = 0; else { cudaGetLastError(); m->h_flag = nullptr; }
    m->heads_l = c.n_heads / c.tp_world; m->kv_heads_l = c.n_kv_heads / c.tp_world;
    m->ffn_l = c.ffn_dim / c.tp_world; m->vocab_l = c.vocab / c.tp_world;
    m->layers.resize(c.n_layers);
    m->host_pos.assign(c.max_batch, 0);
    m->max_rows = std::max(c.max_batch, PREFILL_CHUNK_ROWS);
    m->log_cap = 4096;
    m->magic = MODEL_MAGIC;
    { std::lock_guard<std::mutex> lk(g_model_mu); g_models.insert(m); }
    int32_t st = SKAINET_CUDA_OK;
    auto A = [&](int32_t r) { if (st == SKAINET_CUDA_OK) st = r; };
    const size_t R = m->max_rows, D = c.head_dim;
    const size_t cache = (size_t) c.max_batch * m->kv_heads_l * c.max_seq * D;
    for (auto& L : m->layers) { A(dalloc(&L.kc, cache)); A(dalloc(&L.vc, cache)); A(dalloc(&L.g_attn, c.d_model)); A(dalloc(&L.g_ffn, c.d_model)); }
    A(dalloc(&m->g_out, c.d_model));
    A(dalloc(&m->x, R * c.d_model)); A(dalloc(&m->qkv, R * (m->heads_l + 2 * m->kv_heads_l) * D)); A(dalloc(&m->q, R * m->heads_l * D));
    A(dalloc(&m->attn, R * m->heads_l * D)); A(dalloc(&m->gu, R * 2 * m->ffn_l));
    A(dalloc(&m->tmp, R * std::max<size_t>(c.d_model, 64))); A(dalloc(&m->logits, (size_t) c.max_batch * m->vocab_l));
    if (c.tp_world > 1) A(dalloc(&m->logits_full, (size_t) c.max_batch * c.vocab));
    const int widest = std::max(std::max(c.d_model, m->ffn_l), m->heads_l * (int) D);
    m->act_bytes = std::max(act_scratch_bytes(SKAINET_ENC_Q4_K, SKAINET_ACT_NATIVE, (int) R, widest), act_scratch_bytes(SKAINET_ENC_Q8_0, SKAINET_ACT_NATIVE, (int) R, widest));
    if (st == SKAINET_CUDA_OK && cudaMalloc(&m->act, m->act_bytes) != cudaSuccess) st = cuda_fail(cudaGetLastError(), "cudaMalloc(act)", __FILE__, __LINE__);
    m->attn_scratch_bytes = attn_scratch_bytes(c.max_batch, m->heads_l, c.head_dim, c.max_seq);
    if (st == SKAINET_CUDA_OK && cudaMalloc(&m->attn_scratch, m->attn_scratch_bytes) != cudaSuccess) st = cuda_fail(cudaGetLastError(), "cudaMalloc(attn scratch)", __FILE__, __LINE__);
    A(dalloc(&m->cur_token, R)); A(dalloc(&m->pos, c.max_batch)); A(dalloc(&m->kv_len, c.max_batch));
    A(dalloc(&m->log, (size_t) m->log_cap * c.max_batch)); A(dalloc(&m->log_cursor, 1)); A(dalloc(&m->row_seq, R));
    if (st == SKAINET_CUDA_OK && cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking) != cudaSuccess) st = cuda_fail(cudaGetLastError(), "cudaStreamCreate", __FILE__, __LINE__);
    if (st == SKAINET_CUDA_OK) {
        cudaMemset(m->pos, 0, sizeof(int32_t) * c.max_batch); cudaMemset(m->log_cursor, 0, sizeof(int32_t));
        std::vector<float> ones(c.d_model, 1.0f);
        for (auto& L : m->layers) { cudaMemcpy(L.g_attn, ones.data(), 4 * c.d_model, cudaMemcpyHostToDevice); cudaMemcpy(L.g_ffn, ones.data(), 4 * c.d_model, cudaMemcpyHostToDevice); }
        cudaMemcpy(m->g_out, ones.data(), 4 * c.d_model, cudaMemcpyHostToDevice);
    }
    if (st != SKAINET_CUDA_OK) { { std::lock_guard<std::mutex> lk(g_model_mu); g_models.erase(m); } free_model(m); return st; }
    *out = (skainet_model_t) reinterpret_cast<intptr_t>(m);
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_llama_free(skainet_model_t h) {
    Model* m = model_from_handle(h);
    if (!m) return SKAINET_CUDA_ERR_HANDLE;
    set_device_of(*m);
    cudaStreamSynchronize(m->stream);
    { std::lock_guard<std::mutex> lk(g_model_mu); g_models.erase(m); }
    free_model(m);
    return SKAINET_CUDA_OK;
}

// expected shard shape of a tensor on this rank
static void shard_shape(const Model& m, int which, int* rows, int* cols, int* enc, int64_t* row0, int64_t* col0, int* full_cols) {
    const auto& c = m.cfg;
    const int D = c.head_dim, r = c.tp_rank;
    *enc = c.linear_enc; *row0 = 0; *col0 = 0;
    switch (which) {
        case SKAINET_W_EMBED: *rows = c.vocab; *cols = c.d_model; *enc = c.table_enc; break;
        case SKAINET_W_HEAD:  *rows = m.vocab_l; *cols = c.d_model; *enc = c.table_enc; *row0 = (int64_t) r * m.vocab_l; break;
        case SKAINET_W_Q:     *rows = m.heads_l * D; *cols = c.d_model; *row0 = (int64_t) r * m.heads_l * D; break;
        case SKAINET_W_K: case SKAINET_W_V: *rows = m.kv_heads_l * D; *cols = c.d_model; *row0 = (int64_t) r * m.kv_heads_l * D; break;
        case SKAINET_W_O:     *rows = c.d_model; *cols = m.heads_l * D; *col0 = (int64_t) r * m.heads_l * D; break;
        case SKAINET_W_GATE: case SKAINET_W_UP: *rows = m.ffn_l; *cols = c.d_model; *row0 = (int64_t) r * m.ffn_l; break;
        default:              *rows = c.d_model; *cols = m.ffn_l; *col0 = (int64_t) r * m.ffn_l; break;   // DOWN
    }
    *full_cols = (which == SKAINET_W_O) ? c.n_heads * D : (which == SKAINET_W_DOWN ? c.ffn_dim : c.d_model);
}

static Weight** weight_slot(Model& m, int layer, int which) {
    switch (which) {
        case SKAINET_W_EMBED: return &m.embed;
        case SKAINET_W_HEAD: return &m.head;
        case SKAINET_W_Q: return &m.layers[layer].wq;
        case SKAINET_W_K: return &m.layers[layer].wk;
        case SKAINET_W_V: return &m.layers[layer].wv;
        case SKAINET_W_O: return &m.layers[layer].wo;
        case SKAINET_W_GATE: return &m.layers[layer].wgate;
        case SKAINET_W_UP: return &m.layers[layer].wup;
        case SKAINET_W_DOWN: return &m.layers[layer].wdown;
        case SKAINET_W_QKV: return &m.layers[layer].wqkv;
        case SKAINET_W_GATE_UP: return &m.layers[layer].wgu;
        default: return nullptr;
    }
}

int32_t skainet_cuda_llama_set_weight(skainet_model_t h, int32_t layer, int32_t which, skainet_weight_t wh) {
    Model* m = model_from_handle(h);
    if (!m) return SKAINET_CUDA_ERR_HANDLE;
    Weight* w = weight_from_handle(wh);
    if (!w) return SKAINET_CUDA_ERR_HANDLE;
    SK_REQUIRE(!m->finalized, "llama_set_weight: model already finalized");
    const bool model_level = which == SKAINET_W_EMBED || which == SKAINET_W_HEAD;
    SK_REQUIRE(model_level || (layer >= 0 && layer < m->cfg.n_layers), "llama_set_weight: layer %d out of range", layer);
    Weight** slot = which >= SKAINET_W_QKV ? nullptr : weight_slot(*m, model_level ? 0 : layer, which);
    SK_REQUIRE(slot != nullptr, "llama_set_weight: %d is not a settable packed tensor", which);
    int rows, cols, enc, fc; int64_t r0, c0;
    shard_shape(*m, which, &rows, &cols, &enc, &r0, &c0, &fc);
    SK_TRY(check_weight_shape(w, enc, rows, cols, "llama_set_weight"));
    if (*slot && *slot != w) weight_release(*slot);
    *slot = w;
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_llama_set_norm(skainet_model_t h, int32_t layer, int32_t which, const float* gamma_host) {
    Model* m = model_from_handle(h);
    if (!m) return SKAINET_CUDA_ERR_HANDLE;
    SK_REQUIRE(gamma_host != nullptr, "llama_set_norm: null gains");
    SK_TRY(set_device_of(*m));
    float* dst = nullptr;
    if (which == SKAINET_W_OUT_NORM) dst = m->g_out;
    else {
        SK_REQUIRE(layer >= 0 && layer < m->cfg.n_layers, "llama_set_norm: layer %d out of range", layer);
        dst = which == SKAINET_W_ATTN_NORM ? m->layers[layer].g_attn : (which == SKAINET_W_FFN_NORM ? m->layers[layer].g_ffn : nullptr);
    }
    SK_REQUIRE(dst != nullptr, "llama_set_norm: %d is not a norm", which);
    SK_CUDA(cudaMemcpy(dst, gamma_host, sizeof(float) * m->cfg.d_model, cudaMemcpyHostToDevice));
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_llama_synth(skainet_model_t h, uint64_t seed, float std) {
    Model* m = model_from_handle(h);
    if (!m) return SKAINET_CUDA_ERR_HANDLE;
    SK_REQUIRE(!m->finalized, "llama_synth: model already finalized");
    SK_TRY(set_device_of(*m));
    auto make = [&](int layer, int which) -> int32_t {
        int rows, cols, enc, fc; int64_t r0, c0;
        shard_shape(*m, which, &rows, &cols, &enc, &r0, &c0, &fc);
        Weight* w = nullptr;
        SK_TRY(weight_alloc(enc, rows, cols, &w));
        const uint64_t tensor_seed = seed + 1000003ull * (uint64_t) (layer + 1) + 7919ull * (uint64_t) which;
        const int32_t st = launch_synth(*w, tensor_seed, std, 0, r0, c0, fc, nullptr);
        if (st != SKAINET_CUDA_OK) { weight_release(w); return st; }
        Weight** slot = weight_slot(*m, layer < 0 ? 0 : layer, which);
        if (*slot) weight_release(*slot);
        *slot = w;
        return SKAINET_CUDA_OK;
    };
    SK_TRY(make(-1, SKAINET_W_EMBED));
    SK_TRY(make(-1, SKAINET_W_HEAD));
    const int per_layer[7] = {SKAINET_W_Q, SKAINET_W_K, SKAINET_W_V, SKAINET_W_O, SKAINET_W_GATE, SKAINET_W_UP, SKAINET_W_DOWN};
    for (int l = 0; l < m->cfg.n_layers; ++l)
        for (int w : per_layer) SK_TRY(make(l, w));
    SK_CUDA(cudaDeviceSynchronize());
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_llama_get_weight(skainet_model_t h, int32_t layer, int32_t which, skainet_weight_t* out) {
    Model* m = model_from_handle(h);
    if (!m) return SKAINET_CUDA_ERR_HANDLE;
    SK_REQUIRE(out != nullptr, "llama_get_weight: null output");
    const bool model_level = which == SKAINET_W_EMBED || which == SKAINET_W_HEAD;
    SK_REQUIRE(model_level || (layer >= 0 && layer < m->cfg.n_layers), "llama_get_weight: layer %d out of range", layer);
    Weight** slot = weight_slot(*m, model_level ? 0 : layer, which);
    SK_REQUIRE(slot && *slot, "llama_get_weight: tensor %d of layer %d is not set", which, layer);
    *out = weight_to_handle(*slot);
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_llama_finalize(skainet_model_t h) {
    Model* m = model_from_handle(h);
    if (!m) return SKAINET_CUDA_ERR_HANDLE;
    if (m->finalized) return SKAINET_CUDA_OK;
    SK_TRY(set_device_of(*m));
    SK_REQUIRE(m->embed && m->head, "llama_finalize: embedding table or output head missing");
    for (int l = 0; l < m->cfg.n_layers; ++l) {
        Layer& L = m->layers[l];
        SK_REQUIRE(L.wq && L.wk && L.wv && L.wo && L.wgate && L.wup && L.wdown, "llama_finalize: layer %d is missing a weight", l);
        // parts of one encoding are merged and the merged copy replaces them; mixed encodings (a Q6_K attn_v beside Q4_K
        // q and k) keep their parts and run as separate linears over the same activation
        if (L.wq->enc == L.wk->enc && L.wk->enc == L.wv->enc) {
            SK_TRY(weight_concat_rows(L.wq, L.wk, L.wv, &L.wqkv));
            for (Weight** w : {&L.wq, &L.wk, &L.wv}) { weight_release(*w); *w = nullptr; }
        }
        if (L.wgate->enc == L.wup->enc) {
            SK_TRY(weight_concat_rows(L.wgate, L.wup, nullptr, &L.wgu));
            for (Weight** w : {&L.wgate, &L.wup}) { weight_release(*w); *w = nullptr; }
        }
    }
    // rotation factors: angle = pos * theta^(-2i/d) in double, rounded once
    const int half = m->cfg.head_dim / 2;
    std::vector<float> cs((size_t) m->cfg.max_seq * half), sn(cs.size());
    for (int p = 0; p < m->cfg.max_seq; ++p)
        for (int i = 0; i < half; ++i) {
            const double a = (double) p * pow((double) m->cfg.rope_theta, -2.0 * (double) i / (double) m->cfg.head_dim);
            cs[(size_t) p * half + i] = (float) cos(a); sn[(size_t) p * half + i] = (float) sin(a);
        }
    SK_TRY(dalloc(&m->cos_t, cs.size())); SK_TRY(dalloc(&m->sin_t, sn.size()));
    SK_CUDA(cudaMemcpy(m->cos_t, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice));
    SK_CUDA(cudaMemcpy(m->sin_t, sn.data(), sn.size() * 4, cudaMemcpyHostToDevice));
    SK_CUDA(cudaDeviceSynchronize());
    m->finalized = true;
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_llama_tp_unique_id(uint8_t* id128) {
    SK_REQUIRE(id128 != nullptr, "llama_tp_unique_id: null output");
    return comm_unique_id(id128);
}

int32_t skainet_cuda_llama_tp_init(skainet_model_t h, const uint8_t* id128) {
    Model* m = model_from_handle(h);
    if (!m) return SKAINET_CUDA_ERR_HANDLE;
    SK_REQUIRE(id128 != nullptr, "llama_tp_init: null id");
    if (m->cfg.tp_world <= 1) return SKAINET_CUDA_OK;
    SK_TRY(set_device_of(*m));
    if (m->comm) { comm_destroy(m->comm); m->comm = nullptr; }
    m->comm_broken = false;
    return comm_create(m->cfg.tp_rank, m->cfg.tp_world, id128, &m->comm);
}

// Times the group exchanges of a decode step on their own: `rounds` back-to-back launches captured in one CUDA graph,
// replayed `reps` times between two events on the model's stream. Collective: every rank calls it with the same arguments.
int32_t skainet_cuda_llama_tp_exchange_time(skainet_model_t h, int32_t mode, int32_t rounds, int32_t reps, float* us_per_round) {
    Model* m = model_from_handle(h);
    if (!m) return SKAINET_CUDA_ERR_HANDLE;
    SK_REQUIRE(us_per_round != nullptr && rounds >= 1 && rounds <= 1024 && reps >= 1, "llama_tp_exchange_time: bad arguments");
    SK_REQUIRE(m->cfg.tp_world > 1 && m->comm != nullptr, "llama_tp_exchange_time: not a tensor-parallel model with a communicator");
    SK_REQUIRE(mode >= 0 && mode <= 2, "llama_tp_exchange_time: unknown mode %d", mode);
    SK_TRY(set_device_of(*m));
    const auto& c = m->cfg;
    cudaStream_t s = m->stream;
    SK_CUDA(cudaMemsetAsync(m->x, 0, sizeof(float) * c.d_model, s));         // sums of zeros stay finite however many rounds run
    auto one = [&]() -> int32_t {
        if (mode == 0) return comm_all_reduce_sum(m->comm, m->x, c.d_model, s);
        if (mode == 2) return comm_all_reduce_sum_nccl(m->comm, m->x, c.d_model, s);
        const int32_t st = comm_all_reduce_norm_quant(m->comm, m->x, 1, c.d_model, m->layers[0].g_attn, c.rms_eps, act_q8k_layout(m->act, 1, c.d_model), s);
        if (st == 1) { set_error("llama_tp_exchange_time: the fused exchange does not apply to this model (no peer mapping or d_model outside its slots)"); return SKAINET_CUDA_ERR_INVALID; }
        return st;
    };
    SK_TRY(one());                                                              // outside capture once: lazy initialisation
    SK_CUDA(cudaStreamSynchronize(s));
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    SK_CUDA(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    int32_t st = SKAINET_CUDA_OK;
    for (int i = 0; i < rounds && st == SKAINET_CUDA_OK; ++i) st = one();
    const cudaError_t ce = cudaStreamEndCapture(s, &graph);
    if (st != SKAINET_CUDA_OK) { if (graph) cudaGraphDestroy(graph); return st; }
    SK_CUDA(ce);
    cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    SK_CUDA(e);
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    float ms = 0.0f;
    e = cudaEventCreate(&e0);
    if (e == cudaSuccess) e = cudaEventCreate(&e1);
    for (int i = 0; i < 2 && e == cudaSuccess; ++i) e = cudaGraphLaunch(exec, s);
    if (e == cudaSuccess) e = cudaEventRecord(e0, s);
    for (int i = 0; i < reps && e == cudaSuccess; ++i) e = cudaGraphLaunch(exec, s);
    if (e == cudaSuccess) e = cudaEventRecord(e1, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaGraphExecDestroy(exec);
    SK_CUDA(e);
    *us_per_round = ms * 1000.0f / ((float) rounds * (float) reps);
    SK_TRY(flag_fetch(*m, s));
    SK_CUDA(cudaStreamSynchronize(s));
    return flag_check(*m);
}

int32_t skainet_cuda_llama_reset(skainet_model_t h) {
    Model* m = model_from_handle(h);
    if (!m) return SKAINET_CUDA_ERR_HANDLE;
    SK_TRY(set_device_of(*m));
    SK_CUDA(cudaMemsetAsync(m->pos, 0, sizeof(int32_t) * m->cfg.max_batch, m->stream));
    std::fill(m->host_pos.begin(), m->host_pos.end(), 0);
    return SKAINET_CUDA_OK;
}

static int32_t require_ready(Model* m, const char* who) {
    SK_REQUIRE(m->finalized, "%s: call llama_finalize first", who);
    SK_REQUIRE(m->cfg.tp_world == 1 || m->comm != nullptr, "%s: tensor-parallel model without a communicator", who);
    if (m->comm_broken) { set_error("%s: an earlier step gave up waiting for a tensor-parallel peer; rebuild the group (llama_tp_init) before running again", who); return SKAINET_CUDA_ERR_COMM; }
    return set_device_of(*m);
}

// Greedy token after activation row `xrow` (no position bookkeeping).
static int32_t sample_row(Model& m, const float* xrow, int32_t* token_host) {
    const auto& c = m.cfg;
    cudaStream_t s = m.stream;
    SK_TRY(linear_normed(m, *m.head, xrow, m.g_out, 1, m.logits, s));
    const float* full = m.logits;
    if (c.tp_world > 1) {
        SK_TRY(comm_all_gather(m.comm, m.logits, m.logits_full, (int64_t) m.vocab_l * 4, s));
        full = m.logits_full;
    }
    SK_TRY(launch_argmax(full, 1, c.vocab, m.cur_token, s));
    SK_CUDA(cudaMemcpyAsync(token_host, m.cur_token, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
    SK_TRY(flag_fetch(m, s));
    SK_CUDA(cudaStreamSynchronize(s));
    return flag_check(m);
}

int32_t skainet_cuda_llama_prefill(skainet_model_t h, int32_t seq, const int32_t* tokens_host, int32_t n, int32_t* next_token_host) {
    Model* m = model_from_handle(h);
    if (!m) return SKAINET_CUDA_ERR_HANDLE;
    SK_TRY(require_ready(m, "llama_prefill"));
    SK_REQUIRE(seq >= 0 && seq < m->cfg.max_batch, "llama_prefill: sequence %d out of range", seq);
    SK_REQUIRE(n >= 0 && (n == 0 || tokens_host), "llama_prefill: bad token array");
    SK_REQUIRE(m->host_pos[seq] + n <= m->cfg.max_seq, "llama_prefill: %d + %d tokens exceed max_seq %d", m->host_pos[seq], n, m->cfg.max_seq);
    cudaStream_t s = m->stream;
    std::vector<int32_t> seqs(m->max_rows, seq);
    SK_CUDA(cudaMemcpyAsync(m->row_seq, seqs.data(), sizeof(int32_t) * m->max_rows, cudaMemcpyHostToDevice, s));
    int last_rows = 0;
    for (int done = 0; done < n;) {
        const int rows = std::min(n - done, m->max_rows);
        SK_CUDA(cudaMemcpyAsync(m->cur_token, tokens_host + done, sizeof(int32_t) * rows, cudaMemcpyHostToDevice, s));
        SK_TRY(launch_embed(*m->embed, m->cur_token, rows, m->x, s));
        SK_TRY(body(*m, rows, true, seq, m->host_pos[seq] + rows, s));
        m->host_pos[seq] += rows;
        SK_CUDA(cudaMemcpyAsync(m->pos + seq, &m->host_pos[seq], sizeof(int32_t), cudaMemcpyHostToDevice, s));
        SK_TRY(flag_fetch(*m, s));
        SK_CUDA(cudaStreamSynchronize(s));     // host_pos/tokens buffers are reused by the next chunk
        SK_TRY(flag_check(*m));
        done += rows; last_rows = rows;
    }
    if (next_token_host && n > 0) SK_TRY(sample_row(*m, m->x + (size_t) (last_rows - 1) * m->cfg.d_model, next_token_host));
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_llama_fake_prefill(skainet_model_t h, int32_t seq, int32_t n, uint64_t seed) {
    Model* m = model_from_handle(h);
    if (!m) return SKAINET_CUDA_ERR_HANDLE;
    SK_TRY(require_ready(m, "llama_fake_prefill"));
    SK_REQUIRE(seq >= 0 && seq < m->cfg.max_batch, "llama_fake_prefill: sequence %d out of range", seq);
    SK_REQUIRE(n >= 0 && n <= m->cfg.max_seq, "llama_fake_prefill: %d tokens exceed max_seq %d", n, m->cfg.max_seq);
    const size_t per_seq = (size_t) m->kv_heads_l * m->cfg.max_seq * m->cfg.head_dim;
    for (int l = 0; l < m->cfg.n_layers; ++l)
        fill_cache_kernel<<<592, 256, 0, m->stream>>>(m->layers[l].kc + seq * per_seq, m->layers[l].vc + seq * per_seq, (int64_t) per_seq,
                                                     (int64_t) m->cfg.max_seq * m->cfg.head_dim, m->cfg.tp_rank * m->kv_heads_l,
                                                     seed + 977ull * l + 31ull * seq);
    SK_CUDA(cudaGetLastError());
    m->host_pos[seq] = n;
    SK_CUDA(cudaMemcpyAsync(m->pos + seq, &m->host_pos[seq], sizeof(int32_t), cudaMemcpyHostToDevice, m->stream));
    SK_CUDA(cudaStreamSynchronize(m->stream));
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_llama_decode(skainet_model_t h, int32_t batch, const int32_t* tokens_in_host, int32_t* tokens_out_host) {
    Model* m = model_from_handle(h);
    if (!m) return SKAINET_CUDA_ERR_HANDLE;
    SK_TRY(require_ready(m, "llama_decode"));
    SK_REQUIRE(batch >= 1 && batch <= m->cfg.max_batch, "llama_decode: batch %d out of range (max %d)", batch, m->cfg.max_batch);
    SK_REQUIRE(tokens_in_host && tokens_out_host, "llama_decode: null token array");
    cudaStream_t s = m->stream;
    SK_CUDA(cudaMemcpyAsync(m->cur_token, tokens_in_host, sizeof(int32_t) * batch, cudaMemcpyHostToDevice, s));
    SK_CUDA(cudaMemsetAsync(m->log_cursor, 0, sizeof(int32_t), s));
    SK_TRY(run_steps(*m, batch, 1));
    SK_CUDA(cudaMemcpyAsync(tokens_out_host, m->cur_token, sizeof(int32_t) * batch, cudaMemcpyDeviceToHost, s));
    SK_TRY(flag_fetch(*m, s));
    SK_CUDA(cudaStreamSynchronize(s));
    return flag_check(*m);
}

int32_t skainet_cuda_llama_generate(skainet_model_t h, int32_t batch, const int32_t* first_tokens_host, int32_t n_steps, int32_t* out_tokens_host) {
    Model* m = model_from_handle(h);
    if (!m) return SKAINET_CUDA_ERR_HANDLE;
    SK_TRY(require_ready(m, "llama_generate"));
    SK_REQUIRE(batch >= 1 && batch <= m->cfg.max_batch, "llama_generate: batch %d out of range (max %d)", batch, m->cfg.max_batch);
    SK_REQUIRE(n_steps >= 0 && n_steps <= m->log_cap, "llama_generate: %d steps (max %d per call)", n_steps, m->log_cap);
    SK_REQUIRE(first_tokens_host && (n_steps == 0 || out_tokens_host), "llama_generate: null token array");
    cudaStream_t s = m->stream;
    SK_CUDA(cudaMemcpyAsync(m->cur_token, first_tokens_host, sizeof(int32_t) * batch, cudaMemcpyHostToDevice, s));
    SK_CUDA(cudaMemsetAsync(m->log_cursor, 0, sizeof(int32_t), s));
    SK_TRY(run_steps(*m, batch, n_steps));
    if (n_steps > 0) SK_CUDA(cudaMemcpyAsync(out_tokens_host, m->log, sizeof(int32_t) * (size_t) n_steps * batch, cudaMemcpyDeviceToHost, s));
    SK_TRY(flag_fetch(*m, s));
    SK_CUDA(cudaStreamSynchronize(s));
    return flag_check(*m);
}

int32_t skainet_cuda_llama_logits(skainet_model_t h, int32_t batch, float* logits_host) {
    Model* m = model_from_handle(h);
    if (!m) return SKAINET_CUDA_ERR_HANDLE;
    SK_TRY(require_ready(m, "llama_logits"));
    SK_REQUIRE(batch >= 1 && batch <= m->cfg.max_batch && logits_host, "llama_logits: bad arguments");
    cudaStream_t s = m->stream;
    const auto& c = m->cfg;
    if (c.tp_world == 1) {
        SK_CUDA(cudaMemcpyAsync(logits_host, m->logits, sizeof(float) * (size_t) batch * c.vocab, cudaMemcpyDeviceToHost, s));
        SK_CUDA(cudaStreamSynchronize(s));
        return SKAINET_CUDA_OK;
    }
    SK_TRY(comm_all_gather(m->comm, m->logits, m->logits_full, (int64_t) batch * m->vocab_l * 4, s));
    std::vector<float> tmp((size_t) batch * c.vocab);
    SK_CUDA(cudaMemcpyAsync(tmp.data(), m->logits_full, sizeof(float) * tmp.size(), cudaMemcpyDeviceToHost, s));
    SK_CUDA(cudaStreamSynchronize(s));
    for (int r = 0; r < c.tp_world; ++r)
        for (int b = 0; b < batch; ++b)
            memcpy(logits_host + (size_t) b * c.vocab + (size_t) r * m->vocab_l, tmp.data() + ((size_t) r * batch + b) * m->vocab_l, sizeof(float) * m->vocab_l);
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_llama_step_cost(skainet_model_t h, int32_t batch, int64_t* out2) {
    Model* m = model_from_handle(h);
    if (!m) return SKAINET_CUDA_ERR_HANDLE;
    SK_TRY(require_ready(m, "llama_step_cost"));
    SK_REQUIRE(batch >= 1 && batch <= m->cfg.max_batch && out2, "llama_step_cost: bad arguments");
    const auto& c = m->cfg;
    int64_t bytes = m->head->packed_bytes;
    for (const auto& L : m->layers)
        for (const Weight* w : {L.wqkv, L.wq, L.wk, L.wv, L.wo, L.wgu, L.wgate, L.wup, L.wdown}) if (w) bytes += w->packed_bytes;
    for (int b = 0; b < batch; ++b)
        bytes += (int64_t) c.n_layers * 2 * m->kv_heads_l * c.head_dim * 2 * (m->host_pos[b] + 1)            // K and V visible, f16
               + (int64_t) (c.d_model / block_elems(c.table_enc)) * block_bytes(c.table_enc);                  // one table row
    out2[0] = bytes;
    cudaGraphExec_t ge;
    SK_TRY(step_graph(*m, batch, bucket_of(*m, max_host_pos(*m, batch) + 1), &ge));
    // kernel nodes of the step graph = launches per step
    cudaGraph_t g = nullptr;
    size_t n = 0;
    int64_t kernels = 0;
#if CUDART_VERSION >= 12000
    (void) g;
#endif
    // Count by re-capturing into a throw-away graph (cheap; the exec graph does not expose its nodes).
    SK_CUDA(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
    const int32_t st = enqueue_step(*m, batch, bucket_of(*m, max_host_pos(*m, batch) + 1), m->stream);
    cudaError_t e = cudaStreamEndCapture(m->stream, &g);
    if (st != SKAINET_CUDA_OK) { if (g) cudaGraphDestroy(g); return st; }
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamEndCapture(count)", __FILE__, __LINE__);
    SK_CUDA(cudaGraphGetNodes(g, nullptr, &n));
    std::vector<cudaGraphNode_t> nodes(n);
    SK_CUDA(cudaGraphGetNodes(g, nodes.data(), &n));
    for (size_t i = 0; i < n; ++i) {
        cudaGraphNodeType t;
        if (cudaGraphNodeGetType(nodes[i], &t) == cudaSuccess && t == cudaGraphNodeTypeKernel) ++kernels;
    }
    cudaGraphDestroy(g);
    out2[1] = kernels;
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_llama_peek(skainet_model_t h, int32_t which, float* host_out, int64_t n) {
    Model* m = model_from_handle(h);
    if (!m) return SKAINET_CUDA_ERR_HANDLE;
    SK_REQUIRE(host_out && n >= 0, "llama_peek: bad arguments");
    SK_TRY(set_device_of(*m));
    const float* src = which == 0 ? m->x : which == 1 ? m->qkv : which == 2 ? m->attn : which == 3 ? m->gu : which == 4 ? m->q : nullptr;
    SK_REQUIRE(src != nullptr, "llama_peek: unknown buffer %d", which);
    SK_CUDA(cudaStreamSynchronize(m->stream));
    SK_CUDA(cudaMemcpy(host_out, src, sizeof(float) * (size_t) n, cudaMemcpyDeviceToHost));
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_llama_stream(skainet_model_t h, skainet_stream_t* out) {
    Model* m = model_from_handle(h);
    if (!m) return SKAINET_CUDA_ERR_HANDLE;
    SK_REQUIRE(out != nullptr, "llama_stream: null output");
    *out = (skainet_stream_t) m->stream;
    return SKAINET_CUDA_OK;
}

}  // extern "C"
