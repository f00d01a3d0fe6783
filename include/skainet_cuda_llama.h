/*
 * skainet_cuda_llama.h — a Llama-style decoder runtime over the kernels of skainet_cuda.h, inside the
 * same library: weights and the f16 KV cache resident in HBM, one CUDA graph per decode step, greedy
 * sampling on the device, optional tensor parallelism over NCCL.
 *
 * The reference repository holds no transformer runtime (it moved to the sibling project
 * SKaiNET-transformers: docs/modules/ROOT/pages/tutorials/kllama-getting-started.adoc:1-12), so
 * nothing here replaces a reference entry point one-to-one. The step is composed exactly from the
 * operators the reference does define, in the order a decoder applies them:
 *   gather over a packed table      DefaultCpuOps.kt:3746-3793
 *   rms norm                        native/src/f32_fused.c:255-286
 *   packed matvec (Q4_K / Q8_0)     native/src/q4k_matmul.c:315-357, native/src/q8_0_matmul.c:168-187
 *   scaled dot product attention    native/src/f32_fused.c:304-396 (grouped-query, causal)
 *   silu, mul, add                  native/src/f32_ops.c:107-114,243-245
 *   arg max, lowest index on ties   DefaultCpuOps.kt:3042-3078
 * plus RoPE, which has no reference code (convention declared at skainet_cuda_rope_dev). The nearest
 * in-repo analogue of the loop is the decode harness
 * (skainet-backends/skainet-backend-cpu/src/commonTest/kotlin/sk/ainet/exec/harness/DecodeHarness.kt:49-149).
 */
#ifndef SKAINET_CUDA_LLAMA_H
#define SKAINET_CUDA_LLAMA_H

#include "skainet_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef int64_t skainet_model_t;

typedef struct {
    int32_t n_layers, d_model, n_heads, n_kv_heads, head_dim, ffn_dim, vocab;
    float rms_eps, rope_theta;
    int32_t rope_mode;        /* 0 = pairs (2i, 2i+1), 1 = pairs (i, i + head_dim/2) */
    int32_t max_seq;          /* KV cache capacity in tokens per sequence */
    int32_t max_batch;        /* sequences decoded together */
    int32_t linear_enc;       /* SKAINET_ENC_* of q/k/v/o/gate/up/down (Q4_K in the benchmark configs) */
    int32_t table_enc;        /* SKAINET_ENC_* of the embedding table and the output head */
    int32_t tp_rank, tp_world;/* tensor parallel position; world 1 = single GPU */
} skainet_llama_config;

/* Which tensor of a layer (layer index ignored for the three model-level tensors). */
#define SKAINET_W_EMBED     0   /* [vocab, d_model] packed table (replicated)                         */
#define SKAINET_W_HEAD      1   /* [vocab, d_model] packed, rows sharded under TP                     */
#define SKAINET_W_OUT_NORM  2   /* gamma [d_model]                                                     */
#define SKAINET_W_ATTN_NORM 3   /* gamma [d_model]                                                     */
#define SKAINET_W_Q         4   /* [n_heads*head_dim, d_model]        rows sharded under TP           */
#define SKAINET_W_K         5   /* [n_kv_heads*head_dim, d_model]     rows sharded                    */
#define SKAINET_W_V         6
#define SKAINET_W_O         7   /* [d_model, n_heads*head_dim]        columns sharded                 */
#define SKAINET_W_FFN_NORM  8   /* gamma [d_model]                                                     */
#define SKAINET_W_GATE      9   /* [ffn_dim, d_model]                 rows sharded                    */
#define SKAINET_W_UP        10
#define SKAINET_W_DOWN      11  /* [d_model, ffn_dim]                 columns sharded                 */
/* read-only, after finalize (the parts they were merged from are released then): */
#define SKAINET_W_QKV       12  /* rows of q, k, v in one tensor                                      */
#define SKAINET_W_GATE_UP   13  /* rows of gate then up in one tensor                                 */

SKAINET_CUDA_API int32_t skainet_cuda_llama_create(const skainet_llama_config* cfg, skainet_model_t* out);
SKAINET_CUDA_API int32_t skainet_cuda_llama_free(skainet_model_t m);

/* Hands a resident packed weight to the model (the model owns it afterwards). Under TP the weight is
 * this rank's shard. */
SKAINET_CUDA_API int32_t skainet_cuda_llama_set_weight(skainet_model_t m, int32_t layer, int32_t which, skainet_weight_t w);
/* Norm gains from host floats. */
SKAINET_CUDA_API int32_t skainet_cuda_llama_set_norm(skainet_model_t m, int32_t layer, int32_t which, const float* gamma_host);
/* Random-init model of the configured shape, generated and packed on the device: linears std*N(0,1)
 * in linear_enc, table and head in table_enc, gains 1. Under TP every rank generates its own shard of
 * the same seeded full tensors. */
SKAINET_CUDA_API int32_t skainet_cuda_llama_synth(skainet_model_t m, uint64_t seed, float std);
/* The resident weight behind (layer, which), e.g. to export its bytes for a CPU reference. */
SKAINET_CUDA_API int32_t skainet_cuda_llama_get_weight(skainet_model_t m, int32_t layer, int32_t which, skainet_weight_t* out);
/* Call once after the last set_weight/synth: merges q/k/v and gate/up, builds the RoPE table. */
SKAINET_CUDA_API int32_t skainet_cuda_llama_finalize(skainet_model_t m);
/* One communicator per TP group, from a 128-byte NCCL unique id made on rank 0 (all ranks call). */
SKAINET_CUDA_API int32_t skainet_cuda_llama_tp_unique_id(uint8_t* id128);
SKAINET_CUDA_API int32_t skainet_cuda_llama_tp_init(skainet_model_t m, const uint8_t* id128);

/* Forget all cached tokens of every sequence. */
SKAINET_CUDA_API int32_t skainet_cuda_llama_reset(skainet_model_t m);
/* Runs n prompt tokens of sequence `seq` through the model, filling its cache from its current
 * position. If next_token_host != NULL it receives the greedy token after the last prompt token. */
SKAINET_CUDA_API int32_t skainet_cuda_llama_prefill(skainet_model_t m, int32_t seq, const int32_t* tokens_host, int32_t n,
    int32_t* next_token_host);
/* Fills sequence `seq`'s cache with n tokens worth of seeded random K/V instead of running a prompt
 * (throughput runs at long context, where the reference CPU path could not produce the prefill). */
SKAINET_CUDA_API int32_t skainet_cuda_llama_fake_prefill(skainet_model_t m, int32_t seq, int32_t n, uint64_t seed);
/* One greedy decode step for sequences 0..batch-1: tokens_in_host[b] is fed at each sequence's
 * position, tokens_out_host[b] receives the arg max. Host in, host out: the end-to-end call. */
SKAINET_CUDA_API int32_t skainet_cuda_llama_decode(skainet_model_t m, int32_t batch, const int32_t* tokens_in_host,
    int32_t* tokens_out_host);
/* n_steps greedy steps entirely on the device (each step's arg max feeds the next), one graph replay
 * per step, no host synchronisation inside. first_tokens_host[batch] starts the run;
 * out_tokens_host[n_steps * batch] receives step-major tokens. */
SKAINET_CUDA_API int32_t skainet_cuda_llama_generate(skainet_model_t m, int32_t batch, const int32_t* first_tokens_host,
    int32_t n_steps, int32_t* out_tokens_host);
/* Logits of the last step, [batch, vocab] fp32 (full vocabulary on every rank). */
SKAINET_CUDA_API int32_t skainet_cuda_llama_logits(skainet_model_t m, int32_t batch, float* logits_host);
/* Bytes one decode step must read from HBM at the current positions (weights once + KV visible),
 * and the number of kernels one step launches: the roofline inputs of the bench. out2 = {bytes, launches}. */
SKAINET_CUDA_API int32_t skainet_cuda_llama_step_cost(skainet_model_t m, int32_t batch, int64_t* out2);
/* Diagnostic: the first n floats of an activation buffer as the last step left it
 * (0 residual stream, 1 merged q|k|v as projected — a decode step rotates q and k inside its attention kernel, a prompt
 * chunk rotates q in place —, 2 attention output, 3 gate|up, 4 q). */
SKAINET_CUDA_API int32_t skainet_cuda_llama_peek(skainet_model_t m, int32_t which, float* host_out, int64_t n);
/* Measurement aid (no reference counterpart): the group exchanges of a decode step timed on their own. `rounds` launches
 * are captured back to back in one CUDA graph and replayed `reps` times between two events; *us_per_round = device time of
 * one exchange of a [d_model] fp32 row. mode 0: in-place sum through peer memory; 1: store + gather + sum + RMSNorm +
 * quantize in one kernel (what follows a row-parallel projection); 2: the same sum through NCCL. Collective: every rank
 * of the group calls it with the same arguments. */
SKAINET_CUDA_API int32_t skainet_cuda_llama_tp_exchange_time(skainet_model_t m, int32_t mode, int32_t rounds, int32_t reps, float* us_per_round);
/* The stream the model runs on (for event timing by the caller). */
SKAINET_CUDA_API int32_t skainet_cuda_llama_stream(skainet_model_t m, skainet_stream_t* out);

#ifdef __cplusplus
}
#endif
#endif /* SKAINET_CUDA_LLAMA_H */
