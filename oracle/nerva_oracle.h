/*
 * TEST INFRASTRUCTURE — NOT A PRODUCT CODE PATH.
 *
 * CPU restatement (plain C, fp32, serial reduction order) of the reference's
 * CPU decoder and of the numeric contract of its CUDA layer path.  Only the
 * test-suite, the smoke check and the CPU-baseline leg of the benchmark may
 * link or call this library; the CUDA library never does.
 *
 * Each function cites the reference source it restates (paths relative to the
 * reference repository root).
 */
#ifndef NERVA_ORACLE_H_
#define NERVA_ORACLE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { ORACLE_DTYPE_F16 = 0, ORACLE_DTYPE_BF16 = 1 };

/* Numeric contract selector.
 * ORACLE_MODE_CPU  : crates/nerva-model CPU path — f32 KV cache, f32 (unrounded)
 *                    mat-vec inputs, residual stream re-encoded to the model
 *                    dtype between layers.
 * ORACLE_MODE_CUDA : native/cuda layer path — mat-vec inputs and K/V rounded
 *                    to the model dtype, residual stream kept in f32 across
 *                    layers (hf_decode_sequence/kernels.cu:182-217,434-492,
 *                    577-612,651-687). */
/* ORACLE_MODE_CPU_KV16: the CPU contract with K and V rounded to the model dtype
 * when they enter the cache (the paged cache of the C ABI holds 16-bit values,
 * hf_decode_sequence/types.cuh:328-337).  Used to study contracts; not a
 * reference path by itself. */
enum { ORACLE_MODE_CPU = 0, ORACLE_MODE_CUDA = 1, ORACLE_MODE_CPU_KV16 = 2 };

typedef struct OracleLayer {
  const uint16_t *rms_attn, *rms_mlp;
  const uint16_t *w_q, *w_k, *w_v, *w_o;
  const uint16_t *q_norm, *k_norm;            /* optional, [head_dim] */
  const uint16_t *q_bias, *k_bias, *v_bias, *o_bias; /* optional */
  const uint16_t *w_gate, *w_up, *w_down;     /* dense MLP */
  /* softmax top-k sparse MoE (mlp_kind == 1) */
  uint32_t mlp_kind, moe_intermediate, shared_intermediate;
  uint32_t num_experts, top_k, norm_topk_prob;
  const uint16_t *w_router, *w_expert_gate_up, *w_expert_down;
  const uint16_t *w_shared_gate, *w_shared_up, *w_shared_down, *w_shared_router;
  /* DeepSeek multi-head latent attention (attention_kind == 2), the V2-Lite form without a query
   * low-rank stage: w_q is [heads * (nope + rope)][hidden], w_o is [hidden][heads * v_head_dim]
   * (v_head_dim == model head_dim), and
   *   w_kv_a    [kv_lora_rank + rope][hidden]      latent + shared rotary key
   *   kv_a_norm [kv_lora_rank]                     RMSNorm weight of the latent
   *   w_kv_b    [heads * (nope + v)][kv_lora_rank] per head: nope rows of W_UK, then v rows of W_UV
   * With attention_kind == 2 a sparse-MoE layer's shared experts are ungated (w_shared_router NULL). */
  uint32_t attention_kind, kv_lora_rank, qk_nope_head_dim, qk_rope_head_dim;
  const uint16_t *w_kv_a, *kv_a_norm, *w_kv_b;
} OracleLayer;

typedef struct OracleModel {
  uint32_t dtype, hidden, heads, kv_heads, head_dim, intermediate, vocab, layers;
  float rms_eps, rope_theta; /* rope_theta <= 0 disables RoPE */
  const uint16_t *embeddings, *final_norm, *lm_head;
  const OracleLayer *layer;
} OracleModel;

typedef struct OracleCtx OracleCtx;

/* codecs: crates/nerva-model/src/precision/bits.rs:4-18,20-85 */
float oracle_bf16_to_f32(uint16_t bits);
uint16_t oracle_f32_to_bf16(float value);
float oracle_f16_to_f32(uint16_t bits);
uint16_t oracle_f32_to_f16(float value);

/* precision/block/ops.rs:32-99 */
void oracle_rms_norm(uint32_t dtype, const float *input, const uint16_t *weight,
                     uint32_t n, float eps, float *output);
void oracle_per_head_rms_norm(uint32_t dtype, const uint16_t *weight, uint32_t head_dim,
                              float *values, uint32_t n, float eps);
void oracle_matvec(uint32_t dtype, const uint16_t *matrix, const float *input,
                   uint32_t rows, uint32_t cols, float *output);
/* common/rope.rs:54-79 */
void oracle_rope(float *values, uint32_t heads, uint32_t head_dim, uint32_t position,
                 float theta);
/* attention/exact/run.rs:13-127 with a single visible-KV block (the decoder's
 * use, precision/block/model/kv.rs:176-189).  keys/values: [tokens][kv_heads*head_dim]. */
int oracle_attention(const float *query, const float *keys, const float *values,
                     uint32_t tokens, uint32_t heads, uint32_t kv_heads, uint32_t head_dim,
                     float *output);
/* Same math over a paged, dtype-encoded cache:
 * native/cuda/hf_decode_sequence/types.cuh:328-337 (page addressing, 16-token
 * pages) and attention_kernels.cu:528-760 (K/V decoded to f32, f32 query). */
int oracle_attention_paged(uint32_t dtype, const float *query, const uint16_t *key_pages,
                           const uint16_t *value_pages, const uint32_t *page_table,
                           uint32_t tokens, uint32_t heads, uint32_t kv_heads,
                           uint32_t head_dim, float *output);
/* common/token.rs:33-58 (mode CPU: -1 on a non-finite logit) and
 * native/cuda/hf_decode_sequence/sampler.cu:35-40,89-119 (mode CUDA: non-finite
 * logits skipped, lowest index wins ties, 0 when nothing is finite). */
int64_t oracle_argmax(const float *logits, uint32_t n, int mode);
/* common/math.rs:76-82 */
float oracle_silu(float value);

/* softmax top-k routing: native/cuda/hf_decode_sequence/device_ops.cuh:212-258
 * and crates/nerva-model/src/precision/block/moe.rs:1303-1326. */
void oracle_route_softmax_topk(const float *router_logits, uint32_t num_experts,
                               uint32_t top_k, uint32_t norm_topk_prob,
                               uint32_t *experts, float *weights);

/* Decoder. */
OracleCtx *oracle_create(const OracleModel *model, uint32_t max_context, int mode);
void oracle_destroy(OracleCtx *ctx);
void oracle_reset(OracleCtx *ctx);
uint32_t oracle_position(const OracleCtx *ctx);
/* Timing aid: jump to `position` with a patterned cache (see the definition). */
int oracle_seek_for_timing(OracleCtx *ctx, uint32_t position);
/* Runs one token at the current position through every layer and appends its
 * K/V.  logits (vocab floats) may be NULL to skip final norm + lm_head. */
int oracle_step(OracleCtx *ctx, uint32_t token, float *logits);
/* causal_lm/context.rs:41-120: all prompt rows, first generated token from the
 * last prompt row, then steps-1 decode steps.  logits_out: steps*vocab or NULL.
 * Returns the number of tokens written, or -1. */
int oracle_decode_greedy(OracleCtx *ctx, const uint32_t *prompt, uint32_t prompt_count,
                         uint32_t steps, uint32_t *tokens_out, float *logits_out);
/* Last layer-stack output of the most recent step (f32 view). */
const float *oracle_hidden_state(const OracleCtx *ctx);

/* FNV-1a-64 helpers of the ABI: hf_decode_sequence/weights.cu:78-111. */
uint64_t oracle_hash_tokens(const uint32_t *tokens, uint32_t count);

/* Host thread count used by the row-parallel mat-vec (results do not depend on it). */
/* Summation-order probe for tolerance-floor measurements: 1 = the reference's
 * serial order (default); n > 1 = n interleaved partial sums per row. */
void oracle_set_sum_lanes(int lanes);
void oracle_set_threads(int threads);
int oracle_get_threads(void);

#ifdef __cplusplus
}
#endif
#endif
