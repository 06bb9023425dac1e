/*
 * C ABI of the B200-native resident decode step.
 *
 * Every `nerva_cuda_*` entry point and every `NervaCuda*` struct below has the
 * same name, field order, field types and error convention as its counterpart
 * in the reference's native/cuda/nerva_cuda_api.h, so the reference's FFI crate
 * (crates/nerva-cuda, `repr(C)` mirrors in src/decode/hf_sequence/session/ffi.rs)
 * links against this library unchanged.  The citation after each declaration is
 * the reference declaration it replaces.
 *
 * Error convention (reference: hf_decode_sequence/session_api_lifecycle.inc.cu):
 * return 0 on success and -1 on failure; `out` is zero-filled first, then
 * `status` (0 / -1) and `cuda_error` (a cudaError_t value) are set.  Invalid
 * arguments are rejected before any device call.  Nothing here falls back to
 * the CPU: without a CUDA device `cuda_error` is cudaErrorNoDevice.
 *
 * Entry points named `nerva_b200_*` are additive (no reference counterpart);
 * each says so.
 */
#ifndef NERVA_B200_API_H_
#define NERVA_B200_API_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* dtype codes — hf_decode_sequence/types.cuh:9-11 */
#define NERVA_DTYPE_F16 0u
#define NERVA_DTYPE_BF16 1u
#define NERVA_DTYPE_F32 2u
/* hf_decode_sequence/types.cuh:12-16,37-38,64 */
#define NERVA_MLP_KIND_DENSE 0u
#define NERVA_MLP_KIND_SPARSE_MOE 1u
#define NERVA_ATTENTION_KIND_FULL 0u
#define NERVA_ATTENTION_KIND_LINEAR_GDN 1u
#define NERVA_ATTENTION_KIND_DEEPSEEK_MLA 2u
#define NERVA_WEIGHT_STRATEGY_GPU_RESIDENT 1u
#define NERVA_WEIGHT_STRATEGY_GPU_STAGED 2u
#define NERVA_KV_CACHE_BLOCK_TOKENS 16u

/* nerva_cuda_api.h:29-37 — one entry of the device token ring (40 bytes). */
typedef struct NervaCudaSyntheticTokenSlot {
  uint32_t request_id;
  uint32_t sequence_id;
  uint64_t token_index;
  uint32_t token;
  uint64_t version;
  uint32_t completion;
  uint32_t host_copied;
} NervaCudaSyntheticTokenSlot;

/* nerva_cuda_api.h:255-332 */
typedef struct NervaCudaHfDecodeChainLayer {
  const uint16_t *rms_attn_weight;
  const uint16_t *rms_mlp_weight;
  const uint16_t *w_q;
  const uint16_t *w_q_gate;
  const uint16_t *w_k;
  const uint16_t *q_norm_weight;
  const uint16_t *k_norm_weight;
  const uint16_t *w_v;
  const uint16_t *w_o;
  const uint16_t *q_bias;
  const uint16_t *k_bias;
  const uint16_t *v_bias;
  const uint16_t *o_bias;
  const uint16_t *w_gate;
  const uint16_t *w_up;
  const uint16_t *w_down;
  const uint16_t *w_router;
  const uint16_t *w_expert_gate_up;
  const uint16_t *w_expert_down;
  const uint16_t *w_shared_expert_gate;
  const uint16_t *w_shared_expert_up;
  const uint16_t *w_shared_expert_down;
  const uint16_t *w_shared_expert_router;
  uint32_t linear_key_heads;
  uint32_t linear_value_heads;
  uint32_t linear_key_head_dim;
  uint32_t linear_value_head_dim;
  uint32_t linear_conv_kernel;
  const uint16_t *w_linear_conv;
  const uint16_t *w_linear_qkv;
  const uint16_t *w_linear_z;
  const uint16_t *w_linear_b;
  const uint16_t *w_linear_a;
  const uint16_t *w_linear_dt_bias;
  const float *w_linear_a_log;
  const uint16_t *w_linear_norm;
  const uint16_t *w_linear_out;
  uint32_t mlp_kind;
  uint32_t moe_intermediate;
  uint32_t shared_expert_intermediate;
  uint32_t num_experts;
  uint32_t experts_per_token;
  uint32_t norm_topk_prob;
  uint32_t attention_kind;
  uint32_t deepseek_mode;
  uint32_t deepseek_flags;
  uint32_t deepseek_storage;
  uint32_t deepseek_hc_mult;
  uint32_t deepseek_hc_sinkhorn_iters;
  uint32_t deepseek_q_lora_rank;
  uint32_t deepseek_kv_lora_rank;
  uint32_t deepseek_o_lora_rank;
  uint32_t deepseek_o_groups;
  uint32_t deepseek_qk_nope_head_dim;
  uint32_t deepseek_qk_rope_head_dim;
  uint32_t deepseek_v_head_dim;
  uint32_t deepseek_compress_ratio;
  uint32_t deepseek_index_topk;
  uint32_t deepseek_index_n_heads;
  uint32_t deepseek_index_head_dim;
  uint32_t deepseek_router_num_groups;
  uint32_t deepseek_router_topk_groups;
  float deepseek_routed_scaling_factor;
  float deepseek_hc_eps;
  float deepseek_hc_post_alpha;
  uint32_t deepseek_rope_scaling_type;
  uint32_t deepseek_rope_original_max_position;
  float deepseek_rope_scaling_factor;
  float deepseek_rope_extrapolation_factor;
  float deepseek_rope_attn_factor;
  float deepseek_rope_beta_fast;
  float deepseek_rope_beta_slow;
  float deepseek_rope_mscale;
  float deepseek_rope_mscale_all_dim;
  float deepseek_compress_rope_theta;
  float deepseek_swiglu_limit;
} NervaCudaHfDecodeChainLayer;

/* nerva_cuda_api.h:380-391 */
typedef struct NervaCudaHfDecodeSequenceWeightBlock {
  const uint16_t *host_source;
  const char *source_file;
  uint64_t source_file_len;
  uint64_t file_offset_begin;
  uint64_t block_id;
  uint64_t block_version;
  uint64_t offset_bytes;
  uint64_t bytes;
  uint32_t strategy;
  uint32_t reserved;
} NervaCudaHfDecodeSequenceWeightBlock;

/* nerva_cuda_api.h:393-399 */
typedef struct NervaCudaHfDecodeSamplerConfig {
  float temperature;
  float top_p;
  uint32_t top_k;
  uint32_t reserved;
  uint64_t seed;
} NervaCudaHfDecodeSamplerConfig;

/* nerva_cuda_api.h:401-434 */
typedef struct NervaCudaHfDecodeSequenceRequest {
  uint32_t dtype;
  uint32_t hidden;
  uint32_t heads;
  uint32_t kv_heads;
  uint32_t head_dim;
  uint32_t intermediate;
  uint32_t vocab_size;
  uint32_t layer_count;
  uint32_t steps;
  uint32_t seed_token;
  const uint32_t *prompt_tokens;
  uint32_t prompt_token_count;
  uint32_t has_eos_token;
  uint32_t eos_token;
  float rms_eps;
  float rope_theta;
  const uint16_t *embeddings;
  const NervaCudaHfDecodeChainLayer *layers;
  const uint16_t *final_norm_weight;
  const uint16_t *lm_head;
  uint32_t planned_weight_blocks;
  uint32_t planned_gpu_resident_blocks;
  uint32_t planned_gpu_staged_blocks;
  uint64_t planned_weight_bytes;
  uint64_t planned_gpu_resident_weight_bytes;
  uint64_t planned_gpu_staged_weight_bytes;
  const NervaCudaHfDecodeSequenceWeightBlock *planned_weight_descriptors;
  uint32_t planned_weight_descriptor_count;
  uint64_t planned_weight_descriptor_hash;
  uint32_t *output_tokens;
  uint32_t output_token_capacity;
  NervaCudaHfDecodeSamplerConfig sampler;
} NervaCudaHfDecodeSequenceRequest;

/* nerva_cuda_api.h:436-513 */
typedef struct NervaCudaHfDecodeSequenceResult {
  int32_t status;
  int32_t cuda_error;
  int32_t device_count;
  uint32_t dtype;
  uint32_t hidden;
  uint32_t heads;
  uint32_t kv_heads;
  uint32_t head_dim;
  uint32_t intermediate;
  uint32_t vocab_size;
  uint32_t layer_count;
  uint32_t steps;
  uint32_t seed_token;
  uint32_t observed_tokens;
  uint32_t last_token;
  uint64_t observed_token_hash;
  uint64_t resident_weight_bytes;
  uint32_t planned_weight_blocks;
  uint32_t planned_gpu_resident_blocks;
  uint32_t planned_gpu_staged_blocks;
  uint64_t planned_weight_bytes;
  uint64_t planned_gpu_resident_weight_bytes;
  uint64_t planned_gpu_staged_weight_bytes;
  uint64_t descriptor_gpu_resident_h2d_bytes;
  uint64_t descriptor_gpu_staged_h2d_bytes;
  uint32_t planned_weight_descriptor_count;
  uint64_t planned_weight_descriptor_hash;
  uint64_t resident_kv_bytes;
  uint64_t deepseek_mhc_residual_bytes;
  uint64_t deepseek_mhc_post_mix_bytes;
  uint64_t deepseek_mhc_comb_mix_bytes;
  uint64_t kv_tokens;
  uint64_t device_arena_bytes;
  uint64_t pinned_host_bytes;
  uint64_t h2d_bytes;
  uint64_t d2h_bytes;
  uint64_t graph_replays;
  uint64_t graph_nodes;
  uint64_t graph_launches;
  uint64_t graph_captures;
  uint64_t graph_cache_hits;
  uint64_t kernel_launches;
  uint64_t experimental_rt_selector_launches;
  uint32_t experimental_rt_sparse_attention_active;
  uint32_t experimental_rt_dense_attention_chunks;
  uint32_t experimental_rt_attention_chunks;
  uint32_t experimental_rt_reserved;
  uint64_t device_elapsed_ns;
  uint64_t projection_ns;
  uint64_t qkv_projection_ns;
  uint64_t attention_output_projection_ns;
  uint64_t gate_up_projection_ns;
  uint64_t down_projection_ns;
  uint64_t lm_head_projection_ns;
  uint64_t attention_ns;
  uint64_t mlp_ns;
  uint64_t norm_ns;
  uint64_t sampling_ns;
  uint64_t sync_calls;
  uint64_t host_causality_edges;
  uint64_t hot_path_allocations;
  uint64_t deepseek_compressor_state_writes;
  uint64_t deepseek_compressed_kv_writes;
  uint64_t deepseek_indexer_state_writes;
  uint64_t deepseek_indexer_kv_writes;
  uint64_t deepseek_compressed_kv_attention_reads;
  uint64_t deepseek_compressed_kv_attention_slots_scanned;
  uint64_t deepseek_sparse_topk_selections;
  uint64_t deepseek_sparse_topk_slots_selected;
  uint64_t deepseek_sparse_topk_candidates_scored;
  uint64_t deepseek_sparse_topk_selection_hash;
  uint64_t deepseek_v3_grouped_router_selections;
  uint64_t deepseek_v4_bias_router_selections;
  uint64_t deepseek_v4_hash_router_selections;
  uint64_t deepseek_raw_attention_tokens_scanned;
  uint64_t deepseek_sparse_attention_output_hash;
} NervaCudaHfDecodeSequenceResult;

/* nerva_cuda_api.h:515-525 */
typedef struct NervaCudaHfDecodeSequenceLayoutPlanRequest {
  uint32_t hidden;
  uint32_t heads;
  uint32_t kv_heads;
  uint32_t head_dim;
  uint32_t intermediate;
  uint32_t vocab_size;
  uint32_t layer_count;
  uint32_t layer_index;
  const NervaCudaHfDecodeChainLayer *layers;
} NervaCudaHfDecodeSequenceLayoutPlanRequest;

/* nerva_cuda_api.h:527-602.  Offsets are in 16-bit arena elements;
 * UINT64_MAX marks a tensor the layer does not have. */
typedef struct NervaCudaHfDecodeSequenceLayoutPlanResult {
  int32_t status;
  uint32_t hidden;
  uint32_t heads;
  uint32_t kv_heads;
  uint32_t head_dim;
  uint32_t intermediate;
  uint32_t vocab_size;
  uint32_t layer_count;
  uint32_t layer_index;
  uint32_t attention_kind;
  uint32_t deepseek_mode;
  uint32_t deepseek_flags;
  uint32_t deepseek_hc_mult;
  uint32_t deepseek_hc_sinkhorn_iters;
  uint32_t deepseek_qk_head_dim;
  uint32_t deepseek_q_rows;
  uint32_t deepseek_kv_cache_width;
  uint32_t deepseek_kv_b_rows;
  uint32_t deepseek_value_rows;
  uint64_t resident_weight_bytes;
  uint64_t layout_bytes;
  uint64_t final_norm;
  uint64_t lm_head;
  uint64_t rms_attn;
  uint64_t rms_mlp;
  uint64_t w_q;
  uint64_t q_norm;
  uint64_t w_k;
  uint64_t k_norm;
  uint64_t w_v;
  uint64_t w_o;
  uint64_t w_router;
  uint64_t w_expert_gate_up;
  uint64_t w_expert_down;
  uint64_t w_shared_expert_gate;
  uint64_t w_shared_expert_up;
  uint64_t w_shared_expert_down;
  uint64_t deepseek_q_a_scale;
  uint64_t deepseek_q_b;
  uint64_t deepseek_q_b_scale;
  uint64_t deepseek_kv_a_scale;
  uint64_t deepseek_kv_b_scale;
  uint64_t deepseek_o_a_scale;
  uint64_t deepseek_o_b;
  uint64_t deepseek_o_b_scale;
  uint64_t deepseek_attention_sink;
  uint64_t deepseek_indexer_q;
  uint64_t deepseek_indexer_q_scale;
  uint64_t deepseek_indexer_k;
  uint64_t deepseek_indexer_k_scale;
  uint64_t deepseek_indexer_k_norm;
  uint64_t deepseek_indexer_k_norm_bias;
  uint64_t deepseek_indexer_weights;
  uint64_t deepseek_compressor_ape;
  uint64_t deepseek_compressor_wkv;
  uint64_t deepseek_compressor_wgate;
  uint64_t deepseek_compressor_norm;
  uint64_t deepseek_indexer_compressor_ape;
  uint64_t deepseek_indexer_compressor_wkv;
  uint64_t deepseek_indexer_compressor_wgate;
  uint64_t deepseek_indexer_compressor_norm;
  uint64_t deepseek_hc_head_base;
  uint64_t deepseek_hc_head_fn;
  uint64_t deepseek_hc_head_scale;
  uint64_t deepseek_hc_attn_base;
  uint64_t deepseek_hc_attn_fn;
  uint64_t deepseek_hc_attn_scale;
  uint64_t deepseek_hc_ffn_base;
  uint64_t deepseek_hc_ffn_fn;
  uint64_t deepseek_hc_ffn_scale;
  float deepseek_hc_eps;
  float deepseek_hc_post_alpha;
  float deepseek_compress_rope_theta;
  float deepseek_swiglu_limit;
} NervaCudaHfDecodeSequenceLayoutPlanResult;

/* nerva_cuda_api.h:604 */
typedef struct NervaCudaHfDecodeSequenceSession NervaCudaHfDecodeSequenceSession;

/* nerva_cuda_api.h:606-638 */
typedef struct NervaCudaHfDecodeSequenceSessionCreateRequest {
  uint32_t dtype;
  uint32_t hidden;
  uint32_t heads;
  uint32_t kv_heads;
  uint32_t head_dim;
  uint32_t intermediate;
  uint32_t vocab_size;
  uint32_t layer_count;
  uint32_t max_context_tokens;
  float rms_eps;
  float rope_theta;
  const uint16_t *embeddings;
  const NervaCudaHfDecodeChainLayer *layers;
  const uint16_t *final_norm_weight;
  const uint16_t *lm_head;
  uint32_t planned_weight_blocks;
  uint32_t planned_gpu_resident_blocks;
  uint32_t planned_gpu_staged_blocks;
  uint64_t planned_weight_bytes;
  uint64_t planned_gpu_resident_weight_bytes;
  uint64_t planned_gpu_staged_weight_bytes;
  const NervaCudaHfDecodeSequenceWeightBlock *planned_weight_descriptors;
  uint32_t planned_weight_descriptor_count;
  uint64_t planned_weight_descriptor_hash;
  uint32_t detailed_profile;
  uint32_t experimental_rt_decode;
  uint32_t experimental_rt_mode;
  uint32_t experimental_rt_page_tokens;
  uint32_t experimental_rt_pages;
  uint32_t experimental_rt_local_window_tokens;
  uint32_t experimental_rt_sink_tokens;
} NervaCudaHfDecodeSequenceSessionCreateRequest;

/* nerva_cuda_api.h:640-687 */
typedef struct NervaCudaHfDecodeSequenceSessionCreateResult {
  int32_t status;
  int32_t cuda_error;
  int32_t failure_stage;
  int32_t device_count;
  uint32_t dtype;
  uint32_t hidden;
  uint32_t heads;
  uint32_t kv_heads;
  uint32_t head_dim;
  uint32_t intermediate;
  uint32_t vocab_size;
  uint32_t layer_count;
  uint32_t max_context_tokens;
  uint32_t prefill_chunk_tokens;
  uint32_t head_threads;
  uint64_t resident_weight_bytes;
  uint32_t planned_weight_blocks;
  uint32_t planned_gpu_resident_blocks;
  uint32_t planned_gpu_staged_blocks;
  uint64_t planned_weight_bytes;
  uint64_t planned_gpu_resident_weight_bytes;
  uint64_t planned_gpu_staged_weight_bytes;
  uint64_t descriptor_gpu_resident_h2d_bytes;
  uint64_t descriptor_gpu_staged_h2d_bytes;
  uint32_t planned_weight_descriptor_count;
  uint64_t planned_weight_descriptor_hash;
  uint32_t experimental_rt_decode_requested;
  uint32_t experimental_rt_decode_enabled;
  uint32_t experimental_rt_mode;
  uint32_t experimental_rt_page_tokens;
  uint32_t experimental_rt_pages;
  uint32_t experimental_rt_local_window_tokens;
  uint32_t experimental_rt_sink_tokens;
  uint32_t deepseek_v4_attention_aux_streams;
  uint32_t deepseek_v4_attention_events;
  uint64_t deepseek_v4_swa_kv_bytes;
  uint64_t deepseek_mhc_residual_bytes;
  uint64_t deepseek_mhc_post_mix_bytes;
  uint64_t deepseek_mhc_comb_mix_bytes;
  uint64_t resident_kv_bytes;
  uint64_t device_arena_bytes;
  uint64_t pinned_host_bytes;
  uint64_t h2d_bytes;
  uint64_t sync_calls;
  uint64_t hot_path_allocations;
  uint64_t device_memory_bandwidth_bps;
} NervaCudaHfDecodeSequenceSessionCreateResult;

/* nerva_cuda_api.h:689-692 */
typedef struct NervaCudaHfDecodeSequenceSessionForkSharedWeightsRequest {
  NervaCudaHfDecodeSequenceSession *parent;
  uint32_t detailed_profile;
} NervaCudaHfDecodeSequenceSessionForkSharedWeightsRequest;

/* nerva_cuda_api.h:694-705 */
typedef struct NervaCudaHfDecodeSequenceSessionRunRequest {
  NervaCudaHfDecodeSequenceSession *session;
  uint32_t steps;
  uint32_t seed_token;
  const uint32_t *prompt_tokens;
  uint32_t prompt_token_count;
  uint32_t has_eos_token;
  uint32_t eos_token;
  uint32_t *output_tokens;
  uint32_t output_token_capacity;
  NervaCudaHfDecodeSamplerConfig sampler;
} NervaCudaHfDecodeSequenceSessionRunRequest;

/* nerva_cuda_api.h:707-714 */
typedef struct NervaCudaHfDecodeSequenceSessionStartRequest {
  NervaCudaHfDecodeSequenceSession *session;
  const uint32_t *prompt_tokens;
  uint32_t prompt_token_count;
  uint32_t has_eos_token;
  uint32_t eos_token;
  NervaCudaHfDecodeSamplerConfig sampler;
} NervaCudaHfDecodeSequenceSessionStartRequest;

/* nerva_cuda_api.h:716-721 */
typedef struct NervaCudaHfDecodeSequenceSessionAdvanceRequest {
  NervaCudaHfDecodeSequenceSession *session;
  uint32_t steps;
  uint32_t *output_tokens;
  uint32_t output_token_capacity;
} NervaCudaHfDecodeSequenceSessionAdvanceRequest;

/* nerva_cuda_api.h:936-943.  `sessions` is an array of session_count handles;
 * output_tokens[i] receives the token of sessions[i] when that session took part. */
typedef struct NervaCudaHfDecodeSequenceBatchAdvanceRequest {
  NervaCudaHfDecodeSequenceSession **sessions;
  uint32_t session_count;
  uint32_t target_block_tokens;
  uint32_t min_block_tokens;
  uint32_t *output_tokens;
  uint32_t output_token_capacity;
} NervaCudaHfDecodeSequenceBatchAdvanceRequest;

/* nerva_cuda_api.h:945-976.  reason: 0 ready, 1 invalid request, 2 no sessions,
 * 3 no ready sessions, 4 shared weights unproven (no descriptor hash), 5 fewer compatible
 * ready sessions than min_block_tokens (hf_decode_sequence/session_prelude.inc.cu:56-64). */
typedef struct NervaCudaHfDecodeSequenceBatchAdvanceResult {
  int32_t status;
  int32_t cuda_error;
  int32_t device_count;
  uint32_t reason;
  uint32_t exact;
  uint32_t requested_session_count;
  uint32_t eligible_session_count;
  uint32_t block_tokens;
  uint32_t target_block_tokens;
  uint32_t min_block_tokens;
  uint32_t dtype;
  uint32_t layer_count;
  uint32_t observed_tokens;
  uint32_t last_token;
  uint64_t observed_token_hash;
  uint64_t d2h_bytes;
  uint64_t projection_elapsed_ns;
  uint64_t qkv_elapsed_ns;
  uint64_t attention_output_elapsed_ns;
  uint64_t gate_up_elapsed_ns;
  uint64_t down_elapsed_ns;
  uint64_t lm_head_elapsed_ns;
  uint64_t pack_kernel_launches;
  uint64_t projection_kernel_launches;
  uint64_t scatter_kernel_launches;
  uint64_t dependency_kernel_launches;
  uint64_t experimental_rt_selector_launches;
  uint64_t sampling_kernel_launches;
  uint64_t sync_calls;
  uint64_t hot_path_allocations;
} NervaCudaHfDecodeSequenceBatchAdvanceResult;

/* nerva_cuda_api.h:1075-1082 */
typedef struct NervaCudaProjectionBenchRequest {
  uint32_t dtype;
  uint32_t rows;
  uint32_t cols;
  uint32_t iterations;
  uint32_t warmup_iterations;
  uint32_t block_tokens;
} NervaCudaProjectionBenchRequest;

/* nerva_cuda_api.h:1084-1144.  The single-token `cublaslt_*` fields stay zero: this library
 * links no BLAS.  `custom_*` describe the hand-written single-token projection kernel.  With
 * block_tokens > 1 the `block_cublaslt_*` fields (the reference's block path) carry this
 * library's block kernel on the tensor pipe, which streams the weights once for the block. */
typedef struct NervaCudaProjectionBenchResult {
  int32_t status;
  int32_t cuda_error;
  int32_t device_count;
  int32_t device_ordinal;
  int32_t compute_capability_major;
  int32_t compute_capability_minor;
  uint32_t dtype;
  uint32_t rows;
  uint32_t cols;
  uint32_t block_tokens;
  uint32_t iterations;
  uint32_t warmup_iterations;
  uint64_t matrix_bytes;
  uint64_t input_bytes;
  uint64_t output_bytes;
  uint64_t cublaslt_total_ns;
  uint64_t cublaslt_avg_ns;
  uint64_t cublaslt_default_total_ns;
  uint64_t cublaslt_default_avg_ns;
  uint32_t cublaslt_heuristic_count;
  uint32_t cublaslt_best_heuristic_index;
  uint64_t cublaslt_best_heuristic_total_ns;
  uint64_t cublaslt_best_heuristic_avg_ns;
  uint64_t custom_total_ns;
  uint64_t custom_avg_ns;
  uint64_t cublaslt_graph_total_ns;
  uint64_t cublaslt_graph_avg_ns;
  uint64_t cublaslt_default_graph_total_ns;
  uint64_t cublaslt_default_graph_avg_ns;
  uint64_t cublaslt_best_heuristic_graph_total_ns;
  uint64_t cublaslt_best_heuristic_graph_avg_ns;
  uint64_t custom_graph_total_ns;
  uint64_t custom_graph_avg_ns;
  uint64_t cublaslt_graph_nodes;
  uint64_t custom_graph_nodes;
  uint64_t graph_replays;
  uint64_t graph_captures;
  uint32_t selected_graph_strategy;
  uint64_t cublaslt_effective_bandwidth_bps;
  uint64_t custom_effective_bandwidth_bps;
  uint32_t selected_strategy;
  uint32_t mismatch_count;
  float max_abs_diff;
  uint64_t kernel_launches;
  uint64_t sync_calls;
  uint64_t device_allocations;
  uint64_t device_frees;
  uint64_t device_arena_bytes;
  uint64_t hot_path_allocations;
  uint64_t block_cublaslt_total_ns;
  uint64_t block_cublaslt_avg_ns;
  uint64_t block_cublaslt_per_token_ns;
  uint64_t block_cublaslt_graph_total_ns;
  uint64_t block_cublaslt_graph_avg_ns;
  uint64_t block_cublaslt_graph_per_token_ns;
  uint64_t block_cublaslt_graph_nodes;
  uint64_t block_cublaslt_speedup_x1000;
  uint64_t block_cublaslt_graph_speedup_x1000;
  uint64_t block_cublaslt_effective_bandwidth_bps;
} NervaCudaProjectionBenchResult;

/* ---- resident decode session (the hot path) ---- */

/* nerva_cuda_api.h:2160 */
int nerva_cuda_hf_decode_sequence_plan_layout(
    const NervaCudaHfDecodeSequenceLayoutPlanRequest *request,
    NervaCudaHfDecodeSequenceLayoutPlanResult *out);
/* nerva_cuda_api.h:2163 */
int nerva_cuda_hf_decode_sequence_session_create(
    const NervaCudaHfDecodeSequenceSessionCreateRequest *request,
    NervaCudaHfDecodeSequenceSessionCreateResult *out,
    NervaCudaHfDecodeSequenceSession **session);
/* nerva_cuda_api.h:2167 */
int nerva_cuda_hf_decode_sequence_session_run(
    const NervaCudaHfDecodeSequenceSessionRunRequest *request,
    NervaCudaHfDecodeSequenceResult *out);
/* nerva_cuda_api.h:2170 */
int nerva_cuda_hf_decode_sequence_session_start(
    const NervaCudaHfDecodeSequenceSessionStartRequest *request,
    NervaCudaHfDecodeSequenceResult *out);
/* nerva_cuda_api.h:2173 */
int nerva_cuda_hf_decode_sequence_session_advance(
    const NervaCudaHfDecodeSequenceSessionAdvanceRequest *request,
    NervaCudaHfDecodeSequenceResult *out);
/* nerva_cuda_api.h:2209.  Advances by one token every started, unfinished session of the
 * request that has caught up with its cursor and shares the first such session's weights
 * (same descriptor hash and shape), up to target_block_tokens (at most 32) of them, provided
 * at least min_block_tokens qualify; otherwise status 0 with the reason and no session
 * touched (hf_decode_sequence/session_api_batch_fork_destroy.inc.cu:1-309).  Tokens are
 * the ones session_advance(1) would give.  Here the sessions' steps are replayed on their
 * own streams side by side; the weights are streamed once per session, not once per block. */
int nerva_cuda_hf_decode_sequence_batch_advance_one(
    const NervaCudaHfDecodeSequenceBatchAdvanceRequest *request,
    NervaCudaHfDecodeSequenceBatchAdvanceResult *out);
/* nerva_cuda_api.h:2212 */
int nerva_cuda_hf_decode_sequence_session_fork_shared_weights(
    const NervaCudaHfDecodeSequenceSessionForkSharedWeightsRequest *request,
    NervaCudaHfDecodeSequenceSessionCreateResult *out,
    NervaCudaHfDecodeSequenceSession **session_out);
/* nerva_cuda_api.h:2216 */
int nerva_cuda_hf_decode_sequence_session_destroy(
    NervaCudaHfDecodeSequenceSession *session,
    NervaCudaHfDecodeSequenceSessionCreateResult *out /* nullable */);
/* nerva_cuda_api.h:2157 — one-shot: create, run, destroy. */
int nerva_cuda_hf_decode_sequence_u16(const NervaCudaHfDecodeSequenceRequest *request,
                                      NervaCudaHfDecodeSequenceResult *out);
/* nerva_cuda_api.h:2227 */
int nerva_cuda_projection_bench(const NervaCudaProjectionBenchRequest *request,
                                NervaCudaProjectionBenchResult *out);

/* nerva_cuda_api.h:1480-1495 — DeepSeek expert routing of one token.  router_kind: 1 = V3
 * grouped sigmoid, 2 = V4 sqrt-softplus, 3 = V4 hash table.  Host pointers. */
typedef struct NervaCudaDeepSeekRouterRouteRequest {
  uint32_t router_kind;
  uint32_t num_experts;
  uint32_t num_groups;
  uint32_t top_k_groups;
  uint32_t top_k;
  uint32_t norm_topk_prob;
  uint32_t route_token;
  float routed_scaling_factor;
  const float *logits;
  const float *correction_bias;
  const uint32_t *hash_route_table;
  uint32_t hash_route_table_len;
  uint32_t *expert_ids;
  float *weights;
} NervaCudaDeepSeekRouterRouteRequest;

/* nerva_cuda_api.h:1497-1515 */
typedef struct NervaCudaDeepSeekRouterRouteResult {
  int32_t status;
  int32_t cuda_error;
  int32_t device_count;
  int32_t route_error;
  uint32_t router_kind;
  uint32_t num_experts;
  uint32_t num_groups;
  uint32_t top_k_groups;
  uint32_t top_k;
  uint64_t output_hash;
  uint64_t device_arena_bytes;
  uint64_t pinned_host_bytes;
  uint64_t h2d_bytes;
  uint64_t d2h_bytes;
  uint64_t kernel_launches;
  uint64_t sync_calls;
  uint64_t hot_path_allocations;
} NervaCudaDeepSeekRouterRouteResult;

/* nerva_cuda_api.h:2258 */
int nerva_cuda_deepseek_router_route(const NervaCudaDeepSeekRouterRouteRequest *request,
                                     NervaCudaDeepSeekRouterRouteResult *out);

/* nerva_cuda_api.h:1540-1555 — DeepSeek multi-head latent attention decode of one token in
 * absorbed form.  fp32 host pointers: q_nope [heads][nope], q_pe [heads][rope],
 * kv_c [tokens][kv_lora_rank], k_pe [tokens][rope], w_uk [kv_lora_rank][heads][nope],
 * w_uv [kv_lora_rank][heads][v_head_dim], output [heads][v_head_dim]. */
typedef struct NervaCudaDeepSeekMlaDecodeRequest {
  uint32_t heads;
  uint32_t tokens;
  uint32_t kv_lora_rank;
  uint32_t qk_nope_head_dim;
  uint32_t qk_rope_head_dim;
  uint32_t v_head_dim;
  float softmax_scale;
  const float *q_nope;
  const float *q_pe;
  const float *kv_c;
  const float *k_pe;
  const float *w_uk;
  const float *w_uv;
  float *output;
} NervaCudaDeepSeekMlaDecodeRequest;

/* nerva_cuda_api.h:1557-1577 */
typedef struct NervaCudaDeepSeekMlaDecodeResult {
  int32_t status;
  int32_t cuda_error;
  int32_t device_count;
  int32_t decode_error;
  uint32_t heads;
  uint32_t tokens;
  uint32_t kv_lora_rank;
  uint32_t qk_nope_head_dim;
  uint32_t qk_rope_head_dim;
  uint32_t v_head_dim;
  float softmax_scale;
  uint64_t output_hash;
  uint64_t device_arena_bytes;
  uint64_t pinned_host_bytes;
  uint64_t h2d_bytes;
  uint64_t d2h_bytes;
  uint64_t kernel_launches;
  uint64_t sync_calls;
  uint64_t hot_path_allocations;
} NervaCudaDeepSeekMlaDecodeResult;

/* nerva_cuda_api.h:2262 */
int nerva_cuda_deepseek_mla_decode(const NervaCudaDeepSeekMlaDecodeRequest *request,
                                   NervaCudaDeepSeekMlaDecodeResult *out);

/* nerva_cuda_api.h:2023-2037 — expert MLP of one token over already routed experts.  fp32 host
 * pointers: input [hidden], w_gate / w_up [num_experts][intermediate][hidden],
 * w_down [num_experts][hidden][intermediate], output [hidden]. */
typedef struct NervaCudaDeepSeekMoeForwardRequest {
  uint32_t hidden_size;
  uint32_t intermediate_size;
  uint32_t num_experts;
  uint32_t top_k;
  uint32_t clamp_swiglu;
  float swiglu_limit;
  const float *input;
  const uint32_t *expert_ids;
  const float *expert_weights;
  const float *w_gate;
  const float *w_up;
  const float *w_down;
  float *output;
} NervaCudaDeepSeekMoeForwardRequest;

/* nerva_cuda_api.h:2039-2058 */
typedef struct NervaCudaDeepSeekMoeForwardResult {
  int32_t status;
  int32_t cuda_error;
  int32_t device_count;
  int32_t moe_error;
  uint32_t hidden_size;
  uint32_t intermediate_size;
  uint32_t num_experts;
  uint32_t top_k;
  uint32_t clamp_swiglu;
  float swiglu_limit;
  uint64_t output_hash;
  uint64_t device_arena_bytes;
  uint64_t pinned_host_bytes;
  uint64_t h2d_bytes;
  uint64_t d2h_bytes;
  uint64_t kernel_launches;
  uint64_t sync_calls;
  uint64_t hot_path_allocations;
} NervaCudaDeepSeekMoeForwardResult;

/* nerva_cuda_api.h:2302 */
int nerva_cuda_deepseek_moe_forward(const NervaCudaDeepSeekMoeForwardRequest *request,
                                    NervaCudaDeepSeekMoeForwardResult *out);

/* ---- additive entry points (no counterpart in the reference) ---- */

/* Step engine of a session: 0 = one kernel per operator captured in a CUDA
 * graph, 1 = the persistent whole-step kernel.  Must be called before
 * session_start.  Returns 0, or -1 when the engine cannot run the model. */
int nerva_b200_session_set_engine(NervaCudaHfDecodeSequenceSession *session, uint32_t engine);
/* Copies the f32 logits of the most recent sampled step (vocab_size floats) to
 * host memory.  Synchronises the session stream. */
int nerva_b200_session_read_logits(NervaCudaHfDecodeSequenceSession *session, float *logits,
                                   uint32_t capacity);
/* Replaces the logical->physical KV page table (one uint32 per 16-token page,
 * a permutation of 0..page_count-1).  Only legal before session_start. */
int nerva_b200_session_set_kv_block_table(NervaCudaHfDecodeSequenceSession *session,
                                          const uint32_t *table, uint32_t page_count);
/* Reads the page table back (for page-table parity checks). */
int nerva_b200_session_get_kv_block_table(NervaCudaHfDecodeSequenceSession *session,
                                          uint32_t *table, uint32_t capacity);
/* Copies one token's K or V row (kv_heads*head_dim 16-bit values) of one layer
 * out of the paged cache. which: 0 = K, 1 = V. */
int nerva_b200_session_read_kv_row(NervaCudaHfDecodeSequenceSession *session, uint32_t layer,
                                   uint32_t token, uint32_t which, uint16_t *row,
                                   uint32_t capacity);

/* Runs `steps` further decode steps of the active request un-captured, with a
 * CUDA event between operator groups, and returns summed device nanoseconds per
 * bucket: 0 embedding, 1 QKV projection, 2 attention (q/k norm + RoPE + KV
 * append + split-KV + merge), 3 O projection, 4 gate/up projection, 5 down
 * projection, 6 lm_head projection, 7 sampling.  bucket_launches (nullable)
 * receives kernel launches per bucket per step.  The sequence advances. */
int nerva_b200_session_profile_steps(NervaCudaHfDecodeSequenceSession *session, uint32_t steps,
                                     uint64_t *bucket_ns, uint32_t *bucket_launches,
                                     uint32_t bucket_capacity);

/* Tuning aid of the whole-step kernel: reads and clears 16 counters of SM cycles
 * that block 0 spent per phase (QKV prologue, QKV, barrier, attention, barrier,
 * O prologue, O, barrier, gate/up prologue, gate/up, barrier, down prologue,
 * down, barrier, lm_head, tail).  Only filled when the session was created with
 * the environment variable NERVA_B200_PHASE_PROFILE=1.  Returns the count. */
int nerva_b200_session_read_phase_cycles(NervaCudaHfDecodeSequenceSession *session,
                                         uint64_t *cycles, uint32_t capacity);

/* ---- tensor parallel over the GPUs of one node (no counterpart in the reference, whose
 * multi-GPU plan moves activations between layer islands only) ----
 * One process per GPU.  Every rank creates a session over ITS SHARD of the model with the
 * CUDA device it owns current: the request carries the full hidden size, the rank's share
 * of the query heads, KV heads, intermediate size (rows of gate/up, columns of down) and
 * lm_head rows, the matching slices of the weights, and the WHOLE embedding table
 * (`full_vocab` rows).  QKV, gate/up and lm_head are split by output rows; O and down by
 * input columns, and their partial sums travel between the GPUs inside the projection
 * kernels: the epilogue stores each rank's partial rows into every rank's exchange buffer
 * with plain peer stores, the prologue of the next projection waits (bounded, about a
 * second, then the step fails) for all partials and adds them in rank order, so every rank
 * holds the same residual stream bit for bit.  The arg-max candidates of the vocabulary
 * shards are exchanged the same way by the sampler.  No collective library is involved on
 * the data path.
 *
 * Set-up: create_sharded on every rank -> comm_handle -> exchange the 64-byte handles by
 * any host channel -> attach_peers.  Afterwards start/advance/run are called on all ranks
 * in lock-step with identical arguments.  Not available: planned weight descriptors,
 * forks, the whole-step engine. */
typedef struct NervaB200ShardInfo {
  uint32_t rank;
  uint32_t world;        /* 2, 4 or 8 (any value in 2..8 that divides the head counts) */
  uint32_t full_vocab;   /* rows of the embedding table */
  uint32_t vocab_offset; /* first lm_head row of this rank */
  uint32_t mode;         /* 0: tensor parallel (dense layers: heads, intermediate size and lm_head rows are
                          * cut).  1: expert parallel (sparse-MoE models): every rank holds the whole model
                          * except the routed experts, of which it holds num_experts / world consecutive
                          * ones starting at rank * num_experts / world, and the shared expert, of which it
                          * holds an equal slice of the intermediate dimension (the request's
                          * shared_expert_intermediate is the slice's size, num_experts stays the layer's
                          * total); full_vocab = vocab_size, vocab_offset = 0.  The ranks' partial MLP
                          * outputs are exchanged like the tensor-parallel partial sums.  Needs an even
                          * number of sparse layers. */
} NervaB200ShardInfo;
int nerva_b200_session_create_sharded(const NervaCudaHfDecodeSequenceSessionCreateRequest *request,
                                      const NervaB200ShardInfo *shard,
                                      NervaCudaHfDecodeSequenceSessionCreateResult *out,
                                      NervaCudaHfDecodeSequenceSession **session);
/* Writes the 64-byte inter-process handle of this rank's exchange buffer; returns 64. */
int nerva_b200_session_comm_handle(NervaCudaHfDecodeSequenceSession *session, uint8_t *handle,
                                   uint32_t capacity);
/* handles: world x 64 bytes in rank order (the rank's own entry is ignored). */
int nerva_b200_session_attach_peers(NervaCudaHfDecodeSequenceSession *session,
                                    const uint8_t *handles, uint32_t world);
/* Diagnostic stand-in for attach_peers when no peer exists: every rank's exchange buffer is taken
 * to be this rank's own, so this rank's partial sums arrive and nobody else's ever do.  The first
 * exchange of a step then runs into its wait limit, sets the error word (code 6), and the call
 * that queued the step fails with status -1; the context stays usable.  It lets a test exercise
 * the bounded-wait path on one GPU without faulting or hanging anything. */
int nerva_b200_session_attach_loopback(NervaCudaHfDecodeSequenceSession *session);

/* Tuning aid of the per-operator engine: nanosecond stamps (%globaltimer) of the
 * last step, 8 per launch, launches ordered [layer][QKV, attention, O, gate/up,
 * down] then lm_head.  Slots 0..3: first block at kernel entry, after the wait
 * for the previous kernel, after the prologue, before exit; slots 4..7: the same
 * for the last block.  Only filled when the session was created with the
 * environment variable NERVA_B200_TIMELINE=1.  Returns the number of values. */
int nerva_b200_session_read_timeline(NervaCudaHfDecodeSequenceSession *session, uint64_t *stamps,
                                     uint32_t capacity);

/* Isolated projection: y[m][n] = sum_k W[n][k] * x[m][k], bf16 in, fp32
 * accumulate and out.  All pointers are HOST memory; the call copies in, runs
 * `iterations` launches after `warmup` untimed ones, and copies y back.
 * avg_ns (nullable) receives the mean device time per launch. */
int nerva_b200_projection(const uint16_t *weight, const uint16_t *x, float *y, uint32_t rows,
                          uint32_t cols, uint32_t tokens, uint32_t warmup, uint32_t iterations,
                          uint64_t *avg_ns);
/* Sustained form of the same measurement (no counterpart in the reference): `copies` device copies
 * of the matrix, together larger than the L2, are projected back to back, each launch allowed to
 * start while its predecessor drains, as the projections of consecutive layers follow each other
 * inside a decode step.  avg_ns: time per launch over `iterations` launches after `warmup`. */
int nerva_b200_projection_sustained(const uint16_t *weight, const uint16_t *x, float *y, uint32_t rows,
                                    uint32_t cols, uint32_t tokens, uint32_t copies, uint32_t warmup,
                                    uint32_t iterations, uint64_t *avg_ns);

/* Isolated GQA paged decode attention for `batch` sequences of `context`
 * tokens each: q f32 [batch][heads*head_dim]; K/V pages bf16
 * [batch][pages][16][kv_heads*head_dim]; page_table uint32 [batch][pages];
 * out f32 [batch][heads*head_dim].  Host pointers. */
int nerva_b200_gqa_decode_attention(const float *q, const uint16_t *key_pages,
                                    const uint16_t *value_pages, const uint32_t *page_table,
                                    float *out, uint32_t batch, uint32_t context, uint32_t heads,
                                    uint32_t kv_heads, uint32_t head_dim, uint32_t warmup,
                                    uint32_t iterations, uint64_t *avg_ns);
/* Sustained form (no counterpart in the reference): `copies` device copies of the K and V pages —
 * the caches of that many layers, together larger than the L2 — are attended over back to back on
 * one stream, as the attention launches of the layers of a decode step follow each other.
 * avg_ns: time per launch (attention + merge) over `iterations` launches after `warmup`. */
int nerva_b200_gqa_decode_attention_sustained(const float *q, const uint16_t *key_pages,
                                              const uint16_t *value_pages, const uint32_t *page_table,
                                              float *out, uint32_t batch, uint32_t context, uint32_t heads,
                                              uint32_t kv_heads, uint32_t head_dim, uint32_t copies,
                                              uint32_t warmup, uint32_t iterations, uint64_t *avg_ns);

/* The same attention with DEVICE pointers (layouts as above) and no allocation:
 * the split partials live in a fixed 4 MiB device array inside the library, so
 * the call needs batch*heads*splits*(head_dim+2) <= 1048576 floats (the split
 * count is lowered to fit; a shape that does not fit unsplit returns -1 with
 * the limit in nerva_b200_last_error()).  `stream` is a cudaStream_t (NULL: the
 * default stream); the call returns once the stream has finished the work.
 * Calls on one device share the array, so overlapping calls race: serialise
 * them.  The first call on each device also performs the set-up (the address
 * of the array, the kernels' attributes).  No counterpart in the reference: it is
 * for callers whose arena already owns the device memory, or whose decode loop
 * must report zero hot-path allocations. */
int nerva_b200_gqa_decode_attention_static_scratch(
    const float *q, const uint16_t *key_pages, const uint16_t *value_pages,
    const uint32_t *page_table, float *out, uint32_t batch, uint32_t context, uint32_t heads,
    uint32_t kv_heads, uint32_t head_dim, void *stream);

/* Greedy argmax over f32 logits with the sampler's tie rule (lowest index,
 * non-finite values skipped).  Host pointers. */
int nerva_b200_greedy_argmax(const float *logits, uint32_t count, uint32_t *token);

/* One token from f32 host logits at `position` with the decode step's sampler: arg-max when
 * temperature is 0 or top_k is 1, Gumbel-max when top_k is 0 and top_p >= 0.999999, else the
 * top-k / top-p draw, all seeded by (seed, position) as the reference's final-head sampler
 * (native/cuda/hf_decode_sequence/sampler.cu:66-408) seeds them.  temperature must be finite
 * and >= 0, top_p in (0, 1]; -1 otherwise. */
int nerva_b200_sample_token(const float *logits, uint32_t count, uint32_t position, float temperature,
                            float top_p, uint32_t top_k, uint64_t seed, uint32_t *token);

/* Fills host memory with the synthetic checkpoint generator of
 * include/nerva_synth.h (multi-threaded; same bits as the header). */
void nerva_b200_synth_normal_bf16(uint64_t seed, uint64_t tensor_id, uint64_t count, float std,
                                  uint16_t *out);

/* ---- host-side memory bookkeeping (no device call) ----
 * C++ restatements, used by the session, of the reference's
 * crates/nerva-memory StaticArena (arena/static_arena.rs:71-112: bump offsets
 * rounded up to `align`, requests in the hot-path phase refused) and KvPagePool
 * (kv/pool/{preallocate,allocation,cache}.rs: FIFO free list, reference counts,
 * prefix-key cache).  phase: 0 initialization, 1 warm-up, 2 hot path. */
typedef struct NervaB200StaticArena NervaB200StaticArena;
typedef struct NervaB200KvPagePool NervaB200KvPagePool;
typedef struct NervaB200KvPageInfo {
  uint64_t arena_offset;
  uint64_t page_bytes;
  uint64_t last_use;
  uint32_t token_start;
  uint32_t token_count;
  uint32_t ref_count;
  uint32_t prefix_tokens;
  uint32_t is_free;
  uint32_t has_prefix;
} NervaB200KvPageInfo;

NervaB200StaticArena *nerva_b200_static_arena_new(uint64_t capacity_bytes);
void nerva_b200_static_arena_free(NervaB200StaticArena *arena);
int nerva_b200_static_arena_reserve(NervaB200StaticArena *arena, uint64_t bytes, uint64_t align,
                                    uint32_t phase, uint64_t *offset_out);
uint64_t nerva_b200_static_arena_used(const NervaB200StaticArena *arena);
uint64_t nerva_b200_static_arena_remaining(const NervaB200StaticArena *arena);
int nerva_b200_static_arena_restore(NervaB200StaticArena *arena, uint64_t cursor);

NervaB200KvPagePool *nerva_b200_kv_page_pool_new(NervaB200StaticArena *arena, uint32_t num_pages,
                                                 uint32_t block_size_tokens, uint64_t page_bytes,
                                                 uint64_t align);
void nerva_b200_kv_page_pool_free(NervaB200KvPagePool *pool);
uint32_t nerva_b200_kv_page_pool_len(const NervaB200KvPagePool *pool);
uint32_t nerva_b200_kv_page_pool_free_pages(const NervaB200KvPagePool *pool);
/* page index, -1 pool exhausted, -2 token_count larger than a page */
int64_t nerva_b200_kv_page_pool_allocate(NervaB200KvPagePool *pool, uint32_t token_start,
                                         uint32_t token_count, uint64_t step);
int nerva_b200_kv_page_pool_retain(NervaB200KvPagePool *pool, uint32_t page, uint64_t step);
int nerva_b200_kv_page_pool_release(NervaB200KvPagePool *pool, uint32_t page, uint64_t step);
int nerva_b200_kv_page_pool_cache(NervaB200KvPagePool *pool, uint32_t page, const uint8_t *hash32,
                                  uint32_t group_id, uint32_t prefix_tokens);
int64_t nerva_b200_kv_page_pool_lookup_cached(const NervaB200KvPagePool *pool,
                                              const uint8_t *hash32, uint32_t group_id);
int64_t nerva_b200_kv_page_pool_retain_cached(NervaB200KvPagePool *pool, const uint8_t *hash32,
                                              uint32_t group_id, uint64_t step);
/* 1 a key was evicted, 0 the page had none, -1 bad index */
int nerva_b200_kv_page_pool_evict_cached(NervaB200KvPagePool *pool, uint32_t page);
int nerva_b200_kv_page_pool_page(const NervaB200KvPagePool *pool, uint32_t page,
                                 NervaB200KvPageInfo *out);

/* The block [row_begin, row_begin+rows) x [col_begin, col_begin+cols) of the same generator's
 * row-major tensor with full_cols columns (what a tensor-parallel rank holds), rows*cols values. */
void nerva_b200_synth_normal_bf16_block(uint64_t seed, uint64_t tensor_id, uint64_t full_cols,
                                        uint64_t row_begin, uint64_t rows, uint64_t col_begin,
                                        uint64_t cols, float std, uint16_t *out);

/* Last error text of the calling thread ("" when none). */
const char *nerva_b200_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* NERVA_B200_API_H_ */
