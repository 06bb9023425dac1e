// Host-callable launchers of the decode-step kernels.  All pointers are device
// pointers; every launcher only enqueues work on `stream` (graph-capturable) and
// returns cudaGetLastError().
#pragma once

#include <cuda_runtime.h>

#include <vector>
#include <stdint.h>

#include "../../include/nerva_b200_api.h"

namespace nb {

// Launches `kernel`; with pdl set the launch carries the programmatic
// stream-serialization attribute, so the kernel may begin (up to its
// griddepcontrol.wait) while its predecessor in the stream drains.  Works under
// stream capture (the edge becomes a programmatic graph dependency).
template <class... KernelArgs, class... Args>
cudaError_t launch_with_pdl(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                            cudaStream_t stream, bool pdl, Args &&...args) {
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute{};
  if (pdl) {
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

// ---- projection (weight-streaming GEMV) ----
enum ProjectionPrologue : uint32_t {
  kProloguePlain = 0,     // x_bf16 is the activation vector
  kPrologueAddNorm = 1,   // r = add_a + add_b + add_bias; x = bf16(rmsnorm(r) * norm_weight);
                          // block 0 stores r to resid_out
};
enum ProjectionEpilogue : uint32_t {
  kEpilogueStore = 0,     // out_f32[row] = y
  kEpilogueSwiglu = 1,    // rows interleaved (gate, up): out_bf16[row/2] = bf16(silu(gate) * up)
  kEpilogueArgmax = 2,    // out_f32[row] = y and per-block (best value, lowest index)
};

// ---- tensor-parallel exchange of a row-parallel projection (O, down) ----
// Every rank holds, per phase, a receive buffer of [world][rows] 8-byte entries:
// the f32 value in the low word, a tag in the high word.  The writer's epilogue
// stores each of its result rows, tagged, into slot `rank` of EVERY rank's
// buffer with one 8-byte store per entry (plain peer stores over NVLink; an
// 8-byte store is single-copy atomic, so a matching tag proves the value).  The
// prologue of the next projection polls (bounded) the entries it needs until
// their tags match, and adds the partials in rank order.  Tags only grow:
// tag = *epoch * per_epoch + offset, where *epoch counts the steps this session
// has completed (the same on every rank) and offset numbers the exchange inside
// a step from 1.
constexpr uint32_t kMaxTpWorld = 8;
struct TpPush {
  uint32_t world, rank;                   // world <= 1: off
  unsigned long long *recv[kMaxTpWorld];  // rank q's receive buffer of this phase
  const unsigned long long *epoch;
  uint32_t per_epoch, offset;
};
struct TpGather {
  uint32_t world;                         // world <= 1: off
  const unsigned long long *recv;         // this rank's receive buffer of the phase
  unsigned long long *reduced;            // this rank's [cols] tagged sums of the phase (world > 2)
  const unsigned long long *epoch;
  uint32_t per_epoch, offset;
  uint32_t two_stage;                     // world == 2 only: take the two-stage gather of the larger worlds
};

struct ProjectionParams {
  const uint16_t *weight;  // [rows][cols] bf16 row-major
  uint32_t rows, cols;
  uint32_t prologue;
  const uint16_t *x_bf16;       // kProloguePlain: the vector.  kPrologueAddNorm: `cols`
                                // writable bf16 elements of scratch (used by the toy-shape path)
  const float *add_a;           // kPrologueAddNorm (required)
  const float *add_b;           // optional
  const uint16_t *add_bias;     // optional bf16 vector
  const uint16_t *norm_weight;  // bf16 [cols]
  float eps;
  float *resid_out;             // optional
  uint32_t epilogue;
  const float *resid_in;        // kEpilogueStore, optional: out_f32[row] = y + resid_in[row], the residual
                                // add done by the row's owner so that the next prologue reads one vector
  float *out_f32;
  uint16_t *out_bf16;
  float *best_value;     // [blocks] kEpilogueArgmax
  uint32_t *best_index;  // [blocks]
  uint32_t *error_word;
  uint32_t pdl;          // launch with programmatic dependent launch (see launch_with_pdl)
  unsigned long long *stamps;  // optional kTimelineSlots timeline stamps (common.cuh: stamp)
  TpGather gather;  // kPrologueAddNorm: add_b is the sum of the partials arriving in gather.recv
  TpPush push;      // kEpilogueStore: results go to every rank's receive buffer instead of out_f32
};

constexpr uint32_t kTimelineSlots = 8;

// ---- block projection on the tensor pipe (gemm_tc.cu): 2..256 tokens, weights streamed once ----
constexpr uint32_t kGemmMaxTokens = 256;
struct GemmParams {
  const uint16_t *weight;  // [rows][cols] bf16 row-major, cols a multiple of 64
  uint32_t rows, cols;
  const uint16_t *x;       // [tokens][cols] bf16
  uint32_t tokens;
  uint32_t epilogue;       // kEpilogueStore: out_f32[token][row] = y (+ resid_in[token][row])
                           // kEpilogueSwiglu: rows interleaved (gate, up): out_bf16[token][row/2]
  const float *resid_in;   // optional [tokens][rows]
  float *out_f32;          // [tokens][rows]
  uint16_t *out_bf16;      // [tokens][rows/2]
  float *workspace;        // gemm_tc_workspace_bytes(tokens, sm_count)
  uint32_t *tickets;       // unused (kept so that callers' buffer plans stay as they are)
  uint32_t *error_word;
  uint32_t pdl;
  unsigned long long *stamps;  // optional kTimelineSlots stamps of the first and the last block: entry, first
                               // tile ready for the MMA, last MMA committed, exit
};
bool gemm_tc_eligible(const GemmParams &g);
uint64_t gemm_tc_workspace_bytes(uint32_t tokens, uint32_t sm_count);
uint32_t gemm_tc_ticket_count(uint32_t rows);
bool tensor_map_available();  // the driver exposes the tensor-map encoder the TMA kernels need
// Encodes a CUtensorMap (128 bytes at `map`, 64-byte aligned) over a bf16 [outer][inner] row-major
// tensor with boxes of box_inner x box_outer elements and the 128-byte swizzle (box_inner = 64);
// elements outside the tensor read as zero.
bool encode_bf16_map_2d(void *map, const uint16_t *base, uint64_t inner, uint64_t outer, uint32_t box_inner,
                        uint32_t box_outer);
cudaError_t configure_gemm_tc_kernel();
cudaError_t launch_gemm_tc(cudaStream_t stream, const GemmParams &g, uint32_t sm_count);

// Number of blocks launch_projection will use (= number of arg-max partials).
uint32_t projection_blocks(const ProjectionParams &p, uint32_t sm_count);
cudaError_t launch_projection(cudaStream_t stream, const ProjectionParams &p, uint32_t sm_count);
cudaError_t configure_projection_kernels();

// ---- token / position bookkeeping ----
struct StepState {
  uint32_t *cursor;                       // device step cursor (= position of the token being run)
  const uint32_t *prompt;                 // device prompt ids
  const uint32_t *prompt_count;           // device word: a captured step serves every prompt length
  NervaCudaSyntheticTokenSlot *slots;     // device token ring
  uint32_t max_context;
  uint32_t vocab;
  uint32_t *error_word;
};

// input[h] = embedding[token(cursor)][h] as f32.
cudaError_t launch_embed(cudaStream_t stream, const StepState &st, const uint16_t *embeddings,
                         uint32_t hidden, float *input);

struct QkvPrepareParams {
  float *qkv;  // [heads*d | kv_heads*d | kv_heads*d] f32, q is normalised/rotated in place
  const uint16_t *q_bias, *k_bias, *v_bias;  // optional bf16
  const uint16_t *q_norm, *k_norm;           // optional bf16 [head_dim]
  uint32_t heads, kv_heads, head_dim;
  float eps, rope_theta;
  uint16_t *key_pages, *value_pages;  // this layer's pages: [pages][16][kv_hidden] bf16
  const uint32_t *page_table;
  uint32_t page_count;
};
cudaError_t launch_qkv_prepare(cudaStream_t stream, const StepState &st, const QkvPrepareParams &p);

// ---- GQA paged split-KV decode attention ----
struct AttentionParams {
  const float *q;              // [batch][heads*d] f32 (already normalised / rotated)
  const uint16_t *key_pages;   // [batch][pages][16][kv_hidden] bf16
  const uint16_t *value_pages;
  const uint32_t *page_table;  // [batch][pages]
  uint32_t batch, heads, kv_heads, head_dim, page_count;
  const uint32_t *cursor;      // context = *cursor + 1 when non-null ...
  uint32_t context;            // ... else this
  uint32_t splits;
  float *partial_acc;          // [batch][heads][splits][d]
  float *partial_m;            // [batch][heads][splits]
  float *partial_l;
  float *out_f32;              // [batch][heads*d] optional
  uint16_t *out_bf16;          // optional
  uint32_t *error_word;
  // Row form (launch_attention_rows): sequence b of the batch is row b of a block step; its q
  // (normalised, rotated, fp32, at the start of the row's projection output), cache, page table
  // and context (position + 1) come from rows[b], q / key_pages / value_pages / page_table /
  // cursor / context above are unused.  `layer` selects the layer inside the row's cache.
  const struct FusedAttentionRow *rows;
  uint32_t layer;
};
cudaError_t launch_attention(cudaStream_t stream, const AttentionParams &p);
// 128 opaque bytes of a tensor map, encoded once per cache by encode_bf16_map_2d (gemm_tc.cu).
struct alignas(64) TensorMapStorage {
  unsigned char bytes[128];
};
// Caches one launch of the row form may span (rows[b].map_index selects the pair).
constexpr uint32_t kAttentionRowCaches = 32;
// The row form of the paged tensor-pipe kernel + its merge: head_dim 64 or 128, at most 8 query
// heads per KV head, at most 16 spans (the block steps' partial buffers).  k_maps / v_maps: host
// arrays of `caches` tensor maps over [layers * pages * 16][kv_hidden] bf16, boxes of 64 x 16.
bool attention_rows_supported(uint32_t heads, uint32_t kv_heads, uint32_t head_dim);
uint32_t attention_rows_splits(uint32_t longest_context, uint32_t rows, uint32_t kv_heads, uint32_t sm_count);
cudaError_t launch_attention_rows(cudaStream_t stream, const AttentionParams &p, const TensorMapStorage *k_maps,
                                  const TensorMapStorage *v_maps, uint32_t caches);
cudaError_t configure_attention_kernels();
uint32_t attention_default_splits(uint32_t context, uint32_t batch, uint32_t kv_heads,
                                  uint32_t sm_count);

// ---- fused decode attention of the session (one launch per layer) ----
// One activation row of a block step (several tokens through the layer together): the
// per-row replacements of the single-session fields of FusedAttentionParams.
struct FusedAttentionRow {
  uint32_t position;       // position of this row's token
  uint32_t max_context, page_count;
  uint32_t map_index;      // row form of the paged tensor-pipe kernel: which cache of the launch is this row's
  const float *qkv;        // this row's projection output
  uint16_t *key_pages, *value_pages;  // layer 0 of the row's session; the kernel adds layer * kv_layer_elems
  uint64_t kv_layer_elems;
  const uint32_t *page_table;
  float *partial_acc, *partial_m, *partial_l;
  uint32_t *tickets;
  uint16_t *out_bf16;
  uint32_t *error_word;
};

struct FusedAttentionParams {
  const uint32_t *cursor;  // position of the token being decoded
  uint32_t max_context;
  const float *qkv;        // [heads*d | kv_heads*d | kv_heads*d] f32 projection output
  const uint16_t *q_bias, *k_bias, *v_bias, *q_norm, *k_norm;  // optional
  uint16_t *key_pages, *value_pages;  // this layer's pages
  const uint32_t *page_table;
  uint32_t page_count;
  uint32_t heads, kv_heads, head_dim;
  float eps, rope_theta;
  uint32_t splits;
  float *partial_acc, *partial_m, *partial_l;  // [heads][splits][...]
  uint32_t *tickets;                           // [kv_heads], zero between launches
  uint16_t *out_bf16;                          // [heads*d]
  uint32_t *error_word;
  uint32_t pdl;
  unsigned long long *stamps;  // optional timeline stamps
  // Block step: rows != nullptr launches one set of blocks per row (grid.y = row_count); the row
  // supplies position, qkv, pages, partials, tickets and output.  cached_only: the row's own K/V
  // are already in the cache (published by an earlier kernel of the chunk), so the kernel attends
  // over positions 0..position and appends nothing.
  const FusedAttentionRow *rows;
  uint32_t row_count, layer, cached_only;
};
bool fused_attention_supported(uint32_t heads, uint32_t kv_heads, uint32_t head_dim);
uint32_t fused_attention_splits(uint32_t target_context);
cudaError_t launch_fused_attention(cudaStream_t stream, const FusedAttentionParams &p);
cudaError_t configure_fused_attention_kernel();

// ---- DeepSeek multi-head latent attention of the session (mla_session.cu) ----
struct MlaParams {
  const uint32_t *cursor;  // position of the token being decoded
  uint32_t max_context;
  float *qkv;              // fused projection output: [heads][nope + rope] queries, then [rank + rope]; the
                           // rotary parts of the queries are rotated in place
  const uint16_t *w_kv_b;  // [heads][nope + v_dim][rank]: per head W_UK rows, then W_UV rows
  const uint16_t *kv_a_norm;  // [rank]
  uint16_t *cache;         // this layer's cache rows [pages][16][rank + rope] bf16
  const uint32_t *page_table;
  uint32_t page_count;
  uint32_t heads, rank, nope, rope, v_dim;
  float eps, rope_theta;
  float *ql;               // scratch [heads][rank]
  float *partial_acc, *partial_m, *partial_l;  // [heads][splits][rank], [heads][splits]
  uint16_t *out_bf16;      // [heads * v_dim]
  uint32_t *error_word;
};
bool mla_session_supported(uint32_t heads, uint32_t rank, uint32_t nope, uint32_t rope, uint32_t v_dim);
uint32_t mla_attention_splits(uint32_t target_context);
// Three launches: prepare (rotary, absorbed queries, cache append), split attention, merge + value projection.
cudaError_t launch_mla_attention(cudaStream_t stream, const MlaParams &p, uint32_t splits, bool pdl);
cudaError_t configure_mla_kernels();  // once per device before the first launch

// ---- softmax top-k sparse MoE MLP (moe.cu) ----
struct MoeExpertParams {
  // residual add + RMSNorm prologue (as ProjectionParams), fp32 result
  const float *add_a, *add_b;
  const uint16_t *add_bias, *norm_weight;
  float eps;
  uint32_t hidden, moe_intermediate, shared_intermediate, top_k;
  const uint16_t *w_expert_gate_up;  // expert e's gate matrix at e * expert_stride, its up matrix expert_up_offset
                                     // further: [E][2 * mi][hidden] (stride 2 mi hidden, offset mi hidden), or all
                                     // gate matrices then all up matrices (stride mi hidden, offset E mi hidden)
  uint64_t expert_stride, expert_up_offset;
  const uint16_t *w_expert_down;     // [E][hidden][moe_intermediate]
  const uint16_t *w_shared_gate, *w_shared_up, *w_shared_down;  // shared expert, optional
  const uint16_t *w_shared_router;   // its gate sigmoid(router . x); null: always on (scale 1)
  // Routing happens inside the gate/up launch: router logits W_router . x for all experts, softmax,
  // top-k, optional renormalisation; block 0 stores the new residual stream (resid_out, optional)
  // and the result, which the down launch reads.
  const uint16_t *w_router;          // [num_experts][hidden]
  uint32_t num_experts, norm_topk_prob;
  float *resid_out;
  uint32_t *expert_ids;              // [top_k] scratch: the routing result
  float *route_weights;              // [top_k]
  float *gate_up_out;                // scratch: per expert gate then up rows (+ the shared expert's), fp32
  float *shared_gate;                // scratch: 1 float
  float *out_f32;                    // [hidden] the MLP output
  float *partial;                    // scratch: [17][hidden] per-expert contributions before they are added
  uint32_t *ticket;                  // scratch: one counter, zero between launches
  uint32_t *error_word;
  uint32_t max_intermediate, max_rows_per_block;  // filled by the launcher
  // Expert parallel: this rank holds experts [expert_base, expert_base + expert_local) of the layer
  // (the matrices above are indexed by id - expert_base) and, of the shared expert, a slice of the
  // intermediate dimension; chosen experts held elsewhere are skipped.  With push.world > 1 the
  // partial MLP output goes, tagged, into every rank's receive buffer instead of out_f32, and the
  // next norm prologue adds the ranks' partials in rank order (TpPush / TpGather).
  // expert_local == 0 means all experts are here.
  uint32_t expert_base, expert_local;
  TpPush push;
};
bool moe_supported(uint32_t hidden, uint32_t moe_intermediate, uint32_t shared_intermediate,
                   uint32_t num_experts, uint32_t top_k, uint32_t sm_count);
cudaError_t configure_moe_kernels();
// Two launches: routing + gate/up of the chosen experts, then SwiGLU + down and the weighted sum.
cudaError_t launch_moe_experts(cudaStream_t stream, const MoeExpertParams &p, uint32_t sm_count, bool pdl);

// ---- greedy sampling ----
// Reduces per-block (value, index) partials, writes the token slot at the
// cursor and advances the cursor.  sample == 0: only advances the cursor.
// tp (nullable): the exchange of per-shard arg-max candidates between tensor-parallel ranks;
// tp->epoch (nullable) is incremented at the end of every step.
struct TpSample {
  uint32_t world, rank;
  uint32_t vocab_offset;                      // first vocabulary row of this rank's lm_head shard
  unsigned long long *epoch;
  unsigned long long *recv[kMaxTpWorld];      // rank q's candidates [world]: value bits << 32 | index
  unsigned long long *arrivals[kMaxTpWorld];  // rank q's arrival counters [world]
};
cudaError_t launch_sample_greedy(cudaStream_t stream, const StepState &st, const float *best_value,
                                 const uint32_t *best_index, uint32_t partials, uint32_t sample,
                                 bool pdl = false, const TpSample *tp = nullptr);
// One row of a packed step for the batched sampler: the row's session (cursor, token ring, ...) and
// where that session keeps the logits it sampled from (nullable).
struct BlockSampleRow {
  StepState state;
  float *logits;
};
// Arg-max of every row (from `partials` candidates per row) into the row's own session, and the
// rows' logits into the sessions' own buffers, in one launch.
cudaError_t launch_block_sample(cudaStream_t stream, const BlockSampleRow *rows, uint32_t count, const float *best_value,
                                const uint32_t *best_index, uint32_t partials, const float *logits, uint32_t vocab,
                                bool pdl);
// Waits (bounded) until every rank's entries of one exchange have arrived; closes a step that does
// not sample, whose last exchange no projection reads.
cudaError_t launch_exchange_wait(cudaStream_t stream, const TpGather &gather, uint32_t cols, uint32_t *error_word,
                                 bool pdl);
// ---- temperature / top-k / top-p sampling ----
// Read from device memory at every step, so that a captured graph does not depend on the values.
struct SamplerParams {
  float temperature, top_p;
  uint32_t top_k, reserved;
  uint64_t seed;
};
// One block over the fp32 logits: writes the token slot at the cursor and advances the cursor.
cudaError_t launch_sample_general(cudaStream_t stream, const StepState &st, const float *logits,
                                  const SamplerParams *params, bool pdl = false);
// Stand-alone argmax over logits (used by the per-op entry point).
cudaError_t launch_argmax(cudaStream_t stream, const float *logits, uint32_t count,
                          uint32_t *token_out);

// ---- helpers ----
cudaError_t launch_pack_qkv(cudaStream_t stream, const uint16_t *wq, const uint16_t *wk,
                            const uint16_t *wv, uint16_t *packed, uint64_t q_elems,
                            uint64_t kv_elems);
cudaError_t launch_pack_gate_up(cudaStream_t stream, const uint16_t *gate, const uint16_t *up,
                                uint16_t *packed, uint32_t intermediate, uint32_t hidden);
cudaError_t launch_identity_table(cudaStream_t stream, uint32_t *table, uint32_t count);
cudaError_t launch_fill_normal_bf16(cudaStream_t stream, uint16_t *out, uint64_t count,
                                    uint64_t seed, uint64_t tensor_id, float std);

}  // namespace nb
