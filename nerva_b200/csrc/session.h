// Resident decode session: everything a session owns on the host and on the
// device.  Mirrors the role of the reference's
// hf_decode_sequence/session_state.cuh:1-222 (device pointers, cached graphs,
// cursor, token ring) with a different memory plan: two device allocations per
// session (shared weights, private state), each carved by a StaticArena, and
// nothing allocated after create.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <memory>
#include <string>
#include <deque>
#include <vector>

#include "../../include/nerva_b200_api.h"
#include "host_memory.h"
#include "kernels.cuh"

namespace nb {

constexpr uint64_t kMissingOffset = UINT64_MAX;

// Offsets (16-bit elements) of one layer's tensors in the upload arena; the
// order is the reference's pack_layer (hf_decode_sequence/weights.cu:487-591).
struct LayerLayout {
  uint64_t rms_attn = kMissingOffset, rms_mlp = kMissingOffset;
  uint64_t w_q = kMissingOffset, w_q_gate = kMissingOffset, q_norm = kMissingOffset;
  uint64_t w_k = kMissingOffset, k_norm = kMissingOffset, w_v = kMissingOffset;
  uint64_t w_o = kMissingOffset;
  uint64_t w_gate = kMissingOffset, w_up = kMissingOffset, w_down = kMissingOffset;
  uint64_t w_router = kMissingOffset, w_expert_gate_up = kMissingOffset;
  uint64_t w_expert_down = kMissingOffset;
  uint64_t w_shared_gate = kMissingOffset, w_shared_up = kMissingOffset;
  uint64_t w_shared_down = kMissingOffset, w_shared_router = kMissingOffset;
  uint64_t q_bias = kMissingOffset, k_bias = kMissingOffset, v_bias = kMissingOffset;
  uint64_t o_bias = kMissingOffset;
  uint32_t mlp_kind = 0, moe_intermediate = 0, shared_intermediate = 0;
  uint32_t num_experts = 0, top_k = 0, norm_topk_prob = 0;
  // DeepSeek multi-head latent attention (attention_kind 2): w_q is the query projection
  // [heads * (nope + rope)][hidden], w_k the latent + rotary-key projection [rank + rope][hidden],
  // k_norm the latent's norm weight [rank], w_v the up-projection [heads * (nope + v)][rank]
  // (per head: nope rows of W_UK, then v rows of W_UV), w_o [hidden][heads * v] — the slots the
  // reference's packer uses for them (hf_decode_sequence/deepseek/weights_pack.inc.cu:156-186).
  uint32_t attention_kind = 0, kv_lora_rank = 0, qk_nope = 0, qk_rope = 0;
  // Sparse-MoE expert matrices: Qwen-style layers hold per expert [gate rows | up rows]
  // (expert_up_offset = moe_intermediate * hidden inside a stride of twice that); DeepSeek layers
  // hold all gate matrices, then all up matrices (weights_pack.inc.cu:303-312).
  uint64_t expert_stride = 0, expert_up_offset = 0;
  // expert parallel: the experts whose matrices this arena holds (all of them otherwise)
  uint32_t expert_base = 0, expert_local = 0;
};

struct ArenaLayout {
  uint64_t embeddings = 0, input = 0, scratch = 0, final_norm = 0, lm_head = 0;
  uint64_t elements = 0;
  std::vector<LayerLayout> layers;
};

struct ModelDims {
  uint32_t dtype = 0, hidden = 0, heads = 0, kv_heads = 0, head_dim = 0;
  uint32_t intermediate = 0, vocab = 0, layers = 0;
  // vocab = rows of lm_head held here; a tensor-parallel rank holds a shard of the
  // rows starting at vocab_offset, while the embedding table keeps embed_vocab rows.
  uint32_t embed_vocab = 0, vocab_offset = 0;
  // latent attention (every layer, or none): rows of the fused query + latent projection and width
  // of a cache row; zero for ordinary attention
  uint32_t mla_rank = 0, mla_nope = 0, mla_rope = 0;
  // expert parallel (ep_world > 1): this rank's arena holds num_experts / ep_world routed experts per layer
  uint32_t ep_world = 1, ep_rank = 0;
  uint64_t attention_hidden() const { return static_cast<uint64_t>(heads) * head_dim; }
  uint64_t kv_hidden() const { return static_cast<uint64_t>(kv_heads) * head_dim; }
  bool mla() const { return mla_rank != 0; }
  uint64_t mla_q_rows() const { return static_cast<uint64_t>(heads) * (mla_nope + mla_rope); }
  uint64_t mla_width() const { return static_cast<uint64_t>(mla_rank) + mla_rope; }
  // rows of the packed first projection of a layer: [Q; K; V], or [Q; latent + rotary key]
  uint64_t qkv_rows() const { return mla() ? mla_q_rows() + mla_width() : attention_hidden() + 2 * kv_hidden(); }
  // elements of one cached row per array
  uint64_t kv_row() const { return mla() ? mla_width() : kv_hidden(); }
};

bool valid_layer(const NervaCudaHfDecodeChainLayer &layer, bool require_sources);
bool layer_supported(const NervaCudaHfDecodeChainLayer &layer);
ArenaLayout compute_arena_layout(const ModelDims &dims, const NervaCudaHfDecodeChainLayer *layers);
uint64_t hash_tokens(const uint32_t *tokens, uint32_t count);
uint64_t hash_weight_descriptors(const NervaCudaHfDecodeSequenceWeightBlock *blocks, uint32_t count);
void set_last_error(const std::string &text);

// One token of a block step: where its id comes from and where errors go.
struct BlockTokenRow {
  const uint32_t *prompt;
  const uint32_t *prompt_count;
  const NervaCudaSyntheticTokenSlot *slots;
  uint32_t position, vocab;
  uint32_t *error_word;
};

// Scratch of the block steps (several tokens through every layer together: the packed step of
// batch_advance_one and the chunked prefill of session_start).  One per weight set, allocated at
// create and shared by the forks; a block step runs on one stream at a time.
struct BlockWorkspace {
  void *block = nullptr;
  uint64_t bytes = 0;
  uint32_t max_rows = 0, sample_rows = 0;
  uint16_t *x_bf16 = nullptr;   // [max_rows][x_elems] normalised activations, the B operand of the next GEMM
  float *qkv = nullptr;         // [max_rows][A + 2 KV]
  uint16_t *attn = nullptr;     // [max_rows][A]
  float *h_a = nullptr, *h_b = nullptr;  // [max_rows][hidden] residual stream, ping-pong
  uint16_t *ff = nullptr;       // [max_rows][intermediate]
  float *logits = nullptr;      // [sample_rows][vocab]
  float *partial_acc = nullptr, *partial_m = nullptr, *partial_l = nullptr;  // split attention, per row
  uint32_t *attn_tickets = nullptr;  // [max_rows][kv_heads]
  float *gemm_workspace = nullptr;
  uint32_t *gemm_tickets = nullptr;
  float *best_value = nullptr;  // [sample_rows][kBlockArgmaxChunks]
  uint32_t *best_index = nullptr;
  FusedAttentionRow *attn_rows = nullptr;  // [max_rows] device copies of the row descriptors
  bool paged_rows = false;      // the rows' attention runs on the paged tensor-pipe kernel (attention.cu)
  BlockTokenRow *token_rows = nullptr;
  BlockSampleRow *sample_rows_dev = nullptr;  // [sample_rows] device copies of the sampler's row descriptors
};
constexpr uint32_t kBlockArgmaxChunks = 64;
constexpr uint32_t kBlockMaxRows = 256;       // one MMA N
constexpr uint32_t kBlockSampleRows = 32;     // sessions per packed decode step (hf_decode_sequence/types.cuh:63)

// Device weights shared between a session and its forks.
struct SharedWeights {
  void *block = nullptr;  // one allocation
  uint64_t block_bytes = 0;
  uint16_t *arena = nullptr;          // upload arena (reference layout)
  uint16_t *qkv_packed = nullptr;     // [layers][(A + 2 KV) x H]
  uint16_t *gate_up_packed = nullptr; // [layers][2 I x H], rows interleaved gate/up
  BlockWorkspace block_ws;            // empty when the model has no block-step path
  ~SharedWeights() {
    if (block != nullptr) cudaFree(block);
    if (block_ws.block != nullptr) cudaFree(block_ws.block);
  }
};

// Event-per-launch-group timing of un-captured steps (the reference's
// detailed_profile path, hf_decode_sequence/session_decode_prefill.inc.cu:374-810).
enum ProfileBucket : uint32_t {
  kBucketEmbed = 0, kBucketQkv, kBucketAttention, kBucketO, kBucketGateUp, kBucketDown,
  kBucketLmHead, kBucketSampling, kBucketCount
};
struct StepProfile {
  std::vector<cudaEvent_t> events;
  std::vector<uint32_t> bucket;  // bucket[i] labels the interval events[i] -> events[i+1]
  uint32_t used = 0;
};

struct GraphEntry {
  uint32_t splits = 0, sample = 0, engine = 0;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;  // null: the step is launched directly (capture was refused)
  uint64_t nodes = 0;
};

struct StepLayerDev;
struct JobDesc;
struct StepKernelParams;
uint32_t step_kernel_smem_bytes(uint32_t x_elems, uint32_t row_elems);
bool step_kernel_supported(uint32_t hidden, uint32_t heads, uint32_t kv_heads, uint32_t head_dim,
                           uint32_t intermediate, uint32_t x_elems, uint32_t row_elems);
cudaError_t configure_step_kernel();
cudaError_t launch_step_kernel(cudaStream_t stream, const StepKernelParams &p, uint32_t blocks);

// ---- block steps (block_step.cu) ----
// True when every layer is dense SwiGLU without biases, the fused attention kernel serves the head
// shape and every projection width is a multiple of 64: the shapes the block kernels run.
bool block_step_supported(const NervaCudaHfDecodeSequenceSession *s);
// Allocates s->weights->block_ws (at create).
cudaError_t allocate_block_workspace(NervaCudaHfDecodeSequenceSession *s);
// One token for each of `count` sessions that share weights, on `stream`: the weights are streamed
// once for the block.  Every session must be idle, positioned at its next token, and its stream
// synchronised.  Enqueues only; the caller copies the token slots back and synchronises.
cudaError_t enqueue_block_decode(NervaCudaHfDecodeSequenceSession *const *sessions, uint32_t count,
                                 cudaStream_t stream, uint64_t *launches);
// Prompt positions [0, prompt_count) of one session through every layer in chunks of up to
// kBlockMaxRows tokens, writing the same paged bf16 K/V the decode step reads, then the final
// norm, lm_head and the sampler for the last position.  Leaves the cursor at prompt_count.
cudaError_t enqueue_chunked_prefill(NervaCudaHfDecodeSequenceSession *s, uint32_t prompt_count, uint32_t sample_kind,
                                    uint64_t *launches);

}  // namespace nb

// The opaque handle of the C ABI.
struct NervaCudaHfDecodeSequenceSession {
  nb::ModelDims dims;
  uint32_t max_context = 0;
  float rms_eps = 0.0f, rope_theta = 0.0f;
  uint32_t sm_count = 0;
  uint32_t engine = 0;
  uint32_t detailed_profile = 0;
  nb::ArenaLayout layout;
  std::vector<NervaCudaHfDecodeChainLayer> layer_meta;  // scalars only; pointers cleared

  // planned-weight echo
  uint64_t resident_weight_bytes = 0;
  uint32_t planned_weight_blocks = 0, planned_gpu_resident_blocks = 0, planned_gpu_staged_blocks = 0;
  uint64_t planned_weight_bytes = 0, planned_gpu_resident_weight_bytes = 0;
  uint64_t planned_gpu_staged_weight_bytes = 0;
  uint32_t planned_weight_descriptor_count = 0;
  uint64_t planned_weight_descriptor_hash = 0;

  std::shared_ptr<nb::SharedWeights> weights;
  nb::StaticArena weight_arena, state_arena;
  nb::KvPagePool kv_pool;

  // private device state (one allocation)
  void *state_block = nullptr;
  uint64_t state_bytes = 0;
  uint16_t *kv_keys = nullptr, *kv_values = nullptr;  // [layers][pages][16][kv_hidden]
  uint64_t kv_layer_elems = 0;
  // the two arrays as 2-D tensor maps [layers * pages * 16][kv_hidden] (boxes of 64 dims x one page),
  // encoded once when the state is allocated; read by the row form of the paged attention kernel
  nb::TensorMapStorage kv_map_k{}, kv_map_v{};
  bool kv_maps = false;
  uint32_t kv_pages = 0;
  uint32_t *page_table = nullptr;
  float *h_a = nullptr, *h_b = nullptr, *qkv = nullptr, *o_out = nullptr, *down = nullptr;
  float *logits = nullptr;
  float *partial_acc = nullptr, *partial_m = nullptr, *partial_l = nullptr;
  uint32_t max_splits = 1;
  uint32_t *attn_tickets = nullptr;  // per-head completion tickets of the fused attention kernel
  bool fused_attention = false;      // head_dim 64/128: one attention launch per layer
  bool use_pdl = true;               // programmatic dependent launch between the step's kernels
                                     // (NERVA_B200_PDL=0 at create turns it off)
  uint16_t *attn_bf16 = nullptr, *ff_bf16 = nullptr, *x_scratch = nullptr;
  float *best_value = nullptr;
  uint32_t *best_index = nullptr;
  // whole-step kernel (engine 1)
  nb::StepLayerDev *step_layers = nullptr;
  nb::JobDesc *step_jobs = nullptr;
  uint32_t *barrier_counter = nullptr;
  unsigned long long *phase_cycles = nullptr;  // per-phase SM cycles of block 0 (tuning aid)
  bool phase_profile = false;                  // NERVA_B200_PHASE_PROFILE=1 at create
  // Tuning aid (NERVA_B200_TIMELINE=1 at create): per launch of a step, %globaltimer
  // stamps of the first and the last block (see kTimelineSlots in kernels.cuh).
  unsigned long long *timeline = nullptr;
  uint32_t timeline_nodes = 0;
  bool timeline_on = false;
  // sparse MoE layers: routing scratch
  bool has_moe = false;
  std::vector<int32_t> dense_ordinal;  // per layer: index of its packed gate/up copy, -1 for sparse layers
  // latent attention scratch
  float *mla_ql = nullptr;             // [heads][rank] absorbed queries
  float *router_logits = nullptr, *route_weights = nullptr, *shared_gate = nullptr, *moe_gate_up = nullptr;
  uint32_t *route_ids = nullptr;
  float *moe_partial = nullptr;        // [17][hidden] per-expert contributions of a sparse MLP (moe.cu)
  uint32_t *moe_ticket = nullptr;      // completion counter of the expert down launch, zero between launches
  // tensor parallel (nerva_b200_session_create_sharded)
  uint32_t tp_world = 1, tp_rank = 0;
  bool tp_two_stage = false;   // two ranks only: use the two-stage gather of the larger worlds
  void *comm_block = nullptr;  // this rank's exchange buffer (own allocation, exported to the peers)
  uint64_t comm_bytes = 0;
  void *comm_peers[nb::kMaxTpWorld] = {};  // every rank's exchange buffer as mapped here
  bool tp_attached = false;
  uint32_t x_elems = 0;
  uint32_t row_elems = 0;  // rows of the largest per-block row range of any projection
  bool step_kernel_ok = false;
  NervaCudaSyntheticTokenSlot *device_slots = nullptr;
  uint32_t *device_cursor = nullptr, *device_error = nullptr, *device_prompt = nullptr;
  uint64_t slots_bytes = 0;

  NervaCudaSyntheticTokenSlot *host_slots = nullptr;  // pinned
  uint32_t *host_error = nullptr;                     // pinned, 1 word

  cudaStream_t stream = nullptr;
  cudaEvent_t ev_start = nullptr, ev_stop = nullptr;
  std::deque<nb::GraphEntry> graphs;  // deque: entries keep their address when more are cached

  // active request
  bool started = false, finished = false;
  uint32_t prompt_count = 0, has_eos = 0, eos_token = 0, seed_token = 0;
  uint32_t observed = 0, cursor = 0;
  bool logits_valid = false;
  // Sampler of the active request: 1 = arg-max, 2 = temperature / top-k / top-p from device_sampler.
  uint32_t sample_kind = 1;
  nb::SamplerParams host_sampler{};
  nb::SamplerParams *device_sampler = nullptr;
  uint64_t hot_path_allocations = 0;
};

// Element offset of layer l's packed gate/up copy (dense layers only; sparse layers have none).
inline uint64_t gate_up_packed_offset(const NervaCudaHfDecodeSequenceSession *s, uint32_t l) {
  return static_cast<uint64_t>(s->dense_ordinal[l]) * 2u * s->dims.intermediate * s->dims.hidden;
}
