// C ABI of the resident decode session: create / start / advance / run / fork /
// destroy / plan_layout / one-shot.  Entry-point names, argument structs,
// validation rules and result accounting follow the reference
// (hf_decode_sequence/session_api_lifecycle.inc.cu, weights.cu); the engine
// underneath is this library's own.
#include "session.h"
#include "step_kernel.cuh"

#include <math.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <new>

namespace nb {

// ---------------------------------------------------------------- errors ----
static thread_local std::string g_last_error;
void set_last_error(const std::string &text) { g_last_error = text; }

// Reference create-failure stages that still apply
// (hf_decode_sequence/session_prelude.inc.cu:1-40).
enum CreateStage : int32_t {
  kStageNone = 0,
  kStageInvalidRequest = 1,
  kStageGetDeviceCount = 2,
  kStageSetDevice = 3,
  kStageSessionAlloc = 4,
  kStageHostSlotsAlloc = 6,
  kStageDeviceArenaAlloc = 7,
  kStageDeviceScratchAlloc = 9,
  kStageStreamCreate = 19,
  kStageStartEventCreate = 23,
  kStageStopEventCreate = 24,
  kStageDescriptorCopy = 25,
  kStagePackReplicas = 27,
  kStageSetupSynchronize = 29,
};

// ------------------------------------------------------------ validation ----
// hf_decode_sequence/weights.cu:168-230.
bool valid_layer(const NervaCudaHfDecodeChainLayer &layer, bool require_sources) {
  const bool dense = layer.mlp_kind == NERVA_MLP_KIND_DENSE;
  const bool sparse = layer.mlp_kind == NERVA_MLP_KIND_SPARSE_MOE;
  if (!dense && !sparse) return false;
  if (layer.attention_kind == NERVA_ATTENTION_KIND_LINEAR_GDN) {
    if (layer.linear_key_heads == 0 || layer.linear_value_heads == 0 ||
        layer.linear_key_head_dim == 0 || layer.linear_value_head_dim == 0 ||
        layer.linear_conv_kernel == 0)
      return false;
  } else if (layer.attention_kind == NERVA_ATTENTION_KIND_DEEPSEEK_MLA) {
    if (layer.deepseek_kv_lora_rank == 0 || layer.deepseek_qk_rope_head_dim == 0) return false;
  } else if (layer.attention_kind != NERVA_ATTENTION_KIND_FULL) {
    return false;
  }
  if (sparse && (layer.moe_intermediate == 0 || layer.num_experts == 0 ||
                 layer.experts_per_token == 0 || layer.experts_per_token > layer.num_experts ||
                 layer.num_experts > 256u || layer.experts_per_token > 16u))
    return false;
  if (!require_sources) return true;
  if (layer.rms_attn_weight == nullptr || layer.rms_mlp_weight == nullptr) return false;
  if (layer.attention_kind != NERVA_ATTENTION_KIND_FULL) return false;  // latent-attention tensors only come by descriptor
  if (layer.w_q == nullptr || layer.w_k == nullptr || layer.w_v == nullptr || layer.w_o == nullptr)
    return false;
  if (dense) return layer.w_gate != nullptr && layer.w_up != nullptr && layer.w_down != nullptr;
  if (layer.w_router == nullptr || layer.w_expert_gate_up == nullptr ||
      layer.w_expert_down == nullptr)
    return false;
  if (layer.shared_expert_intermediate != 0 &&
      (layer.w_shared_expert_gate == nullptr || layer.w_shared_expert_up == nullptr ||
       layer.w_shared_expert_down == nullptr || layer.w_shared_expert_router == nullptr))
    return false;
  return true;
}

// What this library's kernels run: full attention, no query gate, dense SwiGLU or
// softmax top-k sparse MoE (whose shape limits are checked once the device is known).
bool layer_supported(const NervaCudaHfDecodeChainLayer &layer) {
  const bool mlp_ok = layer.mlp_kind == NERVA_MLP_KIND_DENSE || layer.mlp_kind == NERVA_MLP_KIND_SPARSE_MOE;
  if (layer.attention_kind == NERVA_ATTENTION_KIND_FULL) return layer.w_q_gate == nullptr && mlp_ok;
  if (layer.attention_kind != NERVA_ATTENTION_KIND_DEEPSEEK_MLA) return false;
  // Latent attention in its plain bf16 form: no query low-rank stage, no indexer, compressor,
  // hyper-connection, FP8 storage or rotary scaling (the DeepSeek-V2-Lite shape).  The reference's
  // own session runs the V3 form with a query low-rank stage and grouped-sigmoid routing; this
  // degenerate form is an extension the reference rejects (session_decode_v3_projection.inc.cu:30-33).
  return mlp_ok && layer.deepseek_q_lora_rank == 0 && layer.deepseek_storage == 1u && layer.deepseek_flags == 0 &&
         layer.deepseek_hc_mult == 0 && layer.deepseek_o_lora_rank == 0 && layer.deepseek_compress_ratio <= 1 &&
         layer.deepseek_rope_scaling_type == 0 && layer.deepseek_kv_lora_rank % 32u == 0 &&
         layer.deepseek_kv_lora_rank <= 512u && layer.deepseek_qk_rope_head_dim % 2u == 0 &&
         layer.deepseek_qk_rope_head_dim <= 64u && layer.deepseek_qk_nope_head_dim != 0 &&
         layer.deepseek_qk_nope_head_dim <= 256u && layer.deepseek_v_head_dim != 0;
}

static bool sampler_valid(const NervaCudaHfDecodeSamplerConfig &s) {
  return isfinite(s.temperature) && s.temperature >= 0.0f && isfinite(s.top_p) && s.top_p > 0.0f &&
         s.top_p <= 1.0f;
}
static bool sampler_greedy(const NervaCudaHfDecodeSamplerConfig &s) {
  return !(s.temperature > 0.0f) || s.top_k == 1;  // sampler.cu:88
}

// ---------------------------------------------------------------- layout ----
static uint64_t push(uint64_t &cursor, uint64_t len) {
  const uint64_t offset = cursor;
  cursor += len;
  return offset;
}
static uint64_t push_optional(uint64_t &cursor, uint64_t len, const void *ptr) {
  return ptr == nullptr ? kMissingOffset : push(cursor, len);
}

// hf_decode_sequence/weights.cu:487-591 (full-attention layers) and
// session_api_lifecycle.inc.cu:124-146 (arena order).
ArenaLayout compute_arena_layout(const ModelDims &d, const NervaCudaHfDecodeChainLayer *layers) {
  ArenaLayout out;
  const uint64_t hidden = d.hidden, ah = d.attention_hidden(), kvh = d.kv_hidden();
  const uint64_t inter = d.intermediate;
  uint64_t c = 0;
  out.embeddings = push(c, static_cast<uint64_t>(d.embed_vocab != 0 ? d.embed_vocab : d.vocab) * hidden);
  out.input = push(c, hidden);
  out.scratch = push(c, hidden);
  out.layers.resize(d.layers);
  for (uint32_t i = 0; i < d.layers; ++i) {
    const NervaCudaHfDecodeChainLayer &layer = layers[i];
    LayerLayout &l = out.layers[i];
    l.mlp_kind = layer.mlp_kind;
    l.moe_intermediate = layer.moe_intermediate;
    l.shared_intermediate = layer.shared_expert_intermediate;
    l.num_experts = layer.num_experts;
    l.top_k = layer.experts_per_token;
    l.norm_topk_prob = layer.norm_topk_prob == 0 ? 0u : 1u;
    l.attention_kind = layer.attention_kind;
    if (layer.attention_kind == NERVA_ATTENTION_KIND_DEEPSEEK_MLA) {
      // hf_decode_sequence/deepseek/weights_pack.inc.cu:156-186,261-322 (bf16 storage), with the query
      // projection in the w_q slot because there is no low-rank stage in front of it
      const uint64_t rank = layer.deepseek_kv_lora_rank, nope = layer.deepseek_qk_nope_head_dim;
      const uint64_t rope = layer.deepseek_qk_rope_head_dim, vdim = layer.deepseek_v_head_dim;
      const uint64_t heads = d.heads;
      l.kv_lora_rank = static_cast<uint32_t>(rank);
      l.qk_nope = static_cast<uint32_t>(nope);
      l.qk_rope = static_cast<uint32_t>(rope);
      l.rms_attn = push(c, hidden);
      l.w_q = push(c, heads * (nope + rope) * hidden);
      l.w_k = push(c, (rank + rope) * hidden);
      l.k_norm = push(c, rank);
      l.w_v = push(c, heads * (nope + vdim) * rank);
      l.w_o = push(c, hidden * heads * vdim);
      l.rms_mlp = push(c, hidden);
      if (layer.mlp_kind == NERVA_MLP_KIND_SPARSE_MOE) {
        const uint64_t mi = layer.moe_intermediate, si = layer.shared_expert_intermediate;
        const uint64_t e = layer.num_experts / d.ep_world;  // the experts held here
        l.expert_local = static_cast<uint32_t>(e);
        l.expert_base = static_cast<uint32_t>(e) * d.ep_rank;
        l.w_router = push(c, static_cast<uint64_t>(layer.num_experts) * hidden);
        if (si != 0) {
          l.w_shared_gate = push(c, si * hidden);
          l.w_shared_up = push(c, si * hidden);
          l.w_shared_down = push(c, hidden * si);
        }
        l.w_expert_gate_up = push(c, e * mi * hidden);  // every expert's gate matrix ...
        push(c, e * mi * hidden);                       // ... then every expert's up matrix
        l.w_expert_down = push(c, e * hidden * mi);
        l.expert_stride = mi * hidden;
        l.expert_up_offset = e * mi * hidden;
      } else {
        l.w_gate = push(c, inter * hidden);
        l.w_up = push(c, inter * hidden);
        l.w_down = push(c, hidden * inter);
      }
      continue;
    }
    l.rms_attn = push(c, hidden);
    l.w_q = push(c, ah * hidden);
    l.w_q_gate = push_optional(c, ah * hidden, layer.w_q_gate);
    l.q_norm = push_optional(c, d.head_dim, layer.q_norm_weight);
    l.w_k = push(c, kvh * hidden);
    l.k_norm = push_optional(c, d.head_dim, layer.k_norm_weight);
    l.w_v = push(c, kvh * hidden);
    l.w_o = push(c, hidden * ah);
    l.rms_mlp = push(c, hidden);
    if (layer.mlp_kind == NERVA_MLP_KIND_SPARSE_MOE) {
      const uint64_t mi = layer.moe_intermediate, e = layer.num_experts / d.ep_world;
      const uint64_t si = layer.shared_expert_intermediate;
      l.expert_local = static_cast<uint32_t>(e);
      l.expert_base = static_cast<uint32_t>(e) * d.ep_rank;
      l.w_router = push(c, static_cast<uint64_t>(layer.num_experts) * hidden);
      l.w_expert_gate_up = push(c, e * mi * 2u * hidden);
      l.w_expert_down = push(c, e * hidden * mi);
      l.expert_stride = 2u * mi * hidden;
      l.expert_up_offset = mi * hidden;
      if (si != 0) {
        l.w_shared_gate = push(c, si * hidden);
        l.w_shared_up = push(c, si * hidden);
        l.w_shared_down = push(c, hidden * si);
        l.w_shared_router = push(c, hidden);
      }
    } else {
      l.w_gate = push(c, inter * hidden);
      l.w_up = push(c, inter * hidden);
      l.w_down = push(c, hidden * inter);
    }
    l.q_bias = push_optional(c, ah, layer.q_bias);
    l.k_bias = push_optional(c, kvh, layer.k_bias);
    l.v_bias = push_optional(c, kvh, layer.v_bias);
    l.o_bias = push_optional(c, hidden, layer.o_bias);
  }
  out.final_norm = push(c, hidden);
  out.lm_head = push(c, static_cast<uint64_t>(d.vocab) * hidden);
  out.elements = c;
  return out;
}

// ---------------------------------------------------------------- hashes ----
constexpr uint64_t kFnvOffset = 0xcbf29ce484222325ull;
constexpr uint64_t kFnvPrime = 0x00000100000001b3ull;
static void fnv_bytes(uint64_t &h, uint64_t v, uint32_t n) {
  for (uint32_t b = 0; b < n; ++b) {
    h ^= (v >> (8u * b)) & 0xffu;
    h *= kFnvPrime;
  }
}
// hf_decode_sequence/weights.cu:78-88
uint64_t hash_tokens(const uint32_t *tokens, uint32_t count) {
  uint64_t h = kFnvOffset;
  for (uint32_t i = 0; i < count; ++i) fnv_bytes(h, tokens[i], 4);
  return h;
}
// hf_decode_sequence/weights.cu:104-111
uint64_t hash_weight_descriptors(const NervaCudaHfDecodeSequenceWeightBlock *blocks, uint32_t n) {
  uint64_t h = kFnvOffset;
  for (uint32_t i = 0; i < n; ++i) {
    fnv_bytes(h, blocks[i].block_id, 8);
    fnv_bytes(h, blocks[i].block_version, 8);
    fnv_bytes(h, blocks[i].offset_bytes, 8);
    fnv_bytes(h, blocks[i].bytes, 8);
    fnv_bytes(h, blocks[i].strategy, 4);
  }
  return h;
}

}  // namespace nb

using namespace nb;
typedef NervaCudaHfDecodeSequenceSession Session;

namespace {

template <class T>
bool carve(StaticArena &arena, void *base, uint64_t count, T **out) {
  ArenaRegion region;
  if (!arena.reserve(count * sizeof(T), 256, AllocationPhase::Initialization, &region)) return false;
  if (base != nullptr) *out = reinterpret_cast<T *>(static_cast<uint8_t *>(base) + region.offset);
  return true;
}

// Carves the shared weight block.  base == nullptr: sizing pass.
bool plan_weights(Session *s, StaticArena &arena, void *base, SharedWeights *w) {
  const ModelDims &d = s->dims;
  const uint64_t qkv_rows = d.qkv_rows();
  uint64_t dense_layers = 0;
  for (int32_t ordinal : s->dense_ordinal) dense_layers += ordinal >= 0 ? 1u : 0u;
  uint16_t *arena_ptr = nullptr, *qkv = nullptr, *gu = nullptr;
  bool ok = carve(arena, base, s->layout.elements, &arena_ptr);
  ok = ok && carve(arena, base, static_cast<uint64_t>(d.layers) * qkv_rows * d.hidden, &qkv);
  ok = ok && carve(arena, base, std::max<uint64_t>(dense_layers, 1u) * 2u * d.intermediate * d.hidden, &gu);
  if (ok && w != nullptr) {
    w->arena = arena_ptr;
    w->qkv_packed = qkv;
    w->gate_up_packed = gu;
  }
  return ok;
}

// Carves the private state block.  base == nullptr: sizing pass.
bool plan_state(Session *s, StaticArena &arena, void *base) {
  const ModelDims &d = s->dims;
  const uint64_t ah = d.attention_hidden(), kvh = d.kv_hidden();
  s->kv_pages = (s->max_context + NERVA_KV_CACHE_BLOCK_TOKENS - 1) / NERVA_KV_CACHE_BLOCK_TOKENS;
  // latent attention caches one row of (rank + rope) values per token in the K array; the V array is not used
  s->kv_layer_elems = static_cast<uint64_t>(s->kv_pages) * NERVA_KV_CACHE_BLOCK_TOKENS * d.kv_row();
  s->max_splits = attention_default_splits(s->max_context, 1, d.kv_heads, s->sm_count);
  const uint64_t max_x = std::max<uint64_t>(std::max<uint64_t>(d.hidden, d.intermediate), ah);
  bool ok = carve(arena, base, d.layers * s->kv_layer_elems, &s->kv_keys);
  ok = ok && carve(arena, base, d.mla() ? uint64_t{16} : d.layers * s->kv_layer_elems, &s->kv_values);
  ok = ok && carve(arena, base, static_cast<uint64_t>(s->kv_pages), &s->page_table);
  ok = ok && carve(arena, base, static_cast<uint64_t>(d.hidden), &s->h_a);
  ok = ok && carve(arena, base, static_cast<uint64_t>(d.hidden), &s->h_b);
  ok = ok && carve(arena, base, std::max<uint64_t>(ah + 2 * kvh, d.qkv_rows()), &s->qkv);
  ok = ok && carve(arena, base, std::max<uint64_t>(static_cast<uint64_t>(d.heads) * d.mla_rank, 4u), &s->mla_ql);
  ok = ok && carve(arena, base, static_cast<uint64_t>(d.hidden), &s->o_out);
  ok = ok && carve(arena, base, static_cast<uint64_t>(d.hidden), &s->down);
  ok = ok && carve(arena, base, static_cast<uint64_t>(d.vocab), &s->logits);
  // fused attention uses up to 16 spans, latent attention up to 64
  const uint64_t split_slots = std::max<uint32_t>(s->max_splits, d.mla() ? 64u : 16u);
  ok = ok && carve(arena, base, static_cast<uint64_t>(d.heads), &s->attn_tickets);
  s->x_elems = static_cast<uint32_t>(max_x);
  ok = ok && carve(arena, base, static_cast<uint64_t>(d.heads) * split_slots * std::max(d.head_dim, d.mla_rank),
                   &s->partial_acc);
  ok = ok && carve(arena, base, static_cast<uint64_t>(d.heads) * split_slots, &s->partial_m);
  ok = ok && carve(arena, base, static_cast<uint64_t>(d.heads) * split_slots, &s->partial_l);
  ok = ok && carve(arena, base, static_cast<uint64_t>(d.layers), &s->step_layers);
  ok = ok && carve(arena, base, static_cast<uint64_t>(d.layers) * 4u + 1u, &s->step_jobs);
  ok = ok && carve(arena, base, uint64_t{4}, &s->barrier_counter);
  ok = ok && carve(arena, base, static_cast<uint64_t>(kPhaseCount), &s->phase_cycles);
  ok = ok && carve(arena, base, ah, &s->attn_bf16);
  ok = ok && carve(arena, base, static_cast<uint64_t>(d.intermediate), &s->ff_bf16);
  ok = ok && carve(arena, base, max_x, &s->x_scratch);
  ok = ok && carve(arena, base, static_cast<uint64_t>(s->sm_count), &s->best_value);
  ok = ok && carve(arena, base, static_cast<uint64_t>(s->sm_count), &s->best_index);
  ok = ok && carve(arena, base, static_cast<uint64_t>(s->max_context), &s->device_slots);
  ok = ok && carve(arena, base, static_cast<uint64_t>(s->max_context), &s->device_prompt);
  ok = ok && carve(arena, base, uint64_t{4}, &s->device_cursor);
  ok = ok && carve(arena, base, uint64_t{4}, &s->device_error);
  ok = ok && carve(arena, base, uint64_t{1}, &s->device_sampler);
  uint64_t moe_scratch = 0;
  for (const LayerLayout &L : s->layout.layers) {
    if (L.mlp_kind == NERVA_MLP_KIND_SPARSE_MOE)
      moe_scratch = std::max<uint64_t>(moe_scratch, 2ull * L.top_k * L.moe_intermediate + 2ull * L.shared_intermediate);
  }
  ok = ok && carve(arena, base, uint64_t{256}, &s->router_logits);
  ok = ok && carve(arena, base, uint64_t{16}, &s->route_ids);
  ok = ok && carve(arena, base, uint64_t{16}, &s->route_weights);
  ok = ok && carve(arena, base, uint64_t{4}, &s->shared_gate);
  ok = ok && carve(arena, base, moe_scratch + 4u, &s->moe_gate_up);
  ok = ok && carve(arena, base, moe_scratch != 0 ? uint64_t{17} * d.hidden : uint64_t{4}, &s->moe_partial);
  ok = ok && carve(arena, base, uint64_t{4}, &s->moe_ticket);
  s->timeline_nodes = 5u * d.layers + 1u;
  ok = ok && carve(arena, base, static_cast<uint64_t>(s->timeline_nodes) * kTimelineSlots, &s->timeline);
  return ok;
}

// Exchange buffer of a tensor-parallel rank (its own allocation, shared with the
// other ranks through an inter-process handle).  Offsets are the same on every rank.
struct CommLayout {
  uint64_t recv_o, recv_d, reduced_o, reduced_d, arrivals_s, candidates, epoch, bytes;
};
CommLayout comm_layout(uint32_t world, uint32_t hidden) {
  CommLayout c{};
  uint64_t at = 0;
  auto take = [&at](uint64_t bytes) {
    const uint64_t begin = at;
    at = (at + bytes + 255u) & ~uint64_t{255};
    return begin;
  };
  c.recv_o = take(static_cast<uint64_t>(world) * hidden * 8u);  // tagged 8-byte entries
  c.recv_d = take(static_cast<uint64_t>(world) * hidden * 8u);
  c.reduced_o = take(static_cast<uint64_t>(hidden) * 8u);  // local sums over the ranks (world > 2)
  c.reduced_d = take(static_cast<uint64_t>(hidden) * 8u);
  c.arrivals_s = take(world * 8u);
  c.candidates = take(world * 8u);
  c.epoch = take(8u);
  c.bytes = at;
  return c;
}
template <class T>
T *comm_at(void *base, uint64_t offset) {
  return reinterpret_cast<T *>(static_cast<uint8_t *>(base) + offset);
}
cudaError_t allocate_comm(Session *s) {
  const CommLayout c = comm_layout(s->tp_world, s->dims.hidden);
  cudaError_t err = cudaMalloc(&s->comm_block, c.bytes);
  if (err == cudaSuccess) err = cudaMemset(s->comm_block, 0, c.bytes);
  s->comm_bytes = c.bytes;
  return err;
}

void destroy_graphs(Session *s) {
  for (GraphEntry &g : s->graphs) {
    if (g.exec != nullptr) cudaGraphExecDestroy(g.exec);
    if (g.graph != nullptr) cudaGraphDestroy(g.graph);
  }
  s->graphs.clear();
}

void destroy_session(Session *s) {
  if (s == nullptr) return;
  if (s->stream != nullptr) cudaStreamSynchronize(s->stream);
  destroy_graphs(s);
  if (s->ev_start != nullptr) cudaEventDestroy(s->ev_start);
  if (s->ev_stop != nullptr) cudaEventDestroy(s->ev_stop);
  if (s->stream != nullptr) cudaStreamDestroy(s->stream);
  if (s->host_slots != nullptr) cudaFreeHost(s->host_slots);
  if (s->host_error != nullptr) cudaFreeHost(s->host_error);
  if (s->state_block != nullptr) cudaFree(s->state_block);
  for (uint32_t q = 0; q < kMaxTpWorld; ++q) {
    if (s->comm_peers[q] != nullptr && s->comm_peers[q] != s->comm_block) cudaIpcCloseMemHandle(s->comm_peers[q]);
  }
  if (s->comm_block != nullptr) cudaFree(s->comm_block);
  delete s;
}

StepState step_state(Session *s) {
  StepState st;
  st.cursor = s->device_cursor;
  st.prompt = s->device_prompt;
  st.prompt_count = s->device_cursor + 1;  // word 1 of the cursor block, written by reset_request_state
  st.slots = s->device_slots;
  st.max_context = s->max_context;
  st.vocab = s->dims.embed_vocab;  // token ids index the (whole) embedding table
  st.error_word = s->device_error;
  return st;
}

const uint16_t *arena_at(Session *s, uint64_t offset) {
  return offset == kMissingOffset ? nullptr : s->weights->arena + offset;
}

// One decode step as a sequence of kernels (engine 0).  Per layer:
//   QKV projection (residual add + RMSNorm fused in front)
//   q/k norm + RoPE + KV append, split-KV attention, merge
//   O projection
//   gate/up projection (residual add + RMSNorm in front, SwiGLU behind)
//   down projection
// then lm_head (final norm in front, arg-max partials behind) and the sampler.
// Same operator order as the reference step
// (hf_decode_sequence/session_decode_prefill.inc.cu:74-372).
// Fills the device tables of the whole-step kernel: one StepLayerDev per layer
// and the projection job list (QKV, O, gate/up, down per layer, then lm_head).
cudaError_t setup_step_kernel(Session *s) {
  const ModelDims &d = s->dims;
  const uint32_t qkv_rows32 = static_cast<uint32_t>(d.qkv_rows());
  s->row_elems = std::max(std::max(max_rows_per_block(qkv_rows32, 1, s->sm_count),
                                   max_rows_per_block(2u * d.intermediate, 2, s->sm_count)),
                          std::max(max_rows_per_block(d.hidden, 1, s->sm_count),
                                   max_rows_per_block(d.vocab, 1, s->sm_count)));
  s->step_kernel_ok = !s->has_moe && !d.mla() && step_kernel_supported(d.hidden, d.heads, d.kv_heads, d.head_dim,
                                                           d.intermediate, s->x_elems, s->row_elems);
  if (!s->step_kernel_ok) return cudaSuccess;
  cudaError_t err = configure_step_kernel();
  if (err != cudaSuccess) return err;
  const char *profile = getenv("NERVA_B200_PHASE_PROFILE");
  s->phase_profile = profile != nullptr && profile[0] == '1';
  err = cudaMemsetAsync(s->phase_cycles, 0, kPhaseCount * sizeof(unsigned long long), s->stream);
  if (err != cudaSuccess) return err;
  const uint64_t ah = d.attention_hidden(), qkv_rows = d.qkv_rows();
  std::vector<StepLayerDev> layers(d.layers);
  std::vector<JobDesc> jobs(static_cast<size_t>(d.layers) * 4u + 1u);
  for (uint32_t l = 0; l < d.layers; ++l) {
    const LayerLayout &L = s->layout.layers[l];
    StepLayerDev &o = layers[l];
    o.rms_attn = arena_at(s, L.rms_attn);
    o.rms_mlp = arena_at(s, L.rms_mlp);
    o.q_norm = arena_at(s, L.q_norm);
    o.k_norm = arena_at(s, L.k_norm);
    o.q_bias = arena_at(s, L.q_bias);
    o.k_bias = arena_at(s, L.k_bias);
    o.v_bias = arena_at(s, L.v_bias);
    o.o_bias = arena_at(s, L.o_bias);
    o.key_pages = s->kv_keys + l * s->kv_layer_elems;
    o.value_pages = s->kv_values + l * s->kv_layer_elems;
    jobs[4 * l + 0] = JobDesc{s->weights->qkv_packed + static_cast<uint64_t>(l) * qkv_rows * d.hidden,
                              static_cast<uint32_t>(qkv_rows), d.hidden, 1, 0};
    jobs[4 * l + 1] = JobDesc{arena_at(s, L.w_o), d.hidden, static_cast<uint32_t>(ah), 1, 0};
    jobs[4 * l + 2] = JobDesc{s->weights->gate_up_packed + gate_up_packed_offset(s, l),
                              2u * d.intermediate, d.hidden, 2, 0};
    jobs[4 * l + 3] = JobDesc{arena_at(s, L.w_down), d.hidden, d.intermediate, 1, 0};
  }
  jobs[4 * d.layers] = JobDesc{arena_at(s, s->layout.lm_head), d.vocab, d.hidden, 1, 0};
  for (const JobDesc &j : jobs) {
    if ((reinterpret_cast<uintptr_t>(j.weight) & 15u) != 0) s->step_kernel_ok = false;  // TMA source alignment
  }
  if (!s->step_kernel_ok) return cudaSuccess;
  err = cudaMemcpyAsync(s->step_layers, layers.data(), layers.size() * sizeof(StepLayerDev),
                        cudaMemcpyHostToDevice, s->stream);
  if (err == cudaSuccess)
    err = cudaMemcpyAsync(s->step_jobs, jobs.data(), jobs.size() * sizeof(JobDesc), cudaMemcpyHostToDevice,
                          s->stream);
  if (err == cudaSuccess) err = cudaStreamSynchronize(s->stream);  // the host vectors go out of scope
  return err;
}

// Attention items per query head in the whole-step kernel: one 32-token tile
// per warp per item where possible, at most kStepMaxSplits items.
uint32_t step_kernel_splits(uint32_t target_context) {
  const uint32_t per_item = kStreamWarps * kStepAttnTile;
  uint32_t s = (target_context + per_item - 1u) / per_item;
  if (s < 1) s = 1;
  if (s > kStepMaxSplits) s = kStepMaxSplits;
  return s;
}

cudaError_t enqueue_step_kernel(Session *s, uint32_t splits, uint32_t sample) {
  const ModelDims &d = s->dims;
  StepKernelParams p{};
  p.st = step_state(s);
  p.embeddings = arena_at(s, s->layout.embeddings);
  p.final_norm = arena_at(s, s->layout.final_norm);
  p.layers = s->step_layers;
  p.jobs = s->step_jobs;
  p.layer_count = d.layers;
  p.job_count = sample != 0 ? d.layers * 4u + 1u : d.layers * 4u;
  p.hidden = d.hidden;
  p.heads = d.heads;
  p.kv_heads = d.kv_heads;
  p.head_dim = d.head_dim;
  p.intermediate = d.intermediate;
  p.vocab = d.vocab;
  p.eps = s->rms_eps;
  p.rope_theta = s->rope_theta;
  p.page_table = s->page_table;
  p.page_count = s->kv_pages;
  p.h_a = s->h_a;
  p.h_b = s->h_b;
  p.qkv = s->qkv;
  p.o_out = s->o_out;
  p.down = s->down;
  p.logits = s->logits;
  p.ff_bf16 = s->ff_bf16;
  p.partial_acc = s->partial_acc;
  p.partial_m = s->partial_m;
  p.partial_l = s->partial_l;
  p.attn_splits = splits;
  p.best_value = s->best_value;
  p.best_index = s->best_index;
  p.barrier_counter = s->barrier_counter;
  p.sample = sample;
  p.x_elems = s->x_elems;
  p.row_elems = s->row_elems;
  p.phase_cycles = s->phase_profile ? s->phase_cycles : nullptr;
  return launch_step_kernel(s->stream, p, s->sm_count);
}

// Router logits of a sparse-MoE layer.  The expert kernels follow the reference's MoE arithmetic
// (unrounded fp32 activations); the router mat-vec does too, through the fp32 router kernel.

// Records the next profile event; the interval that ends here gets `bucket`.
static void profile_mark(Session *s, StepProfile *prof, uint32_t bucket) {
  if (prof == nullptr) return;
  if (prof->used >= prof->events.size()) {
    cudaEvent_t e = nullptr;
    if (cudaEventCreate(&e) != cudaSuccess) return;
    prof->events.push_back(e);
    prof->bucket.push_back(0);
  }
  cudaEventRecord(prof->events[prof->used], s->stream);
  if (prof->used > 0) prof->bucket[prof->used - 1] = bucket;
  prof->used += 1;
}

// head_only: the residual stream after the last layer is already in s->h_b (the chunked prefill
// left it there): only the final norm, lm_head and the sampler are enqueued.
cudaError_t enqueue_step(Session *s, uint32_t splits, uint32_t sample, uint64_t *launches,
                         StepProfile *prof = nullptr, bool head_only = false) {
  const ModelDims &d = s->dims;
  const StepState st = step_state(s);
  const uint64_t ah = d.attention_hidden();
  const uint64_t qkv_rows = d.qkv_rows();
  uint64_t n = 0;
  // tensor parallel: where the partial sums of O and down travel (see kernels.cuh: TpPush)
  // expert parallel uses the same exchange buffers for the sparse MLPs' partial outputs; every
  // other operator runs whole on every rank
  const bool ep_on = s->tp_world > 1 && d.ep_world > 1;
  const bool tp = s->tp_world > 1 && !ep_on;
  if ((tp || ep_on) && (!s->tp_attached || s->engine != 0)) return cudaErrorNotReady;
  const CommLayout comm = comm_layout(s->tp_world, d.hidden);
  // sparse layer number `ordinal` (counted from 0) exchanges through recv_d when even, recv_o when odd
  auto ep_buffer = [&](uint32_t layer) {
    uint32_t ordinal = 0;
    for (uint32_t i = 0; i < layer; ++i) ordinal += s->layout.layers[i].mlp_kind == NERVA_MLP_KIND_SPARSE_MOE ? 1u : 0u;
    return ordinal % 2u == 0 ? comm.recv_d : comm.recv_o;
  };
  auto sparse_layer = [&](uint32_t layer) { return s->layout.layers[layer].mlp_kind == NERVA_MLP_KIND_SPARSE_MOE; };
  auto push_to = [&](uint64_t recv, uint32_t exchange) {
    TpPush push{};
    push.world = s->tp_world;
    push.rank = s->tp_rank;
    for (uint32_t q = 0; q < s->tp_world; ++q) push.recv[q] = comm_at<unsigned long long>(s->comm_peers[q], recv);
    push.epoch = comm_at<unsigned long long>(s->comm_block, comm.epoch);
    push.per_epoch = d.layers;
    push.offset = exchange;
    return push;
  };
  auto gather_from = [&](uint64_t recv, uint32_t exchange) {
    TpGather gather{};
    gather.world = s->tp_world;
    gather.recv = comm_at<unsigned long long>(s->comm_block, recv);
    gather.reduced = comm_at<unsigned long long>(s->comm_block, recv == comm.recv_o ? comm.reduced_o : comm.reduced_d);
    gather.epoch = comm_at<unsigned long long>(s->comm_block, comm.epoch);
    gather.per_epoch = d.layers;
    gather.offset = exchange;
    gather.two_stage = s->tp_two_stage ? 1u : 0u;
    return gather;
  };
  auto stamps_for = [s](uint32_t node) -> unsigned long long * {
    return s->timeline_on && node < s->timeline_nodes ? s->timeline + node * kTimelineSlots : nullptr;
  };
  if (s->engine == 1 && prof == nullptr) {
    if (launches != nullptr) *launches = 1;
    if (sample == 2) return cudaErrorNotSupported;  // the one-kernel engine only has the arg-max sampler
    return enqueue_step_kernel(s, splits, sample);
  }
  // Dense single-GPU models without an O bias: O and down add the residual stream to their
  // own output (row by row, by the row's owner), so the next prologue reads one summed vector.
  // The sum is the same two-operand add the prologue would have done.
  bool fused_resid = !tp && !s->has_moe;
  for (const LayerLayout &L : s->layout.layers) fused_resid = fused_resid && arena_at(s, L.o_bias) == nullptr;
  profile_mark(s, prof, kBucketEmbed);
  cudaError_t err = cudaSuccess;
  if (!head_only) {
    err = launch_embed(s->stream, st, arena_at(s, s->layout.embeddings), d.hidden, s->h_b);
    n += 1;
  }
  profile_mark(s, prof, kBucketEmbed);
  for (uint32_t l = 0; !head_only && err == cudaSuccess && l < d.layers; ++l) {
    const LayerLayout &L = s->layout.layers[l];
    ProjectionParams p{};
    p.error_word = s->device_error;
    p.pdl = s->use_pdl ? 1u : 0u;
    p.eps = s->rms_eps;
    // QKV
    p.weight = s->weights->qkv_packed + static_cast<uint64_t>(l) * qkv_rows * d.hidden;
    p.rows = static_cast<uint32_t>(qkv_rows);
    p.cols = d.hidden;
    p.prologue = kPrologueAddNorm;
    p.x_bf16 = s->x_scratch;
    p.add_a = s->h_b;
    p.add_b = l == 0 || fused_resid ? nullptr : s->down;
    if (tp && l != 0) {
      p.add_b = s->down;  // placeholder: the sum arrives in the exchange buffer
      p.gather = gather_from(comm.recv_d, l);  // down of layer l-1 was exchange number l
    }
    if (ep_on && l != 0 && sparse_layer(l - 1u)) {
      p.add_b = s->down;  // placeholder: the ranks' partial MLP outputs arrive in the exchange buffer
      p.gather = gather_from(ep_buffer(l - 1u), l);
    }
    p.norm_weight = arena_at(s, L.rms_attn);
    p.resid_out = fused_resid ? nullptr : s->h_a;
    p.epilogue = kEpilogueStore;
    p.out_f32 = s->qkv;
    p.stamps = stamps_for(5u * l);
    err = launch_projection(s->stream, p, s->sm_count);
    n += 1;
    profile_mark(s, prof, kBucketQkv);
    if (err != cudaSuccess) break;

    if (d.mla()) {
      // latent attention: rotary + absorbed queries + cache append, split attention over the latent
      // cache, merge + value projection
      MlaParams mp{};
      mp.cursor = s->device_cursor;
      mp.max_context = s->max_context;
      mp.qkv = s->qkv;
      mp.w_kv_b = arena_at(s, L.w_v);
      mp.kv_a_norm = arena_at(s, L.k_norm);
      mp.cache = s->kv_keys + l * s->kv_layer_elems;
      mp.page_table = s->page_table;
      mp.page_count = s->kv_pages;
      mp.heads = d.heads;
      mp.rank = d.mla_rank;
      mp.nope = d.mla_nope;
      mp.rope = d.mla_rope;
      mp.v_dim = d.head_dim;
      mp.eps = s->rms_eps;
      mp.rope_theta = s->rope_theta;
      mp.ql = s->mla_ql;
      mp.partial_acc = s->partial_acc;
      mp.partial_m = s->partial_m;
      mp.partial_l = s->partial_l;
      mp.out_bf16 = s->attn_bf16;
      mp.error_word = s->device_error;
      err = launch_mla_attention(s->stream, mp, splits, s->use_pdl);
      n += 3;
      profile_mark(s, prof, kBucketAttention);
      if (err != cudaSuccess) break;
    } else {
    QkvPrepareParams qp{};
    qp.qkv = s->qkv;
    qp.q_bias = arena_at(s, L.q_bias);
    qp.k_bias = arena_at(s, L.k_bias);
    qp.v_bias = arena_at(s, L.v_bias);
    qp.q_norm = arena_at(s, L.q_norm);
    qp.k_norm = arena_at(s, L.k_norm);
    qp.heads = d.heads;
    qp.kv_heads = d.kv_heads;
    qp.head_dim = d.head_dim;
    qp.eps = s->rms_eps;
    qp.rope_theta = s->rope_theta;
    qp.key_pages = s->kv_keys + l * s->kv_layer_elems;
    qp.value_pages = s->kv_values + l * s->kv_layer_elems;
    qp.page_table = s->page_table;
    qp.page_count = s->kv_pages;
    if (s->fused_attention) {
      // q/k norm + RoPE + KV append + split attention + merge in one launch
      FusedAttentionParams fp{};
      fp.cursor = s->device_cursor;
      fp.max_context = s->max_context;
      fp.qkv = s->qkv;
      fp.q_bias = qp.q_bias;
      fp.k_bias = qp.k_bias;
      fp.v_bias = qp.v_bias;
      fp.q_norm = qp.q_norm;
      fp.k_norm = qp.k_norm;
      fp.key_pages = qp.key_pages;
      fp.value_pages = qp.value_pages;
      fp.page_table = s->page_table;
      fp.page_count = s->kv_pages;
      fp.heads = d.heads;
      fp.kv_heads = d.kv_heads;
      fp.head_dim = d.head_dim;
      fp.eps = s->rms_eps;
      fp.rope_theta = s->rope_theta;
      fp.splits = splits;
      fp.partial_acc = s->partial_acc;
      fp.partial_m = s->partial_m;
      fp.partial_l = s->partial_l;
      fp.tickets = s->attn_tickets;
      fp.out_bf16 = s->attn_bf16;
      fp.error_word = s->device_error;
      fp.pdl = s->use_pdl ? 1u : 0u;
      fp.stamps = stamps_for(5u * l + 1u);
      err = launch_fused_attention(s->stream, fp);
      n += 1;
      profile_mark(s, prof, kBucketAttention);
      if (err != cudaSuccess) break;
    } else {
    err = launch_qkv_prepare(s->stream, st, qp);
    n += 1;
    if (err != cudaSuccess) break;

    AttentionParams ap{};
    ap.q = s->qkv;
    ap.key_pages = qp.key_pages;
    ap.value_pages = qp.value_pages;
    ap.page_table = s->page_table;
    ap.batch = 1;
    ap.heads = d.heads;
    ap.kv_heads = d.kv_heads;
    ap.head_dim = d.head_dim;
    ap.page_count = s->kv_pages;
    ap.cursor = s->device_cursor;
    ap.splits = splits;
    ap.partial_acc = s->partial_acc;
    ap.partial_m = s->partial_m;
    ap.partial_l = s->partial_l;
    ap.out_bf16 = s->attn_bf16;
    ap.error_word = s->device_error;
    err = launch_attention(s->stream, ap);
    n += 2;
    profile_mark(s, prof, kBucketAttention);
    if (err != cudaSuccess) break;
    }
    }

    // O
    p = ProjectionParams{};
    p.error_word = s->device_error;
    p.pdl = s->use_pdl ? 1u : 0u;
    p.eps = s->rms_eps;
    p.weight = arena_at(s, L.w_o);
    p.rows = d.hidden;
    p.cols = static_cast<uint32_t>(ah);
    p.prologue = kProloguePlain;
    p.x_bf16 = s->attn_bf16;
    p.epilogue = kEpilogueStore;
    p.out_f32 = s->o_out;
    if (fused_resid) {
      p.resid_in = s->h_b;  // the stream that entered the layer
      p.out_f32 = s->h_a;   // the stream after attention
    }
    if (tp) p.push = push_to(comm.recv_o, l + 1u);
    p.stamps = stamps_for(5u * l + 2u);
    err = launch_projection(s->stream, p, s->sm_count);
    n += 1;
    profile_mark(s, prof, kBucketO);
    if (err != cudaSuccess) break;

    if (L.mlp_kind == NERVA_MLP_KIND_SPARSE_MOE) {
      MoeExpertParams ep{};
      ep.add_a = s->h_a;
      ep.add_b = s->o_out;
      ep.add_bias = arena_at(s, L.o_bias);
      ep.norm_weight = arena_at(s, L.rms_mlp);
      ep.eps = s->rms_eps;
      ep.hidden = d.hidden;
      ep.moe_intermediate = L.moe_intermediate;
      ep.shared_intermediate = L.shared_intermediate;
      ep.top_k = L.top_k;
      ep.w_expert_gate_up = arena_at(s, L.w_expert_gate_up);
      ep.expert_stride = L.expert_stride;
      ep.expert_up_offset = L.expert_up_offset;
      ep.w_expert_down = arena_at(s, L.w_expert_down);
      ep.w_shared_gate = arena_at(s, L.w_shared_gate);
      ep.w_shared_up = arena_at(s, L.w_shared_up);
      ep.w_shared_down = arena_at(s, L.w_shared_down);
      ep.w_shared_router = arena_at(s, L.w_shared_router);
      ep.w_router = arena_at(s, L.w_router);
      ep.num_experts = L.num_experts;
      ep.norm_topk_prob = L.norm_topk_prob;
      ep.resid_out = s->h_b;
      ep.expert_ids = s->route_ids;
      ep.route_weights = s->route_weights;
      ep.gate_up_out = s->moe_gate_up;
      ep.shared_gate = s->shared_gate;
      ep.out_f32 = s->down;
      ep.partial = s->moe_partial;
      ep.ticket = s->moe_ticket;
      ep.error_word = s->device_error;
      ep.expert_base = L.expert_base;
      ep.expert_local = L.expert_local;
      if (ep_on) ep.push = push_to(ep_buffer(l), l + 1u);
      // routing + gate/up, then down: two launches
      err = launch_moe_experts(s->stream, ep, s->sm_count, s->use_pdl);
      n += 2;
      profile_mark(s, prof, kBucketDown);
      continue;
    }

    // gate/up + SwiGLU
    p = ProjectionParams{};
    p.error_word = s->device_error;
    p.pdl = s->use_pdl ? 1u : 0u;
    p.eps = s->rms_eps;
    p.weight = s->weights->gate_up_packed + gate_up_packed_offset(s, l);
    p.rows = 2u * d.intermediate;
    p.cols = d.hidden;
    p.prologue = kPrologueAddNorm;
    p.x_bf16 = s->x_scratch;
    p.add_a = s->h_a;
    p.add_b = fused_resid ? nullptr : s->o_out;
    if (tp) {
      p.gather = gather_from(comm.recv_o, l + 1u);
    }
    p.add_bias = arena_at(s, L.o_bias);
    p.norm_weight = arena_at(s, L.rms_mlp);
    p.resid_out = fused_resid ? nullptr : s->h_b;
    p.epilogue = kEpilogueSwiglu;
    p.out_bf16 = s->ff_bf16;
    p.stamps = stamps_for(5u * l + 3u);
    err = launch_projection(s->stream, p, s->sm_count);
    n += 1;
    profile_mark(s, prof, kBucketGateUp);
    if (err != cudaSuccess) break;

    // down
    p = ProjectionParams{};
    p.error_word = s->device_error;
    p.pdl = s->use_pdl ? 1u : 0u;
    p.eps = s->rms_eps;
    p.weight = arena_at(s, L.w_down);
    p.rows = d.hidden;
    p.cols = d.intermediate;
    p.prologue = kProloguePlain;
    p.x_bf16 = s->ff_bf16;
    p.epilogue = kEpilogueStore;
    p.out_f32 = s->down;
    if (fused_resid) {
      p.resid_in = s->h_a;
      p.out_f32 = s->h_b;  // the stream that enters the next layer
    }
    if (tp) p.push = push_to(comm.recv_d, l + 1u);
    p.stamps = stamps_for(5u * l + 4u);
    err = launch_projection(s->stream, p, s->sm_count);
    n += 1;
    profile_mark(s, prof, kBucketDown);
  }
  uint32_t partials = 0;
  if (err == cudaSuccess && sample != 0) {
    ProjectionParams p{};
    p.error_word = s->device_error;
    p.pdl = s->use_pdl ? 1u : 0u;
    p.eps = s->rms_eps;
    p.weight = arena_at(s, s->layout.lm_head);
    p.rows = d.vocab;
    p.cols = d.hidden;
    p.prologue = kPrologueAddNorm;
    p.x_bf16 = s->x_scratch;
    p.add_a = s->h_b;
    p.add_b = fused_resid ? nullptr : s->down;
    if (tp) {
      p.gather = gather_from(comm.recv_d, d.layers);
    }
    if (ep_on && sparse_layer(d.layers - 1u)) p.gather = gather_from(ep_buffer(d.layers - 1u), d.layers);
    p.norm_weight = arena_at(s, s->layout.final_norm);
    p.resid_out = fused_resid ? nullptr : s->h_a;
    p.epilogue = kEpilogueArgmax;
    p.out_f32 = s->logits;
    p.best_value = s->best_value;
    p.best_index = s->best_index;
    p.stamps = stamps_for(5u * d.layers);
    partials = projection_blocks(p, s->sm_count);
    err = launch_projection(s->stream, p, s->sm_count);
    n += 1;
    profile_mark(s, prof, kBucketLmHead);
  }
  if (err == cudaSuccess && sample == 0 && !head_only) {
    // no head projection in this step: the last exchange of the layers is read here instead
    if (tp) {
      err = launch_exchange_wait(s->stream, gather_from(comm.recv_d, d.layers), d.hidden, s->device_error, s->use_pdl);
      n += 1;
    } else if (ep_on && sparse_layer(d.layers - 1u)) {
      err = launch_exchange_wait(s->stream, gather_from(ep_buffer(d.layers - 1u), d.layers), d.hidden, s->device_error,
                                 s->use_pdl);
      n += 1;
    }
  }
  if (err == cudaSuccess) {
    TpSample exchange{};
    if (ep_on) {
      // every rank holds the whole head and samples alone; the step counter still advances
      exchange.world = 1;
      exchange.epoch = comm_at<unsigned long long>(s->comm_block, comm.epoch);
    }
    if (tp) {
      exchange.world = s->tp_world;
      exchange.rank = s->tp_rank;
      exchange.vocab_offset = d.vocab_offset;
      exchange.epoch = comm_at<unsigned long long>(s->comm_block, comm.epoch);
      for (uint32_t q = 0; q < s->tp_world; ++q) {
        exchange.recv[q] = comm_at<unsigned long long>(s->comm_peers[q], comm.candidates);
        exchange.arrivals[q] = comm_at<unsigned long long>(s->comm_peers[q], comm.arrivals_s);
      }
    }
    if (sample == 2)
      err = launch_sample_general(s->stream, st, s->logits, s->device_sampler, s->use_pdl);
    else
      err = launch_sample_greedy(s->stream, st, s->best_value, s->best_index, partials, sample, s->use_pdl,
                                 tp || ep_on ? &exchange : nullptr);
    n += 1;
    profile_mark(s, prof, kBucketSampling);
  }
  if (launches != nullptr) *launches = n;
  return err;
}

// Graph cache: one instantiated graph per (attention split bucket, sampler kind, engine) —
// the role of the reference's cached graph key (hf_decode_sequence/session_graph_result.inc.cu:87-209).
// Prompt length, cursor and sampler parameters are read from device memory by the kernels, so a
// session that serves prompts of many lengths keeps a handful of graphs (split buckets x 3 sampler
// kinds x 2 engines at most), never one per request.
cudaError_t ensure_graph(Session *s, uint32_t splits, uint32_t sample, GraphEntry **out,
                         NervaCudaHfDecodeSequenceResult *res) {
  for (GraphEntry &g : s->graphs) {
    if (g.splits == splits && g.sample == sample && g.engine == s->engine) {
      *out = &g;
      if (res != nullptr) {
        res->graph_cache_hits += 1;
        res->graph_nodes = g.nodes;
      }
      return cudaSuccess;
    }
  }
  GraphEntry entry;
  entry.splits = splits;
  entry.sample = sample;
  entry.engine = s->engine;
  const char *no_graph = getenv("NERVA_B200_NO_GRAPH");
  if (no_graph != nullptr && no_graph[0] == '1') {
    // Profiling aid: replay the step as direct launches instead of a graph.
    entry.nodes = 0;
    s->graphs.push_back(entry);
    *out = &s->graphs.back();
    return cudaSuccess;
  }
  cudaError_t err = cudaStreamBeginCapture(s->stream, cudaStreamCaptureModeThreadLocal);
  if (err != cudaSuccess) return err;
  uint64_t launches = 0;
  err = enqueue_step(s, splits, sample, &launches);
  cudaGraph_t graph = nullptr;
  const cudaError_t end_err = cudaStreamEndCapture(s->stream, &graph);
  if (err == cudaSuccess) err = end_err;
  size_t nodes = 0;
  cudaGraphExec_t exec = nullptr;
  if (err == cudaSuccess) err = cudaGraphGetNodes(graph, nullptr, &nodes);
  if (err == cudaSuccess) err = cudaGraphInstantiate(&exec, graph, 0);
  if (err != cudaSuccess) {
    if (graph != nullptr) cudaGraphDestroy(graph);
    graph = nullptr;
    if (s->engine != 1) return err;
    // The whole-step kernel is a cooperative launch; where the runtime will not
    // put one into a graph the step is launched directly (one launch per token).
    cudaGetLastError();
    exec = nullptr;
    nodes = 2;
  }
  entry.graph = graph;
  entry.exec = exec;
  entry.nodes = nodes;
  s->graphs.push_back(entry);
  *out = &s->graphs.back();
  if (res != nullptr) {
    res->graph_captures += 1;
    res->graph_nodes = nodes;
  }
  return cudaSuccess;
}

// Attention split count for a launch that will see contexts up to `target`:
// bucketed to a power of two so that a growing context re-uses the graph.
cudaError_t replay(Session *s, GraphEntry *g) {
  if (g->exec != nullptr) return cudaGraphLaunch(g->exec, s->stream);
  return enqueue_step(s, g->splits, g->sample, nullptr);
}

// Tensor-parallel sessions: a failed exchange (a peer that died or fell behind its wait limit)
// sets the device error word.  Every kPeerCheckInterval replays a copy of that word to pinned
// host memory is queued, and the replay loops stop queueing once a copy shows a failure.  The
// host never waits for the copy, so the value it sees is up to one interval old; the kernels of
// the steps queued meanwhile skip their waits (common.cuh: step_already_failed).
constexpr uint32_t kPeerCheckInterval = 16;
bool peer_failure_seen(Session *s, uint32_t step) {
  if (s->tp_world <= 1) return false;
  if (*reinterpret_cast<volatile uint32_t *>(s->host_error) != 0) return true;
  if (step % kPeerCheckInterval == kPeerCheckInterval - 1u)
    cudaMemcpyAsync(s->host_error, s->device_error, sizeof(uint32_t), cudaMemcpyDeviceToHost, s->stream);
  return false;
}

uint32_t splits_for(Session *s, uint32_t target_context) {
  if (s->engine == 1) return step_kernel_splits(target_context);
  if (s->dims.mla()) return mla_attention_splits(target_context);
  if (s->fused_attention) return fused_attention_splits(target_context);
  uint32_t want = attention_default_splits(target_context, 1, s->dims.kv_heads, s->sm_count);
  uint32_t bucket = 1;
  while (bucket < want) bucket <<= 1;
  if (bucket > s->max_splits) bucket = s->max_splits;
  return bucket == 0 ? 1 : bucket;
}

void fill_header(const Session *s, NervaCudaHfDecodeSequenceResult *out, uint32_t steps,
                 uint32_t seed_token) {
  out->device_count = 1;
  out->dtype = s->dims.dtype;
  out->hidden = s->dims.hidden;
  out->heads = s->dims.heads;
  out->kv_heads = s->dims.kv_heads;
  out->head_dim = s->dims.head_dim;
  out->intermediate = s->dims.intermediate;
  out->vocab_size = s->dims.vocab;
  out->layer_count = s->dims.layers;
  out->steps = steps;
  out->seed_token = seed_token;
  out->resident_weight_bytes = s->resident_weight_bytes;
  out->planned_weight_blocks = s->planned_weight_blocks;
  out->planned_gpu_resident_blocks = s->planned_gpu_resident_blocks;
  out->planned_gpu_staged_blocks = s->planned_gpu_staged_blocks;
  out->planned_weight_bytes = s->planned_weight_bytes;
  out->planned_gpu_resident_weight_bytes = s->planned_gpu_resident_weight_bytes;
  out->planned_gpu_staged_weight_bytes = s->planned_gpu_staged_weight_bytes;
  out->planned_weight_descriptor_count = s->planned_weight_descriptor_count;
  out->planned_weight_descriptor_hash = s->planned_weight_descriptor_hash;
}

uint64_t resident_kv_bytes(const Session *s) {
  return (s->dims.mla() ? 1ull : 2ull) * s->dims.layers * s->kv_layer_elems * sizeof(uint16_t);
}
uint64_t device_footprint(const Session *s) {
  return s->state_bytes + (s->weights ? s->weights->block_bytes : 0);
}

int fail(NervaCudaHfDecodeSequenceResult *out, cudaError_t err) {
  out->status = -1;
  out->cuda_error = static_cast<int32_t>(err);
  set_last_error(cudaGetErrorString(err));
  return -1;
}

// Reads the device error word (after a synchronise).  Non-zero fails the call.
bool device_error_set(Session *s, NervaCudaHfDecodeSequenceResult *out) {
  if (*s->host_error == 0) return false;
  char text[96];
  snprintf(text, sizeof(text), "device kernel reported error code %u", *s->host_error);
  set_last_error(text);
  out->status = -1;
  out->cuda_error = static_cast<int32_t>(cudaErrorLaunchFailure);
  return true;
}

uint32_t observed_from_slots(uint32_t steps, uint32_t has_eos, uint32_t eos,
                             const NervaCudaSyntheticTokenSlot *slots) {
  for (uint32_t i = 0; i < steps; ++i) {
    if (slots[i].completion != 1u) return i;
    if (has_eos != 0 && slots[i].token == eos) return i + 1;
  }
  return steps;
}

bool slots_valid(const NervaCudaSyntheticTokenSlot *slots, uint32_t count, uint32_t first_index) {
  for (uint32_t i = 0; i < count; ++i) {
    if (slots[i].request_id != 1u || slots[i].sequence_id != 1u || slots[i].completion != 1u ||
        slots[i].token_index != static_cast<uint64_t>(first_index) + i)
      return false;
  }
  return true;
}

cudaError_t reset_request_state(Session *s, const uint32_t *prompt, uint32_t count,
                                NervaCudaHfDecodeSequenceResult *out) {
  cudaError_t err = cudaMemsetAsync(s->device_slots, 0, s->slots_bytes, s->stream);
  if (err == cudaSuccess) err = cudaMemsetAsync(s->device_cursor, 0, sizeof(uint32_t), s->stream);
  if (err == cudaSuccess) err = cudaMemsetAsync(s->device_error, 0, sizeof(uint32_t), s->stream);
  // completion counters are zero between launches; a request that failed half-way may have left one mid-count
  if (err == cudaSuccess) err = cudaMemsetAsync(s->moe_ticket, 0, 4 * sizeof(uint32_t), s->stream);
  if (err == cudaSuccess) err = cudaMemsetAsync(s->attn_tickets, 0, s->dims.heads * sizeof(uint32_t), s->stream);
  const uint64_t bytes = static_cast<uint64_t>(count) * sizeof(uint32_t);
  if (err == cudaSuccess)
    err = cudaMemcpyAsync(s->device_prompt, prompt, bytes, cudaMemcpyHostToDevice, s->stream);
  if (err == cudaSuccess)  // pageable source: staged before the call returns
    err = cudaMemcpyAsync(s->device_cursor + 1, &count, sizeof(uint32_t), cudaMemcpyHostToDevice, s->stream);
  out->h2d_bytes = bytes + sizeof(uint32_t);
  if (err == cudaSuccess && s->sample_kind == 2) {
    err = cudaMemcpyAsync(s->device_sampler, &s->host_sampler, sizeof(SamplerParams), cudaMemcpyHostToDevice,
                          s->stream);
    out->h2d_bytes += sizeof(SamplerParams);
  }
  s->logits_valid = false;
  *s->host_error = 0;  // nothing of this session is in flight when a request starts
  return err;
}

// Makes `config` the sampler of the request that is starting: normalised as the reference
// does (hf_decode_sequence/sampler.cu:420-432), arg-max when temperature is 0 or top_k is 1.
// The graphs read temperature, top-k, top-p and seed from device memory, so one captured
// graph serves every non-greedy configuration.
bool activate_sampler(Session *s, const NervaCudaHfDecodeSamplerConfig &config) {
  if (sampler_greedy(config)) {
    s->sample_kind = 1;
    return true;
  }
  if (s->tp_world > 1 || s->engine != 0) {
    set_last_error("temperature / top-k / top-p sampling needs engine 0 on one GPU");
    return false;
  }
  s->sample_kind = 2;
  s->host_sampler = SamplerParams{config.temperature, config.top_p, config.top_k, 0u, config.seed};
  return true;
}

}  // namespace

// ============================================================ C ABI ========

extern "C" const char *nerva_b200_last_error(void) { return g_last_error.c_str(); }

extern "C" int nerva_cuda_hf_decode_sequence_plan_layout(
    const NervaCudaHfDecodeSequenceLayoutPlanRequest *request,
    NervaCudaHfDecodeSequenceLayoutPlanResult *out) {
  if (out == nullptr) return -1;
  memset(out, 0, sizeof(*out));
  out->status = -1;
  if (request == nullptr || request->layers == nullptr || request->layer_count == 0 ||
      request->layer_index >= request->layer_count || request->hidden == 0 ||
      request->heads == 0 || request->kv_heads == 0 || request->head_dim == 0 ||
      request->intermediate == 0 || request->vocab_size == 0 ||
      request->kv_heads > request->heads || request->heads % request->kv_heads != 0)
    return -1;
  for (uint32_t i = 0; i < request->layer_count; ++i) {
    if (!valid_layer(request->layers[i], false)) return -1;
    if (request->layers[i].attention_kind != NERVA_ATTENTION_KIND_FULL) return -1;
  }
  ModelDims d;
  d.dtype = NERVA_DTYPE_BF16;
  d.hidden = request->hidden;
  d.heads = request->heads;
  d.kv_heads = request->kv_heads;
  d.head_dim = request->head_dim;
  d.intermediate = request->intermediate;
  d.vocab = request->vocab_size;
  d.layers = request->layer_count;
  const ArenaLayout layout = compute_arena_layout(d, request->layers);
  const LayerLayout &l = layout.layers[request->layer_index];
  out->status = 0;
  out->hidden = d.hidden;
  out->heads = d.heads;
  out->kv_heads = d.kv_heads;
  out->head_dim = d.head_dim;
  out->intermediate = d.intermediate;
  out->vocab_size = d.vocab;
  out->layer_count = d.layers;
  out->layer_index = request->layer_index;
  out->attention_kind = NERVA_ATTENTION_KIND_FULL;
  out->resident_weight_bytes = layout.elements * 2u - static_cast<uint64_t>(d.hidden) * 2u * 2u;
  out->layout_bytes = static_cast<uint64_t>(d.layers) * 688u;  // sizeof the reference's per-layer layout record
  out->final_norm = layout.final_norm;
  out->lm_head = layout.lm_head;
  out->rms_attn = l.rms_attn;
  out->rms_mlp = l.rms_mlp;
  out->w_q = l.w_q;
  out->q_norm = l.q_norm;
  out->w_k = l.w_k;
  out->k_norm = l.k_norm;
  out->w_v = l.w_v;
  out->w_o = l.w_o;
  out->w_router = l.w_router;
  out->w_expert_gate_up = l.w_expert_gate_up;
  out->w_expert_down = l.w_expert_down;
  out->w_shared_expert_gate = l.w_shared_gate;
  out->w_shared_expert_up = l.w_shared_up;
  out->w_shared_expert_down = l.w_shared_down;
  // The reference leaves every DeepSeek offset of a full-attention layer "missing".
  uint64_t *ds = &out->deepseek_q_a_scale;
  for (uint64_t *p = ds; p <= &out->deepseek_hc_ffn_scale; ++p) *p = kMissingOffset;
  return 0;
}

namespace {

struct UploadCounters {
  uint64_t h2d = 0, resident = 0, staged = 0;
};

cudaError_t copy_tensor(Session *s, uint64_t offset, const uint16_t *src, uint64_t elems,
                        UploadCounters *c) {
  if (offset == kMissingOffset || src == nullptr) return cudaSuccess;
  c->h2d += elems * 2u;
  return cudaMemcpyAsync(s->weights->arena + offset, src, elems * 2u, cudaMemcpyHostToDevice,
                         s->stream);
}

// Pointer mode: every tensor comes from a host pointer in the request
// (hf_decode_sequence/weights.cu:650-726).
cudaError_t upload_from_pointers(Session *s, const NervaCudaHfDecodeSequenceSessionCreateRequest *r,
                                 UploadCounters *c) {
  const ModelDims &d = s->dims;
  const uint64_t hidden = d.hidden, ah = d.attention_hidden(), kvh = d.kv_hidden();
  const uint64_t inter = d.intermediate;
  cudaError_t err = copy_tensor(s, s->layout.embeddings, r->embeddings, d.embed_vocab * hidden, c);
  for (uint32_t i = 0; err == cudaSuccess && i < d.layers; ++i) {
    const NervaCudaHfDecodeChainLayer &L = r->layers[i];
    const LayerLayout &o = s->layout.layers[i];
    struct Item { uint64_t off; const uint16_t *src; uint64_t n; } items[] = {
        {o.rms_attn, L.rms_attn_weight, hidden}, {o.w_q, L.w_q, ah * hidden},
        {o.q_norm, L.q_norm_weight, d.head_dim}, {o.w_k, L.w_k, kvh * hidden},
        {o.k_norm, L.k_norm_weight, d.head_dim}, {o.w_v, L.w_v, kvh * hidden},
        {o.w_o, L.w_o, hidden * ah},             {o.rms_mlp, L.rms_mlp_weight, hidden},
        {o.w_gate, L.w_gate, inter * hidden},    {o.w_up, L.w_up, inter * hidden},
        {o.w_down, L.w_down, hidden * inter},    {o.q_bias, L.q_bias, ah},
        {o.k_bias, L.k_bias, kvh},               {o.v_bias, L.v_bias, kvh},
        {o.o_bias, L.o_bias, hidden}};
    for (const Item &it : items) {
      if (err == cudaSuccess) err = copy_tensor(s, it.off, it.src, it.n, c);
    }
    if (L.mlp_kind == NERVA_MLP_KIND_SPARSE_MOE) {
      const uint64_t mi = L.moe_intermediate, e = L.num_experts, si = L.shared_expert_intermediate;
      const Item moe[] = {{o.w_router, L.w_router, e * hidden},
                          {o.w_expert_gate_up, L.w_expert_gate_up, e * 2u * mi * hidden},
                          {o.w_expert_down, L.w_expert_down, e * hidden * mi},
                          {o.w_shared_gate, L.w_shared_expert_gate, si * hidden},
                          {o.w_shared_up, L.w_shared_expert_up, si * hidden},
                          {o.w_shared_down, L.w_shared_expert_down, hidden * si},
                          {o.w_shared_router, L.w_shared_expert_router, hidden}};
      for (const Item &it : moe) {
        if (err == cudaSuccess && it.off != kMissingOffset) err = copy_tensor(s, it.off, it.src, it.n, c);
      }
    }
  }
  if (err == cudaSuccess) err = copy_tensor(s, s->layout.final_norm, r->final_norm_weight, hidden, c);
  if (err == cudaSuccess) err = copy_tensor(s, s->layout.lm_head, r->lm_head, d.vocab * hidden, c);
  return err;
}

// Descriptor mode: blocks are contiguous over the resident-weight byte space
// (the arena minus its input|scratch gap); each comes from host memory or from
// a byte range of a file, streamed through a pinned staging buffer
// (hf_decode_sequence/weights.cu:728-745,797-908).
cudaError_t upload_from_descriptors(Session *s,
                                    const NervaCudaHfDecodeSequenceSessionCreateRequest *r,
                                    UploadCounters *c) {
  const uint64_t embedding_bytes = static_cast<uint64_t>(s->dims.embed_vocab) * s->dims.hidden * 2u;
  const uint64_t gap_bytes = static_cast<uint64_t>(s->dims.hidden) * 2u * 2u;
  constexpr uint64_t kStagingBytes = 64ull << 20;
  uint8_t *staging = nullptr;
  cudaError_t err = cudaSuccess;
  uint8_t *arena_bytes = reinterpret_cast<uint8_t *>(s->weights->arena);
  for (uint32_t i = 0; err == cudaSuccess && i < r->planned_weight_descriptor_count; ++i) {
    const NervaCudaHfDecodeSequenceWeightBlock &b = r->planned_weight_descriptors[i];
    if (b.offset_bytes < embedding_bytes && b.offset_bytes + b.bytes > embedding_bytes) {
      set_last_error("weight block straddles the embedding boundary");
      err = cudaErrorInvalidValue;
      break;
    }
    const uint64_t dst = b.offset_bytes >= embedding_bytes ? b.offset_bytes + gap_bytes : b.offset_bytes;
    if (b.host_source != nullptr) {
      err = cudaMemcpyAsync(arena_bytes + dst, b.host_source, b.bytes, cudaMemcpyHostToDevice, s->stream);
    } else {
      std::string path(b.source_file, b.source_file_len);
      FILE *f = fopen(path.c_str(), "rb");
      if (f == nullptr) {
        set_last_error("cannot open weight file " + path);
        err = cudaErrorInvalidValue;
        break;
      }
      if (staging == nullptr) err = cudaMallocHost(&staging, kStagingBytes);
      uint64_t done = 0;
      if (err == cudaSuccess && fseek(f, static_cast<long>(b.file_offset_begin), SEEK_SET) != 0)
        err = cudaErrorInvalidValue;
      while (err == cudaSuccess && done < b.bytes) {
        const uint64_t n = std::min<uint64_t>(kStagingBytes, b.bytes - done);
        if (fread(staging, 1, n, f) != n) {
          set_last_error("short read from weight file " + path);
          err = cudaErrorInvalidValue;
          break;
        }
        err = cudaMemcpyAsync(arena_bytes + dst + done, staging, n, cudaMemcpyHostToDevice, s->stream);
        if (err == cudaSuccess) err = cudaStreamSynchronize(s->stream);  // staging is reused
        done += n;
      }
      fclose(f);
    }
    c->h2d += b.bytes;
    if (b.strategy == NERVA_WEIGHT_STRATEGY_GPU_RESIDENT) c->resident += b.bytes;
    else c->staged += b.bytes;
  }
  if (staging != nullptr) {
    cudaStreamSynchronize(s->stream);
    cudaFreeHost(staging);
  }
  return err;
}

// hf_decode_sequence/weights.cu:412-467
bool validate_descriptors(const NervaCudaHfDecodeSequenceSessionCreateRequest *r,
                          uint64_t resident_weight_bytes) {
  uint64_t cursor = 0, resident = 0, staged = 0;
  uint32_t resident_blocks = 0, staged_blocks = 0;
  for (uint32_t i = 0; i < r->planned_weight_descriptor_count; ++i) {
    const NervaCudaHfDecodeSequenceWeightBlock &b = r->planned_weight_descriptors[i];
    const bool has_source = b.host_source != nullptr || (b.source_file != nullptr && b.source_file_len != 0);
    if (b.bytes == 0 || b.reserved != 0 || !has_source || b.offset_bytes != cursor ||
        b.offset_bytes % 2u != 0 || b.bytes % 2u != 0)
      return false;
    if (cursor + b.bytes < cursor) return false;
    cursor += b.bytes;
    if (b.strategy == NERVA_WEIGHT_STRATEGY_GPU_RESIDENT) {
      resident_blocks += 1;
      resident += b.bytes;
    } else if (b.strategy == NERVA_WEIGHT_STRATEGY_GPU_STAGED) {
      staged_blocks += 1;
      staged += b.bytes;
    } else {
      return false;
    }
  }
  return cursor == resident_weight_bytes && cursor == r->planned_weight_bytes &&
         hash_weight_descriptors(r->planned_weight_descriptors, r->planned_weight_descriptor_count) ==
             r->planned_weight_descriptor_hash &&
         resident_blocks == r->planned_gpu_resident_blocks &&
         staged_blocks == r->planned_gpu_staged_blocks &&
         resident == r->planned_gpu_resident_weight_bytes &&
         staged == r->planned_gpu_staged_weight_bytes;
}

void fill_create_header(const NervaCudaHfDecodeSequenceSessionCreateRequest *r,
                        NervaCudaHfDecodeSequenceSessionCreateResult *out) {
  out->dtype = r->dtype;
  out->hidden = r->hidden;
  out->heads = r->heads;
  out->kv_heads = r->kv_heads;
  out->head_dim = r->head_dim;
  out->intermediate = r->intermediate;
  out->vocab_size = r->vocab_size;
  out->layer_count = r->layer_count;
  out->max_context_tokens = r->max_context_tokens;
  out->planned_weight_blocks = r->planned_weight_blocks;
  out->planned_gpu_resident_blocks = r->planned_gpu_resident_blocks;
  out->planned_gpu_staged_blocks = r->planned_gpu_staged_blocks;
  out->planned_weight_bytes = r->planned_weight_bytes;
  out->planned_gpu_resident_weight_bytes = r->planned_gpu_resident_weight_bytes;
  out->planned_gpu_staged_weight_bytes = r->planned_gpu_staged_weight_bytes;
  out->planned_weight_descriptor_count = r->planned_weight_descriptor_count;
  out->experimental_rt_decode_requested = r->experimental_rt_decode == 0 ? 0u : 1u;
  out->experimental_rt_mode = r->experimental_rt_mode;
  out->experimental_rt_page_tokens = r->experimental_rt_page_tokens;
  out->experimental_rt_pages = r->experimental_rt_pages;
  out->experimental_rt_local_window_tokens = r->experimental_rt_local_window_tokens;
  out->experimental_rt_sink_tokens = r->experimental_rt_sink_tokens;
}

int create_fail(Session *s, NervaCudaHfDecodeSequenceSessionCreateResult *out, cudaError_t err,
                int32_t stage) {
  out->status = -1;
  out->cuda_error = static_cast<int32_t>(err);
  out->failure_stage = stage;
  // a more specific text set just before the failure (file errors, layout errors) is kept
  if (err != cudaSuccess && g_last_error.empty()) set_last_error(cudaGetErrorString(err));
  destroy_session(s);
  return -1;
}

// Allocates and carves the private state of a session whose dims, max_context
// and sm_count are set.
cudaError_t allocate_state(Session *s, int32_t *stage) {
  StaticArena sizing(UINT64_MAX / 2);
  if (!plan_state(s, sizing, nullptr)) return cudaErrorMemoryAllocation;
  s->state_bytes = sizing.used();
  *stage = kStageDeviceScratchAlloc;
  cudaError_t err = cudaMalloc(&s->state_block, s->state_bytes);
  if (err != cudaSuccess) return err;
  s->state_arena = StaticArena(s->state_bytes);
  if (!plan_state(s, s->state_arena, s->state_block)) return cudaErrorMemoryAllocation;
  s->slots_bytes = static_cast<uint64_t>(s->max_context) * sizeof(NervaCudaSyntheticTokenSlot);
  *stage = kStageHostSlotsAlloc;
  err = cudaMallocHost(&s->host_slots, s->slots_bytes);
  if (err == cudaSuccess) err = cudaMallocHost(&s->host_error, sizeof(uint32_t));
  if (err != cudaSuccess) return err;
  *s->host_error = 0;
  *stage = kStageStreamCreate;
  err = cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking);
  if (err != cudaSuccess) return err;
  *stage = kStageStartEventCreate;
  err = cudaEventCreate(&s->ev_start);
  if (err != cudaSuccess) return err;
  *stage = kStageStopEventCreate;
  err = cudaEventCreate(&s->ev_stop);
  if (err != cudaSuccess) return err;
  // KV pages come out of the pool in FIFO order, which makes the initial
  // logical->physical table the identity, as the reference initialises it
  // (hf_decode_sequence/kernels.cu:732-739).
  StaticArena page_space(2ull * s->dims.layers * s->kv_layer_elems * 2u + 64u);
  const uint64_t page_bytes = NERVA_KV_CACHE_BLOCK_TOKENS * s->dims.kv_row() * 2u;
  if (!s->kv_pool.preallocate(page_space, s->kv_pages, NERVA_KV_CACHE_BLOCK_TOKENS, page_bytes, 16))
    return cudaErrorMemoryAllocation;
  std::vector<uint32_t> table(s->kv_pages);
  for (uint32_t i = 0; i < s->kv_pages; ++i) {
    const int64_t page = s->kv_pool.allocate_page(i * NERVA_KV_CACHE_BLOCK_TOKENS, 0, 0);
    if (page < 0) return cudaErrorMemoryAllocation;
    table[i] = static_cast<uint32_t>(page);
  }
  err = cudaMemcpyAsync(s->page_table, table.data(), table.size() * sizeof(uint32_t),
                        cudaMemcpyHostToDevice, s->stream);
  if (err == cudaSuccess) err = cudaMemsetAsync(s->device_error, 0, sizeof(uint32_t), s->stream);
  if (err == cudaSuccess) err = cudaMemsetAsync(s->device_cursor, 0, sizeof(uint32_t), s->stream);
  if (err == cudaSuccess)
    err = cudaMemsetAsync(s->attn_tickets, 0, s->dims.heads * sizeof(uint32_t), s->stream);
  if (err == cudaSuccess) err = cudaMemsetAsync(s->moe_ticket, 0, 4 * sizeof(uint32_t), s->stream);
  s->fused_attention = !s->dims.mla() && fused_attention_supported(s->dims.heads, s->dims.kv_heads, s->dims.head_dim);
  if (!s->dims.mla() && attention_rows_supported(s->dims.heads, s->dims.kv_heads, s->dims.head_dim)) {
    const uint64_t rows = static_cast<uint64_t>(s->dims.layers) * s->kv_pages * NERVA_KV_CACHE_BLOCK_TOKENS;
    s->kv_maps = encode_bf16_map_2d(&s->kv_map_k, s->kv_keys, s->dims.kv_hidden(), rows, 64, NERVA_KV_CACHE_BLOCK_TOKENS) &&
                 encode_bf16_map_2d(&s->kv_map_v, s->kv_values, s->dims.kv_hidden(), rows, 64, NERVA_KV_CACHE_BLOCK_TOKENS);
  }
  const char *timeline_env = getenv("NERVA_B200_TIMELINE");
  s->timeline_on = timeline_env != nullptr && timeline_env[0] == '1';
  if (err == cudaSuccess)
    err = cudaMemsetAsync(s->timeline, 0, static_cast<size_t>(s->timeline_nodes) * kTimelineSlots * 8u, s->stream);
  const char *pdl_env = getenv("NERVA_B200_PDL");
  s->use_pdl = !(pdl_env != nullptr && pdl_env[0] == '0');
  if (err == cudaSuccess) err = cudaStreamSynchronize(s->stream);
  return err;
}

}  // namespace

static int create_session(const NervaCudaHfDecodeSequenceSessionCreateRequest *request,
                          const NervaB200ShardInfo *shard,
                          NervaCudaHfDecodeSequenceSessionCreateResult *out,
                          NervaCudaHfDecodeSequenceSession **session_out) {
  if (out == nullptr) return -1;
  memset(out, 0, sizeof(*out));
  out->status = -1;
  if (session_out == nullptr) return -1;
  *session_out = nullptr;
  set_last_error("");
  // session_api_lifecycle.inc.cu:15-55 and weights.cu:232-340
  if (request == nullptr || request->layers == nullptr || request->layer_count == 0 ||
      request->hidden == 0 || request->heads == 0 || request->kv_heads == 0 ||
      request->head_dim == 0 || request->intermediate == 0 || request->vocab_size == 0 ||
      request->max_context_tokens == 0 || request->kv_heads > request->heads ||
      request->heads % request->kv_heads != 0 || request->dtype > NERVA_DTYPE_BF16 ||
      (request->rope_theta > 0.0f && request->head_dim % 2 != 0)) {
    out->failure_stage = kStageInvalidRequest;
    return -1;
  }
  const bool declared_plan = request->planned_weight_blocks != 0;
  if (!declared_plan && (request->embeddings == nullptr || request->final_norm_weight == nullptr ||
                         request->lm_head == nullptr)) {
    out->failure_stage = kStageInvalidRequest;
    return -1;
  }
  for (uint32_t i = 0; i < request->layer_count; ++i) {
    const NervaCudaHfDecodeChainLayer &layer = request->layers[i];
    if (!valid_layer(layer, !declared_plan) ||
        (layer.mlp_kind == NERVA_MLP_KIND_SPARSE_MOE &&
         (layer.moe_intermediate > request->intermediate ||
          layer.shared_expert_intermediate > request->intermediate))) {
      out->failure_stage = kStageInvalidRequest;
      return -1;
    }
  }
  if (declared_plan &&
      (request->planned_weight_bytes == 0 || request->planned_weight_descriptors == nullptr ||
       request->planned_weight_descriptor_count != request->planned_weight_blocks ||
       request->planned_weight_descriptor_hash == 0 ||
       request->planned_gpu_resident_blocks > request->planned_weight_blocks ||
       request->planned_gpu_staged_blocks >
           request->planned_weight_blocks - request->planned_gpu_resident_blocks ||
       request->planned_gpu_resident_weight_bytes > request->planned_weight_bytes ||
       request->planned_gpu_staged_weight_bytes >
           request->planned_weight_bytes - request->planned_gpu_resident_weight_bytes)) {
    out->failure_stage = kStageInvalidRequest;
    return -1;
  }
  fill_create_header(request, out);

  ModelDims d;
  d.dtype = request->dtype;
  d.hidden = request->hidden;
  d.heads = request->heads;
  d.kv_heads = request->kv_heads;
  d.head_dim = request->head_dim;
  d.intermediate = request->intermediate;
  d.vocab = request->vocab_size;
  d.layers = request->layer_count;
  d.embed_vocab = d.vocab;
  if (shard != nullptr) {
    // A tensor-parallel rank: the request describes this rank's shard (local heads,
    // KV heads, intermediate size and lm_head rows); the embedding table is whole.
    if ((shard->world != 2 && shard->world != 4 && shard->world != 8) || shard->rank >= shard->world ||
        shard->full_vocab < request->vocab_size ||
        static_cast<uint64_t>(shard->vocab_offset) + request->vocab_size > shard->full_vocab || shard->mode > 1u ||
        (shard->mode == 0u && request->planned_weight_blocks != 0)) {
      out->failure_stage = kStageInvalidRequest;
      return -1;
    }
    d.embed_vocab = shard->full_vocab;
    d.vocab_offset = shard->vocab_offset;
    if (shard->mode == 1u) {
      // An expert-parallel rank: the whole model except the routed experts (num_experts / world of
      // every sparse layer) and the shared expert (a slice of its intermediate dimension).  The
      // exchange alternates between two receive buffers from one sparse layer to the next, which
      // closes over a step boundary only for an even number of sparse layers.
      uint32_t sparse = 0;
      bool ok = shard->full_vocab == request->vocab_size && shard->vocab_offset == 0;
      for (uint32_t i = 0; ok && i < request->layer_count; ++i) {
        const NervaCudaHfDecodeChainLayer &layer = request->layers[i];
        if (layer.mlp_kind != NERVA_MLP_KIND_SPARSE_MOE) continue;
        sparse += 1;
        ok = layer.num_experts % shard->world == 0;
      }
      if (!ok || sparse == 0 || sparse % 2u != 0) {
        out->failure_stage = kStageInvalidRequest;
        return -1;
      }
      d.ep_world = shard->world;
      d.ep_rank = shard->rank;
    }
  }
  // Latent attention: every layer or none, one shape, value width = head_dim; its tensors have no
  // pointer fields in the layer struct, so they come through planned descriptors.
  uint32_t mla_layers = 0;
  for (uint32_t i = 0; i < request->layer_count; ++i) {
    const NervaCudaHfDecodeChainLayer &layer = request->layers[i];
    if (layer.attention_kind != NERVA_ATTENTION_KIND_DEEPSEEK_MLA) continue;
    mla_layers += 1;
    if (mla_layers == 1) {
      d.mla_rank = layer.deepseek_kv_lora_rank;
      d.mla_nope = layer.deepseek_qk_nope_head_dim;
      d.mla_rope = layer.deepseek_qk_rope_head_dim;
    }
    if (layer.deepseek_kv_lora_rank != d.mla_rank || layer.deepseek_qk_nope_head_dim != d.mla_nope ||
        layer.deepseek_qk_rope_head_dim != d.mla_rope || layer.deepseek_v_head_dim != d.head_dim || !declared_plan) {
      out->failure_stage = kStageInvalidRequest;
      return -1;
    }
  }
  if (mla_layers != 0 && (mla_layers != request->layer_count || (shard != nullptr && shard->mode != 1u))) {
    out->failure_stage = kStageInvalidRequest;
    return -1;
  }
  ArenaLayout layout = compute_arena_layout(d, request->layers);
  const uint64_t resident_weight_bytes = layout.elements * 2u - static_cast<uint64_t>(d.hidden) * 4u;
  out->resident_weight_bytes = resident_weight_bytes;
  if (declared_plan && (request->planned_weight_bytes != resident_weight_bytes ||
                        !validate_descriptors(request, resident_weight_bytes))) {
    out->failure_stage = kStageInvalidRequest;
    return -1;
  }
  if (declared_plan) out->planned_weight_descriptor_hash = request->planned_weight_descriptor_hash;

  // Device work starts here.
  int device_count = 0;
  cudaError_t err = cudaGetDeviceCount(&device_count);
  if (err != cudaSuccess || device_count == 0) {
    out->cuda_error = static_cast<int32_t>(err != cudaSuccess ? err : cudaErrorNoDevice);
    out->failure_stage = kStageGetDeviceCount;
    set_last_error("no CUDA device");
    cudaGetLastError();
    return -1;
  }
  out->device_count = device_count;
  // Shapes this library does not run are refused, never emulated.
  bool supported = request->dtype == NERVA_DTYPE_BF16 && request->head_dim <= 256;
  for (uint32_t i = 0; supported && i < request->layer_count; ++i)
    supported = layer_supported(request->layers[i]);
  if (!supported) {
    out->cuda_error = static_cast<int32_t>(cudaErrorNotSupported);
    out->failure_stage = kStageInvalidRequest;
    set_last_error("model not supported: needs bf16, full attention or plain bf16 latent attention without a "
                   "query low-rank stage, dense SwiGLU or softmax top-k sparse MoE, head_dim <= 256");
    return -1;
  }

  Session *s = new (std::nothrow) Session();
  if (s == nullptr) {
    out->cuda_error = static_cast<int32_t>(cudaErrorMemoryAllocation);
    out->failure_stage = kStageSessionAlloc;
    return -1;
  }
  s->dims = d;
  s->max_context = request->max_context_tokens;
  s->rms_eps = request->rms_eps;
  s->rope_theta = request->rope_theta;
  s->detailed_profile = request->detailed_profile;
  s->layout = layout;
  s->resident_weight_bytes = resident_weight_bytes;
  s->planned_weight_blocks = request->planned_weight_blocks;
  s->planned_gpu_resident_blocks = request->planned_gpu_resident_blocks;
  s->planned_gpu_staged_blocks = request->planned_gpu_staged_blocks;
  s->planned_weight_bytes = request->planned_weight_bytes;
  s->planned_gpu_resident_weight_bytes = request->planned_gpu_resident_weight_bytes;
  s->planned_gpu_staged_weight_bytes = request->planned_gpu_staged_weight_bytes;
  s->planned_weight_descriptor_count = request->planned_weight_descriptor_count;
  s->planned_weight_descriptor_hash = declared_plan ? request->planned_weight_descriptor_hash : 0;
  s->layer_meta.assign(request->layers, request->layers + request->layer_count);
  int32_t dense_count = 0;
  for (const LayerLayout &L : s->layout.layers)
    s->dense_ordinal.push_back(L.mlp_kind == NERVA_MLP_KIND_DENSE ? dense_count++ : -1);
  if (shard != nullptr) {
    s->tp_world = shard->world;
    s->tp_rank = shard->rank;
    // NERVA_B200_TWO_STAGE_GATHER=1: two ranks take the gather of four and eight (each block adds the
    // ranks for its slice, then every block reads the sums), so that path can run where two GPUs are
    const char *two_stage = getenv("NERVA_B200_TWO_STAGE_GATHER");
    s->tp_two_stage = two_stage != nullptr && two_stage[0] == '1';
  }

  int device = 0;
  err = cudaGetDevice(&device);
  cudaDeviceProp prop{};
  if (err == cudaSuccess) err = cudaGetDeviceProperties(&prop, device);
  if (err != cudaSuccess) return create_fail(s, out, err, kStageSetDevice);
  s->sm_count = static_cast<uint32_t>(prop.multiProcessorCount);
  out->device_memory_bandwidth_bps =
      static_cast<uint64_t>(prop.memoryClockRate) * 1000ull * (static_cast<uint64_t>(prop.memoryBusWidth) / 8ull);
  err = configure_projection_kernels();
  if (err == cudaSuccess) err = configure_attention_kernels();
  if (err == cudaSuccess) err = configure_fused_attention_kernel();
  if (err == cudaSuccess) err = configure_moe_kernels();
  if (err == cudaSuccess) err = configure_mla_kernels();
  if (err != cudaSuccess) return create_fail(s, out, err, kStageSetDevice);
  if (d.mla() && !mla_session_supported(d.heads, d.mla_rank, d.mla_nope, d.mla_rope, d.head_dim)) {
    set_last_error("latent attention shape not supported: needs at most 16 heads, latent rank 128, 256 or 512, "
                   "rotary width a multiple of 8 up to 64");
    return create_fail(s, out, cudaErrorNotSupported, kStageInvalidRequest);
  }
  for (const LayerLayout &L : s->layout.layers) {
    if (L.mlp_kind != NERVA_MLP_KIND_SPARSE_MOE) continue;
    s->has_moe = true;
    if ((shard != nullptr && shard->mode != 1u) || !moe_supported(d.hidden, L.moe_intermediate, L.shared_intermediate, L.num_experts, L.top_k,
                                           s->sm_count)) {
      set_last_error("sparse MoE layer not supported: needs hidden and intermediate sizes that are multiples of 8, "
                     "at most 256 experts and 16 per token; several GPUs only as expert parallel");
      return create_fail(s, out, cudaErrorNotSupported, kStageInvalidRequest);
    }
  }

  // shared weights: one allocation
  s->weights = std::make_shared<SharedWeights>();
  {
    StaticArena sizing(UINT64_MAX / 2);
    plan_weights(s, sizing, nullptr, nullptr);
    s->weights->block_bytes = sizing.used();
    err = cudaMalloc(&s->weights->block, s->weights->block_bytes);
    if (err != cudaSuccess) return create_fail(s, out, err, kStageDeviceArenaAlloc);
    s->weight_arena = StaticArena(s->weights->block_bytes);
    plan_weights(s, s->weight_arena, s->weights->block, s->weights.get());
  }
  int32_t stage = kStageDeviceScratchAlloc;
  err = allocate_state(s, &stage);
  if (err != cudaSuccess) return create_fail(s, out, err, stage);
  if (s->tp_world > 1) {
    err = allocate_comm(s);
    if (err != cudaSuccess) return create_fail(s, out, err, kStageDeviceScratchAlloc);
  }
  if (block_step_supported(s)) {
    err = allocate_block_workspace(s);
    if (err != cudaSuccess) return create_fail(s, out, err, kStageDeviceScratchAlloc);
  }

  UploadCounters counters;
  err = declared_plan ? upload_from_descriptors(s, request, &counters)
                      : upload_from_pointers(s, request, &counters);
  if (err != cudaSuccess) return create_fail(s, out, err, kStageDescriptorCopy);
  // packed replicas
  const uint64_t ah = d.attention_hidden(), kvh = d.kv_hidden();
  const uint64_t qkv_rows = d.qkv_rows();
  for (uint32_t l = 0; err == cudaSuccess && l < d.layers; ++l) {
    const LayerLayout &L = s->layout.layers[l];
    uint16_t *packed = s->weights->qkv_packed + l * qkv_rows * d.hidden;
    if (d.mla()) {
      // [query projection; latent + rotary-key projection]: one launch streams both
      err = cudaMemcpyAsync(packed, arena_at(s, L.w_q), d.mla_q_rows() * d.hidden * 2u, cudaMemcpyDeviceToDevice,
                            s->stream);
      if (err == cudaSuccess)
        err = cudaMemcpyAsync(packed + d.mla_q_rows() * d.hidden, arena_at(s, L.w_k), d.mla_width() * d.hidden * 2u,
                              cudaMemcpyDeviceToDevice, s->stream);
    } else {
      err = launch_pack_qkv(s->stream, arena_at(s, L.w_q), arena_at(s, L.w_k), arena_at(s, L.w_v), packed,
                            ah * d.hidden, kvh * d.hidden);
    }
    if (err == cudaSuccess && L.mlp_kind == NERVA_MLP_KIND_DENSE)
      err = launch_pack_gate_up(s->stream, arena_at(s, L.w_gate), arena_at(s, L.w_up),
                                s->weights->gate_up_packed + gate_up_packed_offset(s, l), d.intermediate, d.hidden);
  }
  if (err == cudaSuccess) err = setup_step_kernel(s);
  if (err != cudaSuccess) return create_fail(s, out, err, kStagePackReplicas);
  err = cudaStreamSynchronize(s->stream);
  if (err != cudaSuccess) return create_fail(s, out, err, kStageSetupSynchronize);

  out->descriptor_gpu_resident_h2d_bytes = counters.resident;
  out->descriptor_gpu_staged_h2d_bytes = counters.staged;
  out->h2d_bytes = counters.h2d;
  out->sync_calls = 2;
  out->resident_kv_bytes = resident_kv_bytes(s);
  out->device_arena_bytes = device_footprint(s);
  out->pinned_host_bytes = s->slots_bytes;
  out->head_threads = 128;
  // chunk of the block prefill; 1 when the prompt is pushed through the decode step token by token
  out->prefill_chunk_tokens = s->weights->block_ws.block != nullptr ? s->weights->block_ws.max_rows : 1;
  out->hot_path_allocations = 0;
  out->status = 0;
  *session_out = s;
  return 0;
}

extern "C" int nerva_cuda_hf_decode_sequence_session_create(
    const NervaCudaHfDecodeSequenceSessionCreateRequest *request,
    NervaCudaHfDecodeSequenceSessionCreateResult *out,
    NervaCudaHfDecodeSequenceSession **session_out) {
  return create_session(request, nullptr, out, session_out);
}

extern "C" int nerva_b200_session_create_sharded(
    const NervaCudaHfDecodeSequenceSessionCreateRequest *request, const NervaB200ShardInfo *shard,
    NervaCudaHfDecodeSequenceSessionCreateResult *out, NervaCudaHfDecodeSequenceSession **session_out) {
  if (shard == nullptr) {
    if (out != nullptr) {
      memset(out, 0, sizeof(*out));
      out->status = -1;
      out->failure_stage = kStageInvalidRequest;
    }
    return -1;
  }
  return create_session(request, shard, out, session_out);
}

// The 64-byte inter-process handle of this rank's exchange buffer.
extern "C" int nerva_b200_session_comm_handle(Session *s, uint8_t *handle, uint32_t capacity) {
  if (s == nullptr || handle == nullptr || capacity < sizeof(cudaIpcMemHandle_t) || s->comm_block == nullptr)
    return -1;
  cudaIpcMemHandle_t h;
  const cudaError_t err = cudaIpcGetMemHandle(&h, s->comm_block);
  if (err != cudaSuccess) {
    set_last_error(cudaGetErrorString(err));
    return -1;
  }
  memcpy(handle, &h, sizeof(h));
  return static_cast<int>(sizeof(h));
}

// handles: world x 64 bytes, in rank order (this rank's own entry is ignored).
extern "C" int nerva_b200_session_attach_peers(Session *s, const uint8_t *handles, uint32_t world) {
  if (s == nullptr || handles == nullptr || world != s->tp_world || s->comm_block == nullptr || s->tp_attached)
    return -1;
  for (uint32_t q = 0; q < world; ++q) {
    if (q == s->tp_rank) {
      s->comm_peers[q] = s->comm_block;
      continue;
    }
    cudaIpcMemHandle_t h;
    memcpy(&h, handles + static_cast<size_t>(q) * sizeof(h), sizeof(h));
    void *mapped = nullptr;
    const cudaError_t err = cudaIpcOpenMemHandle(&mapped, h, cudaIpcMemLazyEnablePeerAccess);
    if (err != cudaSuccess) {
      set_last_error(std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(err));
      return -1;
    }
    s->comm_peers[q] = mapped;
  }
  s->tp_attached = true;
  return 0;
}

extern "C" int nerva_b200_session_attach_loopback(Session *s) {
  if (s == nullptr || s->tp_world <= 1 || s->comm_block == nullptr || s->tp_attached) return -1;
  for (uint32_t q = 0; q < s->tp_world; ++q) s->comm_peers[q] = s->comm_block;  // destroy skips own pointers
  s->tp_attached = true;
  return 0;
}

// session_api_batch_fork_destroy.inc.cu:716-732: `out` (nullable) receives the
// session's identity one last time.
extern "C" int nerva_cuda_hf_decode_sequence_session_destroy(
    Session *session, NervaCudaHfDecodeSequenceSessionCreateResult *out) {
  if (out != nullptr) {
    memset(out, 0, sizeof(*out));
    out->status = -1;
  }
  if (session == nullptr) return -1;
  if (out != nullptr) {
    out->device_count = 1;
    out->dtype = session->dims.dtype;
    out->hidden = session->dims.hidden;
    out->heads = session->dims.heads;
    out->kv_heads = session->dims.kv_heads;
    out->head_dim = session->dims.head_dim;
    out->intermediate = session->dims.intermediate;
    out->vocab_size = session->dims.vocab;
    out->layer_count = session->dims.layers;
    out->max_context_tokens = session->max_context;
    out->resident_weight_bytes = session->resident_weight_bytes;
    out->resident_kv_bytes = resident_kv_bytes(session);
    out->device_arena_bytes = device_footprint(session);
    out->pinned_host_bytes = session->slots_bytes;
    out->status = 0;
  }
  destroy_session(session);
  return 0;
}

extern "C" int nerva_b200_session_read_timeline(Session *s, uint64_t *stamps, uint32_t capacity) {
  if (s == nullptr || stamps == nullptr || !s->timeline_on) return -1;
  const uint32_t count = s->timeline_nodes * kTimelineSlots;
  if (capacity < count) return -1;
  cudaError_t err = cudaStreamSynchronize(s->stream);
  if (err == cudaSuccess) err = cudaMemcpy(stamps, s->timeline, static_cast<size_t>(count) * 8u, cudaMemcpyDeviceToHost);
  if (err != cudaSuccess) {
    set_last_error(cudaGetErrorString(err));
    return -1;
  }
  return static_cast<int>(count);
}

extern "C" int nerva_b200_session_set_engine(Session *s, uint32_t engine) {
  if (s == nullptr || engine > 1 || s->started) return -1;
  if (engine == 1 && s->tp_world > 1) {
    set_last_error("the whole-step kernel has no tensor-parallel exchange");
    return -1;
  }
  if (engine == 1 && !s->step_kernel_ok) {
    set_last_error("whole-step kernel needs head_dim 64 or 128, dims that are multiples of 8, and "
                   "an activation vector that fits beside the weight ring in shared memory");
    return -1;
  }
  s->engine = engine;
  return 0;
}

extern "C" int nerva_cuda_hf_decode_sequence_session_start(
    const NervaCudaHfDecodeSequenceSessionStartRequest *request,
    NervaCudaHfDecodeSequenceResult *out) {
  if (out == nullptr) return -1;
  memset(out, 0, sizeof(*out));
  out->status = -1;
  if (request == nullptr || request->session == nullptr || request->prompt_tokens == nullptr ||
      request->prompt_token_count == 0 || !sampler_valid(request->sampler))
    return -1;
  Session *s = request->session;
  if (request->prompt_token_count > s->max_context) return -1;
  for (uint32_t i = 0; i < request->prompt_token_count; ++i) {
    if (request->prompt_tokens[i] >= s->dims.embed_vocab) return -1;
  }
  fill_header(s, out, 0, request->prompt_tokens[request->prompt_token_count - 1u]);
  if (!activate_sampler(s, request->sampler)) {
    out->cuda_error = static_cast<int32_t>(cudaErrorNotSupported);
    return -1;
  }
  s->prompt_count = request->prompt_token_count;
  s->started = false;
  cudaError_t err = reset_request_state(s, request->prompt_tokens, request->prompt_token_count, out);
  const uint32_t splits = splits_for(s, s->prompt_count);
  // NERVA_B200_PREFILL=decode keeps the token-by-token prefill on models that have the block path
  // (comparison runs); read per call.
  const char *prefill_env = getenv("NERVA_B200_PREFILL");
  const bool chunked = s->weights->block_ws.block != nullptr && s->engine == 0 && s->prompt_count > 1 &&
                       !(prefill_env != nullptr && prefill_env[0] == 'd');
  if (chunked) {
    // Chunked prefill: up to block_ws.max_rows prompt positions through every layer at a time
    // (block projections on the tensor pipe, paged K/V published per chunk), then the head for the
    // last position (session_decode_prefill.inc.cu:1879-2245 is the reference's counterpart).
    if (err == cudaSuccess) err = cudaEventRecord(s->ev_start, s->stream);
    uint64_t launches = 0;
    if (err == cudaSuccess) err = enqueue_chunked_prefill(s, s->prompt_count, s->sample_kind, &launches);
    const uint32_t last = s->prompt_count - 1u;
    if (err == cudaSuccess)  // the head samples at the cursor: the last prompt position
      err = cudaMemcpyAsync(s->device_cursor, &last, sizeof(uint32_t), cudaMemcpyHostToDevice, s->stream);
    uint64_t head_launches = 0;
    if (err == cudaSuccess) err = enqueue_step(s, splits, s->sample_kind, &head_launches, nullptr, true);
    out->kernel_launches += launches + head_launches;
  } else {
  // Prefill by decode: prompt_count - 1 steps without sampling, then one with
  // (the reference's serial prefill, session_decode_prefill.inc.cu:2245-2297).
  GraphEntry *quiet = nullptr, *sampled = nullptr;
  if (err == cudaSuccess && s->prompt_count > 1) err = ensure_graph(s, splits, 0, &quiet, out);
  if (err == cudaSuccess) err = ensure_graph(s, splits, s->sample_kind, &sampled, out);
  if (err == cudaSuccess) err = cudaEventRecord(s->ev_start, s->stream);
  for (uint32_t i = 0; err == cudaSuccess && i + 1 < s->prompt_count; ++i) {
    if (peer_failure_seen(s, i)) break;
    err = replay(s, quiet);
    out->graph_replays += 1;
    out->graph_launches += 1;
    out->kernel_launches += quiet->nodes;
  }
  if (err == cudaSuccess) {
    err = replay(s, sampled);
    out->graph_replays += 1;
    out->graph_launches += 1;
    out->kernel_launches += sampled->nodes;
  }
  }
  if (err == cudaSuccess) err = cudaEventRecord(s->ev_stop, s->stream);
  if (err == cudaSuccess)
    err = cudaMemcpyAsync(s->host_error, s->device_error, sizeof(uint32_t), cudaMemcpyDeviceToHost, s->stream);
  if (err == cudaSuccess) {
    err = cudaStreamSynchronize(s->stream);
    out->sync_calls += 1;
    out->d2h_bytes += sizeof(uint32_t);
  }
  if (err != cudaSuccess) return fail(out, err);
  if (device_error_set(s, out)) return -1;
  float ms = 0.0f;
  if (cudaEventElapsedTime(&ms, s->ev_start, s->ev_stop) == cudaSuccess && ms > 0.0f)
    out->device_elapsed_ns = static_cast<uint64_t>(ms * 1.0e6f);
  s->has_eos = request->has_eos_token;
  s->eos_token = request->eos_token;
  s->seed_token = request->prompt_tokens[request->prompt_token_count - 1u];
  s->observed = 0;
  s->cursor = s->prompt_count;
  s->started = true;
  s->finished = false;
  s->logits_valid = true;
  out->resident_kv_bytes = resident_kv_bytes(s);
  out->kv_tokens = s->prompt_count;
  out->device_arena_bytes = device_footprint(s);
  out->pinned_host_bytes = s->slots_bytes;
  out->hot_path_allocations = s->hot_path_allocations;
  out->status = 0;
  return 0;
}

extern "C" int nerva_cuda_hf_decode_sequence_session_advance(
    const NervaCudaHfDecodeSequenceSessionAdvanceRequest *request,
    NervaCudaHfDecodeSequenceResult *out) {
  if (out == nullptr) return -1;
  memset(out, 0, sizeof(*out));
  out->status = -1;
  if (request == nullptr || request->session == nullptr || request->output_tokens == nullptr ||
      request->steps == 0 || request->output_token_capacity < request->steps)
    return -1;
  Session *s = request->session;
  if (!s->started || s->finished || s->prompt_count == 0) return -1;
  // session_api_lifecycle.inc.cu:1137-1153
  const uint32_t slot_start = s->prompt_count - 1u + s->observed;
  const uint64_t target64 = static_cast<uint64_t>(s->prompt_count) + s->observed + request->steps - 1u;
  if (target64 > s->max_context || target64 < s->cursor) return -1;
  const uint32_t target = static_cast<uint32_t>(target64);
  const uint32_t run_count = target - s->cursor;
  const uint32_t seed = s->observed == 0 ? s->seed_token : s->host_slots[slot_start - 1u].token;
  fill_header(s, out, request->steps, seed);

  cudaError_t err = cudaSuccess;
  GraphEntry *graph = nullptr;
  if (run_count != 0) err = ensure_graph(s, splits_for(s, target), s->sample_kind, &graph, out);
  if (err == cudaSuccess && run_count != 0) err = cudaEventRecord(s->ev_start, s->stream);
  for (uint32_t step = 0; err == cudaSuccess && step < run_count; ++step) {
    if (peer_failure_seen(s, step)) break;
    err = replay(s, graph);  // the hot loop: one graph launch per token, nothing else
    if (err != cudaSuccess) break;
    out->graph_replays += 1;
    out->graph_launches += 1;
    out->kernel_launches += graph->nodes;
    if (s->has_eos != 0) {
      // Stop launching once the stop token has been produced
      // (session_api_lifecycle.inc.cu:1217-1234).
      const uint32_t position = s->cursor + step;
      err = cudaStreamSynchronize(s->stream);
      out->sync_calls += 1;
      if (err == cudaSuccess)
        err = cudaMemcpy(&s->host_slots[position], &s->device_slots[position],
                         sizeof(NervaCudaSyntheticTokenSlot), cudaMemcpyDeviceToHost);
      out->d2h_bytes += sizeof(NervaCudaSyntheticTokenSlot);
      if (err == cudaSuccess && s->host_slots[position].completion == 1u &&
          s->host_slots[position].token == s->eos_token)
        break;
    }
  }
  if (err == cudaSuccess && run_count != 0) err = cudaEventRecord(s->ev_stop, s->stream);
  const uint64_t bytes = static_cast<uint64_t>(request->steps) * sizeof(NervaCudaSyntheticTokenSlot);
  if (err == cudaSuccess)
    err = cudaMemcpyAsync(s->host_slots + slot_start, s->device_slots + slot_start, bytes,
                          cudaMemcpyDeviceToHost, s->stream);
  if (err == cudaSuccess)
    err = cudaMemcpyAsync(s->host_error, s->device_error, sizeof(uint32_t), cudaMemcpyDeviceToHost, s->stream);
  out->d2h_bytes += bytes + sizeof(uint32_t);
  if (err == cudaSuccess) {
    err = cudaStreamSynchronize(s->stream);
    out->sync_calls += 1;
  }
  if (err != cudaSuccess) return fail(out, err);
  if (device_error_set(s, out)) return -1;
  if (run_count != 0) {
    float ms = 0.0f;
    if (cudaEventElapsedTime(&ms, s->ev_start, s->ev_stop) == cudaSuccess && ms > 0.0f) {
      out->device_elapsed_ns = static_cast<uint64_t>(ms * 1.0e6f);
      if (out->device_elapsed_ns == 0) out->device_elapsed_ns = 1;
    }
    s->logits_valid = true;
  }
  const NervaCudaSyntheticTokenSlot *slots = s->host_slots + slot_start;
  out->observed_tokens = observed_from_slots(request->steps, s->has_eos, s->eos_token, slots);
  for (uint32_t i = 0; i < out->observed_tokens; ++i) request->output_tokens[i] = slots[i].token;
  out->last_token = out->observed_tokens == 0 ? 0 : request->output_tokens[out->observed_tokens - 1];
  out->observed_token_hash = hash_tokens(request->output_tokens, out->observed_tokens);
  out->resident_kv_bytes = resident_kv_bytes(s);
  out->kv_tokens = static_cast<uint64_t>(slot_start) + out->observed_tokens;
  out->device_arena_bytes = device_footprint(s);
  out->pinned_host_bytes = s->slots_bytes;
  out->host_causality_edges = 0;
  out->hot_path_allocations = s->hot_path_allocations;
  out->status = out->observed_tokens > 0 && slots_valid(slots, out->observed_tokens, slot_start) ? 0 : -1;
  if (out->status == 0) {
    s->observed += out->observed_tokens;
    s->cursor = out->observed_tokens < request->steps ? s->max_context : target;
    s->finished = out->observed_tokens < request->steps || out->kv_tokens >= s->max_context;
  }
  return out->status == 0 ? 0 : -1;
}

extern "C" int nerva_cuda_hf_decode_sequence_session_run(
    const NervaCudaHfDecodeSequenceSessionRunRequest *request,
    NervaCudaHfDecodeSequenceResult *out) {
  if (out == nullptr) return -1;
  memset(out, 0, sizeof(*out));
  out->status = -1;
  if (request == nullptr || request->session == nullptr || request->prompt_tokens == nullptr ||
      request->output_tokens == nullptr || request->steps == 0 ||
      request->prompt_token_count == 0 || request->output_token_capacity < request->steps ||
      request->prompt_tokens[request->prompt_token_count - 1u] != request->seed_token ||
      !sampler_valid(request->sampler) ||
      request->prompt_token_count > UINT32_MAX - request->steps + 1u)
    return -1;
  Session *s = request->session;
  const uint32_t context_steps = request->prompt_token_count + request->steps - 1u;
  if (context_steps > s->max_context) return -1;
  for (uint32_t i = 0; i < request->prompt_token_count; ++i) {
    if (request->prompt_tokens[i] >= s->dims.embed_vocab) return -1;
  }
  fill_header(s, out, request->steps, request->seed_token);
  if (!activate_sampler(s, request->sampler)) {
    out->cuda_error = static_cast<int32_t>(cudaErrorNotSupported);
    return -1;
  }
  s->prompt_count = request->prompt_token_count;
  s->started = false;
  cudaError_t err = reset_request_state(s, request->prompt_tokens, request->prompt_token_count, out);
  GraphEntry *graph = nullptr;
  const char *prefill_env = getenv("NERVA_B200_PREFILL");
  const bool chunked = s->weights->block_ws.block != nullptr && s->engine == 0 && s->prompt_count > 1 &&
                       !(prefill_env != nullptr && prefill_env[0] == 'd');
  if (err == cudaSuccess) err = ensure_graph(s, splits_for(s, context_steps), s->sample_kind, &graph, out);
  if (err == cudaSuccess) err = cudaEventRecord(s->ev_start, s->stream);
  uint32_t first_step = 0;
  if (chunked) {
    // The prompt goes through the chunked prefill, exactly as session_start runs it, so that
    // run == start + advance bit for bit; the decode steps follow.
    uint64_t launches = 0, head_launches = 0;
    if (err == cudaSuccess) err = enqueue_chunked_prefill(s, s->prompt_count, s->sample_kind, &launches);
    const uint32_t last = s->prompt_count - 1u;
    if (err == cudaSuccess)
      err = cudaMemcpyAsync(s->device_cursor, &last, sizeof(uint32_t), cudaMemcpyHostToDevice, s->stream);
    if (err == cudaSuccess)
      err = enqueue_step(s, splits_for(s, s->prompt_count), s->sample_kind, &head_launches, nullptr, true);
    out->kernel_launches += launches + head_launches;
    first_step = s->prompt_count;
  }
  // One sampling graph replayed for every (remaining) position; samples at prompt positions are
  // never read (session_api_lifecycle.inc.cu:849-920).
  for (uint32_t step = first_step; err == cudaSuccess && step < context_steps; ++step) {
    if (peer_failure_seen(s, step)) break;
    err = replay(s, graph);
    if (err == cudaSuccess) {
      out->graph_replays += 1;
      out->graph_launches += 1;
      out->kernel_launches += graph->nodes;
    }
  }
  if (err == cudaSuccess) err = cudaEventRecord(s->ev_stop, s->stream);
  const uint64_t bytes = static_cast<uint64_t>(context_steps) * sizeof(NervaCudaSyntheticTokenSlot);
  if (err == cudaSuccess)
    err = cudaMemcpyAsync(s->host_slots, s->device_slots, bytes, cudaMemcpyDeviceToHost, s->stream);
  if (err == cudaSuccess)
    err = cudaMemcpyAsync(s->host_error, s->device_error, sizeof(uint32_t), cudaMemcpyDeviceToHost, s->stream);
  out->d2h_bytes = bytes + sizeof(uint32_t);
  if (err == cudaSuccess) {
    err = cudaStreamSynchronize(s->stream);
    out->sync_calls += 1;
  }
  if (err != cudaSuccess) return fail(out, err);
  if (device_error_set(s, out)) return -1;
  float ms = 0.0f;
  if (cudaEventElapsedTime(&ms, s->ev_start, s->ev_stop) == cudaSuccess && ms > 0.0f)
    out->device_elapsed_ns = static_cast<uint64_t>(ms * 1.0e6f);
  s->logits_valid = true;
  const uint32_t output_start = request->prompt_token_count - 1u;
  const NervaCudaSyntheticTokenSlot *slots = s->host_slots + output_start;
  out->observed_tokens = observed_from_slots(request->steps, request->has_eos_token, request->eos_token, slots);
  for (uint32_t i = 0; i < out->observed_tokens; ++i) request->output_tokens[i] = slots[i].token;
  out->last_token = out->observed_tokens == 0 ? 0 : request->output_tokens[out->observed_tokens - 1];
  out->observed_token_hash = hash_tokens(request->output_tokens, out->observed_tokens);
  out->resident_kv_bytes = resident_kv_bytes(s);
  out->kv_tokens = static_cast<uint64_t>(output_start) + out->observed_tokens;
  out->device_arena_bytes = device_footprint(s);
  out->pinned_host_bytes = s->slots_bytes;
  out->hot_path_allocations = s->hot_path_allocations;
  out->status = out->observed_tokens > 0 && slots_valid(slots, out->observed_tokens, output_start) ? 0 : -1;
  return out->status == 0 ? 0 : -1;
}

// Clones an active session's KV cache, token ring, cursor and request state;
// the device weights are shared (session_api_batch_fork_destroy.inc.cu:311+).
// One token for a block of sessions that share weights (reference:
// hf_decode_sequence/session_api_batch_fork_destroy.inc.cu:1-309; selection, reasons, state
// updates and result fields follow it).
extern "C" int nerva_cuda_hf_decode_sequence_batch_advance_one(
    const NervaCudaHfDecodeSequenceBatchAdvanceRequest *request,
    NervaCudaHfDecodeSequenceBatchAdvanceResult *out) {
  constexpr uint32_t kReady = 0, kInvalidRequest = 1, kNoSessions = 2, kNoReadySessions = 3,
                     kSharedWeightsUnproven = 4, kInsufficientCompatibleReady = 5;
  constexpr uint32_t kWorkspaceTokens = 32;  // hf_decode_sequence/types.cuh:63
  if (out == nullptr) return -1;
  memset(out, 0, sizeof(*out));
  out->status = -1;
  out->reason = kInvalidRequest;
  if (request == nullptr) return -1;
  out->requested_session_count = request->session_count;
  out->target_block_tokens = request->target_block_tokens == 0 ? 1u : request->target_block_tokens;
  out->min_block_tokens = request->min_block_tokens == 0 ? 1u : request->min_block_tokens;
  if (request->session_count == 0) {
    out->reason = kNoSessions;
    out->status = 0;
    return 0;
  }
  if (request->sessions == nullptr || request->output_tokens == nullptr ||
      request->output_token_capacity < request->session_count)
    return -1;
  cudaError_t err = cudaGetDeviceCount(&out->device_count);
  if (err != cudaSuccess) {
    out->cuda_error = static_cast<int32_t>(err);
    return -1;
  }
  auto ready = [](const Session *s) {
    if (s == nullptr || !s->started || s->finished || s->prompt_count == 0 || s->cursor >= s->max_context)
      return false;
    // dense full-attention models whose heads span the hidden size (session_common.inc.cu:1078-1090),
    // on the per-kernel engine of one GPU
    if (s->dims.hidden < 128 || s->dims.heads * s->dims.head_dim != s->dims.hidden || s->has_moe ||
        s->tp_world > 1 || s->engine != 0)
      return false;
    return s->prompt_count + s->observed == s->cursor + 1u;
  };
  auto same_model = [](const Session *a, const Session *b) {
    return a->planned_weight_descriptor_hash != 0 &&
           a->planned_weight_descriptor_hash == b->planned_weight_descriptor_hash &&
           a->dims.dtype == b->dims.dtype && a->dims.hidden == b->dims.hidden && a->dims.heads == b->dims.heads &&
           a->dims.kv_heads == b->dims.kv_heads && a->dims.head_dim == b->dims.head_dim &&
           a->dims.intermediate == b->dims.intermediate && a->dims.vocab == b->dims.vocab &&
           a->dims.layers == b->dims.layers && a->weights == b->weights;
  };
  uint32_t ready_count = 0;
  bool any_hash = false;
  for (uint32_t i = 0; i < request->session_count; ++i) {
    const Session *s = request->sessions[i];
    if (!ready(s)) continue;
    ready_count += 1;
    any_hash = any_hash || s->planned_weight_descriptor_hash != 0;
  }
  if (ready_count == 0 || !any_hash) {
    out->reason = ready_count == 0 ? kNoReadySessions : kSharedWeightsUnproven;
    out->status = 0;
    return 0;
  }
  const Session *best = nullptr;
  uint32_t best_count = 0;
  for (uint32_t i = 0; i < request->session_count; ++i) {
    const Session *candidate = request->sessions[i];
    if (!ready(candidate) || candidate->planned_weight_descriptor_hash == 0) continue;
    uint32_t compatible = 0;
    for (uint32_t j = 0; j < request->session_count; ++j) {
      if (ready(request->sessions[j]) && same_model(candidate, request->sessions[j])) compatible += 1;
    }
    if (compatible > best_count) {
      best = candidate;
      best_count = compatible;
    }
  }
  out->eligible_session_count = best_count;
  std::vector<uint32_t> selected;
  const uint32_t max_block = std::min(out->target_block_tokens, kWorkspaceTokens);
  for (uint32_t i = 0; best != nullptr && i < request->session_count && selected.size() < max_block; ++i) {
    if (ready(request->sessions[i]) && same_model(best, request->sessions[i])) selected.push_back(i);
  }
  if (best == nullptr || best_count < out->min_block_tokens || selected.size() < out->min_block_tokens) {
    out->reason = kInsufficientCompatibleReady;
    out->status = 0;
    return 0;
  }
  for (size_t a = 0; a < selected.size(); ++a) {  // a handle listed twice would be stepped twice
    for (size_t b = a + 1; b < selected.size(); ++b) {
      if (request->sessions[selected[a]] == request->sessions[selected[b]]) return -1;
    }
  }
  out->reason = kReady;
  out->exact = 1;
  out->block_tokens = static_cast<uint32_t>(selected.size());
  out->dtype = best->dims.dtype;
  out->layer_count = best->dims.layers;

  // Packed block step: the selected sessions' tokens go through every projection together, so the
  // weights are streamed once for the block (the reference: one cublasLtMatmul per projection,
  // session_api_batch_fork_destroy.inc.cu:1-310).  Models without the block path (sparse MoE,
  // biases, odd widths) and blocks of one replay the sessions' own captured steps side by side.
  bool packed = selected.size() >= 2 && selected.size() <= kBlockSampleRows;
  for (uint32_t index : selected) {
    const Session *s = request->sessions[index];
    packed = packed && s->weights->block_ws.block != nullptr && s->sample_kind == 1 && s->engine == 0;
  }
  if (packed) {
    std::vector<Session *> block;
    for (uint32_t index : selected) block.push_back(request->sessions[index]);
    cudaStream_t stream = block[0]->stream;
    for (Session *s : block) {  // idle sessions: this only orders their earlier work before the block's
      if (err == cudaSuccess) err = cudaStreamSynchronize(s->stream);
      out->sync_calls += 1;
    }
    uint64_t launches = 0;
    if (err == cudaSuccess) err = enqueue_block_decode(block.data(), static_cast<uint32_t>(block.size()), stream, &launches);
    for (Session *s : block) {
      const uint32_t slot = s->prompt_count - 1u + s->observed;
      if (err == cudaSuccess)
        err = cudaMemcpyAsync(s->host_slots + slot, s->device_slots + slot, sizeof(NervaCudaSyntheticTokenSlot),
                              cudaMemcpyDeviceToHost, stream);
      if (err == cudaSuccess)
        err = cudaMemcpyAsync(s->host_error, s->device_error, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream);
      out->d2h_bytes += sizeof(NervaCudaSyntheticTokenSlot);
      out->sampling_kernel_launches += 1;
    }
    out->projection_kernel_launches += 4ull * block[0]->dims.layers + 1u;
    const cudaError_t sync = cudaStreamSynchronize(stream);
    out->sync_calls += 1;
    if (err == cudaSuccess) err = sync;
  } else {
  // Launch every session's step before waiting for any of them.
  for (uint32_t index : selected) {
    Session *s = request->sessions[index];
    GraphEntry *graph = nullptr;
    err = ensure_graph(s, splits_for(s, s->cursor + 1u), s->sample_kind, &graph, nullptr);
    if (err == cudaSuccess) err = replay(s, graph);
    const uint32_t slot = s->prompt_count - 1u + s->observed;
    if (err == cudaSuccess)
      err = cudaMemcpyAsync(s->host_slots + slot, s->device_slots + slot, sizeof(NervaCudaSyntheticTokenSlot),
                            cudaMemcpyDeviceToHost, s->stream);
    if (err == cudaSuccess)
      err = cudaMemcpyAsync(s->host_error, s->device_error, sizeof(uint32_t), cudaMemcpyDeviceToHost, s->stream);
    if (err != cudaSuccess) break;
    out->d2h_bytes += sizeof(NervaCudaSyntheticTokenSlot);
    out->projection_kernel_launches += 4ull * s->dims.layers + 1u;
    out->sampling_kernel_launches += 1;
  }
  for (uint32_t index : selected) {  // also after a failed launch: nothing stays in flight
    const cudaError_t sync = cudaStreamSynchronize(request->sessions[index]->stream);
    out->sync_calls += 1;
    if (err == cudaSuccess) err = sync;
  }
  }
  if (err != cudaSuccess) {
    set_last_error(cudaGetErrorString(err));
    out->cuda_error = static_cast<int32_t>(err);
    out->exact = 0;
    return -1;
  }
  std::vector<uint32_t> observed;
  for (uint32_t index : selected) {
    Session *s = request->sessions[index];
    out->hot_path_allocations += s->hot_path_allocations;
    const uint32_t slot_start = s->prompt_count - 1u + s->observed;
    const NervaCudaSyntheticTokenSlot &slot = s->host_slots[slot_start];
    if (*s->host_error != 0 || !slots_valid(&slot, 1, slot_start)) {
      out->status = -1;
      return -1;
    }
    request->output_tokens[index] = slot.token;
    observed.push_back(slot.token);
    out->last_token = slot.token;
    s->observed += 1;
    s->cursor += 1;
    s->logits_valid = true;
    s->finished = (s->has_eos != 0 && slot.token == s->eos_token) || slot_start + 1u >= s->max_context;
  }
  out->observed_tokens = static_cast<uint32_t>(observed.size());
  out->observed_token_hash = hash_tokens(observed.data(), out->observed_tokens);
  out->status = out->observed_tokens == out->block_tokens ? 0 : -1;
  return out->status == 0 ? 0 : -1;
}

extern "C" int nerva_cuda_hf_decode_sequence_session_fork_shared_weights(
    const NervaCudaHfDecodeSequenceSessionForkSharedWeightsRequest *request,
    NervaCudaHfDecodeSequenceSessionCreateResult *out,
    NervaCudaHfDecodeSequenceSession **session_out) {
  if (out == nullptr) return -1;
  memset(out, 0, sizeof(*out));
  out->status = -1;
  if (session_out == nullptr) return -1;
  *session_out = nullptr;
  if (request == nullptr || request->parent == nullptr) {
    out->failure_stage = kStageInvalidRequest;
    return -1;
  }
  set_last_error("");
  Session *parent = request->parent;
  if (parent->tp_world > 1) {
    // A tensor-parallel rank's step needs the exchange buffers of all ranks; a fork would need
    // its own set on every rank, which this entry point cannot arrange.
    out->cuda_error = static_cast<int32_t>(cudaErrorNotSupported);
    out->failure_stage = kStageInvalidRequest;
    set_last_error("a tensor-parallel session cannot be forked");
    return -1;
  }
  Session *s = new (std::nothrow) Session();
  if (s == nullptr) {
    out->cuda_error = static_cast<int32_t>(cudaErrorMemoryAllocation);
    out->failure_stage = kStageSessionAlloc;
    return -1;
  }
  s->dims = parent->dims;
  s->max_context = parent->max_context;
  s->rms_eps = parent->rms_eps;
  s->rope_theta = parent->rope_theta;
  s->sm_count = parent->sm_count;
  s->engine = parent->engine;
  s->detailed_profile = request->detailed_profile;
  s->layout = parent->layout;
  s->layer_meta = parent->layer_meta;
  s->has_moe = parent->has_moe;
  s->dense_ordinal = parent->dense_ordinal;
  s->resident_weight_bytes = parent->resident_weight_bytes;
  s->planned_weight_blocks = parent->planned_weight_blocks;
  s->planned_gpu_resident_blocks = parent->planned_gpu_resident_blocks;
  s->planned_gpu_staged_blocks = parent->planned_gpu_staged_blocks;
  s->planned_weight_bytes = parent->planned_weight_bytes;
  s->planned_gpu_resident_weight_bytes = parent->planned_gpu_resident_weight_bytes;
  s->planned_gpu_staged_weight_bytes = parent->planned_gpu_staged_weight_bytes;
  s->planned_weight_descriptor_count = parent->planned_weight_descriptor_count;
  s->planned_weight_descriptor_hash = parent->planned_weight_descriptor_hash;
  s->weights = parent->weights;
  int32_t stage = kStageDeviceScratchAlloc;
  cudaError_t err = allocate_state(s, &stage);
  if (err != cudaSuccess) return create_fail(s, out, err, stage);
  // The two state blocks have the same carve-up, so one copy clones KV, page
  // table, ring, prompt and cursor.
  err = cudaStreamSynchronize(parent->stream);
  if (err == cudaSuccess)
    err = cudaMemcpyAsync(s->state_block, parent->state_block, s->state_bytes, cudaMemcpyDeviceToDevice, s->stream);
  if (err == cudaSuccess) err = cudaStreamSynchronize(s->stream);
  if (err != cudaSuccess) return create_fail(s, out, err, kStageSetupSynchronize);
  // the copied layer table points at the parent's KV pages: rebuild it for this session
  err = setup_step_kernel(s);
  if (err != cudaSuccess) return create_fail(s, out, err, kStageSetupSynchronize);
  memcpy(s->host_slots, parent->host_slots, s->slots_bytes);
  s->started = parent->started;
  s->finished = parent->finished;
  s->prompt_count = parent->prompt_count;
  s->has_eos = parent->has_eos;
  s->eos_token = parent->eos_token;
  s->seed_token = parent->seed_token;
  s->observed = parent->observed;
  s->cursor = parent->cursor;
  s->logits_valid = parent->logits_valid;
  s->sample_kind = parent->sample_kind;  // the parameters themselves came with the state block
  s->host_sampler = parent->host_sampler;
  out->device_count = 1;
  out->dtype = s->dims.dtype;
  out->hidden = s->dims.hidden;
  out->heads = s->dims.heads;
  out->kv_heads = s->dims.kv_heads;
  out->head_dim = s->dims.head_dim;
  out->intermediate = s->dims.intermediate;
  out->vocab_size = s->dims.vocab;
  out->layer_count = s->dims.layers;
  out->max_context_tokens = s->max_context;
  out->resident_weight_bytes = s->resident_weight_bytes;
  out->resident_kv_bytes = resident_kv_bytes(s);
  out->device_arena_bytes = device_footprint(s);
  out->pinned_host_bytes = s->slots_bytes;
  out->head_threads = 128;
  out->prefill_chunk_tokens = 1;
  out->sync_calls = 2;
  out->status = 0;
  *session_out = s;
  return 0;
}

// One-shot: create, run, destroy (session_api_oneshot.inc.cu).
extern "C" int nerva_cuda_hf_decode_sequence_u16(const NervaCudaHfDecodeSequenceRequest *request,
                                                 NervaCudaHfDecodeSequenceResult *out) {
  if (out == nullptr) return -1;
  memset(out, 0, sizeof(*out));
  out->status = -1;
  // weights.cu:232-262
  if (request == nullptr || request->layers == nullptr || request->output_tokens == nullptr ||
      request->prompt_tokens == nullptr || request->output_token_capacity < request->steps ||
      request->layer_count == 0 || request->steps == 0 || request->prompt_token_count == 0 ||
      request->vocab_size == 0 || request->seed_token >= request->vocab_size ||
      !sampler_valid(request->sampler) ||
      request->prompt_token_count > UINT32_MAX - request->steps + 1u)
    return -1;
  for (uint32_t i = 0; i < request->prompt_token_count; ++i) {
    if (request->prompt_tokens[i] >= request->vocab_size) return -1;
  }
  if (request->prompt_tokens[request->prompt_token_count - 1u] != request->seed_token) return -1;
  NervaCudaHfDecodeSequenceSessionCreateRequest create{};
  create.dtype = request->dtype;
  create.hidden = request->hidden;
  create.heads = request->heads;
  create.kv_heads = request->kv_heads;
  create.head_dim = request->head_dim;
  create.intermediate = request->intermediate;
  create.vocab_size = request->vocab_size;
  create.layer_count = request->layer_count;
  create.max_context_tokens = request->prompt_token_count + request->steps - 1u;
  create.rms_eps = request->rms_eps;
  create.rope_theta = request->rope_theta;
  create.embeddings = request->embeddings;
  create.layers = request->layers;
  create.final_norm_weight = request->final_norm_weight;
  create.lm_head = request->lm_head;
  create.planned_weight_blocks = request->planned_weight_blocks;
  create.planned_gpu_resident_blocks = request->planned_gpu_resident_blocks;
  create.planned_gpu_staged_blocks = request->planned_gpu_staged_blocks;
  create.planned_weight_bytes = request->planned_weight_bytes;
  create.planned_gpu_resident_weight_bytes = request->planned_gpu_resident_weight_bytes;
  create.planned_gpu_staged_weight_bytes = request->planned_gpu_staged_weight_bytes;
  create.planned_weight_descriptors = request->planned_weight_descriptors;
  create.planned_weight_descriptor_count = request->planned_weight_descriptor_count;
  create.planned_weight_descriptor_hash = request->planned_weight_descriptor_hash;
  Session *s = nullptr;
  NervaCudaHfDecodeSequenceSessionCreateResult created{};
  if (nerva_cuda_hf_decode_sequence_session_create(&create, &created, &s) != 0) {
    out->cuda_error = created.cuda_error;
    out->device_count = created.device_count;
    return -1;
  }
  NervaCudaHfDecodeSequenceSessionRunRequest run{};
  run.session = s;
  run.steps = request->steps;
  run.seed_token = request->seed_token;
  run.prompt_tokens = request->prompt_tokens;
  run.prompt_token_count = request->prompt_token_count;
  run.has_eos_token = request->has_eos_token;
  run.eos_token = request->eos_token;
  run.output_tokens = request->output_tokens;
  run.output_token_capacity = request->output_token_capacity;
  run.sampler = request->sampler;
  const int rc = nerva_cuda_hf_decode_sequence_session_run(&run, out);
  out->h2d_bytes += created.h2d_bytes;
  out->descriptor_gpu_resident_h2d_bytes = created.descriptor_gpu_resident_h2d_bytes;
  out->descriptor_gpu_staged_h2d_bytes = created.descriptor_gpu_staged_h2d_bytes;
  destroy_session(s);
  return rc;
}

// ------------------------------------------------------- additive exports ----

extern "C" int nerva_b200_session_read_logits(Session *s, float *logits, uint32_t capacity) {
  if (s == nullptr || logits == nullptr || capacity < s->dims.vocab || !s->logits_valid) return -1;
  if (cudaStreamSynchronize(s->stream) != cudaSuccess) return -1;
  return cudaMemcpy(logits, s->logits, static_cast<uint64_t>(s->dims.vocab) * 4u, cudaMemcpyDeviceToHost) ==
                 cudaSuccess
             ? 0
             : -1;
}

extern "C" int nerva_b200_session_set_kv_block_table(Session *s, const uint32_t *table,
                                                     uint32_t page_count) {
  if (s == nullptr || table == nullptr || page_count != s->kv_pages || s->started) return -1;
  std::vector<uint8_t> seen(page_count, 0);
  for (uint32_t i = 0; i < page_count; ++i) {
    if (table[i] >= page_count || seen[table[i]]) return -1;  // must be a permutation
    seen[table[i]] = 1;
  }
  if (cudaMemcpy(s->page_table, table, static_cast<uint64_t>(page_count) * 4u, cudaMemcpyHostToDevice) !=
      cudaSuccess)
    return -1;
  return 0;
}

extern "C" int nerva_b200_session_get_kv_block_table(Session *s, uint32_t *table, uint32_t capacity) {
  if (s == nullptr || table == nullptr || capacity < s->kv_pages) return -1;
  if (cudaStreamSynchronize(s->stream) != cudaSuccess) return -1;
  return cudaMemcpy(table, s->page_table, static_cast<uint64_t>(s->kv_pages) * 4u, cudaMemcpyDeviceToHost) ==
                 cudaSuccess
             ? static_cast<int>(s->kv_pages)
             : -1;
}

extern "C" int nerva_b200_session_read_kv_row(Session *s, uint32_t layer, uint32_t token,
                                              uint32_t which, uint16_t *row, uint32_t capacity) {
  if (s == nullptr || row == nullptr || layer >= s->dims.layers || token >= s->max_context ||
      which > 1 || capacity < s->dims.kv_row() || (which == 1 && s->dims.mla()))
    return -1;
  if (cudaStreamSynchronize(s->stream) != cudaSuccess) return -1;
  uint32_t physical = 0;
  if (cudaMemcpy(&physical, s->page_table + token / NERVA_KV_CACHE_BLOCK_TOKENS, 4, cudaMemcpyDeviceToHost) !=
      cudaSuccess)
    return -1;
  // hf_decode_sequence/types.cuh:328-337
  const uint64_t offset = ((static_cast<uint64_t>(layer) * s->kv_pages + physical) * NERVA_KV_CACHE_BLOCK_TOKENS +
                           token % NERVA_KV_CACHE_BLOCK_TOKENS) * s->dims.kv_row();
  const uint16_t *src = (which == 0 ? s->kv_keys : s->kv_values) + offset;
  return cudaMemcpy(row, src, s->dims.kv_row() * 2u, cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : -1;
}

// Runs `steps` further decode steps of the active request outside any graph,
// with a CUDA event between launch groups, and sums the device time per
// operator bucket (the reference's detailed_profile path,
// session_decode_prefill.inc.cu:374-810, fills the same buckets).  The steps are
// real: the sequence advances by `steps` tokens.
extern "C" int nerva_b200_session_profile_steps(Session *s, uint32_t steps, uint64_t *bucket_ns,
                                                uint32_t *bucket_launches, uint32_t bucket_capacity) {
  if (s == nullptr || bucket_ns == nullptr || bucket_capacity < kBucketCount || steps == 0) return -1;
  if (!s->started || s->finished) return -1;
  const uint64_t target = static_cast<uint64_t>(s->cursor) + steps;
  if (target > s->max_context) return -1;
  for (uint32_t b = 0; b < bucket_capacity; ++b) {
    bucket_ns[b] = 0;
    if (bucket_launches != nullptr) bucket_launches[b] = 0;
  }
  const uint32_t kLaunchesPerMark[kBucketCount] = {1, 1, s->fused_attention ? 1u : 3u, 1, 1, 1, 1, 1};
  StepProfile prof;
  const uint32_t splits = splits_for(s, static_cast<uint32_t>(target));
  cudaError_t err = cudaSuccess;
  for (uint32_t step = 0; err == cudaSuccess && step < steps; ++step) {
    prof.used = 0;
    uint64_t launches = 0;
    err = enqueue_step(s, splits, 1, &launches, &prof);
    if (err == cudaSuccess) err = cudaStreamSynchronize(s->stream);
    for (uint32_t i = 0; err == cudaSuccess && i + 1 < prof.used; ++i) {
      float ms = 0.0f;
      if (cudaEventElapsedTime(&ms, prof.events[i], prof.events[i + 1]) != cudaSuccess) continue;
      const uint32_t b = prof.bucket[i];
      bucket_ns[b] += static_cast<uint64_t>(ms * 1.0e6f);
      if (bucket_launches != nullptr && step == 0) bucket_launches[b] += kLaunchesPerMark[b];
    }
  }
  for (cudaEvent_t e : prof.events) cudaEventDestroy(e);
  if (err == cudaSuccess)
    err = cudaMemcpy(s->host_slots + s->cursor - 0, s->device_slots + s->cursor,
                     static_cast<uint64_t>(steps) * sizeof(NervaCudaSyntheticTokenSlot), cudaMemcpyDeviceToHost);
  if (err != cudaSuccess) {
    set_last_error(cudaGetErrorString(err));
    return -1;
  }
  s->observed += steps;
  s->cursor = static_cast<uint32_t>(target);
  s->logits_valid = true;
  return 0;
}

// Reads and clears the per-phase cycle counters of the whole-step kernel (only
// filled when the session was created with NERVA_B200_PHASE_PROFILE=1).
extern "C" int nerva_b200_session_read_phase_cycles(Session *s, uint64_t *cycles, uint32_t capacity) {
  if (s == nullptr || cycles == nullptr || capacity < kPhaseCount || s->phase_cycles == nullptr) return -1;
  if (cudaStreamSynchronize(s->stream) != cudaSuccess) return -1;
  if (cudaMemcpy(cycles, s->phase_cycles, kPhaseCount * sizeof(uint64_t), cudaMemcpyDeviceToHost) != cudaSuccess)
    return -1;
  if (cudaMemset(s->phase_cycles, 0, kPhaseCount * sizeof(uint64_t)) != cudaSuccess) return -1;
  return static_cast<int>(kPhaseCount);
}
