// Block steps: several tokens through every layer together, so that the weights are streamed from
// HBM once for the block instead of once per token.  Two callers:
//   * the packed step of nerva_cuda_hf_decode_sequence_batch_advance_one — one token for each of up
//     to 32 sessions that share weights (reference: hf_decode_sequence/
//     session_api_batch_fork_destroy.inc.cu:1-310, kernels.cu:804-930 pack/scatter,
//     projection.cu:192-262 one skinny GEMM per projection);
//   * the chunked prefill of session_start — up to 256 prompt positions of one session at a time
//     (reference: session_decode_prefill.inc.cu:1879-2245, prefill_kernels.cu:66-170).
// Per layer: RMSNorm of the block -> QKV block projection -> (prefill: q/k-norm + RoPE + paged KV
// publish for all rows) -> split attention, one set of blocks per row -> O block projection with
// the residual add in its epilogue -> RMSNorm -> gate/up block projection with SwiGLU in its
// epilogue -> down block projection with the residual add.  The projections are the tcgen05 block
// kernel (gemm_tc.cu); attention is the session's own fused kernel in its row form.
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <vector>

#include "attention_device.cuh"
#include "session.h"
#include "step_device.cuh"

namespace nb {
namespace {

typedef NervaCudaHfDecodeSequenceSession Session;

constexpr uint32_t kNormThreads = 256;  // the thread count the single-token prologue normalises with

__device__ __forceinline__ uint32_t row_token(const BlockTokenRow &r) {
  // hf_decode_sequence/kernels.cu:195-206: a prompt id, or the token the previous step wrote to the ring
  return r.position < *r.prompt_count ? r.prompt[r.position] : r.slots[r.position - 1u].token;
}

// h[row][:] = embedding row of the row's token, as f32.
__global__ void block_embed_kernel(const BlockTokenRow *rows, const uint16_t *embeddings, uint32_t hidden, float *h) {
  pdl_trigger();
  const BlockTokenRow r = rows[blockIdx.x];
  uint32_t token = row_token(r);
  if (token >= r.vocab) {
    if (threadIdx.x == 0) report_error(r.error_word, kErrTokenOutOfRange);
    token = 0;
  }
  const uint16_t *src = embeddings + static_cast<uint64_t>(token) * hidden;
  float *dst = h + static_cast<uint64_t>(blockIdx.x) * hidden;
  for (uint32_t i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = bf16_bits_to_f32(src[i]);
}

// x[row][:] = bf16(h[row][:] * rsqrt(mean(h^2) + eps) * w): the arithmetic, thread mapping and
// summation order of the single-token prologue (step_device.cuh norm_single_*), so a token
// normalises to the same bits whichever path carries it.
__global__ void __launch_bounds__(kNormThreads) block_norm_kernel(const float *h, const uint16_t *w, float eps,
                                                                  uint32_t cols, uint16_t *x, uint32_t x_stride) {
  __shared__ float scratch[40];
  pdl_trigger();
  NormWeightRegs weights;
  norm_weights_preload(weights, w, cols);
  pdl_wait();
  NormValueRegs values;
  norm_single_load(values, h + static_cast<uint64_t>(blockIdx.x) * cols, cols);
  norm_single_finish(x + static_cast<uint64_t>(blockIdx.x) * x_stride, values, weights, eps, cols, scratch);
}

// Prefill: K (k-norm + RoPE) and V of every row of the chunk, rounded to bf16, into the row's page.
// One warp per (KV head, row); the same functions, in the same order, as the decode step's append
// (attention_fused.cu), so the cached bits are those the decode step would have written.
// Blocks beyond the KV heads (the grid has kv_heads + heads of them per row when prepare_q is set)
// do the query side for the paged attention kernel: bias, q-norm and RoPE of one query head, written
// back in place as fp32 (that kernel reads its queries ready-made).
template <uint32_t PER>
__global__ void block_kv_publish_kernel(const FusedAttentionRow *rows, uint32_t layer, uint32_t heads, uint32_t kv_heads,
                                        const uint16_t *k_bias, const uint16_t *v_bias, const uint16_t *k_norm,
                                        const uint16_t *q_bias, const uint16_t *q_norm, float eps, float rope_theta) {
  constexpr uint32_t D = PER * 32u;
  pdl_trigger();
  const FusedAttentionRow r = rows[blockIdx.y];
  const uint32_t lane = threadIdx.x & 31u;
  const bool query = blockIdx.x >= kv_heads;
  const uint32_t kvh = blockIdx.x;
  const uint32_t attention_hidden = heads * D, kv_hidden = kv_heads * D;
  const uint16_t *norm = query ? q_norm : k_norm;
  float norm_w[PER];
#pragma unroll
  for (uint32_t k = 0; k < PER; ++k) norm_w[k] = norm != nullptr ? bf16_bits_to_f32(norm[lane + 32u * k]) : 1.0f;
  RopeFactors<PER> rope;
  rope_factors<PER>(rope, rope_theta, r.position);
  pdl_wait();
  if (r.position >= r.max_context) return;
  if (query) {
    const uint32_t h = blockIdx.x - kv_heads;
    float *q = const_cast<float *>(r.qkv) + h * D;  // the row's projection output is scratch of the block step
    float qn[PER];
#pragma unroll
    for (uint32_t k = 0; k < PER; ++k) {
      const uint32_t e = lane + 32u * k;
      qn[k] = __ldcg(q + e);
      if (q_bias != nullptr) qn[k] += bf16_bits_to_f32(q_bias[h * D + e]);
    }
    head_norm_rope_pre<PER>(qn, q_norm != nullptr, norm_w, eps, rope);
#pragma unroll
    for (uint32_t k = 0; k < PER; ++k) q[lane + 32u * k] = qn[k];
    return;
  }
  float kn[PER], vn[PER];
#pragma unroll
  for (uint32_t k = 0; k < PER; ++k) {
    const uint32_t e = lane + 32u * k;
    kn[k] = __ldcg(r.qkv + attention_hidden + kvh * D + e);
    vn[k] = __ldcg(r.qkv + attention_hidden + kv_hidden + kvh * D + e);
    if (k_bias != nullptr) kn[k] += bf16_bits_to_f32(k_bias[kvh * D + e]);
    if (v_bias != nullptr) vn[k] += bf16_bits_to_f32(v_bias[kvh * D + e]);
  }
  head_norm_rope_pre<PER>(kn, k_norm != nullptr, norm_w, eps, rope);
  uint32_t page = r.page_table[r.position / NERVA_KV_CACHE_BLOCK_TOKENS];
  if (page >= r.page_count) {
    report_error(r.error_word, kErrPageOutOfRange);
    return;
  }
  // hf_decode_sequence/types.cuh:328-337
  const uint64_t base = layer * r.kv_layer_elems +
                        (static_cast<uint64_t>(page) * NERVA_KV_CACHE_BLOCK_TOKENS +
                         r.position % NERVA_KV_CACHE_BLOCK_TOKENS) * kv_hidden + kvh * D;
#pragma unroll
  for (uint32_t k = 0; k < PER; ++k) {
    const uint32_t e = lane + 32u * k;
    r.key_pages[base + e] = f32_to_bf16_bits(kn[k]);
    r.value_pages[base + e] = f32_to_bf16_bits(vn[k]);
  }
}

// Per (chunk, row): arg-max of one slice of the row's logits, reference tie rule (larger value,
// then lower index, non-finite skipped: sampler.cu:35-40).
__global__ void block_argmax_partials_kernel(const float *logits, uint32_t vocab, float *best_value,
                                             uint32_t *best_index) {
  __shared__ float sv[32];
  __shared__ uint32_t si[32];
  constexpr uint32_t kNone = 0xffffffffu;
  pdl_wait();
  const uint32_t chunk = blockIdx.x, chunks = gridDim.x, row = blockIdx.y;
  const uint32_t begin = static_cast<uint32_t>(static_cast<uint64_t>(vocab) * chunk / chunks);
  const uint32_t end = static_cast<uint32_t>(static_cast<uint64_t>(vocab) * (chunk + 1u) / chunks);
  const float *src = logits + static_cast<uint64_t>(row) * vocab;
  float bv = -INFINITY;
  uint32_t bi = kNone;
  for (uint32_t i = begin + threadIdx.x; i < end; i += blockDim.x) {
    const float v = __ldcg(src + i);
    if (isfinite(v) && (v > bv || (v == bv && i < bi))) {
      bv = v;
      bi = i;
    }
  }
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, offset);
    const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, offset);
    if (oi != kNone && (ov > bv || (ov == bv && oi < bi))) {
      bv = ov;
      bi = oi;
    }
  }
  if ((threadIdx.x & 31u) == 0) {
    sv[threadIdx.x >> 5] = bv;
    si[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    bv = -INFINITY;
    bi = kNone;
    for (uint32_t w = 0; w < (blockDim.x >> 5); ++w) {
      if (si[w] != kNone && (sv[w] > bv || (sv[w] == bv && si[w] < bi))) {
        bv = sv[w];
        bi = si[w];
      }
    }
    best_value[row * chunks + chunk] = bv;
    best_index[row * chunks + chunk] = bi;
  }
}

template <class T>
bool carve(StaticArena &arena, void *base, uint64_t count, T **out) {
  ArenaRegion region;
  if (!arena.reserve(count * sizeof(T), 1024, AllocationPhase::Initialization, &region)) return false;
  if (base != nullptr) *out = reinterpret_cast<T *>(static_cast<uint8_t *>(base) + region.offset);
  return true;
}

bool plan_workspace(const Session *s, BlockWorkspace *ws, StaticArena &arena, void *base) {
  const ModelDims &d = s->dims;
  const uint64_t ah = d.attention_hidden(), kvh = d.kv_hidden(), qkv_rows = ah + 2 * kvh;
  const uint64_t rows = ws->max_rows, sample = ws->sample_rows;
  const uint64_t max_x = std::max<uint64_t>(std::max<uint64_t>(d.hidden, d.intermediate), ah);
  const uint32_t max_out = std::max(std::max<uint32_t>(static_cast<uint32_t>(qkv_rows), 2u * d.intermediate),
                                    std::max(d.hidden, d.vocab));
  bool ok = carve(arena, base, rows * max_x, &ws->x_bf16);
  ok = ok && carve(arena, base, rows * qkv_rows, &ws->qkv);
  ok = ok && carve(arena, base, rows * ah, &ws->attn);
  ok = ok && carve(arena, base, rows * d.hidden, &ws->h_a);
  ok = ok && carve(arena, base, rows * d.hidden, &ws->h_b);
  ok = ok && carve(arena, base, rows * d.intermediate, &ws->ff);
  ok = ok && carve(arena, base, sample * d.vocab, &ws->logits);
  ok = ok && carve(arena, base, rows * d.heads * 16u * d.head_dim, &ws->partial_acc);
  ok = ok && carve(arena, base, rows * d.heads * 16u, &ws->partial_m);
  ok = ok && carve(arena, base, rows * d.heads * 16u, &ws->partial_l);
  ok = ok && carve(arena, base, rows * d.kv_heads, &ws->attn_tickets);
  ok = ok && carve(arena, base, gemm_tc_workspace_bytes(ws->max_rows, s->sm_count) / sizeof(float), &ws->gemm_workspace);
  ok = ok && carve(arena, base, static_cast<uint64_t>(gemm_tc_ticket_count(max_out)), &ws->gemm_tickets);
  ok = ok && carve(arena, base, sample * kBlockArgmaxChunks, &ws->best_value);
  ok = ok && carve(arena, base, sample * kBlockArgmaxChunks, &ws->best_index);
  ok = ok && carve(arena, base, rows, &ws->attn_rows);
  ok = ok && carve(arena, base, rows, &ws->token_rows);
  ok = ok && carve(arena, base, sample, &ws->sample_rows_dev);
  return ok;
}

const uint16_t *arena_at(const Session *s, uint64_t offset) {
  return offset == kMissingOffset ? nullptr : s->weights->arena + offset;
}

struct BlockPlan {
  Session *model;        // any session of the block: dims, layout, weights, workspace
  cudaStream_t stream;
  uint32_t rows;
  uint32_t splits;       // attention spans per KV head (covers the longest row)
  bool publish;          // prefill: K/V of all rows published before attention (cached_only)
  bool pdl;
  // Attention on the paged tensor-pipe kernel (attention.cu) instead of the fused kernel's row form:
  // the tensor maps of the caches the rows live in (rows[r].map_index), or empty for the fused kernel.
  std::vector<TensorMapStorage> k_maps, v_maps;
  uint32_t longest = 0;  // longest context among the rows
};

cudaError_t block_gemm(const BlockPlan &b, const uint16_t *weight, uint32_t rows, uint32_t cols, const uint16_t *x,
                       uint32_t x_stride_check, uint32_t epilogue, const float *resid, float *out_f32,
                       uint16_t *out_bf16) {
  (void)x_stride_check;
  const BlockWorkspace &ws = b.model->weights->block_ws;
  GemmParams g{};
  g.weight = weight;
  g.rows = rows;
  g.cols = cols;
  g.x = x;
  g.tokens = b.rows;
  g.epilogue = epilogue;
  g.resid_in = resid;
  g.out_f32 = out_f32;
  g.out_bf16 = out_bf16;
  g.workspace = ws.gemm_workspace;
  g.tickets = ws.gemm_tickets;
  g.error_word = b.model->device_error;
  g.pdl = b.pdl ? 1u : 0u;
  return launch_gemm_tc(b.stream, g, b.model->sm_count);
}

// Embedding + all layers for the rows whose descriptors are already on the device.  On return
// ws.h_b holds the residual stream after the last layer, one row per token.
cudaError_t enqueue_block_layers(const BlockPlan &b, uint64_t *launches) {
  Session *s = b.model;
  const ModelDims &d = s->dims;
  const BlockWorkspace &ws = s->weights->block_ws;
  const uint32_t ah = static_cast<uint32_t>(d.attention_hidden()), kvh = static_cast<uint32_t>(d.kv_hidden());
  const uint32_t qkv_rows = ah + 2u * kvh;
  uint64_t n = 0;
  cudaError_t err = launch_with_pdl(block_embed_kernel, dim3(b.rows), dim3(256), 0, b.stream, false, ws.token_rows,
                                    arena_at(s, s->layout.embeddings), d.hidden, ws.h_b);
  n += 1;
  for (uint32_t l = 0; err == cudaSuccess && l < d.layers; ++l) {
    const LayerLayout &L = s->layout.layers[l];
    // attention half
    err = launch_with_pdl(block_norm_kernel, dim3(b.rows), dim3(kNormThreads), 0, b.stream, b.pdl, ws.h_b,
                          arena_at(s, L.rms_attn), s->rms_eps, d.hidden, ws.x_bf16, d.hidden);
    if (err == cudaSuccess)
      err = block_gemm(b, s->weights->qkv_packed + static_cast<uint64_t>(l) * qkv_rows * d.hidden, qkv_rows, d.hidden,
                       ws.x_bf16, d.hidden, kEpilogueStore, nullptr, ws.qkv, nullptr);
    n += 2;
    const bool paged = !b.k_maps.empty();
    if (err == cudaSuccess && (b.publish || paged)) {
      const dim3 grid(d.kv_heads + (paged ? d.heads : 0u), b.rows);
      if (d.head_dim == 128)
        err = launch_with_pdl(block_kv_publish_kernel<4>, grid, dim3(32), 0, b.stream, b.pdl, ws.attn_rows, l, d.heads,
                              d.kv_heads, arena_at(s, L.k_bias), arena_at(s, L.v_bias), arena_at(s, L.k_norm),
                              arena_at(s, L.q_bias), arena_at(s, L.q_norm), s->rms_eps, s->rope_theta);
      else
        err = launch_with_pdl(block_kv_publish_kernel<2>, grid, dim3(32), 0, b.stream, b.pdl, ws.attn_rows, l, d.heads,
                              d.kv_heads, arena_at(s, L.k_bias), arena_at(s, L.v_bias), arena_at(s, L.k_norm),
                              arena_at(s, L.q_bias), arena_at(s, L.q_norm), s->rms_eps, s->rope_theta);
      n += 1;
    }
    if (err != cudaSuccess) break;
    if (paged) {
      // every row's K/V (its own newest row included) is in its cache and its queries are prepared
      AttentionParams ap{};
      ap.batch = b.rows;
      ap.heads = d.heads;
      ap.kv_heads = d.kv_heads;
      ap.head_dim = d.head_dim;
      ap.splits = attention_rows_splits(b.longest, b.rows, d.kv_heads, s->sm_count);
      ap.partial_acc = ws.partial_acc;
      ap.partial_m = ws.partial_m;
      ap.partial_l = ws.partial_l;
      ap.out_bf16 = ws.attn;
      ap.error_word = s->device_error;
      ap.rows = ws.attn_rows;
      ap.layer = l;
      err = launch_attention_rows(b.stream, ap, b.k_maps.data(), b.v_maps.data(), static_cast<uint32_t>(b.k_maps.size()));
      n += 2;
      if (err != cudaSuccess) break;
    } else {
    FusedAttentionParams fp{};
    fp.max_context = s->max_context;
    fp.q_bias = arena_at(s, L.q_bias);
    fp.k_bias = arena_at(s, L.k_bias);
    fp.v_bias = arena_at(s, L.v_bias);
    fp.q_norm = arena_at(s, L.q_norm);
    fp.k_norm = arena_at(s, L.k_norm);
    fp.heads = d.heads;
    fp.kv_heads = d.kv_heads;
    fp.head_dim = d.head_dim;
    fp.eps = s->rms_eps;
    fp.rope_theta = s->rope_theta;
    fp.splits = b.splits;
    fp.pdl = b.pdl ? 1u : 0u;
    fp.rows = ws.attn_rows;
    fp.row_count = b.rows;
    fp.layer = l;
    fp.cached_only = b.publish ? 1u : 0u;
    err = launch_fused_attention(b.stream, fp);
    n += 1;
    if (err != cudaSuccess) break;
    }
    // h_a = h_b + O(attention)
    err = block_gemm(b, arena_at(s, L.w_o), d.hidden, ah, ws.attn, ah, kEpilogueStore, ws.h_b, ws.h_a, nullptr);
    // MLP half
    if (err == cudaSuccess)
      err = launch_with_pdl(block_norm_kernel, dim3(b.rows), dim3(kNormThreads), 0, b.stream, b.pdl, ws.h_a,
                            arena_at(s, L.rms_mlp), s->rms_eps, d.hidden, ws.x_bf16, d.hidden);
    if (err == cudaSuccess)
      err = block_gemm(b, s->weights->gate_up_packed + gate_up_packed_offset(s, l),
                       2u * d.intermediate, d.hidden, ws.x_bf16, d.hidden, kEpilogueSwiglu, nullptr, nullptr, ws.ff);
    // h_b = h_a + down(ff)
    if (err == cudaSuccess)
      err = block_gemm(b, arena_at(s, L.w_down), d.hidden, d.intermediate, ws.ff, d.intermediate, kEpilogueStore,
                       ws.h_a, ws.h_b, nullptr);
    n += 4;
  }
  if (launches != nullptr) *launches += n;
  return err;
}

// Attention spans per KV head in a block step.  A single token wants many short spans (latency);
// a block of rows already fills the machine with rows x kv_heads blocks per span, so it takes as
// few spans as keep about six blocks per SM in flight, and never more than the context needs.
uint32_t block_attention_splits(const Session *s, uint32_t rows, uint32_t longest_context) {
  const uint32_t by_context = fused_attention_splits(longest_context);
  uint32_t by_machine = (6u * s->sm_count) / (rows * s->dims.kv_heads);
  if (by_machine < 1u) by_machine = 1u;
  return by_context < by_machine ? by_context : by_machine;
}

FusedAttentionRow attention_row(Session *s, const BlockWorkspace &ws, uint32_t row, uint32_t position) {
  const ModelDims &d = s->dims;
  const uint64_t qkv_rows = d.attention_hidden() + 2 * d.kv_hidden();
  FusedAttentionRow r{};
  r.position = position;
  r.max_context = s->max_context;
  r.page_count = s->kv_pages;
  r.qkv = ws.qkv + row * qkv_rows;
  r.key_pages = s->kv_keys;
  r.value_pages = s->kv_values;
  r.kv_layer_elems = s->kv_layer_elems;
  r.page_table = s->page_table;
  r.partial_acc = ws.partial_acc + static_cast<uint64_t>(row) * d.heads * 16u * d.head_dim;
  r.partial_m = ws.partial_m + static_cast<uint64_t>(row) * d.heads * 16u;
  r.partial_l = ws.partial_l + static_cast<uint64_t>(row) * d.heads * 16u;
  r.tickets = ws.attn_tickets + static_cast<uint64_t>(row) * d.kv_heads;
  r.out_bf16 = ws.attn + static_cast<uint64_t>(row) * d.attention_hidden();
  r.error_word = s->device_error;
  return r;
}

BlockTokenRow token_row(Session *s, uint32_t position) {
  BlockTokenRow t{};
  t.prompt = s->device_prompt;
  t.prompt_count = s->device_cursor + 1;  // word 1 of the cursor block (session.cu: step_state)
  t.slots = s->device_slots;
  t.position = position;
  t.vocab = s->dims.embed_vocab;
  t.error_word = s->device_error;
  return t;
}

cudaError_t upload_rows(const BlockWorkspace &ws, const std::vector<FusedAttentionRow> &attn,
                        const std::vector<BlockTokenRow> &tokens, cudaStream_t stream) {
  // pageable sources: staged by the runtime before the calls return
  cudaError_t err = cudaMemcpyAsync(ws.attn_rows, attn.data(), attn.size() * sizeof(FusedAttentionRow),
                                    cudaMemcpyHostToDevice, stream);
  if (err == cudaSuccess)
    err = cudaMemcpyAsync(ws.token_rows, tokens.data(), tokens.size() * sizeof(BlockTokenRow), cudaMemcpyHostToDevice,
                          stream);
  return err;
}

}  // namespace

bool block_step_supported(const NervaCudaHfDecodeSequenceSession *s) {
  const ModelDims &d = s->dims;
  if (s->tp_world > 1 || s->has_moe || d.mla() || !s->fused_attention || d.dtype != NERVA_DTYPE_BF16) return false;
  const uint64_t ah = d.attention_hidden();
  if (d.hidden % 64u != 0 || ah % 64u != 0 || d.intermediate % 64u != 0) return false;
  if (d.hidden % 4u != 0 || d.hidden / 4u > kNormRegIters * kNormThreads) return false;  // block_norm_kernel's reach
  for (const LayerLayout &L : s->layout.layers) {
    if (L.mlp_kind != NERVA_MLP_KIND_DENSE || L.o_bias != kMissingOffset) return false;
  }
  return tensor_map_available();
}

cudaError_t allocate_block_workspace(NervaCudaHfDecodeSequenceSession *s) {
  BlockWorkspace &ws = s->weights->block_ws;
  const uint32_t context_rows = (s->max_context + 15u) & ~15u;
  ws.max_rows = std::max(kBlockSampleRows, std::min(kBlockMaxRows, context_rows));
  ws.sample_rows = kBlockSampleRows;
  StaticArena sizing(UINT64_MAX / 2);
  if (!plan_workspace(s, &ws, sizing, nullptr)) return cudaErrorMemoryAllocation;
  ws.bytes = sizing.used();
  cudaError_t err = cudaMalloc(&ws.block, ws.bytes);
  if (err != cudaSuccess) return err;
  StaticArena arena(ws.bytes);
  if (!plan_workspace(s, &ws, arena, ws.block)) return cudaErrorMemoryAllocation;
  const ModelDims &d = s->dims;
  const uint32_t max_out = std::max(std::max<uint32_t>(static_cast<uint32_t>(d.attention_hidden() + 2 * d.kv_hidden()),
                                                      2u * d.intermediate),
                                    std::max(d.hidden, d.vocab));
  err = cudaMemsetAsync(ws.attn_tickets, 0, static_cast<uint64_t>(ws.max_rows) * d.kv_heads * sizeof(uint32_t), s->stream);
  if (err == cudaSuccess)
    err = cudaMemsetAsync(ws.gemm_tickets, 0, static_cast<uint64_t>(gemm_tc_ticket_count(max_out)) * sizeof(uint32_t),
                          s->stream);
  if (err == cudaSuccess) err = configure_gemm_tc_kernel();
  // NERVA_B200_ROW_ATTENTION=fused keeps the fused kernel's row form (comparison and fallback)
  const char *row_attention = getenv("NERVA_B200_ROW_ATTENTION");
  ws.paged_rows = attention_rows_supported(d.heads, d.kv_heads, d.head_dim) &&
                  !(row_attention != nullptr && strcmp(row_attention, "fused") == 0);
  return err;
}

cudaError_t enqueue_block_decode(NervaCudaHfDecodeSequenceSession *const *sessions, uint32_t count,
                                 cudaStream_t stream, uint64_t *launches) {
  if (count == 0 || count > kBlockSampleRows) return cudaErrorInvalidValue;
  Session *model = sessions[0];
  const BlockWorkspace &ws = model->weights->block_ws;
  if (ws.block == nullptr || count > ws.max_rows) return cudaErrorNotSupported;
  const ModelDims &d = model->dims;
  std::vector<FusedAttentionRow> attn(count);
  std::vector<BlockTokenRow> tokens(count);
  uint32_t longest = 0;
  bool paged = ws.paged_rows && count <= kAttentionRowCaches;
  for (uint32_t r = 0; r < count; ++r) {
    Session *s = sessions[r];
    attn[r] = attention_row(s, ws, r, s->cursor);
    attn[r].map_index = r;  // every session brings its own cache
    tokens[r] = token_row(s, s->cursor);
    longest = std::max(longest, s->cursor + 1u);
    paged = paged && s->kv_maps;
  }
  cudaError_t err = upload_rows(ws, attn, tokens, stream);
  if (err != cudaSuccess) return err;
  BlockPlan b{model, stream, count, block_attention_splits(model, count, longest), false, model->use_pdl};
  b.longest = longest;
  if (paged) {
    for (uint32_t r = 0; r < count; ++r) {
      b.k_maps.push_back(sessions[r]->kv_map_k);
      b.v_maps.push_back(sessions[r]->kv_map_v);
    }
  }
  uint64_t n = 0;
  err = enqueue_block_layers(b, &n);
  // final norm, lm_head, arg-max: per row
  if (err == cudaSuccess)
    err = launch_with_pdl(block_norm_kernel, dim3(count), dim3(kNormThreads), 0, stream, b.pdl, ws.h_b,
                          arena_at(model, model->layout.final_norm), model->rms_eps, d.hidden, ws.x_bf16, d.hidden);
  if (err == cudaSuccess)
    err = block_gemm(b, arena_at(model, model->layout.lm_head), d.vocab, d.hidden, ws.x_bf16, d.hidden, kEpilogueStore,
                     nullptr, ws.logits, nullptr);
  if (err == cudaSuccess)
    err = launch_with_pdl(block_argmax_partials_kernel, dim3(kBlockArgmaxChunks, count), dim3(256), 0, stream, b.pdl,
                          ws.logits, d.vocab, ws.best_value, ws.best_index);
  n += 3;
  // every row's token into its own session's ring, and its logits into the session's own buffer
  // (nerva_b200_session_read_logits), in one launch
  std::vector<BlockSampleRow> sample(count);
  for (uint32_t r = 0; r < count; ++r) {
    Session *s = sessions[r];
    StepState &st = sample[r].state;
    st.cursor = s->device_cursor;
    st.prompt = s->device_prompt;
    st.prompt_count = s->device_cursor + 1;
    st.slots = s->device_slots;
    st.max_context = s->max_context;
    st.vocab = d.embed_vocab;
    st.error_word = s->device_error;
    sample[r].logits = s->logits;
  }
  if (err == cudaSuccess)  // pageable source: staged before the call returns
    err = cudaMemcpyAsync(ws.sample_rows_dev, sample.data(), sample.size() * sizeof(BlockSampleRow),
                          cudaMemcpyHostToDevice, stream);
  if (err == cudaSuccess)
    err = launch_block_sample(stream, ws.sample_rows_dev, count, ws.best_value, ws.best_index, kBlockArgmaxChunks,
                              ws.logits, d.vocab, false);
  n += 1;
  if (launches != nullptr) *launches += n;
  return err;
}

cudaError_t enqueue_chunked_prefill(NervaCudaHfDecodeSequenceSession *s, uint32_t prompt_count, uint32_t sample_kind,
                                    uint64_t *launches) {
  (void)sample_kind;
  const BlockWorkspace &ws = s->weights->block_ws;
  if (ws.block == nullptr || prompt_count == 0) return cudaErrorNotSupported;
  const ModelDims &d = s->dims;
  cudaError_t err = cudaSuccess;
  for (uint32_t begin = 0; err == cudaSuccess && begin < prompt_count; begin += ws.max_rows) {
    const uint32_t rows = std::min(ws.max_rows, prompt_count - begin);
    std::vector<FusedAttentionRow> attn(rows);
    std::vector<BlockTokenRow> tokens(rows);
    for (uint32_t r = 0; r < rows; ++r) {
      attn[r] = attention_row(s, ws, r, begin + r);
      tokens[r] = token_row(s, begin + r);
    }
    err = upload_rows(ws, attn, tokens, s->stream);
    if (err != cudaSuccess) break;
    BlockPlan b{s, s->stream, rows, block_attention_splits(s, rows, begin + rows), true, s->use_pdl};
    b.longest = begin + rows;
    if (ws.paged_rows && s->kv_maps) {
      b.k_maps.push_back(s->kv_map_k);  // all rows of a chunk live in this session's cache (map_index 0)
      b.v_maps.push_back(s->kv_map_v);
    }
    err = enqueue_block_layers(b, launches);
    if (err == cudaSuccess && begin + rows == prompt_count) {
      // the last position's residual stream becomes the session's own, where the head expects it
      err = cudaMemcpyAsync(s->h_b, ws.h_b + static_cast<uint64_t>(rows - 1u) * d.hidden,
                            static_cast<uint64_t>(d.hidden) * sizeof(float), cudaMemcpyDeviceToDevice, s->stream);
    }
  }
  return err;
}

}  // namespace nb
