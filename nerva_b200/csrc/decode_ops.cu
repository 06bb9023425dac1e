// Small kernels of the decode step: token fetch + embedding, per-head q/k
// RMSNorm + RoPE + paged KV append, greedy sampling, and set-up helpers.
#include <math.h>

#include "../../include/nerva_synth.h"
#include "common.cuh"
#include "kernels.cuh"

namespace nb {
namespace {

constexpr uint32_t kNoIndex = 0xffffffffu;
constexpr uint32_t kRequestId = 1;          // hf_decode_sequence/types.cuh:34-36
constexpr uint32_t kSequenceId = 1;
constexpr uint32_t kCompletionDeviceComplete = 1;

// Token of the position being decoded: a prompt id, or the token the previous
// step wrote to the ring (hf_decode_sequence/kernels.cu:195-206).
__device__ __forceinline__ uint32_t current_token(const StepState &st, uint32_t position) {
  return position < *st.prompt_count ? st.prompt[position] : st.slots[position - 1].token;
}

__global__ void embed_kernel(StepState st, const uint16_t *embeddings, uint32_t hidden,
                             float *input) {
  pdl_trigger();  // the first projection may start prefetching its weights now
  const uint32_t position = *st.cursor;
  if (position >= st.max_context) {
    if (threadIdx.x == 0) report_error(st.error_word, kErrCursorOutOfRange);
    return;
  }
  uint32_t token = current_token(st, position);
  if (token >= st.vocab) {
    if (threadIdx.x == 0) report_error(st.error_word, kErrTokenOutOfRange);
    token = 0;
  }
  const uint16_t *row = embeddings + static_cast<uint64_t>(token) * hidden;
  for (uint32_t i = threadIdx.x; i < hidden; i += blockDim.x) input[i] = bf16_bits_to_f32(row[i]);
}

// One block per head: blocks [0, heads) are query heads, [heads, heads+kv_heads)
// are key/value heads.  Order of operations per head follows the reference
// (hf_decode_sequence/kernels.cu:434-492): bias, per-head RMSNorm, RoPE with
// pairs (i, i + d/2) and angle pos / theta^(2i/d), then K and V rounded to bf16
// into the page selected by page_table[pos / 16]
// (hf_decode_sequence/types.cuh:328-337).
__global__ void qkv_prepare_kernel(StepState st, QkvPrepareParams p) {
  extern __shared__ float head_values[];  // head_dim floats
  __shared__ float scratch[40];
  const uint32_t position = *st.cursor;
  if (position >= st.max_context) return;
  const uint32_t d = p.head_dim;
  const bool is_query = blockIdx.x < p.heads;
  const uint32_t head = is_query ? blockIdx.x : blockIdx.x - p.heads;
  const uint32_t attention_hidden = p.heads * d;
  const uint32_t kv_hidden = p.kv_heads * d;
  float *values = is_query ? p.qkv + head * d : p.qkv + attention_hidden + head * d;
  const uint16_t *bias = is_query ? p.q_bias : p.k_bias;
  const uint16_t *norm = is_query ? p.q_norm : p.k_norm;

  float sumsq = 0.0f;
  for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {
    float v = values[i];
    if (bias != nullptr) v += bf16_bits_to_f32(bias[head * d + i]);
    head_values[i] = v;
    sumsq += v * v;
  }
  if (norm != nullptr) {
    const float total = block_sum(sumsq, scratch);
    const float scale = rsqrtf(total / static_cast<float>(d) + p.eps);
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {
      head_values[i] *= scale * bf16_bits_to_f32(norm[i]);
    }
  }
  __syncthreads();
  if (p.rope_theta > 0.0f) {
    const uint32_t half = d / 2;
    for (uint32_t i = threadIdx.x; i < half; i += blockDim.x) {
      const float exponent = static_cast<float>(2 * i) / static_cast<float>(d);
      const float angle = static_cast<float>(position) / powf(p.rope_theta, exponent);
      float s, c;
      sincosf(angle, &s, &c);
      const float left = head_values[i];
      const float right = head_values[i + half];
      head_values[i] = left * c - right * s;
      head_values[i + half] = right * c + left * s;
    }
    __syncthreads();
  }
  if (is_query) {
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) values[i] = head_values[i];
    return;
  }
  const uint32_t logical_page = position / NERVA_KV_CACHE_BLOCK_TOKENS;
  uint32_t physical_page = p.page_table[logical_page];
  if (physical_page >= p.page_count) {
    if (threadIdx.x == 0) report_error(st.error_word, kErrPageOutOfRange);
    return;
  }
  const uint64_t base =
      (static_cast<uint64_t>(physical_page) * NERVA_KV_CACHE_BLOCK_TOKENS +
       position % NERVA_KV_CACHE_BLOCK_TOKENS) * kv_hidden + head * d;
  const float *v_in = p.qkv + attention_hidden + kv_hidden + head * d;
  for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {
    float v = v_in[i];
    if (p.v_bias != nullptr) v += bf16_bits_to_f32(p.v_bias[head * d + i]);
    p.key_pages[base + i] = f32_to_bf16_bits(head_values[i]);
    p.value_pages[base + i] = f32_to_bf16_bits(v);
  }
}

__device__ __forceinline__ bool candidate_better(float v, uint32_t i, float best_v,
                                                 uint32_t best_i) {
  return v > best_v || (v == best_v && i < best_i);
}

// hf_decode_sequence/sampler.cu:394-407: slot fields and cursor advance.
//
// Tensor parallel (tp.world > 1): every rank holds the arg-max of its vocabulary
// shard.  Thread 0 stores (value, global index) into slot `rank` of every rank's
// candidate array, bumps the arrival counters, waits (bounded) for the other
// ranks' candidates of this step and applies the same tie rule, so all ranks
// write the same token.  Quiet steps exchange an empty candidate to keep the
// counters equal to the number of completed steps.
__device__ __forceinline__ void sample_greedy_block(const StepState &st, const float *best_value,
                                                    const uint32_t *best_index, uint32_t partials,
                                                    uint32_t sample, const TpSample &tp) {
  __shared__ float sv[32];
  __shared__ uint32_t si[32];
  const uint32_t position = *st.cursor;
  if (position >= st.max_context) return;
  float bv = -INFINITY;
  uint32_t bi = kNoIndex;
  if (sample != 0) {
    for (uint32_t i = threadIdx.x; i < partials; i += blockDim.x) {
      const uint32_t idx = best_index[i];
      if (idx != kNoIndex && candidate_better(best_value[i], idx, bv, bi)) {
        bv = best_value[i];
        bi = idx;
      }
    }
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, offset);
      const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, offset);
      if (oi != kNoIndex && candidate_better(ov, oi, bv, bi)) {
        bv = ov;
        bi = oi;
      }
    }
    if ((threadIdx.x & 31u) == 0) {
      sv[threadIdx.x >> 5] = bv;
      si[threadIdx.x >> 5] = bi;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (sample != 0) {
      bv = -INFINITY;
      bi = kNoIndex;
      for (uint32_t w = 0; w < (blockDim.x >> 5); ++w) {
        if (si[w] != kNoIndex && candidate_better(sv[w], si[w], bv, bi)) {
          bv = sv[w];
          bi = si[w];
        }
      }
      if (bi != kNoIndex) bi += tp.vocab_offset;
    }
    if (tp.world > 1) {
      const unsigned long long mine =
          (static_cast<unsigned long long>(__float_as_uint(bv)) << 32) | (sample != 0 ? bi : kNoIndex);
      for (uint32_t q = 0; q < tp.world; ++q) tp.recv[q][tp.rank] = mine;
      __threadfence_system();
      for (uint32_t q = 0; q < tp.world; ++q) atomicAdd_system(tp.arrivals[q] + tp.rank, 1ull);
      const unsigned long long expected = *tp.epoch + 1ull;
      bv = -INFINITY;
      bi = kNoIndex;
      bool failed = step_already_failed(st.error_word);  // an earlier exchange gave up: do not wait again
      for (uint32_t q = 0; q < tp.world; ++q) {
        if (failed) continue;
        if (!wait_counter_bounded(tp.arrivals[tp.rank] + q, expected)) {
          report_error(st.error_word, kErrPeerWaitTimeout);
          failed = true;
          continue;
        }
        const unsigned long long cand = ld_acquire_sys(tp.recv[tp.rank] + q);
        const float cv = __uint_as_float(static_cast<uint32_t>(cand >> 32));
        const uint32_t ci = static_cast<uint32_t>(cand & 0xffffffffull);
        if (ci != kNoIndex && candidate_better(cv, ci, bv, bi)) {
          bv = cv;
          bi = ci;
        }
      }
    }
    if (sample != 0) {
      NervaCudaSyntheticTokenSlot *slot = st.slots + position;
      slot->request_id = kRequestId;
      slot->sequence_id = kSequenceId;
      slot->token_index = position;
      slot->token = bi == kNoIndex ? 0u : bi;  // nothing finite: index 0, as the reference
      slot->version = static_cast<uint64_t>(position) + 1u;
      slot->completion = kCompletionDeviceComplete;
      slot->host_copied = 0;
    }
    *st.cursor = position + 1;
    if (tp.epoch != nullptr) *tp.epoch += 1ull;
  }
}

__global__ void sample_greedy_kernel(StepState st, const float *best_value,
                                     const uint32_t *best_index, uint32_t partials,
                                     uint32_t sample, TpSample tp) {
  pdl_wait();  // the arg-max partials come from the lm_head projection
  sample_greedy_block(st, best_value, best_index, partials, sample, tp);
}

// The rows of a packed step, one block each: row r's token goes to its own session's ring at that
// session's cursor (rows[r].state), from the row's `partials` arg-max candidates; blocks with
// blockIdx.y > 0 copy a slice of the row's logits into the session's own logits buffer instead.
__global__ void block_sample_kernel(const BlockSampleRow *rows, const float *best_value, const uint32_t *best_index,
                                    uint32_t partials, const float *logits, uint32_t vocab) {
  pdl_wait();
  const BlockSampleRow row = rows[blockIdx.x];
  if (blockIdx.y == 0) {
    TpSample none{};
    sample_greedy_block(row.state, best_value + blockIdx.x * partials, best_index + blockIdx.x * partials, partials, 1u,
                        none);
    return;
  }
  if (row.logits == nullptr) return;
  const uint32_t slices = gridDim.y - 1u, slice = blockIdx.y - 1u;
  const float *src = logits + static_cast<uint64_t>(blockIdx.x) * vocab;
  if (vocab % 4u == 0) {  // rows start on 16-byte boundaries
    const uint32_t quads = vocab / 4u;
    const uint32_t begin = static_cast<uint32_t>(static_cast<uint64_t>(quads) * slice / slices);
    const uint32_t end = static_cast<uint32_t>(static_cast<uint64_t>(quads) * (slice + 1u) / slices);
    for (uint32_t i = begin + threadIdx.x; i < end; i += blockDim.x)
      reinterpret_cast<float4 *>(row.logits)[i] = __ldcg(reinterpret_cast<const float4 *>(src) + i);
  } else {
    const uint32_t begin = static_cast<uint32_t>(static_cast<uint64_t>(vocab) * slice / slices);
    const uint32_t end = static_cast<uint32_t>(static_cast<uint64_t>(vocab) * (slice + 1u) / slices);
    for (uint32_t i = begin + threadIdx.x; i < end; i += blockDim.x) row.logits[i] = __ldcg(src + i);
  }
}

__global__ void argmax_kernel(const float *logits, uint32_t count, uint32_t *token_out) {
  __shared__ float sv[32];
  __shared__ uint32_t si[32];
  float bv = -INFINITY;
  uint32_t bi = kNoIndex;
  for (uint32_t i = threadIdx.x; i < count; i += blockDim.x) {
    const float v = logits[i];
    if (isfinite(v) && candidate_better(v, i, bv, bi)) {
      bv = v;
      bi = i;
    }
  }
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, offset);
    const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, offset);
    if (oi != kNoIndex && candidate_better(ov, oi, bv, bi)) {
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
    bi = kNoIndex;
    for (uint32_t w = 0; w < (blockDim.x >> 5); ++w) {
      if (si[w] != kNoIndex && candidate_better(sv[w], si[w], bv, bi)) {
        bv = sv[w];
        bi = si[w];
      }
    }
    *token_out = bi == kNoIndex ? 0u : bi;
  }
}

// Packed replicas (the reference keeps the same two, kernels.cu:741-802):
// [Wq; Wk; Wv] and the gate/up matrix with rows interleaved (g0, u0, g1, u1, ...)
// so that one warp finishes a SwiGLU pair on its own.
__global__ void copy_u16_kernel(const uint16_t *src, uint16_t *dst, uint64_t count) {
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
       i += stride) {
    dst[i] = src[i];
  }
}

__global__ void pack_gate_up_kernel(const uint16_t *gate, const uint16_t *up, uint16_t *packed,
                                    uint32_t intermediate, uint32_t hidden) {
  const uint64_t total = static_cast<uint64_t>(intermediate) * hidden;
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += stride) {
    const uint64_t row = i / hidden;
    const uint64_t col = i - row * hidden;
    packed[(2 * row) * hidden + col] = gate[i];
    packed[(2 * row + 1) * hidden + col] = up[i];
  }
}

__global__ void identity_table_kernel(uint32_t *table, uint32_t count) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) table[i] = i;
}

__global__ void fill_normal_bf16_kernel(uint16_t *out, uint64_t count, uint64_t key, float scale) {
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
       i += stride) {
    out[i] = nerva_synth_normal_bf16(key, i, scale);
  }
}

uint32_t grid_for(uint64_t count) {
  const uint64_t blocks = (count + 255) / 256;
  return static_cast<uint32_t>(blocks < 148ull * 16 ? (blocks == 0 ? 1 : blocks) : 148ull * 16);
}

}  // namespace

cudaError_t launch_embed(cudaStream_t stream, const StepState &st, const uint16_t *embeddings,
                         uint32_t hidden, float *input) {
  embed_kernel<<<1, 256, 0, stream>>>(st, embeddings, hidden, input);
  return cudaGetLastError();
}

cudaError_t launch_qkv_prepare(cudaStream_t stream, const StepState &st,
                               const QkvPrepareParams &p) {
  uint32_t threads = ((p.head_dim + 31u) / 32u) * 32u;
  if (threads > 256) threads = 256;
  qkv_prepare_kernel<<<p.heads + p.kv_heads, threads, p.head_dim * sizeof(float), stream>>>(st, p);
  return cudaGetLastError();
}

cudaError_t launch_sample_greedy(cudaStream_t stream, const StepState &st, const float *best_value,
                                 const uint32_t *best_index, uint32_t partials, uint32_t sample,
                                 bool pdl, const TpSample *tp) {
  TpSample exchange{};
  if (tp != nullptr) exchange = *tp;
  return launch_with_pdl(sample_greedy_kernel, dim3(1), dim3(256), 0, stream, pdl, st, best_value,
                         best_index, partials, sample, exchange);
}

// A step that does not sample has no head projection, so nothing reads the last exchange of its
// layers.  This kernel reads it instead: one block waits (bounded, like every peer wait) until all
// ranks' entries of that exchange carry the step's tag.  With it every push of a step is followed
// by a wait on the same exchange before the rank can push into that buffer again, which is what
// keeps a rank that runs ahead from overwriting entries a slower rank is still polling.
__global__ void __launch_bounds__(256) exchange_wait_kernel(TpGather g, uint32_t cols, uint32_t *error_word) {
  pdl_trigger();
  pdl_wait();
  const uint32_t tag = static_cast<uint32_t>(*g.epoch) * g.per_epoch + g.offset;
  const uint32_t total = g.world * cols;
  const long long start = clock64();
  bool gave_up = false;
  for (uint32_t i = threadIdx.x; i < total && !gave_up; i += blockDim.x) {
    uint32_t polls = 0;
    for (;;) {
      unsigned long long v;
      asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(g.recv + i) : "memory");
      if (static_cast<uint32_t>(v >> 32) == tag) break;
      if ((polls++ & 63u) == 0) {
        if (step_already_failed(error_word)) {
          gave_up = true;
        } else if (clock64() - start > kPeerWaitCycleLimit) {
          gave_up = true;
          report_error(error_word, kErrPeerWaitTimeout);
        }
        if (gave_up) break;
      }
    }
  }
}

cudaError_t launch_exchange_wait(cudaStream_t stream, const TpGather &gather, uint32_t cols, uint32_t *error_word,
                                 bool pdl) {
  return launch_with_pdl(exchange_wait_kernel, dim3(1), dim3(256), 0, stream, pdl, gather, cols, error_word);
}

cudaError_t launch_block_sample(cudaStream_t stream, const BlockSampleRow *rows, uint32_t count, const float *best_value,
                                const uint32_t *best_index, uint32_t partials, const float *logits, uint32_t vocab,
                                bool pdl) {
  return launch_with_pdl(block_sample_kernel, dim3(count, 9u), dim3(256), 0, stream, pdl, rows, best_value, best_index,
                         partials, logits, vocab);
}

cudaError_t launch_argmax(cudaStream_t stream, const float *logits, uint32_t count,
                          uint32_t *token_out) {
  argmax_kernel<<<1, 1024, 0, stream>>>(logits, count, token_out);
  return cudaGetLastError();
}

cudaError_t launch_pack_qkv(cudaStream_t stream, const uint16_t *wq, const uint16_t *wk,
                            const uint16_t *wv, uint16_t *packed, uint64_t q_elems,
                            uint64_t kv_elems) {
  copy_u16_kernel<<<grid_for(q_elems), 256, 0, stream>>>(wq, packed, q_elems);
  copy_u16_kernel<<<grid_for(kv_elems), 256, 0, stream>>>(wk, packed + q_elems, kv_elems);
  copy_u16_kernel<<<grid_for(kv_elems), 256, 0, stream>>>(wv, packed + q_elems + kv_elems, kv_elems);
  return cudaGetLastError();
}

cudaError_t launch_pack_gate_up(cudaStream_t stream, const uint16_t *gate, const uint16_t *up,
                                uint16_t *packed, uint32_t intermediate, uint32_t hidden) {
  pack_gate_up_kernel<<<grid_for(static_cast<uint64_t>(intermediate) * hidden), 256, 0, stream>>>(
      gate, up, packed, intermediate, hidden);
  return cudaGetLastError();
}

cudaError_t launch_identity_table(cudaStream_t stream, uint32_t *table, uint32_t count) {
  identity_table_kernel<<<(count + 255) / 256, 256, 0, stream>>>(table, count);
  return cudaGetLastError();
}

cudaError_t launch_fill_normal_bf16(cudaStream_t stream, uint16_t *out, uint64_t count,
                                    uint64_t seed, uint64_t tensor_id, float std) {
  const float scale = std * (1.0f / 65536.0f);
  fill_normal_bf16_kernel<<<grid_for(count), 256, 0, stream>>>(out, count,
                                                               nerva_synth_key(seed, tensor_id), scale);
  return cudaGetLastError();
}

}  // namespace nb
