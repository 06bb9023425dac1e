// Decode attention of the resident session as ONE launch per layer: q/k RMSNorm
// + RoPE + paged KV append + split attention + merge.  The reference spends
// three launches on this (hf_decode_sequence/kernels.cu:434-492,
// attention_kernels.cu:528-760, kernels.cu:494-555).
//
// Grid = heads x splits blocks.  Every block runs one (head, split) item
// (attention_device.cuh) and leaves its partial in global memory; the block that
// finishes a head last (a ticket counter per head, no waiting) merges the
// head's partials and writes the bf16 attention output.
#include "attention_device.cuh"
#include "kernels.cuh"

namespace nb {
namespace {

constexpr uint32_t kFusedWarps = 8;
constexpr uint32_t kFusedMaxSplits = 8;

template <uint32_t PER>
__global__ void __launch_bounds__(kFusedWarps * 32, 1) fused_decode_attention_kernel(FusedAttentionParams p) {
  constexpr uint32_t D = PER * 32u;
  __shared__ AttnItemShared<kFusedWarps> sh;
  __shared__ __align__(16) float merge[kFusedWarps * kAttnMergeStride];
  __shared__ uint32_t ticket;
  pdl_trigger();
  // The cursor only changes in the last kernel of a step, which has completed.
  const uint32_t position = *p.cursor;
  if (position >= p.max_context) return;
  AttnItemCtx c;
  c.qkv = p.qkv;
  c.q_bias = p.q_bias;
  c.k_bias = p.k_bias;
  c.v_bias = p.v_bias;
  c.q_norm = p.q_norm;
  c.k_norm = p.k_norm;
  c.key_pages = p.key_pages;
  c.value_pages = p.value_pages;
  c.page_table = p.page_table;
  c.page_count = p.page_count;
  c.heads = p.heads;
  c.kv_heads = p.kv_heads;
  c.eps = p.eps;
  c.rope_theta = p.rope_theta;
  c.position = position;
  c.splits = p.splits;
  c.partial_acc = p.partial_acc;
  c.partial_m = p.partial_m;
  c.partial_l = p.partial_l;
  c.error_word = p.error_word;
  c.wait_dependency = true;  // a no-op when the launch carries no programmatic dependency
  const uint32_t S = p.splits;
  const uint32_t h = blockIdx.x / S, s = blockIdx.x - h * S;
  attention_item<PER, kFusedWarps>(c, sh, merge, h, s);

  // Publish the partial, then take a ticket: the block that draws the last
  // ticket of its head sees every partial of that head.
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) ticket = atomicAdd(p.tickets + h, 1u);
  __syncthreads();
  if (ticket != S - 1u) return;
  __threadfence();
  float ms[kFusedMaxSplits], ls[kFusedMaxSplits];
  float m = -INFINITY;
#pragma unroll
  for (uint32_t i = 0; i < kFusedMaxSplits; ++i) {
    ms[i] = i < S ? __ldcg(p.partial_m + h * S + i) : -INFINITY;
    ls[i] = i < S ? __ldcg(p.partial_l + h * S + i) : 0.0f;
    if (ls[i] > 0.0f) m = fmaxf(m, ms[i]);
  }
  float l = 0.0f;
#pragma unroll
  for (uint32_t i = 0; i < kFusedMaxSplits; ++i) {
    ms[i] = ls[i] > 0.0f ? exp2f(ms[i] - m) : 0.0f;  // weight of split i
    l = fmaf(ls[i], ms[i], l);
  }
  const float inv = l > 0.0f ? 1.0f / l : 0.0f;
  for (uint32_t d = threadIdx.x; d < D; d += blockDim.x) {
    float a = 0.0f;
#pragma unroll
    for (uint32_t i = 0; i < kFusedMaxSplits; ++i) {
      if (i < S) a = fmaf(__ldcg(p.partial_acc + (static_cast<uint64_t>(h) * S + i) * D + d), ms[i], a);
    }
    p.out_bf16[h * D + d] = f32_to_bf16_bits(a * inv);
  }
  if (threadIdx.x == 0) p.tickets[h] = 0;  // ready for the next launch
}

}  // namespace

bool fused_attention_supported(uint32_t heads, uint32_t kv_heads, uint32_t head_dim) {
  return (head_dim == 64 || head_dim == 128) && kv_heads != 0 && heads % kv_heads == 0;
}

uint32_t fused_attention_splits(uint32_t target_context) {
  const uint32_t per_item = kFusedWarps * kAttnItemTile;  // one 32-token tile per warp
  uint32_t s = (target_context + per_item - 1u) / per_item;
  if (s < 1) s = 1;
  if (s > kFusedMaxSplits) s = kFusedMaxSplits;
  return s;
}

cudaError_t launch_fused_attention(cudaStream_t stream, const FusedAttentionParams &p) {
  if (!fused_attention_supported(p.heads, p.kv_heads, p.head_dim) || p.splits == 0 ||
      p.splits > kFusedMaxSplits)
    return cudaErrorInvalidValue;
  const uint32_t blocks = p.heads * p.splits;
  if (p.head_dim == 128) {
    return launch_with_pdl(fused_decode_attention_kernel<4>, dim3(blocks), dim3(kFusedWarps * 32), 0,
                           stream, p.pdl != 0, p);
  }
  return launch_with_pdl(fused_decode_attention_kernel<2>, dim3(blocks), dim3(kFusedWarps * 32), 0, stream,
                         p.pdl != 0, p);
}

}  // namespace nb
