// The whole decode step as ONE persistent kernel (engine 1).
//
// One block per SM runs every operator of the token: per layer QKV projection,
// q/k norm + RoPE + KV append + attention, O projection, gate/up projection with
// SwiGLU, down projection; then lm_head with greedy arg-max and the token-ring
// write.  Blocks meet at a grid barrier between operators.  What makes this
// faster than one launch per operator is the weight stream (row_stream.cuh):
// each warp's TMA ring keeps prefetching the next projection's rows through the
// barriers, the norms and the attention, so HBM never drains between operators
// and there is no per-kernel ramp-up or tail.
//
// Numerics are those of the per-operator engine (same rounding points, same
// per-row summation order in the projections).
#include <math.h>

#include "step_kernel.cuh"

namespace nb {
namespace {

constexpr uint32_t kNoIndex = 0xffffffffu;

__device__ __forceinline__ bool better(float v, uint32_t i, float bv, uint32_t bi) {
  return v > bv || (v == bv && i < bi);
}

// Attention of one layer: work items (query head, split of the cached tokens)
// are dealt round-robin to the blocks.
template <uint32_t PER>
__device__ void attention_phase(const StepKernelParams &p, StepShared &sh, float *merge,
                                const StepLayerDev &L, uint32_t position) {
  AttnItemCtx c;
  c.qkv = p.qkv;
  c.q_bias = L.q_bias;
  c.k_bias = L.k_bias;
  c.v_bias = L.v_bias;
  c.q_norm = L.q_norm;
  c.k_norm = L.k_norm;
  c.key_pages = L.key_pages;
  c.value_pages = L.value_pages;
  c.page_table = p.page_table;
  c.page_count = p.page_count;
  c.heads = p.heads;
  c.kv_heads = p.kv_heads;
  c.eps = p.eps;
  c.rope_theta = p.rope_theta;
  c.position = position;
  c.splits = p.attn_splits;
  c.partial_acc = p.partial_acc;
  c.partial_m = p.partial_m;
  c.partial_l = p.partial_l;
  c.error_word = p.st.error_word;
  c.wait_dependency = false;
  for (uint32_t item = blockIdx.x; item < p.heads * p.attn_splits; item += gridDim.x) {
    attention_item<PER, kStreamWarps>(c, sh.attn, merge, item / p.attn_splits, item % p.attn_splits);
  }
}

// x[h*D + d] = bf16( sum_s acc_s w_s ),  w_s = 2^{m_s - M} / sum_s l_s 2^{m_s - M}.
// Two round trips to L2 per block: first the (m, l) pairs of every (head, split)
// become normalised weights in shared memory, then every thread issues all of its
// partial-accumulator loads before it uses any of them.
__device__ void merge_attention_to_smem(const StepKernelParams &p, StepShared &sh, uint16_t *x) {
  const uint32_t D = p.head_dim, S = p.attn_splits;
  float *weights = sh.weights;  // [heads][S]
  for (uint32_t h = threadIdx.x; h < p.heads; h += blockDim.x) {
    float ms[kStepMaxSplits], ls[kStepMaxSplits];
#pragma unroll
    for (uint32_t s = 0; s < kStepMaxSplits; ++s) {
      ms[s] = s < S ? __ldcg(p.partial_m + h * S + s) : -INFINITY;
      ls[s] = s < S ? __ldcg(p.partial_l + h * S + s) : 0.0f;
    }
    float m = -INFINITY;
#pragma unroll
    for (uint32_t s = 0; s < kStepMaxSplits; ++s)
      if (ls[s] > 0.0f) m = fmaxf(m, ms[s]);
    float l = 0.0f;
#pragma unroll
    for (uint32_t s = 0; s < kStepMaxSplits; ++s)
      if (ls[s] > 0.0f) l = fmaf(ls[s], exp2f(ms[s] - m), l);
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (uint32_t s = 0; s < kStepMaxSplits; ++s)
      if (s < S) weights[h * S + s] = ls[s] > 0.0f ? exp2f(ms[s] - m) * inv : 0.0f;
  }
  __syncthreads();
  constexpr uint32_t kBatch = 8;
  const uint32_t total = p.heads * D;
  for (uint32_t base = 0; base < total; base += kBatch * blockDim.x) {
    float v[kBatch][kStepMaxSplits];
#pragma unroll
    for (uint32_t k = 0; k < kBatch; ++k) {
      const uint32_t idx = base + k * blockDim.x + threadIdx.x;
      const uint32_t h = idx / D, d = idx - h * D;
#pragma unroll
      for (uint32_t s = 0; s < kStepMaxSplits; ++s) {
        v[k][s] = (idx < total && s < S)
                      ? __ldcg(p.partial_acc + (static_cast<uint64_t>(h) * S + s) * D + d)
                      : 0.0f;
      }
    }
#pragma unroll
    for (uint32_t k = 0; k < kBatch; ++k) {
      const uint32_t idx = base + k * blockDim.x + threadIdx.x;
      if (idx < total) {
        const uint32_t h = idx / D;
        float a = 0.0f;
#pragma unroll
        for (uint32_t s = 0; s < kStepMaxSplits; ++s)
          if (s < S) a = fmaf(v[k][s], weights[h * S + s], a);
        x[idx] = f32_to_bf16_bits(a);
      }
    }
  }
}

}  // namespace
}  // namespace nb

#include "step_kernel_main.cuh"  // the kernel body and its launcher (second half of this file)
