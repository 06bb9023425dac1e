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

}  // namespace
}  // namespace nb

#include "step_kernel_main.cuh"  // the kernel body and its launcher (second half of this file)
