// Parameters and device helpers of the whole-step kernel (engine 1).
#pragma once

#include "kernels.cuh"
#include "step_device.cuh"
#include "weight_stream_multi.cuh"

namespace nb {

struct StepLayerDev {
  const uint16_t *rms_attn, *rms_mlp, *q_norm, *k_norm;
  const uint16_t *q_bias, *k_bias, *v_bias, *o_bias;
  uint16_t *key_pages, *value_pages;  // this layer's [pages][16][kv_hidden] bf16
};

struct StepKernelParams {
  StepState st;
  const uint16_t *embeddings, *final_norm;
  const StepLayerDev *layers;
  const JobDesc *jobs;  // 4 per layer (QKV, O, gate/up, down) + lm_head
  uint32_t layer_count, job_count;
  uint32_t hidden, heads, kv_heads, head_dim, intermediate, vocab;
  float eps, rope_theta;
  const uint32_t *page_table;
  uint32_t page_count;
  float *h_a, *h_b, *qkv, *o_out, *down, *logits;
  uint16_t *ff_bf16;
  float *partial_acc, *partial_m, *partial_l;  // [heads][attn_splits][...]
  uint32_t attn_splits;
  float *best_value;
  uint32_t *best_index;
  uint32_t *barrier_counter;  // zeroed before every launch
  uint32_t sample;
  uint32_t x_elems;  // capacity of the shared activation vector (bf16 elements)
};

constexpr uint32_t kStepMaxSplits = 4;  // attention items per query head
constexpr uint32_t kStepAttnTile = 32;
constexpr uint32_t kStepMaxHeadDim = 128;

// Shared memory beyond the ring and the activation vector.
struct StepShared {
  uint64_t bars[kStreamWarps * kStreamSlots];
  float scratch[64];
  uint32_t dead;                                   // a grid barrier timed out
  alignas(16) float q[kStepMaxHeadDim];            // this item's query, pre-scaled (read as float4)
  alignas(16) float k_new[kStepMaxHeadDim];        // current token's K and V, bf16-rounded
  alignas(16) float v_new[kStepMaxHeadDim];
  alignas(16) float p[kStreamWarps][kStepAttnTile];
  alignas(16) float merge[kStreamWarps][kStepMaxHeadDim + 2];
};

// Grid-wide barrier number `index` (1-based) of this launch.  All threads of
// all blocks call it.  A block that waits longer than the cycle limit records
// kErrGridBarrierTimeout, marks itself dead and stops waiting at later barriers,
// so the kernel always terminates.
__device__ __forceinline__ void grid_barrier(const StepKernelParams &p, StepShared &sh,
                                             uint32_t index) {
  __syncthreads();
  if (threadIdx.x == 0 && sh.dead == 0) {
    __threadfence();
    atomicAdd(p.barrier_counter, 1u);
    const uint32_t target = index * gridDim.x;
    const long long start = clock64();
    for (;;) {
      uint32_t seen;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.barrier_counter) : "memory");
      if (seen >= target) break;
      if (clock64() - start > kWaitCycleLimit) {
        sh.dead = 1;
        report_error(p.st.error_word, kErrGridBarrierTimeout);
        break;
      }
    }
    __threadfence();
  }
  __syncthreads();
}

// Per-head RMSNorm + RoPE of one head held four-elements-per-lane by one warp
// (element e = lane + 32 k).  head_dim is a multiple of 64, so both members of
// every rotary pair (e, e + d/2) live in the same lane.
template <uint32_t PER>  // elements per lane; head_dim = 32 * PER
__device__ __forceinline__ void head_norm_rope(float (&v)[PER], const uint16_t *norm, float eps,
                                               float theta, uint32_t position) {
  constexpr uint32_t D = PER * 32u;
  constexpr uint32_t HALF = PER / 2u;  // v[k] pairs with v[k + HALF]
  const uint32_t lane = threadIdx.x & 31u;
  if (norm != nullptr) {
    float ss = 0.0f;
#pragma unroll
    for (uint32_t k = 0; k < PER; ++k) ss += v[k] * v[k];
    ss = warp_sum(ss);
    const float scale = rsqrtf(ss / static_cast<float>(D) + eps);
#pragma unroll
    for (uint32_t k = 0; k < PER; ++k) v[k] *= scale * bf16_bits_to_f32(norm[lane + 32u * k]);
  }
  if (theta > 0.0f) {
#pragma unroll
    for (uint32_t k = 0; k < HALF; ++k) {
      const uint32_t i = lane + 32u * k;
      const float exponent = static_cast<float>(2u * i) / static_cast<float>(D);
      const float angle = static_cast<float>(position) / powf(theta, exponent);
      float s, c;
      sincosf(angle, &s, &c);
      const float left = v[k], right = v[k + HALF];
      v[k] = left * c - right * s;
      v[k + HALF] = right * c + left * s;
    }
  }
}

}  // namespace nb
