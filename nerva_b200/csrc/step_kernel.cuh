// Parameters and device helpers of the whole-step kernel (engine 1).
#pragma once

#include "attention_device.cuh"
#include "kernels.cuh"
#include "row_stream.cuh"
#include "step_device.cuh"

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
  uint32_t x_elems;    // capacity of the shared activation vector (bf16 elements)
  uint32_t row_elems;  // capacity of the shared row-total buffer (floats)
  // Optional: block 0 adds the SM cycles it spent in each phase of the step
  // (kPhase* slots), for tuning.  Null in normal operation.
  unsigned long long *phase_cycles;
};

enum StepPhase : uint32_t {
  kPhaseQkvPrologue = 0, kPhaseQkv, kPhaseBarrierQkv, kPhaseAttention, kPhaseBarrierAttention,
  kPhaseOPrologue, kPhaseO, kPhaseBarrierO, kPhaseGateUpPrologue, kPhaseGateUp, kPhaseBarrierGateUp,
  kPhaseDownPrologue, kPhaseDown, kPhaseBarrierDown, kPhaseLmHead, kPhaseTail, kPhaseCount
};

constexpr uint32_t kStepMaxSplits = 4;  // attention items per query head
constexpr uint32_t kStepAttnTile = 32;
constexpr uint32_t kStepMaxHeadDim = 128;
constexpr uint32_t kStepMaxHeads = 64;

// Shared memory beyond the ring, the activation vector and the row totals.
struct StepShared {
  StreamShared stream;
  float scratch[64];
  uint32_t dead;                                   // a grid barrier timed out
  AttnItemShared<kStreamWarps> attn;
  alignas(16) float weights[kStepMaxHeads * kStepMaxSplits];  // merge weights per (head, item)
};
// The per-warp merge records of the attention phase ([warps][head_dim + 2]
// floats) overlay the activation vector, which is dead between the QKV
// projection and the O prologue.
constexpr uint32_t kStepMergeStride = kAttnMergeStride;
constexpr uint32_t kStepMergeBytes = kStreamWarps * kStepMergeStride * 4u;
__host__ __device__ inline uint32_t step_round128(uint32_t v) { return (v + 127u) & ~127u; }
// Bytes reserved for the activation vector (and the merge records that overlay it).
__host__ __device__ inline uint32_t step_x_bytes(uint32_t x_elems) {
  const uint32_t x = step_round128(x_elems * 2u);
  const uint32_t m = step_round128(kStepMergeBytes);
  return x > m ? x : m;
}

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

}  // namespace nb
