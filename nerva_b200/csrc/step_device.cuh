// Device functions shared by the per-operator kernels and the whole-step
// kernel: the residual-add + RMSNorm prologue that turns the f32 residual
// stream into the bf16 activation vector of the next projection.
#pragma once

#include "common.cuh"

namespace nb {

// r = (b + bias) + a   (b, bias optional);  x = bf16(r * rsqrt(mean(r^2) + eps) * w)
// Every thread of the block calls it; `x` is shared memory, `resid_out` (global,
// optional) receives r.  Same arithmetic as the reference's residual + RMSNorm
// kernels (hf_decode_sequence/kernels.cu:577-593,651-687, device_ops.cuh:334-358):
// the O/down output (+ bias) is added to the stream, the scale is rsqrtf of the
// mean square plus eps, and (value * scale) * weight is rounded to bf16.
//
// The values stay in registers between the two passes and the loads are 128-bit,
// so a block touches each input once: with cols <= kNormRegCols the whole
// prologue is one round trip to L2.
constexpr uint32_t kNormRegIters = 8;  // float4 per thread held in registers

//
// b_count > 1 (tensor parallel): b holds b_count partial vectors of `cols`
// floats, one per rank; they are added in rank order, so every rank computes
// the same r bit for bit.
__device__ __forceinline__ void add_norm_to_smem(uint16_t *x, const float *a, const float *b,
                                                 const uint16_t *bias, const uint16_t *w, float eps,
                                                 uint32_t cols, float *resid_out, float *scratch,
                                                 uint32_t b_count = 1) {
  const uint32_t vecs = cols / 4u;
  const bool fast = cols % 4u == 0 && bias == nullptr && vecs <= kNormRegIters * blockDim.x &&
                    (reinterpret_cast<uintptr_t>(a) & 15u) == 0 &&
                    (b == nullptr || (reinterpret_cast<uintptr_t>(b) & 15u) == 0) &&
                    (resid_out == nullptr || (reinterpret_cast<uintptr_t>(resid_out) & 15u) == 0) &&
                    (reinterpret_cast<uintptr_t>(w) & 7u) == 0;
  if (fast) {
    float4 r[kNormRegIters];
    uint2 wk[kNormRegIters];
    float sumsq = 0.0f;
#pragma unroll
    for (uint32_t k = 0; k < kNormRegIters; ++k) {
      const uint32_t i = threadIdx.x + k * blockDim.x;
      if (i < vecs) {
        // L2 loads: in the whole-step kernel these vectors were written by other blocks
        float4 v = __ldcg(reinterpret_cast<const float4 *>(a) + i);
        if (b != nullptr) {
          float4 t = __ldcg(reinterpret_cast<const float4 *>(b) + i);
          for (uint32_t q = 1; q < b_count; ++q) {
            const float4 u = __ldcg(reinterpret_cast<const float4 *>(b + static_cast<uint64_t>(q) * cols) + i);
            t.x += u.x;
            t.y += u.y;
            t.z += u.z;
            t.w += u.w;
          }
          v.x = t.x + v.x;
          v.y = t.y + v.y;
          v.z = t.z + v.z;
          v.w = t.w + v.w;
        }
        r[k] = v;
        wk[k] = reinterpret_cast<const uint2 *>(w)[i];  // in flight together with a and b
        sumsq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
    }
    const float total = block_sum(sumsq, scratch);
    const float scale = rsqrtf(total / static_cast<float>(cols) + eps);
#pragma unroll
    for (uint32_t k = 0; k < kNormRegIters; ++k) {
      const uint32_t i = threadIdx.x + k * blockDim.x;
      if (i < vecs) {
        const float4 v = r[k];
        if (resid_out != nullptr) reinterpret_cast<float4 *>(resid_out)[i] = v;
        const uint2 wb = wk[k];
        uint2 out;
        out.x = static_cast<uint32_t>(f32_to_bf16_bits(v.x * scale * bf16x2_lo(wb.x))) |
                (static_cast<uint32_t>(f32_to_bf16_bits(v.y * scale * bf16x2_hi(wb.x))) << 16);
        out.y = static_cast<uint32_t>(f32_to_bf16_bits(v.z * scale * bf16x2_lo(wb.y))) |
                (static_cast<uint32_t>(f32_to_bf16_bits(v.w * scale * bf16x2_hi(wb.y))) << 16);
        reinterpret_cast<uint2 *>(x)[i] = out;
      }
    }
    return;
  }
  auto b_sum = [&](uint32_t i) {
    float t = __ldcg(b + i);
    for (uint32_t q = 1; q < b_count; ++q) t += __ldcg(b + static_cast<uint64_t>(q) * cols + i);
    return t;
  };
  float sumsq = 0.0f;
  for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) {
    float r = b != nullptr ? b_sum(i) : __ldcg(a + i);
    if (bias != nullptr) r += bf16_bits_to_f32(bias[i]);
    if (b != nullptr) r += __ldcg(a + i);
    sumsq += r * r;
  }
  const float total = block_sum(sumsq, scratch);
  const float scale = rsqrtf(total / static_cast<float>(cols) + eps);
  for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) {
    float r = b != nullptr ? b_sum(i) : __ldcg(a + i);
    if (bias != nullptr) r += bf16_bits_to_f32(bias[i]);
    if (b != nullptr) r += __ldcg(a + i);
    if (resid_out != nullptr) resid_out[i] = r;
    x[i] = f32_to_bf16_bits(r * scale * bf16_bits_to_f32(w[i]));
  }
}

// Prologue of the O projection: merges the split-attention partials of every
// head into the bf16 activation vector,
//   x[h*D + d] = bf16( sum_s acc[h][s][d] w[h][s] ),
//   w[h][s] = 2^{m_s - M} / sum_s l_s 2^{m_s - M}
// (the algebra of hf_decode_sequence/kernels.cu:494-555, base 2).  Two round
// trips to L2 per block: first the (m, l) pairs become normalised weights in
// shared memory (`weights`, heads * S floats), then every thread issues all of
// its partial-accumulator loads before it uses any of them.
constexpr uint32_t kMergeMaxSplits = 8;

__device__ __forceinline__ void merge_attention_to_smem(uint16_t *x, float *weights,
                                                        const float *partial_acc,
                                                        const float *partial_m,
                                                        const float *partial_l, uint32_t heads,
                                                        uint32_t D, uint32_t S) {
  for (uint32_t h = threadIdx.x; h < heads; h += blockDim.x) {
    float ms[kMergeMaxSplits], ls[kMergeMaxSplits];
#pragma unroll
    for (uint32_t s = 0; s < kMergeMaxSplits; ++s) {
      ms[s] = s < S ? __ldcg(partial_m + h * S + s) : -INFINITY;
      ls[s] = s < S ? __ldcg(partial_l + h * S + s) : 0.0f;
    }
    float m = -INFINITY;
#pragma unroll
    for (uint32_t s = 0; s < kMergeMaxSplits; ++s)
      if (ls[s] > 0.0f) m = fmaxf(m, ms[s]);
    float l = 0.0f;
#pragma unroll
    for (uint32_t s = 0; s < kMergeMaxSplits; ++s)
      if (ls[s] > 0.0f) l = fmaf(ls[s], exp2f(ms[s] - m), l);
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (uint32_t s = 0; s < kMergeMaxSplits; ++s)
      if (s < S) weights[h * S + s] = ls[s] > 0.0f ? exp2f(ms[s] - m) * inv : 0.0f;
  }
  __syncthreads();
  constexpr uint32_t kBatch = 4;
  const uint32_t total = heads * D;
  for (uint32_t base = 0; base < total; base += kBatch * blockDim.x) {
    float v[kBatch][kMergeMaxSplits];
#pragma unroll
    for (uint32_t k = 0; k < kBatch; ++k) {
      const uint32_t idx = base + k * blockDim.x + threadIdx.x;
      const uint32_t h = idx / D, d = idx - h * D;
#pragma unroll
      for (uint32_t s = 0; s < kMergeMaxSplits; ++s) {
        v[k][s] = (idx < total && s < S)
                      ? __ldcg(partial_acc + (static_cast<uint64_t>(h) * S + s) * D + d)
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
        for (uint32_t s = 0; s < kMergeMaxSplits; ++s)
          if (s < S) a = fmaf(v[k][s], weights[h * S + s], a);
        x[idx] = f32_to_bf16_bits(a);
      }
    }
  }
}

}  // namespace nb
