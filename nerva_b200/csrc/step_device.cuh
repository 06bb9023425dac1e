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

__device__ __forceinline__ void add_norm_to_smem(uint16_t *x, const float *a, const float *b,
                                                 const uint16_t *bias, const uint16_t *w, float eps,
                                                 uint32_t cols, float *resid_out, float *scratch) {
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
          const float4 t = __ldcg(reinterpret_cast<const float4 *>(b) + i);
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
  float sumsq = 0.0f;
  for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) {
    float r = b != nullptr ? __ldcg(b + i) : __ldcg(a + i);
    if (bias != nullptr) r += bf16_bits_to_f32(bias[i]);
    if (b != nullptr) r += __ldcg(a + i);
    sumsq += r * r;
  }
  const float total = block_sum(sumsq, scratch);
  const float scale = rsqrtf(total / static_cast<float>(cols) + eps);
  for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) {
    float r = b != nullptr ? __ldcg(b + i) : __ldcg(a + i);
    if (bias != nullptr) r += bf16_bits_to_f32(bias[i]);
    if (b != nullptr) r += __ldcg(a + i);
    if (resid_out != nullptr) resid_out[i] = r;
    x[i] = f32_to_bf16_bits(r * scale * bf16_bits_to_f32(w[i]));
  }
}

}  // namespace nb
