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

// The same prologue for a residual stream that is already summed (the producer's epilogue
// added its output to it): x = bf16(a * rsqrt(mean(a^2) + eps) * w).  The norm weights do not
// depend on the previous kernel, so norm_weights_preload fetches them before the dependency
// wait and the wait is followed by one 16-byte load per thread and iteration.
struct NormWeightRegs {
  uint2 w[kNormRegIters];
};
__device__ __forceinline__ bool norm_single_eligible(const float *a, const uint16_t *w, uint32_t cols) {
  return cols % 4u == 0 && cols / 4u <= kNormRegIters * blockDim.x && (reinterpret_cast<uintptr_t>(a) & 15u) == 0 &&
         (reinterpret_cast<uintptr_t>(w) & 7u) == 0;
}
__device__ __forceinline__ void norm_weights_preload(NormWeightRegs &regs, const uint16_t *w, uint32_t cols) {
  const uint32_t vecs = cols / 4u;
#pragma unroll
  for (uint32_t k = 0; k < kNormRegIters; ++k) {
    const uint32_t i = threadIdx.x + k * blockDim.x;
    regs.w[k] = i < vecs ? reinterpret_cast<const uint2 *>(w)[i] : make_uint2(0u, 0u);
  }
}
// Two halves, so that the caller can issue other memory traffic (the rest of its weight ring)
// behind the activation loads instead of in front of them: norm_single_load issues the loads,
// norm_single_finish consumes them.
struct NormValueRegs {
  float4 v[kNormRegIters];
};
__device__ __forceinline__ void norm_single_load(NormValueRegs &r, const float *a, uint32_t cols) {
  const uint32_t vecs = cols / 4u;
#pragma unroll
  for (uint32_t k = 0; k < kNormRegIters; ++k) {
    const uint32_t i = threadIdx.x + k * blockDim.x;
    r.v[k] = i < vecs ? __ldcg(reinterpret_cast<const float4 *>(a) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
}
__device__ __forceinline__ void norm_single_finish(uint16_t *x, const NormValueRegs &loaded, const NormWeightRegs &regs,
                                                   float eps, uint32_t cols, float *scratch) {
  const uint32_t vecs = cols / 4u;
  const float4 *r = loaded.v;
  float sumsq = 0.0f;
#pragma unroll
  for (uint32_t k = 0; k < kNormRegIters; ++k) {
    const uint32_t i = threadIdx.x + k * blockDim.x;
    if (i < vecs) {
      const float4 v = r[k];
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
      const uint2 wb = regs.w[k];
      uint2 out;
      out.x = static_cast<uint32_t>(f32_to_bf16_bits(v.x * scale * bf16x2_lo(wb.x))) |
              (static_cast<uint32_t>(f32_to_bf16_bits(v.y * scale * bf16x2_hi(wb.x))) << 16);
      out.y = static_cast<uint32_t>(f32_to_bf16_bits(v.z * scale * bf16x2_lo(wb.y))) |
              (static_cast<uint32_t>(f32_to_bf16_bits(v.w * scale * bf16x2_hi(wb.y))) << 16);
      reinterpret_cast<uint2 *>(x)[i] = out;
    }
  }
}

// Tensor-parallel form of the same prologue: `b` is the sum over the ranks of
// partial vectors that arrive from the other GPUs while this runs.  recv holds
// [world][cols] 8-byte entries, value bits in the low word and a tag in the high
// word; a writer stores an entry with ONE 8-byte store, so an entry whose tag is
// the expected one carries its value (no fence, no separate flag).  Each thread
// polls exactly the entries it needs (bounded, see kPeerWaitCycleLimit; on expiry the error
// word is set and the step fails) and adds the partials in rank order, so every rank
// computes the same r bit for bit.  cols % 4 == 0 and cols <= 4 * kNormRegIters *
// blockDim.x.
constexpr uint32_t kMaxGatherWorld = 8;

__device__ __forceinline__ ulonglong2 ld_volatile_16(const ulonglong2 *p) {
  ulonglong2 v;
  asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(v.x), "=l"(v.y) : "l"(p) : "memory");
  return v;
}

// WORLD is the number of ranks (compile time, so that the entries in flight live
// in registers); a thread keeps BATCH of its float4 groups from all ranks in
// flight at once, so the whole gather is one or two round trips to L2 once the
// data has arrived.
template <uint32_t WORLD>
__device__ __forceinline__ void gather_norm_to_smem(uint16_t *x, const float *a,
                                                    const unsigned long long *recv, uint32_t tag,
                                                    const uint16_t *bias, const uint16_t *w, float eps,
                                                    uint32_t cols, float *resid_out, float *scratch,
                                                    uint32_t *error_word) {
  constexpr uint32_t BATCH = WORLD <= 4 ? 4 : 2;
  static_assert(kNormRegIters % BATCH == 0, "batches tile the register-resident groups");
  const uint32_t vecs = cols / 4u;
  float4 r[kNormRegIters];
  uint2 wk[kNormRegIters];
  float sumsq = 0.0f;
  const long long start = clock64();
  bool gave_up = false;
#pragma unroll
  for (uint32_t k0 = 0; k0 < kNormRegIters; k0 += BATCH) {
    if (k0 * blockDim.x >= vecs) break;
    float4 av[BATCH];
#pragma unroll
    for (uint32_t kb = 0; kb < BATCH; ++kb) {
      const uint32_t i = threadIdx.x + (k0 + kb) * blockDim.x;
      if (i < vecs) {
        av[kb] = __ldcg(reinterpret_cast<const float4 *>(a) + i);
        wk[k0 + kb] = reinterpret_cast<const uint2 *>(w)[i];
      }
    }
    ulonglong2 lo[BATCH][WORLD], hi[BATCH][WORLD];
    uint32_t polls = 0;
    for (;;) {
#pragma unroll
      for (uint32_t kb = 0; kb < BATCH; ++kb) {
        const uint32_t i = threadIdx.x + (k0 + kb) * blockDim.x;
        if (i < vecs) {
#pragma unroll
          for (uint32_t q = 0; q < WORLD; ++q) {
            const ulonglong2 *src =
                reinterpret_cast<const ulonglong2 *>(recv + static_cast<uint64_t>(q) * cols + 4u * i);
            lo[kb][q] = ld_volatile_16(src);
            hi[kb][q] = ld_volatile_16(src + 1);
          }
        }
      }
      bool ok = true;
#pragma unroll
      for (uint32_t kb = 0; kb < BATCH; ++kb) {
        const uint32_t i = threadIdx.x + (k0 + kb) * blockDim.x;
        if (i < vecs) {
#pragma unroll
          for (uint32_t q = 0; q < WORLD; ++q) {
            ok = ok && static_cast<uint32_t>(lo[kb][q].x >> 32) == tag &&
                 static_cast<uint32_t>(lo[kb][q].y >> 32) == tag &&
                 static_cast<uint32_t>(hi[kb][q].x >> 32) == tag &&
                 static_cast<uint32_t>(hi[kb][q].y >> 32) == tag;
          }
        }
      }
      if (ok || gave_up) break;
      // looked at only while waiting: first whether an earlier exchange of this step gave up, then the clock
      if ((polls++ & 63u) == 0) {
        if (step_already_failed(error_word)) {
          gave_up = true;
        } else if (clock64() - start > kPeerWaitCycleLimit) {
          gave_up = true;
          report_error(error_word, kErrPeerWaitTimeout);
        }
      }
    }
#pragma unroll
    for (uint32_t kb = 0; kb < BATCH; ++kb) {
      const uint32_t i = threadIdx.x + (k0 + kb) * blockDim.x;
      if (i < vecs) {
        float4 t = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (uint32_t q = 0; q < WORLD; ++q) {
          const float4 u = make_float4(__uint_as_float(static_cast<uint32_t>(lo[kb][q].x)),
                                       __uint_as_float(static_cast<uint32_t>(lo[kb][q].y)),
                                       __uint_as_float(static_cast<uint32_t>(hi[kb][q].x)),
                                       __uint_as_float(static_cast<uint32_t>(hi[kb][q].y)));
          if (q == 0) {
            t = u;
          } else {
            t.x += u.x;
            t.y += u.y;
            t.z += u.z;
            t.w += u.w;
          }
        }
        if (bias != nullptr) {
          t.x += bf16_bits_to_f32(bias[4u * i]);
          t.y += bf16_bits_to_f32(bias[4u * i + 1u]);
          t.z += bf16_bits_to_f32(bias[4u * i + 2u]);
          t.w += bf16_bits_to_f32(bias[4u * i + 3u]);
        }
        float4 v = av[kb];
        v.x = t.x + v.x;
        v.y = t.y + v.y;
        v.z = t.z + v.z;
        v.w = t.w + v.w;
        r[k0 + kb] = v;
        sumsq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
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
}

// First stage of the tensor-parallel gather when every block would otherwise read all
// WORLD partial vectors: block b adds the ranks' partials (in rank order) for ITS slice of
// the vector only, and publishes the sums as tagged 8-byte entries in `reduced` (local
// memory, same layout as one rank's slot).  Every block then gathers the whole vector from
// `reduced` with gather_norm_to_smem<1>.  Blocks of one launch wait on each other's slices
// here: the launch must fit the device in one wave (one block per SM), and the waits are
// bounded like all others.
template <uint32_t WORLD>
__device__ __forceinline__ void reduce_partials_slice(const unsigned long long *recv,
                                                      unsigned long long *reduced, uint32_t tag,
                                                      uint32_t cols, uint32_t *error_word) {
  const uint32_t groups = cols / 4u;
  const uint32_t begin = static_cast<uint32_t>(static_cast<uint64_t>(groups) * blockIdx.x / gridDim.x);
  const uint32_t end = static_cast<uint32_t>(static_cast<uint64_t>(groups) * (blockIdx.x + 1u) / gridDim.x);
  const long long start = clock64();
  bool gave_up = false;
  for (uint32_t g = begin + threadIdx.x; g < end; g += blockDim.x) {
    ulonglong2 lo[WORLD], hi[WORLD];
    uint32_t polls = 0;
    for (;;) {
#pragma unroll
      for (uint32_t q = 0; q < WORLD; ++q) {
        const ulonglong2 *src = reinterpret_cast<const ulonglong2 *>(recv + static_cast<uint64_t>(q) * cols + 4u * g);
        lo[q] = ld_volatile_16(src);
        hi[q] = ld_volatile_16(src + 1);
      }
      bool ok = true;
#pragma unroll
      for (uint32_t q = 0; q < WORLD; ++q) {
        ok = ok && static_cast<uint32_t>(lo[q].x >> 32) == tag && static_cast<uint32_t>(lo[q].y >> 32) == tag &&
             static_cast<uint32_t>(hi[q].x >> 32) == tag && static_cast<uint32_t>(hi[q].y >> 32) == tag;
      }
      if (ok || gave_up) break;
      // looked at only while waiting: first whether an earlier exchange of this step gave up, then the clock
      if ((polls++ & 63u) == 0) {
        if (step_already_failed(error_word)) {
          gave_up = true;
        } else if (clock64() - start > kPeerWaitCycleLimit) {
          gave_up = true;
          report_error(error_word, kErrPeerWaitTimeout);
        }
      }
    }
    float4 t = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (uint32_t q = 0; q < WORLD; ++q) {
      const float4 u = make_float4(__uint_as_float(static_cast<uint32_t>(lo[q].x)),
                                   __uint_as_float(static_cast<uint32_t>(lo[q].y)),
                                   __uint_as_float(static_cast<uint32_t>(hi[q].x)),
                                   __uint_as_float(static_cast<uint32_t>(hi[q].y)));
      if (q == 0) {
        t = u;
      } else {
        t.x += u.x;
        t.y += u.y;
        t.z += u.z;
        t.w += u.w;
      }
    }
    const unsigned long long high = static_cast<unsigned long long>(tag) << 32;
    unsigned long long *dst = reduced + 4u * g;
    asm volatile("st.volatile.global.v2.u64 [%0], {%1, %2};" ::"l"(dst), "l"(high | __float_as_uint(t.x)),
                 "l"(high | __float_as_uint(t.y))
                 : "memory");
    asm volatile("st.volatile.global.v2.u64 [%0], {%1, %2};" ::"l"(dst + 2), "l"(high | __float_as_uint(t.z)),
                 "l"(high | __float_as_uint(t.w))
                 : "memory");
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
