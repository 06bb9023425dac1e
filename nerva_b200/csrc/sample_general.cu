// Temperature / top-k / top-p sampling of the resident decode step with the reference's
// seeded, counter-based randomness: a (logits, position, seed) triple always gives the same
// token (behaviour of hf_decode_sequence/sampler.cu:18-33 and 120-392).
//
//   greedy          temperature <= 0 or top_k == 1: the arg-max path, not this kernel
//   Gumbel-max      top_k == 0 and top_p >= 0.999999: arg-max over the finite logits of
//                   logit / temperature - log(-log(u(seed, position, index, salt 0)))
//   top-k / top-p   the c = min(top_k or 128, 128, vocab) largest finite logits by (value
//                   descending, index ascending); softmax with temperature over them; the
//                   shortest prefix whose mass reaches top_p; one draw
//                   u(seed, position, 0, salt 1) * kept mass walks that prefix
//
// One block of 1024 threads over the fp32 logits that the lm_head projection left in global
// memory (600 KB for a 152k vocabulary: L2-resident, so the repeated scans cost microseconds).
// The top-c set is exact.  Every candidate has a unique 64-bit key (sign-flipped float bits
// above the inverted index), the c-th largest key is found by a radix descent from the most
// significant byte (at most eight scans, usually four since the index bytes rarely matter),
// the keys at or above it are gathered and sorted by a 128-wide bitonic network.  The softmax
// weights are computed once, in parallel; one thread then accumulates them in rank order, the
// order the reference accumulates in, so the three sums see the same rounding.
#include <math.h>

#include "common.cuh"
#include "kernels.cuh"

namespace nb {
namespace {

constexpr uint32_t kThreads = 1024;
constexpr uint32_t kWarps = kThreads / 32;
constexpr uint32_t kCandidates = 128;  // the reference's top-k ceiling (sampler.cu:11)

// splitmix64 finaliser over seed ^ position<<32 ^ token ^ salt<<48, top 24 bits -> (0, 1).
__device__ __forceinline__ float counter_uniform(uint64_t seed, uint32_t position, uint32_t token, uint32_t salt) {
  uint64_t z = (seed ^ (uint64_t(position) << 32) ^ uint64_t(token) ^ (uint64_t(salt) << 48)) + 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  z ^= z >> 31;
  return (float(uint32_t(z >> 40) & 0xffffffu) + 1.0f) / 16777217.0f;
}
// Radix-sortable float: negative values have all bits flipped, the others only the sign.
__device__ __forceinline__ uint32_t sortable(float value) {
  const uint32_t bits = __float_as_uint(value);
  return bits ^ (uint32_t(int32_t(bits) >> 31) | 0x80000000u);
}
__device__ __forceinline__ float unsortable(uint32_t s) {
  return __uint_as_float(s ^ (((s >> 31) - 1u) | 0x80000000u));
}
// Larger key = larger value, then smaller index.
__device__ __forceinline__ uint64_t make_key(float value, uint32_t index) {
  return (uint64_t(sortable(value)) << 32) | uint64_t(~index);
}

struct Pick {
  float value;
  uint32_t index;
  __device__ __forceinline__ void take(float v, uint32_t i) {
    if (v > value || (v == value && i < index)) {
      value = v;
      index = i;
    }
  }
};

__global__ void __launch_bounds__(kThreads) sample_general_kernel(StepState st, const float *logits,
                                                                  const SamplerParams *params) {
  __shared__ Pick warp_pick[kWarps];
  __shared__ uint32_t hist[256];
  __shared__ uint64_t keys[kCandidates];
  __shared__ float weight[kCandidates];
  __shared__ uint64_t prefix_sh;
  __shared__ uint32_t need_sh, count_sh, token_sh;
  pdl_wait();  // the logits come from the lm_head projection
  const uint32_t position = *st.cursor;
  if (position >= st.max_context) return;
  const SamplerParams sp = *params;
  const uint32_t tid = threadIdx.x;
  const float inv_temperature = 1.0f / sp.temperature;

  if (sp.top_k == 0 && sp.top_p >= 0.999999f) {
    Pick mine{-INFINITY, 0u};
    for (uint32_t i = tid; i < st.vocab; i += kThreads) {
      const float v = logits[i];
      if (!isfinite(v)) continue;
      const float gumbel = -logf(-logf(counter_uniform(sp.seed, position, i, 0)));
      mine.take(v * inv_temperature + gumbel, i);
    }
    for (int offset = 16; offset > 0; offset >>= 1)
      mine.take(__shfl_xor_sync(0xffffffffu, mine.value, offset), __shfl_xor_sync(0xffffffffu, mine.index, offset));
    if ((tid & 31u) == 0) warp_pick[tid >> 5] = mine;
    __syncthreads();
    if (tid == 0) {
      Pick all{-INFINITY, 0u};
      for (uint32_t w = 0; w < kWarps; ++w) all.take(warp_pick[w].value, warp_pick[w].index);
      token_sh = all.index;
    }
  } else {
    if (tid == 0) {
      uint32_t want = sp.top_k == 0 || sp.top_k > kCandidates ? kCandidates : sp.top_k;
      need_sh = want < st.vocab ? want : st.vocab;
      prefix_sh = 0;
      count_sh = 0;
    }
    // Radix descent to the need-th largest key.  `open` turns false when fewer finite
    // candidates exist than wanted: then every finite candidate is taken.
    bool open = true;
    uint64_t decided = 0;  // mask of the key bits that prefix_sh fixes
    for (int shift = 56; shift >= 0 && open; shift -= 8) {
      if (tid < 256) hist[tid] = 0;
      __syncthreads();
      const uint64_t prefix = prefix_sh;
      for (uint32_t i = tid; i < st.vocab; i += kThreads) {
        const float v = logits[i];
        if (!isfinite(v)) continue;
        const uint64_t key = make_key(v, i);
        if ((key & decided) == prefix) atomicAdd(hist + uint32_t((key >> shift) & 0xffu), 1u);
      }
      __syncthreads();
      if (tid == 0) {
        uint32_t above = 0, need = need_sh;
        int digit = 255;
        while (digit >= 0 && above + hist[digit] < need) above += hist[digit--];
        if (digit < 0) {
          need_sh = 0;  // not enough candidates under this prefix (only possible at the top digit)
        } else {
          prefix_sh = prefix | (uint64_t(uint32_t(digit)) << shift);
          need_sh = need - above;
        }
      }
      __syncthreads();
      open = need_sh != 0;
      decided |= 0xffull << shift;
    }
    const uint64_t threshold = open ? prefix_sh : 0ull;
    for (uint32_t i = tid; i < st.vocab; i += kThreads) {
      const float v = logits[i];
      if (!isfinite(v)) continue;
      const uint64_t key = make_key(v, i);
      if (key >= threshold) {
        const uint32_t at = atomicAdd(&count_sh, 1u);
        if (at < kCandidates) keys[at] = key;
      }
    }
    __syncthreads();
    const uint32_t selected = count_sh < kCandidates ? count_sh : kCandidates;
    if (tid >= selected && tid < kCandidates) keys[tid] = 0;  // below every real key
    __syncthreads();
    for (uint32_t width = 2; width <= kCandidates; width <<= 1) {
      for (uint32_t stride = width >> 1; stride != 0; stride >>= 1) {
        const uint32_t partner = tid ^ stride;
        if (tid < kCandidates && partner > tid) {
          const uint64_t a = keys[tid], b = keys[partner];
          const bool down = (tid & width) == 0;
          if (down ? a < b : a > b) {
            keys[tid] = b;
            keys[partner] = a;
          }
        }
        __syncthreads();
      }
    }
    if (tid < selected) {
      const float top = unsortable(uint32_t(keys[0] >> 32));
      weight[tid] = expf((unsortable(uint32_t(keys[tid] >> 32)) - top) * inv_temperature);
    }
    __syncthreads();
    if (tid == 0) {
      uint32_t token = 0;
      if (selected != 0) {
        float total = 0.0f;
        for (uint32_t r = 0; r < selected; ++r) total += weight[r];
        uint32_t kept = selected;
        float kept_mass = total;
        if (sp.top_p < 0.999999f) {
          kept_mass = 0.0f;
          for (kept = 0; kept < selected;) {
            kept_mass += weight[kept++];
            if (total > 0.0f && kept_mass / total >= sp.top_p) break;
          }
        }
        token = ~uint32_t(keys[0]);
        if (kept_mass > 0.0f && kept != 0) {
          const float draw = counter_uniform(sp.seed, position, 0, 1) * kept_mass;
          float running = 0.0f;
          uint32_t r = 0;
          for (; r + 1 < kept; ++r) {
            running += weight[r];
            if (draw <= running) break;
          }
          token = ~uint32_t(keys[r]);  // the last kept rank when the draw passes every earlier one
        }
      }
      token_sh = token;
    }
  }
  __syncthreads();
  if (tid == 0) {
    NervaCudaSyntheticTokenSlot *slot = st.slots + position;
    slot->request_id = 1;
    slot->sequence_id = 1;
    slot->token_index = position;
    slot->token = token_sh;
    slot->version = uint64_t(position) + 1u;
    slot->completion = 1;  // device complete
    slot->host_copied = 0;
    *st.cursor = position + 1;
  }
}

}  // namespace

cudaError_t launch_sample_general(cudaStream_t stream, const StepState &st, const float *logits,
                                  const SamplerParams *params, bool pdl) {
  return launch_with_pdl(sample_general_kernel, dim3(1), dim3(kThreads), 0, stream, pdl, st, logits, params);
}

}  // namespace nb
