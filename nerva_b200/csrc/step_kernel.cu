// The whole decode step as ONE persistent kernel (engine 1).
//
// One block per SM runs every operator of the token: per layer QKV projection,
// q/k norm + RoPE + KV append + attention, O projection, gate/up projection with
// SwiGLU, down projection; then lm_head with greedy arg-max and the token-ring
// write.  Blocks meet at a grid barrier between operators.  What makes this
// faster than one launch per operator is the weight stream (weight_stream_multi.cuh):
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
constexpr float kLog2e = 1.4426950408889634f;

struct StoreEpi {
  float *out;
  __device__ __forceinline__ void row(uint32_t r, float v) {
    if ((threadIdx.x & 31u) == 0) out[r] = v;
  }
};
struct SwigluEpi {
  uint16_t *out;
  float gate;
  __device__ __forceinline__ void row(uint32_t r, float v) {
    if ((r & 1u) == 0) {
      gate = v;
    } else if ((threadIdx.x & 31u) == 0) {
      out[r >> 1] = f32_to_bf16_bits(silu(gate) * v);
    }
  }
};
__device__ __forceinline__ bool better(float v, uint32_t i, float bv, uint32_t bi) {
  return v > bv || (v == bv && i < bi);
}
struct ArgmaxEpi {
  float *out;
  float best_v;
  uint32_t best_i;
  __device__ __forceinline__ void row(uint32_t r, float v) {
    if ((threadIdx.x & 31u) == 0) out[r] = v;
    if (isfinite(v) && better(v, r, best_v, best_i)) {
      best_v = v;
      best_i = r;
    }
  }
};

__device__ __forceinline__ float exp2_or_zero(float x) { return exp2f(x); }  // exp2f(-inf) == 0

// Attention of one layer: work item = (query head, split of the cached tokens).
// The current token's K/V row is computed by every item that needs it and kept
// in shared memory; only one item per KV head stores it to the page.
template <uint32_t PER>
__device__ void attention_phase(const StepKernelParams &p, StepShared &sh, const StepLayerDev &L,
                                uint32_t position) {
  constexpr uint32_t D = PER * 32u;
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const uint32_t group = p.heads / p.kv_heads;
  const uint32_t attention_hidden = p.heads * D, kv_hidden = p.kv_heads * D;
  const uint32_t S = p.attn_splits;
  const uint32_t hist = position;  // tokens already in the cache
  const uint32_t tiles_total = (hist + kStepAttnTile - 1u) / kStepAttnTile;
  const uint32_t tiles_per_split = (tiles_total + S - 1u) / S;
  const float qscale = kLog2e * rsqrtf(static_cast<float>(D));

  for (uint32_t item = blockIdx.x; item < p.heads * S; item += gridDim.x) {
    const uint32_t h = item / S, s = item - h * S, kvh = h / group;
    const uint32_t tile_begin = s * tiles_per_split;
    uint32_t tile_end = tile_begin + tiles_per_split;
    if (tile_end > tiles_total) tile_end = tiles_total;
    const bool owns_current = s + 1u == S;

    if (warp == 0) {
      float v[PER];
#pragma unroll
      for (uint32_t k = 0; k < PER; ++k) {
        const uint32_t e = lane + 32u * k;
        v[k] = __ldcg(p.qkv + h * D + e);
        if (L.q_bias != nullptr) v[k] += bf16_bits_to_f32(L.q_bias[h * D + e]);
      }
      head_norm_rope<PER>(v, L.q_norm, p.eps, p.rope_theta, position);
#pragma unroll
      for (uint32_t k = 0; k < PER; ++k) sh.q[lane + 32u * k] = v[k] * qscale;
    } else if (warp == 1 && owns_current) {
      float kk[PER], vv[PER];
#pragma unroll
      for (uint32_t k = 0; k < PER; ++k) {
        const uint32_t e = lane + 32u * k;
        kk[k] = __ldcg(p.qkv + attention_hidden + kvh * D + e);
        vv[k] = __ldcg(p.qkv + attention_hidden + kv_hidden + kvh * D + e);
        if (L.k_bias != nullptr) kk[k] += bf16_bits_to_f32(L.k_bias[kvh * D + e]);
        if (L.v_bias != nullptr) vv[k] += bf16_bits_to_f32(L.v_bias[kvh * D + e]);
      }
      head_norm_rope<PER>(kk, L.k_norm, p.eps, p.rope_theta, position);
      const uint32_t logical = position / NERVA_KV_CACHE_BLOCK_TOKENS;
      uint32_t phys = p.page_table[logical];
      const bool store = h == kvh * group;
      if (phys >= p.page_count) {
        report_error(p.st.error_word, kErrPageOutOfRange);
        phys = 0;
      }
      const uint64_t base = (static_cast<uint64_t>(phys) * NERVA_KV_CACHE_BLOCK_TOKENS +
                             position % NERVA_KV_CACHE_BLOCK_TOKENS) * kv_hidden + kvh * D;
#pragma unroll
      for (uint32_t k = 0; k < PER; ++k) {
        const uint32_t e = lane + 32u * k;
        const uint16_t kb = f32_to_bf16_bits(kk[k]), vb = f32_to_bf16_bits(vv[k]);
        sh.k_new[e] = bf16_bits_to_f32(kb);
        sh.v_new[e] = bf16_bits_to_f32(vb);
        if (store) {
          L.key_pages[base + e] = kb;
          L.value_pages[base + e] = vb;
        }
      }
    }
    __syncthreads();

    float m_run = -INFINITY, l_run = 0.0f, acc[PER];
#pragma unroll
    for (uint32_t i = 0; i < PER; ++i) acc[i] = 0.0f;
    for (uint32_t tile = tile_begin + warp; tile < tile_end; tile += kStreamWarps) {
      const uint32_t token = tile * kStepAttnTile + lane;
      const bool valid = token < hist;
      uint32_t phys = 0;
      if (valid) {
        phys = p.page_table[token / NERVA_KV_CACHE_BLOCK_TOKENS];
        if (phys >= p.page_count) {
          report_error(p.st.error_word, kErrPageOutOfRange);
          phys = 0;
        }
      }
      const uint64_t row = (static_cast<uint64_t>(phys) * NERVA_KV_CACHE_BLOCK_TOKENS +
                            token % NERVA_KV_CACHE_BLOCK_TOKENS) * kv_hidden + kvh * D;
      float score = 0.0f;
      if (valid) {
        const uint4 *k_row = reinterpret_cast<const uint4 *>(L.key_pages + row);
        uint4 kk[D / 8u];
#pragma unroll
        for (uint32_t b = 0; b < D / 8u; ++b) kk[b] = __ldcg(k_row + b);
#pragma unroll
        for (uint32_t b = 0; b < D / 8u; ++b) {
          const float4 qa = *reinterpret_cast<const float4 *>(sh.q + b * 8u);
          const float4 qb = *reinterpret_cast<const float4 *>(sh.q + b * 8u + 4u);
          score = fmaf(bf16x2_lo(kk[b].x), qa.x, score);
          score = fmaf(bf16x2_hi(kk[b].x), qa.y, score);
          score = fmaf(bf16x2_lo(kk[b].y), qa.z, score);
          score = fmaf(bf16x2_hi(kk[b].y), qa.w, score);
          score = fmaf(bf16x2_lo(kk[b].z), qb.x, score);
          score = fmaf(bf16x2_hi(kk[b].z), qb.y, score);
          score = fmaf(bf16x2_lo(kk[b].w), qb.z, score);
          score = fmaf(bf16x2_hi(kk[b].w), qb.w, score);
        }
      } else {
        score = -INFINITY;
      }
      const float m_new = fmaxf(m_run, warp_max(score));
      const float pr = exp2_or_zero(score - m_new);
      const float corr = exp2_or_zero(m_run - m_new);
      l_run = l_run * corr + warp_sum(pr);
      m_run = m_new;
#pragma unroll
      for (uint32_t i = 0; i < PER; ++i) acc[i] *= corr;
      sh.p[warp][lane] = pr;
      __syncwarp();
      const uint32_t count = hist - tile * kStepAttnTile < kStepAttnTile ? hist - tile * kStepAttnTile
                                                                         : kStepAttnTile;
#pragma unroll 8
      for (uint32_t t = 0; t < kStepAttnTile; ++t) {
        const uint32_t phys_t = __shfl_sync(0xffffffffu, phys, t);
        if (t < count) {
          const uint64_t vrow = (static_cast<uint64_t>(phys_t) * NERVA_KV_CACHE_BLOCK_TOKENS +
                                 (tile * kStepAttnTile + t) % NERVA_KV_CACHE_BLOCK_TOKENS) * kv_hidden +
                                kvh * D + lane * PER;
          const float pt = sh.p[warp][t];
          if (PER == 4) {
            const uint2 w = __ldcg(reinterpret_cast<const uint2 *>(L.value_pages + vrow));
            acc[0] = fmaf(pt, bf16x2_lo(w.x), acc[0]);
            acc[1 % PER] = fmaf(pt, bf16x2_hi(w.x), acc[1 % PER]);
            acc[2 % PER] = fmaf(pt, bf16x2_lo(w.y), acc[2 % PER]);
            acc[3 % PER] = fmaf(pt, bf16x2_hi(w.y), acc[3 % PER]);
          } else {
            const uint32_t w = __ldcg(reinterpret_cast<const uint32_t *>(L.value_pages + vrow));
            acc[0] = fmaf(pt, bf16x2_lo(w), acc[0]);
            acc[1 % PER] = fmaf(pt, bf16x2_hi(w), acc[1 % PER]);
          }
        }
      }
      __syncwarp();
    }
    // merge the warps; warp 0 then folds in the current token
#pragma unroll
    for (uint32_t i = 0; i < PER; ++i) sh.merge[warp][lane * PER + i] = acc[i];
    if (lane == 0) {
      sh.merge[warp][D] = m_run;
      sh.merge[warp][D + 1] = l_run;
    }
    __syncthreads();
    if (warp == 0) {
      float m = -INFINITY;
      for (uint32_t w = 0; w < kStreamWarps; ++w) m = fmaxf(m, sh.merge[w][D]);
      float a[PER], l = 0.0f;
#pragma unroll
      for (uint32_t i = 0; i < PER; ++i) a[i] = 0.0f;
      if (m > -INFINITY) {
        for (uint32_t w = 0; w < kStreamWarps; ++w) {
          const float wgt = exp2_or_zero(sh.merge[w][D] - m);
          l = fmaf(sh.merge[w][D + 1], wgt, l);
#pragma unroll
          for (uint32_t i = 0; i < PER; ++i) a[i] = fmaf(sh.merge[w][lane * PER + i], wgt, a[i]);
        }
      }
      if (owns_current) {
        float dot = 0.0f;
#pragma unroll
        for (uint32_t i = 0; i < PER; ++i) dot = fmaf(sh.q[lane * PER + i], sh.k_new[lane * PER + i], dot);
        const float s_new = warp_sum(dot);
        const float m2 = fmaxf(m, s_new);
        const float corr = exp2_or_zero(m - m2);
        const float pr = exp2_or_zero(s_new - m2);
        l = l * corr + pr;
#pragma unroll
        for (uint32_t i = 0; i < PER; ++i) a[i] = a[i] * corr + pr * sh.v_new[lane * PER + i];
        m = m2;
      }
      const uint64_t slot = static_cast<uint64_t>(h) * S + s;
#pragma unroll
      for (uint32_t i = 0; i < PER; ++i) p.partial_acc[slot * D + lane * PER + i] = a[i];
      if (lane == 0) {
        p.partial_m[slot] = m;
        p.partial_l[slot] = l;
      }
    }
    __syncthreads();
  }
}

// x[h*D + d] = bf16( sum_s acc 2^{m_s - M} / sum_s l_s 2^{m_s - M} )
__device__ void merge_attention_to_smem(const StepKernelParams &p, uint16_t *x) {
  const uint32_t D = p.head_dim, S = p.attn_splits;
  for (uint32_t idx = threadIdx.x; idx < p.heads * D; idx += blockDim.x) {
    const uint32_t h = idx / D, d = idx - h * D;
    const uint64_t slot0 = static_cast<uint64_t>(h) * S;
    float m = -INFINITY;
    for (uint32_t s = 0; s < S; ++s) {
      if (__ldcg(p.partial_l + slot0 + s) > 0.0f) m = fmaxf(m, __ldcg(p.partial_m + slot0 + s));
    }
    float l = 0.0f, a = 0.0f;
    for (uint32_t s = 0; s < S; ++s) {
      const float ls = __ldcg(p.partial_l + slot0 + s);
      if (ls > 0.0f) {
        const float wgt = exp2_or_zero(__ldcg(p.partial_m + slot0 + s) - m);
        l = fmaf(ls, wgt, l);
        a = fmaf(__ldcg(p.partial_acc + (slot0 + s) * D + d), wgt, a);
      }
    }
    x[idx] = f32_to_bf16_bits(l > 0.0f ? a / l : 0.0f);
  }
}

template <uint32_t PER>
__global__ void __launch_bounds__(kStreamThreads, 1) decode_step_kernel(StepKernelParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t *ring = smem;
  uint16_t *x = reinterpret_cast<uint16_t *>(smem + kRingBytes);
  StepShared &sh = *reinterpret_cast<StepShared *>(smem + kRingBytes + ((p.x_elems * 2u + 127u) & ~127u));

  const uint32_t position = *p.st.cursor;
  if (position >= p.st.max_context) {
    if (blockIdx.x == 0 && threadIdx.x == 0) report_error(p.st.error_word, kErrCursorOutOfRange);
    return;  // uniform over the grid: nobody reaches a barrier
  }
  if (threadIdx.x == 0) sh.dead = 0;
  MultiStream ms;
  multi_init(ms, ring, sh.bars, p.jobs, p.job_count);
  __syncthreads();
  multi_fill(ms);

  uint32_t token = position < p.st.prompt_count ? p.st.prompt[position] : p.st.slots[position - 1].token;
  if (token >= p.st.vocab) {
    if (blockIdx.x == 0 && threadIdx.x == 0) report_error(p.st.error_word, kErrTokenOutOfRange);
    token = 0;
  }
  uint32_t barrier = 0;
  for (uint32_t l = 0; l < p.layer_count; ++l) {
    const StepLayerDev &L = p.layers[l];
    // ---- QKV ----
    if (l == 0) {
      const uint16_t *row = p.embeddings + static_cast<uint64_t>(token) * p.hidden;
      float sumsq = 0.0f;
      for (uint32_t i = threadIdx.x; i < p.hidden; i += blockDim.x) {
        const float r = bf16_bits_to_f32(row[i]);
        sumsq += r * r;
      }
      const float total = block_sum(sumsq, sh.scratch);
      const float scale = rsqrtf(total / static_cast<float>(p.hidden) + p.eps);
      for (uint32_t i = threadIdx.x; i < p.hidden; i += blockDim.x) {
        const float r = bf16_bits_to_f32(row[i]);
        if (blockIdx.x == 0) p.h_a[i] = r;
        x[i] = f32_to_bf16_bits(r * scale * bf16_bits_to_f32(L.rms_attn[i]));
      }
    } else {
      add_norm_to_smem(x, p.h_b, p.down, nullptr, L.rms_attn, p.eps, p.hidden,
                       blockIdx.x == 0 ? p.h_a : nullptr, sh.scratch);
    }
    __syncthreads();
    {
      StoreEpi epi{p.qkv};
      multi_consume(ms, 4u * l, x, epi, p.st.error_word);
    }
    grid_barrier(p, sh, ++barrier);
    // ---- attention ----
    attention_phase<PER>(p, sh, L, position);
    grid_barrier(p, sh, ++barrier);
    // ---- O ----
    merge_attention_to_smem(p, x);
    __syncthreads();
    {
      StoreEpi epi{p.o_out};
      multi_consume(ms, 4u * l + 1u, x, epi, p.st.error_word);
    }
    grid_barrier(p, sh, ++barrier);
    // ---- gate/up + SwiGLU ----
    add_norm_to_smem(x, p.h_a, p.o_out, L.o_bias, L.rms_mlp, p.eps, p.hidden,
                     blockIdx.x == 0 ? p.h_b : nullptr, sh.scratch);
    __syncthreads();
    {
      SwigluEpi epi{p.ff_bf16, 0.0f};
      multi_consume(ms, 4u * l + 2u, x, epi, p.st.error_word);
    }
    grid_barrier(p, sh, ++barrier);
    // ---- down ----
    for (uint32_t i = threadIdx.x; i < p.intermediate / 8u; i += blockDim.x) {
      reinterpret_cast<uint4 *>(x)[i] = __ldcg(reinterpret_cast<const uint4 *>(p.ff_bf16) + i);
    }
    __syncthreads();
    {
      StoreEpi epi{p.down};
      multi_consume(ms, 4u * l + 3u, x, epi, p.st.error_word);
    }
    grid_barrier(p, sh, ++barrier);
  }
  if (p.sample != 0) {
    add_norm_to_smem(x, p.h_b, p.down, nullptr, p.final_norm, p.eps, p.hidden,
                     blockIdx.x == 0 ? p.h_a : nullptr, sh.scratch);
    __syncthreads();
    ArgmaxEpi epi{p.logits, -INFINITY, kNoIndex};
    multi_consume(ms, 4u * p.layer_count, x, epi, p.st.error_word);
    float *wv = sh.scratch;
    uint32_t *wi = reinterpret_cast<uint32_t *>(sh.scratch + 16);
    if ((threadIdx.x & 31u) == 0) {
      wv[threadIdx.x >> 5] = epi.best_v;
      wi[threadIdx.x >> 5] = epi.best_i;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float bv = -INFINITY;
      uint32_t bi = kNoIndex;
      for (uint32_t w = 0; w < kStreamWarps; ++w) {
        if (wi[w] != kNoIndex && better(wv[w], wi[w], bv, bi)) {
          bv = wv[w];
          bi = wi[w];
        }
      }
      p.best_value[blockIdx.x] = bv;
      p.best_index[blockIdx.x] = bi;
    }
    grid_barrier(p, sh, ++barrier);
  }
  stream_drain(ms.ws);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    if (p.sample != 0) {
      float bv = -INFINITY;
      uint32_t bi = kNoIndex;
      for (uint32_t b = 0; b < gridDim.x; ++b) {
        const uint32_t idx = __ldcg(p.best_index + b);
        const float val = __ldcg(p.best_value + b);
        if (idx != kNoIndex && better(val, idx, bv, bi)) {
          bv = val;
          bi = idx;
        }
      }
      // hf_decode_sequence/sampler.cu:394-407
      NervaCudaSyntheticTokenSlot *slot = p.st.slots + position;
      slot->request_id = 1;
      slot->sequence_id = 1;
      slot->token_index = position;
      slot->token = bi == kNoIndex ? 0u : bi;
      slot->version = static_cast<uint64_t>(position) + 1u;
      slot->completion = 1;
      slot->host_copied = 0;
    }
    *p.st.cursor = position + 1;
  }
}

}  // namespace

uint32_t step_kernel_smem_bytes(uint32_t x_elems) {
  return kRingBytes + ((x_elems * 2u + 127u) & ~127u) + static_cast<uint32_t>(sizeof(StepShared));
}

bool step_kernel_supported(uint32_t hidden, uint32_t heads, uint32_t kv_heads, uint32_t head_dim,
                           uint32_t intermediate, uint32_t x_elems) {
  return (head_dim == 64 || head_dim == 128) && hidden % 8 == 0 && intermediate % 8 == 0 &&
         (heads * head_dim) % 8 == 0 && heads % kv_heads == 0 &&
         step_kernel_smem_bytes(x_elems) <= 227u * 1024u;
}

cudaError_t configure_step_kernel() {
  cudaError_t err = cudaFuncSetAttribute(decode_step_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         227 * 1024);
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(decode_step_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  return err;
}

// Cooperative launch: the runtime refuses the launch unless every block can be
// resident at once, which the grid barrier needs.
cudaError_t launch_step_kernel(cudaStream_t stream, const StepKernelParams &p, uint32_t blocks) {
  cudaError_t err = cudaMemsetAsync(p.barrier_counter, 0, sizeof(uint32_t), stream);
  if (err != cudaSuccess) return err;
  StepKernelParams params = p;
  void *args[] = {&params};
  const void *fn = p.head_dim == 128 ? reinterpret_cast<const void *>(decode_step_kernel<4>)
                                     : reinterpret_cast<const void *>(decode_step_kernel<2>);
  return cudaLaunchCooperativeKernel(fn, dim3(blocks), dim3(kStreamThreads), args,
                                     step_kernel_smem_bytes(p.x_elems), stream);
}

}  // namespace nb
