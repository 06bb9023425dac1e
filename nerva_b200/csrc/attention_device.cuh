// Decode attention of one (query head, token split) work item by one thread
// block, shared by the per-operator engine's fused attention kernel and by the
// whole-step kernel.  Includes what the reference does in three launches
// (hf_decode_sequence/kernels.cu:434-492 q/k norm + RoPE + KV append,
// attention_kernels.cu:528-760 chunked attention, kernels.cu:494-555 merge).
//
// Latency is what matters at decode context lengths (a few hundred KB of KV per
// layer), so each warp puts the page-table entries, then the whole K tile and V
// tile of its 32 tokens in flight (registers) before anyone needs them, while
// warp 0 prepares q and warp 1 the current token's K/V row: an item costs about
// three dependent trips to L2, not one per operand.
#pragma once

#include "common.cuh"
#include "kernels.cuh"

namespace nb {

constexpr uint32_t kAttnItemTile = 32;
constexpr uint32_t kAttnItemMaxHeadDim = 128;
constexpr float kAttnLog2e = 1.4426950408889634f;

struct AttnItemCtx {
  const float *qkv;  // [heads*d | kv_heads*d | kv_heads*d] f32 projection output of this token
  const uint16_t *q_bias, *k_bias, *v_bias, *q_norm, *k_norm;  // optional
  uint16_t *key_pages, *value_pages;  // this layer's [pages][16][kv_hidden] bf16
  const uint32_t *page_table;
  uint32_t page_count;
  uint32_t heads, kv_heads;
  float eps, rope_theta;
  uint32_t position;  // token being decoded; tokens [0, position) are in the cache
  uint32_t splits;
  float *partial_acc, *partial_m, *partial_l;  // [heads][splits][...]
  uint32_t *error_word;
  // The kernel was launched with programmatic dependent launch: the cached K/V
  // tiles (written by earlier steps) are put in flight first, then the item
  // waits for the QKV projection before it touches `qkv`.
  bool wait_dependency;
  unsigned long long *stamps = nullptr;  // optional timeline stamps (common.cuh: stamp)
};

template <uint32_t WARPS>
struct AttnItemShared {
  alignas(16) float q[kAttnItemMaxHeadDim];      // pre-scaled by log2(e)/sqrt(d)
  alignas(16) float k_new[kAttnItemMaxHeadDim];  // current token's K and V, bf16-rounded
  alignas(16) float v_new[kAttnItemMaxHeadDim];
  alignas(16) float p[WARPS][kAttnItemTile];
};
constexpr uint32_t kAttnMergeStride = kAttnItemMaxHeadDim + 2;  // per-warp merge record, floats

// Per-head RMSNorm + RoPE of one head held PER-elements-per-lane by one warp
// (element e = lane + 32 k).  head_dim = 32 PER is a multiple of 64, so both
// members of every rotary pair (e, e + d/2) live in the same lane.
template <uint32_t PER>
__device__ __forceinline__ void head_norm_rope(float (&v)[PER], const uint16_t *norm, float eps,
                                               float theta, uint32_t position) {
  constexpr uint32_t D = PER * 32u;
  constexpr uint32_t HALF = PER / 2u;
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

// The same in two steps, for kernels that know the position before their input
// arrives: rope_factors() needs only the position; head_norm_rope_pre() then
// applies norm weights already held in registers and the prepared rotation.
template <uint32_t PER>
struct RopeFactors {
  float c[PER / 2u], s[PER / 2u];
  bool on;
};
template <uint32_t PER>
__device__ __forceinline__ void rope_factors(RopeFactors<PER> &f, float theta, uint32_t position) {
  constexpr uint32_t D = PER * 32u;
  const uint32_t lane = threadIdx.x & 31u;
  f.on = theta > 0.0f;
#pragma unroll
  for (uint32_t k = 0; k < PER / 2u; ++k) {
    f.c[k] = 1.0f;
    f.s[k] = 0.0f;
    if (f.on) {
      const uint32_t i = lane + 32u * k;
      const float exponent = static_cast<float>(2u * i) / static_cast<float>(D);
      const float angle = static_cast<float>(position) / powf(theta, exponent);
      sincosf(angle, &f.s[k], &f.c[k]);
    }
  }
}
template <uint32_t PER>
__device__ __forceinline__ void head_norm_rope_pre(float (&v)[PER], bool has_norm, const float (&w)[PER],
                                                   float eps, const RopeFactors<PER> &f) {
  constexpr uint32_t D = PER * 32u;
  constexpr uint32_t HALF = PER / 2u;
  if (has_norm) {
    float ss = 0.0f;
#pragma unroll
    for (uint32_t k = 0; k < PER; ++k) ss += v[k] * v[k];
    ss = warp_sum(ss);
    const float scale = rsqrtf(ss / static_cast<float>(D) + eps);
#pragma unroll
    for (uint32_t k = 0; k < PER; ++k) v[k] *= scale * w[k];
  }
  if (f.on) {
#pragma unroll
    for (uint32_t k = 0; k < HALF; ++k) {
      const float left = v[k], right = v[k + HALF];
      v[k] = left * f.c[k] - right * f.s[k];
      v[k + HALF] = right * f.c[k] + left * f.s[k];
    }
  }
}

// Runs item (head h, split s).  All WARPS*32 threads of the block call it.
// `merge` is WARPS * kAttnMergeStride floats of shared memory.  On return the
// item's partial (acc, m, l) is in global memory (written by warp 0).
template <uint32_t PER, uint32_t WARPS>
__device__ __forceinline__ void attention_item(const AttnItemCtx &c, AttnItemShared<WARPS> &sh,
                                               float *merge, uint32_t h, uint32_t s) {
  constexpr uint32_t D = PER * 32u;
  constexpr uint32_t KV4 = D / 8u;  // 16-byte pieces of a K row
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const uint32_t group = c.heads / c.kv_heads;
  const uint32_t attention_hidden = c.heads * D, kv_hidden = c.kv_heads * D;
  const uint32_t S = c.splits;
  const uint32_t hist = c.position;
  const uint32_t tiles_total = (hist + kAttnItemTile - 1u) / kAttnItemTile;
  const uint32_t tiles_per_split = (tiles_total + S - 1u) / S;
  const float qscale = kAttnLog2e * rsqrtf(static_cast<float>(D));
  const uint32_t kvh = h / group;
  const uint32_t tile_begin = s * tiles_per_split;
  uint32_t tile_end = tile_begin + tiles_per_split;
  if (tile_end > tiles_total) tile_end = tiles_total;
  const bool owns_current = s + 1u == S;

  uint4 kk[KV4];
  uint32_t vw[kAttnItemTile * PER / 2u];  // this lane's PER dims of the tile's 32 V rows
  auto load_tile = [&](uint32_t tile) {
    const uint32_t token = tile * kAttnItemTile + lane;
    uint32_t phys = 0;
    if (token < hist) {
      phys = c.page_table[token / NERVA_KV_CACHE_BLOCK_TOKENS];
      if (phys >= c.page_count) {
        report_error(c.error_word, kErrPageOutOfRange);
        phys = 0;
      }
      const uint64_t row = (static_cast<uint64_t>(phys) * NERVA_KV_CACHE_BLOCK_TOKENS +
                            token % NERVA_KV_CACHE_BLOCK_TOKENS) * kv_hidden + kvh * D;
      const uint4 *k_row = reinterpret_cast<const uint4 *>(c.key_pages + row);
#pragma unroll
      for (uint32_t b = 0; b < KV4; ++b) kk[b] = __ldcg(k_row + b);
    }
#pragma unroll
    for (uint32_t t = 0; t < kAttnItemTile; ++t) {
      const uint32_t phys_t = __shfl_sync(0xffffffffu, phys, t);
      const uint32_t tok = tile * kAttnItemTile + t;
      if (tok < hist) {
        const uint64_t vrow = (static_cast<uint64_t>(phys_t) * NERVA_KV_CACHE_BLOCK_TOKENS +
                               tok % NERVA_KV_CACHE_BLOCK_TOKENS) * kv_hidden + kvh * D + lane * PER;
        if (PER == 4) {
          const uint2 w = __ldcg(reinterpret_cast<const uint2 *>(c.value_pages + vrow));
          vw[t * (PER / 2u)] = w.x;
          vw[t * (PER / 2u) + (PER / 2u - 1u)] = w.y;
        } else {
          vw[t * (PER / 2u)] = __ldcg(reinterpret_cast<const uint32_t *>(c.value_pages + vrow));
        }
      }
    }
  };
  uint32_t tile = tile_begin + warp;
  if (tile < tile_end) load_tile(tile);
  stamp(c.stamps, kStampAfterWait);      // attention: cached K/V tile loads issued
  if (c.wait_dependency) pdl_wait();
  stamp(c.stamps, kStampAfterPrologue);  // attention: the QKV projection has completed

  if (warp == 0) {
    float v[PER];
#pragma unroll
    for (uint32_t k = 0; k < PER; ++k) {
      const uint32_t e = lane + 32u * k;
      v[k] = __ldcg(c.qkv + h * D + e);
      if (c.q_bias != nullptr) v[k] += bf16_bits_to_f32(c.q_bias[h * D + e]);
    }
    head_norm_rope<PER>(v, c.q_norm, c.eps, c.rope_theta, c.position);
#pragma unroll
    for (uint32_t k = 0; k < PER; ++k) sh.q[lane + 32u * k] = v[k] * qscale;
  } else if (warp == 1 % WARPS && owns_current) {
    float kn[PER], vn[PER];
#pragma unroll
    for (uint32_t k = 0; k < PER; ++k) {
      const uint32_t e = lane + 32u * k;
      kn[k] = __ldcg(c.qkv + attention_hidden + kvh * D + e);
      vn[k] = __ldcg(c.qkv + attention_hidden + kv_hidden + kvh * D + e);
      if (c.k_bias != nullptr) kn[k] += bf16_bits_to_f32(c.k_bias[kvh * D + e]);
      if (c.v_bias != nullptr) vn[k] += bf16_bits_to_f32(c.v_bias[kvh * D + e]);
    }
    head_norm_rope<PER>(kn, c.k_norm, c.eps, c.rope_theta, c.position);
    uint32_t page = c.page_table[c.position / NERVA_KV_CACHE_BLOCK_TOKENS];
    const bool store = h == kvh * group;  // one item per KV head appends the row
    if (page >= c.page_count) {
      report_error(c.error_word, kErrPageOutOfRange);
      page = 0;
    }
    const uint64_t base = (static_cast<uint64_t>(page) * NERVA_KV_CACHE_BLOCK_TOKENS +
                           c.position % NERVA_KV_CACHE_BLOCK_TOKENS) * kv_hidden + kvh * D;
#pragma unroll
    for (uint32_t k = 0; k < PER; ++k) {
      const uint32_t e = lane + 32u * k;
      const uint16_t kb = f32_to_bf16_bits(kn[k]), vb = f32_to_bf16_bits(vn[k]);
      sh.k_new[e] = bf16_bits_to_f32(kb);
      sh.v_new[e] = bf16_bits_to_f32(vb);
      if (store) {
        c.key_pages[base + e] = kb;
        c.value_pages[base + e] = vb;
      }
    }
  }
  __syncthreads();

  float m_run = -INFINITY, l_run = 0.0f, acc[PER];
#pragma unroll
  for (uint32_t i = 0; i < PER; ++i) acc[i] = 0.0f;
  while (tile < tile_end) {
    const bool valid = tile * kAttnItemTile + lane < hist;
    float score = -INFINITY;
    if (valid) {
      score = 0.0f;
#pragma unroll
      for (uint32_t b = 0; b < KV4; ++b) {
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
    }
    const float m_new = fmaxf(m_run, warp_max(score));
    const float pr = exp2f(score - m_new);    // masked tokens: exp2(-inf) = 0
    const float corr = exp2f(m_run - m_new);  // first tile: 0
    l_run = l_run * corr + warp_sum(pr);
    m_run = m_new;
#pragma unroll
    for (uint32_t i = 0; i < PER; ++i) acc[i] *= corr;
    sh.p[warp][lane] = pr;
    __syncwarp();
    const uint32_t left = hist - tile * kAttnItemTile;
#pragma unroll
    for (uint32_t t = 0; t < kAttnItemTile; ++t) {
      if (t < left) {
        const float pt = sh.p[warp][t];
        if (PER == 4) {
          const uint32_t w0 = vw[t * (PER / 2u)], w1 = vw[t * (PER / 2u) + (PER / 2u - 1u)];
          acc[0] = fmaf(pt, bf16x2_lo(w0), acc[0]);
          acc[1 % PER] = fmaf(pt, bf16x2_hi(w0), acc[1 % PER]);
          acc[2 % PER] = fmaf(pt, bf16x2_lo(w1), acc[2 % PER]);
          acc[3 % PER] = fmaf(pt, bf16x2_hi(w1), acc[3 % PER]);
        } else {
          const uint32_t w0 = vw[t * (PER / 2u)];
          acc[0] = fmaf(pt, bf16x2_lo(w0), acc[0]);
          acc[1 % PER] = fmaf(pt, bf16x2_hi(w0), acc[1 % PER]);
        }
      }
    }
    __syncwarp();
    tile += WARPS;
    if (tile < tile_end) load_tile(tile);
  }
  // merge the warps; warp 0 then folds in the current token
#pragma unroll
  for (uint32_t i = 0; i < PER; ++i) merge[warp * kAttnMergeStride + lane * PER + i] = acc[i];
  if (lane == 0) {
    merge[warp * kAttnMergeStride + D] = m_run;
    merge[warp * kAttnMergeStride + D + 1] = l_run;
  }
  __syncthreads();
  if (warp == 0) {
    float m = -INFINITY;
    for (uint32_t w = 0; w < WARPS; ++w) m = fmaxf(m, merge[w * kAttnMergeStride + D]);
    float a[PER], l = 0.0f;
#pragma unroll
    for (uint32_t i = 0; i < PER; ++i) a[i] = 0.0f;
    if (m > -INFINITY) {
      for (uint32_t w = 0; w < WARPS; ++w) {
        const float wgt = exp2f(merge[w * kAttnMergeStride + D] - m);
        l = fmaf(merge[w * kAttnMergeStride + D + 1], wgt, l);
#pragma unroll
        for (uint32_t i = 0; i < PER; ++i) a[i] = fmaf(merge[w * kAttnMergeStride + lane * PER + i], wgt, a[i]);
      }
    }
    if (owns_current) {
      float dot = 0.0f;
#pragma unroll
      for (uint32_t i = 0; i < PER; ++i) dot = fmaf(sh.q[lane * PER + i], sh.k_new[lane * PER + i], dot);
      const float s_new = warp_sum(dot);
      const float m2 = fmaxf(m, s_new);
      const float corr = exp2f(m - m2);
      const float pr = exp2f(s_new - m2);
      l = l * corr + pr;
#pragma unroll
      for (uint32_t i = 0; i < PER; ++i) a[i] = a[i] * corr + pr * sh.v_new[lane * PER + i];
      m = m2;
    }
    const uint64_t slot = static_cast<uint64_t>(h) * S + s;
#pragma unroll
    for (uint32_t i = 0; i < PER; ++i) c.partial_acc[slot * D + lane * PER + i] = a[i];
    if (lane == 0) {
      c.partial_m[slot] = m;
      c.partial_l[slot] = l;
    }
  }
  __syncthreads();
}

}  // namespace nb
