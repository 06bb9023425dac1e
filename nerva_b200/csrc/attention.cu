// GQA paged split-KV decode attention (one query token per sequence).
//
// Replaces the reference's chunked decode attention and its merge kernel
// (hf_decode_sequence/attention_kernels.cu:528-760, kernels.cu:494-555) with the
// same mathematics: s = q.k / sqrt(d), online softmax, acc += p v per split,
// then out = sum_s acc_s e^{m_s - M} / sum_s l_s e^{m_s - M}.
//
// Layout of the work: grid (splits, kv_heads, batch).  Inside a block every warp
// walks its own 32-token tiles of the split through a private 3-stage cp.async
// ring (K and V stay bf16 in shared memory, 16.5 KiB per stage), so up to ~128
// KiB of KV reads are in flight per SM and no block-level barrier sits in the
// loop.  All G query heads of the KV head share each tile: in the QK pass a lane
// owns one token (K rows are padded by 16 B so the 128-bit row reads are bank
// conflict free) and produces G scores; in the PV pass a lane owns d/32 output
// dimensions of all G heads.
#include <math.h>

#include "common.cuh"
#include "kernels.cuh"

namespace nb {
namespace {

constexpr uint32_t kAttnWarps = 4;
constexpr uint32_t kAttnStages = 3;
constexpr uint32_t kAttnTile = 32;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gmem_src, bool valid) {
  const uint32_t bytes = valid ? 16u : 0u;  // 0 source bytes -> the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(smem_dst)),
               "l"(gmem_src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <uint32_t D>
struct AttnLayout {
  static constexpr uint32_t kKRow = D * 2u + 16u;
  static constexpr uint32_t kVRow = D * 2u;
  static constexpr uint32_t kStageBytes = kAttnTile * (kKRow + kVRow);
  static constexpr uint32_t kWarpBytes = kAttnStages * kStageBytes;
};

template <uint32_t D, uint32_t G>
constexpr uint32_t attn_smem_bytes() {
  // q [G][D] f32 | per-warp p [32][G] f32 | per-warp stage rings
  return G * D * 4u + kAttnWarps * kAttnTile * G * 4u + kAttnWarps * AttnLayout<D>::kWarpBytes;
}

template <uint32_t D, uint32_t G>
__global__ void __launch_bounds__(kAttnWarps * 32, 1) gqa_decode_kernel(AttentionParams p) {
  using L = AttnLayout<D>;
  constexpr uint32_t DPL = D / 32u;  // output dims per lane
  extern __shared__ __align__(128) uint8_t smem[];
  float *q_s = reinterpret_cast<float *>(smem);
  float *p_all = q_s + G * D;
  uint8_t *rings = reinterpret_cast<uint8_t *>(p_all + kAttnWarps * kAttnTile * G);

  const uint32_t split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const uint32_t context = p.cursor != nullptr ? *p.cursor + 1u : p.context;
  const uint32_t kv_hidden = p.kv_heads * D;
  const uint32_t tiles_total = (context + kAttnTile - 1u) / kAttnTile;
  const uint32_t tiles_per_split = (tiles_total + p.splits - 1u) / p.splits;
  const uint32_t tile_begin = split * tiles_per_split;
  uint32_t tile_end = tile_begin + tiles_per_split;
  if (tile_end > tiles_total) tile_end = tiles_total;

  const uint32_t *table = p.page_table + static_cast<uint64_t>(b) * p.page_count;
  const uint64_t seq_elems = static_cast<uint64_t>(p.page_count) * NERVA_KV_CACHE_BLOCK_TOKENS * kv_hidden;
  const uint16_t *key_pages = p.key_pages + b * seq_elems;
  const uint16_t *value_pages = p.value_pages + b * seq_elems;

  // q, pre-multiplied by log2(e)/sqrt(d) so that the softmax runs on exp2.
  const float qscale = kLog2e * rsqrtf(static_cast<float>(D));
  const float *q_in = p.q + (static_cast<uint64_t>(b) * p.heads + kvh * G) * D;
  for (uint32_t i = threadIdx.x; i < G * D; i += blockDim.x) q_s[i] = q_in[i] * qscale;
  __syncthreads();

  uint8_t *ring = rings + warp * L::kWarpBytes;
  float *p_s = p_all + warp * kAttnTile * G;

  auto load_tile = [&](uint32_t tile, uint32_t stage) {
    uint8_t *k_dst = ring + stage * L::kStageBytes;
    uint8_t *v_dst = k_dst + kAttnTile * L::kKRow;
    constexpr uint32_t kSegs = D * 2u / 16u;  // 16-byte segments per row
    const uint32_t token0 = tile * kAttnTile;
    uint32_t page[2];
#pragma unroll
    for (uint32_t h = 0; h < 2; ++h) {
      const uint32_t logical = tile * 2u + h;
      uint32_t phys = 0;
      if (token0 + h * 16u < context && logical < p.page_count) {
        phys = table[logical];
        if (phys >= p.page_count) {
          report_error(p.error_word, kErrPageOutOfRange);
          phys = 0;
        }
      }
      page[h] = phys;
    }
#pragma unroll
    for (uint32_t it = 0; it < kAttnTile * kSegs / 32u; ++it) {
      const uint32_t s = it * 32u + lane;
      const uint32_t row = s / kSegs, seg = s % kSegs;
      const uint32_t token = token0 + row;
      const bool valid = token < context;
      const uint64_t elem =
          (static_cast<uint64_t>(page[row >> 4]) * NERVA_KV_CACHE_BLOCK_TOKENS + (row & 15u)) * kv_hidden +
          kvh * D + seg * 8u;
      cp_async16(k_dst + row * L::kKRow + seg * 16u, key_pages + elem, valid);
      cp_async16(v_dst + row * L::kVRow + seg * 16u, value_pages + elem, valid);
    }
  };

  float m_run[G], l_run[G], acc[G][DPL];
#pragma unroll
  for (uint32_t g = 0; g < G; ++g) {
    m_run[g] = -INFINITY;
    l_run[g] = 0.0f;
#pragma unroll
    for (uint32_t i = 0; i < DPL; ++i) acc[g][i] = 0.0f;
  }

  // This warp's tiles: tile_begin + warp, + kAttnWarps, ...
  const uint32_t first = tile_begin + warp;
  const uint32_t my_tiles = first < tile_end ? (tile_end - first + kAttnWarps - 1u) / kAttnWarps : 0u;
#pragma unroll
  for (uint32_t s = 0; s < kAttnStages - 1u; ++s) {
    if (s < my_tiles) load_tile(first + s * kAttnWarps, s);
    cp_async_commit();
  }
  for (uint32_t i = 0; i < my_tiles; ++i) {
    cp_async_wait<kAttnStages - 2>();
    __syncwarp();
    // refill the stage that the previous iteration finished with
    const uint32_t ahead = i + kAttnStages - 1u;
    if (ahead < my_tiles) load_tile(first + ahead * kAttnWarps, ahead % kAttnStages);
    cp_async_commit();

    const uint32_t tile = first + i * kAttnWarps;
    const uint8_t *k_s = ring + (i % kAttnStages) * L::kStageBytes;
    const uint8_t *v_s = k_s + kAttnTile * L::kKRow;

    // ---- scores: this lane's token against the G query heads ----
    float s[G];
#pragma unroll
    for (uint32_t g = 0; g < G; ++g) s[g] = 0.0f;
    const uint8_t *k_row = k_s + lane * L::kKRow;
#pragma unroll 4
    for (uint32_t blk = 0; blk < D / 8u; ++blk) {
      const uint4 kk = lds128(k_row + blk * 16u);
      const float k0 = bf16x2_lo(kk.x), k1 = bf16x2_hi(kk.x), k2 = bf16x2_lo(kk.y), k3 = bf16x2_hi(kk.y);
      const float k4 = bf16x2_lo(kk.z), k5 = bf16x2_hi(kk.z), k6 = bf16x2_lo(kk.w), k7 = bf16x2_hi(kk.w);
#pragma unroll
      for (uint32_t g = 0; g < G; ++g) {
        const float4 qa = *reinterpret_cast<const float4 *>(q_s + g * D + blk * 8u);
        const float4 qb = *reinterpret_cast<const float4 *>(q_s + g * D + blk * 8u + 4u);
        float t = s[g];
        t = fmaf(k0, qa.x, t);
        t = fmaf(k1, qa.y, t);
        t = fmaf(k2, qa.z, t);
        t = fmaf(k3, qa.w, t);
        t = fmaf(k4, qb.x, t);
        t = fmaf(k5, qb.y, t);
        t = fmaf(k6, qb.z, t);
        t = fmaf(k7, qb.w, t);
        s[g] = t;
      }
    }
    const bool token_valid = tile * kAttnTile + lane < context;
    // ---- online softmax (base 2) ----
#pragma unroll
    for (uint32_t g = 0; g < G; ++g) {
      const float sg = token_valid ? s[g] : -INFINITY;
      const float m_new = fmaxf(m_run[g], warp_max(sg));
      const float pr = exp2f(sg - m_new);       // masked tokens -> 0
      const float corr = exp2f(m_run[g] - m_new);  // first tile: exp2(-inf) = 0
      l_run[g] = l_run[g] * corr + warp_sum(pr);
      m_run[g] = m_new;
#pragma unroll
      for (uint32_t d = 0; d < DPL; ++d) acc[g][d] *= corr;
      p_s[lane * G + g] = pr;
    }
    __syncwarp();
    // ---- acc += p v: this lane's DPL dims of every head ----
#pragma unroll 8
    for (uint32_t t = 0; t < kAttnTile; ++t) {
      float v[DPL];
      const uint8_t *v_ptr = v_s + t * L::kVRow + lane * DPL * 2u;
      if (DPL == 4) {
        const uint2 w = *reinterpret_cast<const uint2 *>(v_ptr);
        v[0] = bf16x2_lo(w.x);
        v[1] = bf16x2_hi(w.x);
        v[2 % DPL] = bf16x2_lo(w.y);
        v[3 % DPL] = bf16x2_hi(w.y);
      } else {
        const uint32_t w = *reinterpret_cast<const uint32_t *>(v_ptr);
        v[0] = bf16x2_lo(w);
        v[1 % DPL] = bf16x2_hi(w);
      }
      float pg[G];
      if (G == 4) {
        const float4 pv = *reinterpret_cast<const float4 *>(p_s + t * G);
        pg[0] = pv.x;
        pg[1 % G] = pv.y;
        pg[2 % G] = pv.z;
        pg[3 % G] = pv.w;
      } else {
#pragma unroll
        for (uint32_t g = 0; g < G; ++g) pg[g] = p_s[t * G + g];
      }
#pragma unroll
      for (uint32_t g = 0; g < G; ++g) {
#pragma unroll
        for (uint32_t d = 0; d < DPL; ++d) acc[g][d] = fmaf(pg[g], v[d], acc[g][d]);
      }
    }
    __syncwarp();
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- merge the block's warps (stage memory is free now) ----
  float *merge = reinterpret_cast<float *>(rings);  // [warps][G][D + 2]
  constexpr uint32_t kRec = D + 2u;
#pragma unroll
  for (uint32_t g = 0; g < G; ++g) {
    float *rec = merge + (warp * G + g) * kRec;
#pragma unroll
    for (uint32_t d = 0; d < DPL; ++d) rec[lane * DPL + d] = acc[g][d];
    if (lane == 0) {
      rec[D] = m_run[g];
      rec[D + 1] = l_run[g];
    }
  }
  __syncthreads();
  for (uint32_t idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const uint32_t g = idx / D, d = idx % D;
    float m = -INFINITY;
    for (uint32_t w = 0; w < kAttnWarps; ++w) m = fmaxf(m, merge[(w * G + g) * kRec + D]);
    float a = 0.0f, l = 0.0f;
    if (m > -INFINITY) {
      for (uint32_t w = 0; w < kAttnWarps; ++w) {
        const float *rec = merge + (w * G + g) * kRec;
        const float wgt = exp2f(rec[D] - m);
        a = fmaf(rec[d], wgt, a);
        l = fmaf(rec[D + 1], wgt, l);
      }
    }
    const uint64_t slot = (static_cast<uint64_t>(b) * p.heads + kvh * G + g) * p.splits + split;
    p.partial_acc[slot * D + d] = a;
    if (d == 0) {
      p.partial_m[slot] = m;
      p.partial_l[slot] = l;
    }
  }
}

// Any head_dim <= 256 and any group size: one warp per query head, no split.
__global__ void gqa_decode_generic_kernel(AttentionParams p) {
  const uint32_t head = blockIdx.x, b = blockIdx.y, lane = threadIdx.x;
  const uint32_t d = p.head_dim;
  const uint32_t kvh = head / (p.heads / p.kv_heads);
  const uint32_t kv_hidden = p.kv_heads * d;
  const uint32_t context = p.cursor != nullptr ? *p.cursor + 1u : p.context;
  const uint32_t *table = p.page_table + static_cast<uint64_t>(b) * p.page_count;
  const uint64_t seq_elems = static_cast<uint64_t>(p.page_count) * NERVA_KV_CACHE_BLOCK_TOKENS * kv_hidden;
  const uint16_t *key_pages = p.key_pages + b * seq_elems;
  const uint16_t *value_pages = p.value_pages + b * seq_elems;
  const float *q = p.q + (static_cast<uint64_t>(b) * p.heads + head) * d;
  const float scale = kLog2e * rsqrtf(static_cast<float>(d));
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  float m = -INFINITY, l = 0.0f;
  for (uint32_t token = 0; token < context; ++token) {
    uint32_t phys = table[token / NERVA_KV_CACHE_BLOCK_TOKENS];
    if (phys >= p.page_count) {
      report_error(p.error_word, kErrPageOutOfRange);
      phys = 0;
    }
    const uint64_t base = (static_cast<uint64_t>(phys) * NERVA_KV_CACHE_BLOCK_TOKENS +
                           token % NERVA_KV_CACHE_BLOCK_TOKENS) * kv_hidden + kvh * d;
    float dot = 0.0f;
    for (uint32_t i = lane; i < d; i += 32u) dot = fmaf(q[i], bf16_bits_to_f32(key_pages[base + i]), dot);
    const float s = warp_sum(dot) * scale;
    const float m_new = fmaxf(m, s);
    const float corr = exp2f(m - m_new);
    const float pr = exp2f(s - m_new);
    l = l * corr + pr;
    m = m_new;
    for (uint32_t j = 0, i = lane; i < d; i += 32u, ++j) {
      acc[j] = acc[j] * corr + pr * bf16_bits_to_f32(value_pages[base + i]);
    }
  }
  const uint64_t slot0 = (static_cast<uint64_t>(b) * p.heads + head) * p.splits;
  for (uint32_t j = 0, i = lane; i < d; i += 32u, ++j) p.partial_acc[slot0 * d + i] = acc[j];
  if (lane == 0) {
    p.partial_m[slot0] = m;
    p.partial_l[slot0] = l;
    for (uint32_t s = 1; s < p.splits; ++s) {
      p.partial_m[slot0 + s] = -INFINITY;
      p.partial_l[slot0 + s] = 0.0f;
    }
  }
}

// out = sum_s acc_s 2^{m_s - M} / sum_s l_s 2^{m_s - M}; one block per (head, batch).
__global__ void gqa_merge_kernel(AttentionParams p) {
  const uint32_t head = blockIdx.x, b = blockIdx.y;
  const uint32_t d = p.head_dim;
  const uint64_t slot0 = (static_cast<uint64_t>(b) * p.heads + head) * p.splits;
  float m = -INFINITY;
  for (uint32_t s = 0; s < p.splits; ++s) {
    if (p.partial_l[slot0 + s] > 0.0f) m = fmaxf(m, p.partial_m[slot0 + s]);
  }
  float l = 0.0f;
  for (uint32_t s = 0; s < p.splits; ++s) {
    const float ls = p.partial_l[slot0 + s];
    if (ls > 0.0f) l = fmaf(ls, exp2f(p.partial_m[slot0 + s] - m), l);
  }
  const float inv = l > 0.0f ? 1.0f / l : 0.0f;
  for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {
    float a = 0.0f;
    for (uint32_t s = 0; s < p.splits; ++s) {
      if (p.partial_l[slot0 + s] > 0.0f) {
        a = fmaf(p.partial_acc[(slot0 + s) * d + i], exp2f(p.partial_m[slot0 + s] - m), a);
      }
    }
    const float v = a * inv;
    const uint64_t o = (static_cast<uint64_t>(b) * p.heads + head) * d + i;
    if (p.out_f32 != nullptr) p.out_f32[o] = v;
    if (p.out_bf16 != nullptr) p.out_bf16[o] = f32_to_bf16_bits(v);
  }
}

}  // namespace

cudaError_t configure_attention_kernels() {
  cudaError_t err = cudaFuncSetAttribute(gqa_decode_kernel<128, 4>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(attn_smem_bytes<128, 4>()));
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(gqa_decode_kernel<64, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(attn_smem_bytes<64, 4>()));
  return err;
}

uint32_t attention_default_splits(uint32_t context, uint32_t batch, uint32_t kv_heads,
                                  uint32_t sm_count) {
  // Enough blocks to cover the SMs about twice, but at least one 32-token tile
  // per warp of a block.
  const uint32_t tiles = (context + kAttnTile - 1u) / kAttnTile;
  uint32_t by_work = (tiles + kAttnWarps - 1u) / kAttnWarps;
  if (by_work == 0) by_work = 1;
  uint32_t by_sms = (2u * sm_count + batch * kv_heads - 1u) / (batch * kv_heads);
  if (by_sms == 0) by_sms = 1;
  uint32_t splits = by_work < by_sms ? by_work : by_sms;
  if (splits > 256u) splits = 256u;
  return splits;
}

cudaError_t launch_attention(cudaStream_t stream, const AttentionParams &p) {
  const uint32_t group = p.heads / p.kv_heads;
  const dim3 grid(p.splits, p.kv_heads, p.batch);
  if (p.head_dim == 128 && group == 4) {
    gqa_decode_kernel<128, 4><<<grid, kAttnWarps * 32, attn_smem_bytes<128, 4>(), stream>>>(p);
  } else if (p.head_dim == 64 && group == 4) {
    gqa_decode_kernel<64, 4><<<grid, kAttnWarps * 32, attn_smem_bytes<64, 4>(), stream>>>(p);
  } else {
    if (p.head_dim > 256) return cudaErrorNotSupported;
    gqa_decode_generic_kernel<<<dim3(p.heads, p.batch), 32, 0, stream>>>(p);
  }
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return err;
  uint32_t threads = ((p.head_dim + 31u) / 32u) * 32u;
  if (threads > 256) threads = 256;
  gqa_merge_kernel<<<dim3(p.heads, p.batch), threads, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace nb
