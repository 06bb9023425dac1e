// Decode attention of the resident session as ONE launch per layer: q/k RMSNorm
// + RoPE + paged KV append + split attention + merge.  The reference spends
// three launches on this (hf_decode_sequence/kernels.cu:434-492,
// attention_kernels.cu:528-760, kernels.cu:494-555).
//
// Grid = kv_heads x splits blocks of (2 * group + 1) warps.  A block serves the
// `group` query heads that share one KV head over one span of the context, so
// every cached K/V byte is fetched once per block (not once per query head):
//   * all threads copy the span's K and V rows into shared memory with 16-byte
//     cp.async in 64-token stages (two stages in flight).  Consecutive threads
//     copy consecutive pieces of a row, so a request covers whole 128-byte
//     lines.  These rows were written by earlier steps, so the copies are issued
//     BEFORE the kernel waits for the QKV projection of this step;
//   * warps w and group + w (w < group) own query head kv*group + w: warp w does the
//     q RMSNorm + RoPE and takes the first 32-token tile of every stage, warp
//     group + w the second; scores with one token per lane, base-2 online softmax,
//     P.V with D/32 dims per lane; the two softmax states are merged at the end;
//   * warp 2*group normalises and rotates the new K row, rounds K and V to bf16,
//     appends them to the page and hands them to the query warps (only in the
//     block of the last span);
//   * the partial (acc, m, l) of every (head, span) goes to global memory; the
//     block that draws the last ticket of its KV head (one atomicAdd, no
//     waiting) merges the spans and writes the bf16 attention vector.
#include "attention_device.cuh"
#include "kernels.cuh"

namespace nb {
namespace {

constexpr uint32_t kChunkTokens = 64;     // tokens per shared-memory stage (two 32-token tiles)
constexpr uint32_t kStages = 2;
constexpr uint32_t kFusedMaxSplits = 16;
constexpr uint32_t kFusedMaxGroup = 8;

__device__ __forceinline__ void cp_async_16(void *smem_dst, const void *gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(smem_dst)), "l"(gmem_src)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <uint32_t D>
struct FusedLayout {
  static constexpr uint32_t kRowK = D * 2u + 16u;  // bytes; the pad keeps 16-byte row reads conflict-free
  static constexpr uint32_t kRowV = D * 2u;
  static constexpr uint32_t kStageBytes = kChunkTokens * (kRowK + kRowV);
  static constexpr uint32_t kPieces = D * 2u / 16u;  // 16-byte pieces of one row
  // stages | q [group][D] f32 | k_new [D] | v_new [D] | p [2 * group][32]
  __host__ __device__ static constexpr uint32_t bytes(uint32_t group) {
    return kStages * kStageBytes + (group * D + 2u * D + 2u * group * 32u) * 4u;
  }
};

// ROWS: block-step form (one set of blocks per activation row, fields taken from p.rows[blockIdx.y]).
template <uint32_t PER, bool ROWS>
__global__ void fused_decode_attention_kernel(FusedAttentionParams p) {
  constexpr uint32_t D = PER * 32u;
  using Layout = FusedLayout<D>;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ uint32_t ticket;
  const uint32_t group = p.heads / p.kv_heads;
  float *q_sh = reinterpret_cast<float *>(smem + kStages * Layout::kStageBytes);
  float *k_new = q_sh + group * D;
  float *v_new = k_new + D;
  float *p_sh = v_new + D;

  pdl_trigger();
  stamp(p.stamps, kStampEntry);
  uint32_t position;
  if (ROWS) {
    const FusedAttentionRow r = p.rows[blockIdx.y];
    position = r.position;
    p.max_context = r.max_context;
    p.page_count = r.page_count;
    p.qkv = r.qkv;
    p.key_pages = r.key_pages + p.layer * r.kv_layer_elems;
    p.value_pages = r.value_pages + p.layer * r.kv_layer_elems;
    p.page_table = r.page_table;
    p.partial_acc = r.partial_acc;
    p.partial_m = r.partial_m;
    p.partial_l = r.partial_l;
    p.tickets = r.tickets;
    p.out_bf16 = r.out_bf16;
    p.error_word = r.error_word;
  } else {
    // The cursor only changes in the last kernel of a step, which has completed.
    position = *p.cursor;
  }
  if (position >= p.max_context) return;
  const bool cached_only = ROWS && p.cached_only != 0;
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const uint32_t S = p.splits;
  const uint32_t kvh = blockIdx.x / S, s = blockIdx.x - kvh * S;
  const uint32_t kv_hidden = p.kv_heads * D, attention_hidden = p.heads * D;
  // cached tokens 0 .. position-1, the new one comes from qkv; cached_only: 0 .. position, all cached
  const uint32_t hist = cached_only ? position + 1u : position;
  const uint32_t chunks_total = (hist + kChunkTokens - 1u) / kChunkTokens;
  const uint32_t chunks_per_split = (chunks_total + S - 1u) / S;
  const uint32_t chunk_begin = s * chunks_per_split;
  uint32_t chunk_end = chunk_begin + chunks_per_split;
  if (chunk_end > chunks_total) chunk_end = chunks_total;
  const bool owns_current = !cached_only && s + 1u == S;

  // Copies the cached rows of one 64-token chunk into a stage (one commit group).
  // A warp copies whole tokens: half of its lanes (or a quarter, for D = 64) take
  // the 16-byte pieces of the K row, the other half those of the V row, so every
  // request covers complete 128-byte lines.  The chunk's four page-table entries
  // are read once per warp, before the loop, and handed out by shuffle.
  auto chunk_pages = [&](uint32_t chunk) -> uint32_t {
    constexpr uint32_t kPagesPerChunk = kChunkTokens / NERVA_KV_CACHE_BLOCK_TOKENS;
    const uint32_t first = chunk * kChunkTokens;
    uint32_t my_page = 0;
    if (lane < kPagesPerChunk && first + lane * NERVA_KV_CACHE_BLOCK_TOKENS < hist) {
      my_page = p.page_table[first / NERVA_KV_CACHE_BLOCK_TOKENS + lane];
      if (my_page >= p.page_count) {
        report_error(p.error_word, kErrPageOutOfRange);
        my_page = 0;
      }
    }
    return my_page;
  };
  auto issue = [&](uint32_t chunk, uint32_t stage, uint32_t my_page) {
    uint8_t *k_stage = smem + stage * Layout::kStageBytes;
    uint8_t *v_stage = k_stage + kChunkTokens * Layout::kRowK;
    constexpr uint32_t kLanesPerToken = 2u * Layout::kPieces;          // 32 (D = 128) or 16 (D = 64)
    constexpr uint32_t kTokensPerIter = 32u / kLanesPerToken;
    const uint32_t first = chunk * kChunkTokens;
    const uint32_t sub = lane / kLanesPerToken, r = lane % kLanesPerToken;
    const bool is_v = r >= Layout::kPieces;
    const uint32_t piece = is_v ? r - Layout::kPieces : r;
    const uint32_t warps = blockDim.x >> 5;
    for (uint32_t base = warp * kTokensPerIter; base < kChunkTokens; base += warps * kTokensPerIter) {
      const uint32_t t = base + sub;
      const uint32_t page = __shfl_sync(0xffffffffu, my_page, t / NERVA_KV_CACHE_BLOCK_TOKENS);
      if (first + t >= hist) continue;
      const uint64_t row = (static_cast<uint64_t>(page) * NERVA_KV_CACHE_BLOCK_TOKENS +
                            t % NERVA_KV_CACHE_BLOCK_TOKENS) * kv_hidden + kvh * D;
      if (is_v) {
        cp_async_16(v_stage + t * Layout::kRowV + piece * 16u, p.value_pages + row + piece * 8u);
      } else {
        cp_async_16(k_stage + t * Layout::kRowK + piece * 16u, p.key_pages + row + piece * 8u);
      }
    }
    cp_async_commit();
  };
  // Everything that depends only on the position happens before the wait; the
  // page-table and norm-weight loads are in flight while the rotation is computed.
  // cached_only: the newest cached rows come from the kernel just before this one, so nothing may
  // be fetched ahead of the dependency wait.
  if (cached_only) pdl_wait();
  const uint32_t pages0 = chunk_begin < chunk_end ? chunk_pages(chunk_begin) : 0u;
  const uint32_t pages1 = chunk_begin + 1u < chunk_end ? chunk_pages(chunk_begin + 1u) : 0u;
  // Warps 0 .. group-1 and group .. 2*group-1 serve the same query heads: the first set takes the
  // first 32-token tile of every 64-token chunk, the second set the second tile, and the two
  // partial softmax states are merged once at the end.  Warp 2*group prepares the new K/V row.
  const uint32_t head_warps = 2u * group;
  const uint32_t hw = warp < group ? warp : warp - group;  // head within the group (warp < head_warps)
  const uint32_t my_tile = warp < group ? 0u : 1u;
  const uint32_t h = kvh * group + hw;
  const float qscale = kAttnLog2e * rsqrtf(static_cast<float>(D));
  const uint16_t *norm_ptr = warp < group ? p.q_norm : p.k_norm;
  float norm_w[PER];
#pragma unroll
  for (uint32_t k = 0; k < PER; ++k)
    norm_w[k] = norm_ptr != nullptr ? bf16_bits_to_f32(norm_ptr[lane + 32u * k]) : 1.0f;
  if (chunk_begin < chunk_end) issue(chunk_begin, 0, pages0);
  if (chunk_begin + 1u < chunk_end) issue(chunk_begin + 1u, 1, pages1);
  RopeFactors<PER> rope;
  rope_factors<PER>(rope, p.rope_theta, position);
  stamp(p.stamps, kStampAfterWait);      // cached K/V copies issued
  pdl_wait();
  stamp(p.stamps, kStampAfterPrologue);  // the QKV projection has completed

  if (warp < group) {
    float v[PER];
#pragma unroll
    for (uint32_t k = 0; k < PER; ++k) {
      const uint32_t e = lane + 32u * k;
      v[k] = __ldcg(p.qkv + h * D + e);
      if (p.q_bias != nullptr) v[k] += bf16_bits_to_f32(p.q_bias[h * D + e]);
    }
    head_norm_rope_pre<PER>(v, p.q_norm != nullptr, norm_w, p.eps, rope);
#pragma unroll
    for (uint32_t k = 0; k < PER; ++k) q_sh[warp * D + lane + 32u * k] = v[k] * qscale;
  } else if (warp == head_warps && owns_current) {
    float kn[PER], vn[PER];
#pragma unroll
    for (uint32_t k = 0; k < PER; ++k) {
      const uint32_t e = lane + 32u * k;
      kn[k] = __ldcg(p.qkv + attention_hidden + kvh * D + e);
      vn[k] = __ldcg(p.qkv + attention_hidden + kv_hidden + kvh * D + e);
      if (p.k_bias != nullptr) kn[k] += bf16_bits_to_f32(p.k_bias[kvh * D + e]);
      if (p.v_bias != nullptr) vn[k] += bf16_bits_to_f32(p.v_bias[kvh * D + e]);
    }
    head_norm_rope_pre<PER>(kn, p.k_norm != nullptr, norm_w, p.eps, rope);
    uint32_t page = p.page_table[position / NERVA_KV_CACHE_BLOCK_TOKENS];
    if (page >= p.page_count) {
      report_error(p.error_word, kErrPageOutOfRange);
      page = 0;
    }
    const uint64_t base = (static_cast<uint64_t>(page) * NERVA_KV_CACHE_BLOCK_TOKENS +
                           position % NERVA_KV_CACHE_BLOCK_TOKENS) * kv_hidden + kvh * D;
#pragma unroll
    for (uint32_t k = 0; k < PER; ++k) {
      const uint32_t e = lane + 32u * k;
      const uint16_t kb = f32_to_bf16_bits(kn[k]), vb = f32_to_bf16_bits(vn[k]);
      k_new[e] = bf16_bits_to_f32(kb);
      v_new[e] = bf16_bits_to_f32(vb);
      p.key_pages[base + e] = kb;
      p.value_pages[base + e] = vb;
    }
  }

  float m_run = -INFINITY, l_run = 0.0f, acc[PER];
#pragma unroll
  for (uint32_t i = 0; i < PER; ++i) acc[i] = 0.0f;
  for (uint32_t chunk = chunk_begin; chunk < chunk_end; ++chunk) {
    const uint32_t stage = (chunk - chunk_begin) & 1u;
    if (chunk + 1u < chunk_end) {
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();  // every thread's copies of this stage (and q, k_new, v_new) are visible
    if (warp < head_warps) {
      const uint8_t *k_stage = smem + stage * Layout::kStageBytes;
      const uint8_t *v_stage = k_stage + kChunkTokens * Layout::kRowK;
      const float *q = q_sh + hw * D;
      const uint32_t tile = my_tile;
      const uint32_t first = chunk * kChunkTokens + tile * 32u;
      if (first < hist) {
        const bool valid = first + lane < hist;
        float score = -INFINITY;
        if (valid) {
          score = 0.0f;
          const uint4 *k_row = reinterpret_cast<const uint4 *>(k_stage + (tile * 32u + lane) * Layout::kRowK);
#pragma unroll
          for (uint32_t b = 0; b < Layout::kPieces; ++b) {
            const uint4 kk = k_row[b];
            const float4 qa = *reinterpret_cast<const float4 *>(q + b * 8u);
            const float4 qb = *reinterpret_cast<const float4 *>(q + b * 8u + 4u);
            score = fmaf(bf16x2_lo(kk.x), qa.x, score);
            score = fmaf(bf16x2_hi(kk.x), qa.y, score);
            score = fmaf(bf16x2_lo(kk.y), qa.z, score);
            score = fmaf(bf16x2_hi(kk.y), qa.w, score);
            score = fmaf(bf16x2_lo(kk.z), qb.x, score);
            score = fmaf(bf16x2_hi(kk.z), qb.y, score);
            score = fmaf(bf16x2_lo(kk.w), qb.z, score);
            score = fmaf(bf16x2_hi(kk.w), qb.w, score);
          }
        }
        const float m_new = fmaxf(m_run, warp_max(score));
        const float pr = exp2f(score - m_new);    // masked tokens: exp2(-inf) = 0
        const float corr = exp2f(m_run - m_new);  // first tile: 0
        l_run = l_run * corr + warp_sum(pr);
        m_run = m_new;
#pragma unroll
        for (uint32_t i = 0; i < PER; ++i) acc[i] *= corr;
        p_sh[warp * 32u + lane] = pr;
        __syncwarp();
        const uint32_t left = hist - first < 32u ? hist - first : 32u;
        const uint8_t *v_tile = v_stage + tile * 32u * Layout::kRowV + lane * PER * 2u;
        // Eight tokens' loads are issued before their multiply-adds (same order of additions as
        // the one-token loop below, which takes the remainder).
        uint32_t t = 0;
        if (PER == 4) {
          for (; t + 8u <= left; t += 8u) {
            uint2 w[8];
            float pt[8];
#pragma unroll
            for (uint32_t u = 0; u < 8u; ++u) {
              w[u] = *reinterpret_cast<const uint2 *>(v_tile + (t + u) * Layout::kRowV);
              pt[u] = p_sh[warp * 32u + t + u];
            }
#pragma unroll
            for (uint32_t u = 0; u < 8u; ++u) {
              acc[0] = fmaf(pt[u], bf16x2_lo(w[u].x), acc[0]);
              acc[1 % PER] = fmaf(pt[u], bf16x2_hi(w[u].x), acc[1 % PER]);
              acc[2 % PER] = fmaf(pt[u], bf16x2_lo(w[u].y), acc[2 % PER]);
              acc[3 % PER] = fmaf(pt[u], bf16x2_hi(w[u].y), acc[3 % PER]);
            }
          }
        }
        for (; t < left; ++t) {
          const float pt = p_sh[warp * 32u + t];
          if (PER == 4) {
            const uint2 w = *reinterpret_cast<const uint2 *>(v_tile + t * Layout::kRowV);
            acc[0] = fmaf(pt, bf16x2_lo(w.x), acc[0]);
            acc[1 % PER] = fmaf(pt, bf16x2_hi(w.x), acc[1 % PER]);
            acc[2 % PER] = fmaf(pt, bf16x2_lo(w.y), acc[2 % PER]);
            acc[3 % PER] = fmaf(pt, bf16x2_hi(w.y), acc[3 % PER]);
          } else {
            const uint32_t w = *reinterpret_cast<const uint32_t *>(v_tile + t * Layout::kRowV);
            acc[0] = fmaf(pt, bf16x2_lo(w), acc[0]);
            acc[1 % PER] = fmaf(pt, bf16x2_hi(w), acc[1 % PER]);
          }
        }
        __syncwarp();
      }
    }
    __syncthreads();  // the stage is free again
    if (chunk + kStages < chunk_end) issue(chunk + kStages, stage, chunk_pages(chunk + kStages));
  }
  if (chunk_begin >= chunk_end) __syncthreads();  // q, k_new, v_new visible when no chunk ran

  // The second warp set hands its softmax state to the first through the stage memory, which is
  // idle now (every copy has landed and every warp is past its last read of it).
  float *handoff = reinterpret_cast<float *>(smem);  // [group][32 lanes][PER acc | m | l]
  if (warp >= group && warp < head_warps) {
    float *dst = handoff + (hw * 32u + lane) * (PER + 2u);
#pragma unroll
    for (uint32_t i = 0; i < PER; ++i) dst[i] = acc[i];
    dst[PER] = m_run;
    dst[PER + 1u] = l_run;
  }
  __syncthreads();
  if (warp < group) {
    const float *src = handoff + (warp * 32u + lane) * (PER + 2u);
    const float m1 = src[PER], l1 = src[PER + 1u];
    if (l1 > 0.0f) {  // the second tiles held tokens
      const float m = fmaxf(m_run, m1);
      const float c0 = exp2f(m_run - m), c1 = exp2f(m1 - m);
      l_run = l_run * c0 + l1 * c1;
#pragma unroll
      for (uint32_t i = 0; i < PER; ++i) acc[i] = acc[i] * c0 + src[i] * c1;
      m_run = m;
    }
  }

  if (warp < group) {
    float m = m_run, l = l_run;
    if (owns_current) {
      const float *q = q_sh + warp * D;
      float dot = 0.0f;
#pragma unroll
      for (uint32_t i = 0; i < PER; ++i) dot = fmaf(q[lane * PER + i], k_new[lane * PER + i], dot);
      const float s_new = warp_sum(dot);
      const float m2 = fmaxf(m, s_new);
      const float corr = exp2f(m - m2);
      const float pr = exp2f(s_new - m2);
      l = l * corr + pr;
#pragma unroll
      for (uint32_t i = 0; i < PER; ++i) acc[i] = acc[i] * corr + pr * v_new[lane * PER + i];
      m = m2;
    }
    const uint64_t slot = static_cast<uint64_t>(h) * S + s;
    if (PER == 4) {
      *reinterpret_cast<float4 *>(p.partial_acc + slot * D + lane * PER) =
          make_float4(acc[0], acc[1 % PER], acc[2 % PER], acc[3 % PER]);
    } else {
      *reinterpret_cast<float2 *>(p.partial_acc + slot * D + lane * PER) = make_float2(acc[0], acc[1 % PER]);
    }
    if (lane == 0) {
      p.partial_m[slot] = m;
      p.partial_l[slot] = l;
    }
  }
  stamp(p.stamps, kStampExit);  // partial written (a merging block stamps again at its end)

  // Publish the partials, then take a ticket: the block that draws the last
  // ticket of its KV head sees every partial of the group's heads.  The barrier
  // orders every warp's partial stores before thread 0's release, and thread 0's
  // acquire before every warp's loads after the second barrier, so one acq_rel
  // atomic replaces a device-wide fence by every thread on each side.
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t drawn;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(drawn) : "l"(p.tickets + kvh) : "memory");
    ticket = drawn;
  }
  __syncthreads();
  if (ticket != S - 1u) return;
  if (warp < group) {
    // Every load of the merge is issued before anything is computed from them (every slot was
    // written by this launch; an empty span holds zeros and gets weight 0): one round trip to L2.
    float ms[kFusedMaxSplits], ls[kFusedMaxSplits];
    float part[kFusedMaxSplits][PER];
#pragma unroll
    for (uint32_t i = 0; i < kFusedMaxSplits; ++i) {
      ms[i] = i < S ? __ldcg(p.partial_m + h * S + i) : -INFINITY;
      ls[i] = i < S ? __ldcg(p.partial_l + h * S + i) : 0.0f;
      const float *src = p.partial_acc + (static_cast<uint64_t>(h) * S + (i < S ? i : 0u)) * D + lane * PER;
      if (PER == 4) {
        const float4 t4 = i < S ? __ldcg(reinterpret_cast<const float4 *>(src)) : make_float4(0.f, 0.f, 0.f, 0.f);
        part[i][0] = t4.x;
        part[i][1 % PER] = t4.y;
        part[i][2 % PER] = t4.z;
        part[i][3 % PER] = t4.w;
      } else {
        const float2 t2 = i < S ? __ldcg(reinterpret_cast<const float2 *>(src)) : make_float2(0.f, 0.f);
        part[i][0] = t2.x;
        part[i][1 % PER] = t2.y;
      }
    }
    float m = -INFINITY;
#pragma unroll
    for (uint32_t i = 0; i < kFusedMaxSplits; ++i) {
      if (ls[i] > 0.0f) m = fmaxf(m, ms[i]);
    }
    float l = 0.0f;
#pragma unroll
    for (uint32_t i = 0; i < kFusedMaxSplits; ++i) {
      ms[i] = ls[i] > 0.0f ? exp2f(ms[i] - m) : 0.0f;  // weight of span i
      l = fmaf(ls[i], ms[i], l);
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    float a[PER];
#pragma unroll
    for (uint32_t k = 0; k < PER; ++k) a[k] = 0.0f;
#pragma unroll
    for (uint32_t i = 0; i < kFusedMaxSplits; ++i) {
#pragma unroll
      for (uint32_t k = 0; k < PER; ++k) a[k] = fmaf(part[i][k], ms[i], a[k]);
    }
#pragma unroll
    for (uint32_t k = 0; k < PER; ++k) p.out_bf16[h * D + lane * PER + k] = f32_to_bf16_bits(a[k] * inv);
  }
  if (threadIdx.x == 0) p.tickets[kvh] = 0;  // ready for the next launch
  stamp(p.stamps, kStampExit);
}

}  // namespace

bool fused_attention_supported(uint32_t heads, uint32_t kv_heads, uint32_t head_dim) {
  return (head_dim == 64 || head_dim == 128) && kv_heads != 0 && heads % kv_heads == 0 &&
         heads / kv_heads <= kFusedMaxGroup;
}

// Spans per KV head for a step whose context is at most target_context: one
// 64-token chunk per block while that needs no more than 16 blocks per KV head,
// in powers of two so that a growing context re-captures the step rarely.
uint32_t fused_attention_splits(uint32_t target_context) {
  const uint32_t chunks = (target_context + kChunkTokens - 1u) / kChunkTokens;
  uint32_t s = 1;
  while (s < chunks && s < kFusedMaxSplits) s <<= 1;
  return s;
}

cudaError_t configure_fused_attention_kernel() {
  cudaError_t err = cudaSuccess;
  auto set = [&](void (*kernel)(FusedAttentionParams), uint32_t bytes) {
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
  };
  set(fused_decode_attention_kernel<4, false>, FusedLayout<128>::bytes(kFusedMaxGroup));
  set(fused_decode_attention_kernel<4, true>, FusedLayout<128>::bytes(kFusedMaxGroup));
  set(fused_decode_attention_kernel<2, false>, FusedLayout<64>::bytes(kFusedMaxGroup));
  set(fused_decode_attention_kernel<2, true>, FusedLayout<64>::bytes(kFusedMaxGroup));
  return err;
}

cudaError_t launch_fused_attention(cudaStream_t stream, const FusedAttentionParams &p) {
  if (!fused_attention_supported(p.heads, p.kv_heads, p.head_dim) || p.splits == 0 ||
      p.splits > kFusedMaxSplits)
    return cudaErrorInvalidValue;
  const uint32_t group = p.heads / p.kv_heads;
  const uint32_t blocks = p.kv_heads * p.splits;
  const uint32_t threads = (2u * group + 1u) * 32u;
  if (p.rows != nullptr) {
    if (p.row_count == 0 || p.row_count > 65535u) return cudaErrorInvalidValue;
    const dim3 grid(blocks, p.row_count);
    if (p.head_dim == 128)
      return launch_with_pdl(fused_decode_attention_kernel<4, true>, grid, dim3(threads),
                             FusedLayout<128>::bytes(group), stream, p.pdl != 0, p);
    return launch_with_pdl(fused_decode_attention_kernel<2, true>, grid, dim3(threads), FusedLayout<64>::bytes(group),
                           stream, p.pdl != 0, p);
  }
  if (p.head_dim == 128) {
    return launch_with_pdl(fused_decode_attention_kernel<4, false>, dim3(blocks), dim3(threads),
                           FusedLayout<128>::bytes(group), stream, p.pdl != 0, p);
  }
  return launch_with_pdl(fused_decode_attention_kernel<2, false>, dim3(blocks), dim3(threads),
                         FusedLayout<64>::bytes(group), stream, p.pdl != 0, p);
}

}  // namespace nb
