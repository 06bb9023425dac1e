// GQA paged split-KV decode attention (one query token per sequence).
//
// Replaces the reference's chunked decode attention and its merge kernel
// (hf_decode_sequence/attention_kernels.cu:528-760, kernels.cu:494-555) with the
// same mathematics: s = q.k / sqrt(d), online softmax, acc += p v per split,
// then out = sum_s acc_s e^{m_s - M} / sum_s l_s e^{m_s - M}.
//
// Layout of the work: grid (splits, kv_heads, batch), 4 warps per block, two blocks per SM.  A
// block serves the G <= 8 query heads that share one KV head over its span of 16-token pages, so
// every cached byte is fetched once per group.  Each warp walks its own pages (span page w, w + 4,
// ...) through a private ring of shared-memory stages: lane 0 looks the physical page up and asks
// for the page's K and V slices of this KV head with 2-D bulk tensor copies (one 16 x 64 element
// box per 64 dims, 128-byte swizzle, completion on the stage's mbarrier) — 24 pages, 192 KiB, in
// flight per SM, and no block-level barrier in the loop.  The merge of the spans is a second,
// small launch; both carry the programmatic-serialization attribute, so when attention launches
// follow each other (one per layer of a decode step) the next one streams its pages while this
// one's merge runs, and only its last step — writing its partials — waits for that merge.
//
// Arithmetic on the tensor pipe (mma.sync m16n8k16, bf16 in, fp32 accumulate).  The 16 rows of the
// M dimension hold the group's queries twice: rows 0..7 the bf16 roundings of the (pre-scaled) fp32
// queries, rows 8..15 the bf16 roundings of what the first rounding lost, so q.k keeps fp32-level
// accuracy although K is multiplied as bf16; the accumulator fragment puts rows r and r + 8 into
// the same thread, which adds the two parts.  The probabilities are split the same way for P.V.
// K fragments come from shared memory with ldmatrix, V fragments with ldmatrix.trans; the swizzle
// of the copies makes both conflict-free without padding.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <math.h>
#include <string.h>

#include "common.cuh"
#include "kernels.cuh"
#include "mma_bf16.cuh"

namespace nb {
namespace {

constexpr uint32_t kAttnWarps = 4;
constexpr uint32_t kAttnBlocksPerSm = 2;
constexpr uint32_t kAttnStages = 3;
constexpr uint32_t kPageTokens = NERVA_KV_CACHE_BLOCK_TOKENS;  // 16: one page = the K dimension of one P.V mma
constexpr uint32_t kMaxGroupHeads = 8;
constexpr uint32_t kMaxSplits = 256;   // the merge kernel's weight table
constexpr float kLog2e = 1.4426950408889634f;

template <uint32_t D>
struct PagedLayout {
  static constexpr uint32_t kHalves = D / 64u;                    // 64-dim boxes per row
  static constexpr uint32_t kBoxBytes = kPageTokens * 128u;       // 16 rows x 128 bytes
  static constexpr uint32_t kStageBytes = 2u * kHalves * kBoxBytes;  // K boxes then V boxes
  static constexpr uint32_t kWarpBytes = kAttnStages * kStageBytes;
};

struct PagedShared {
  uint64_t full[kAttnWarps][kAttnStages];
};

template <uint32_t D>
constexpr uint32_t paged_smem_bytes() {
  // rings (1024-byte aligned) | q fp32 [8][D] | PagedShared
  return 1024u + kAttnWarps * PagedLayout<D>::kWarpBytes + kMaxGroupHeads * D * 4u +
         static_cast<uint32_t>(sizeof(PagedShared)) + 64u;
}

__device__ __forceinline__ void tma_load_box(void *dst, const CUtensorMap *map, uint32_t x, uint32_t y, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
          "r"(smem_addr(dst)),
      "l"(map), "r"(x), "r"(y), "r"(smem_addr(bar))
      : "memory");
}
// Byte offset of 16-byte piece `piece` of row `row` inside a 128-byte-swizzled 16 x 128 B box.
__device__ __forceinline__ uint32_t swizzled(uint32_t row, uint32_t piece) {
  return row * 128u + ((piece ^ (row & 7u)) << 4);
}

// The K / V tensor-map pairs of the caches a row-form launch spans (kernel parameter space).
struct RowCacheMaps {
  CUtensorMap k[kAttentionRowCaches], v[kAttentionRowCaches];
};

// One block's work.  ROWS: sequence b is row b of a block step (p.rows[b]); the maps are that
// row's cache, whose pages of layer p.layer start at row p.layer * pages * 16 of the 2-D view.
template <uint32_t D, bool ROWS>
__device__ __forceinline__ void gqa_decode_block(const CUtensorMap *map_k_all, const CUtensorMap *map_v_all,
                                                 const AttentionParams &p) {
  using L = PagedLayout<D>;
  constexpr uint32_t kKSteps = D / 16u;   // mma k-steps of q.k
  constexpr uint32_t kNTiles = D / 8u;    // mma n-tiles of p.v
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *rings = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t{1023});
  float *q_s = reinterpret_cast<float *>(rings + kAttnWarps * L::kWarpBytes);
  PagedShared &sh = *reinterpret_cast<PagedShared *>(q_s + kMaxGroupHeads * D);

  pdl_trigger();
  const uint32_t split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const uint32_t G = p.heads / p.kv_heads;
  // q, the cache, the page table and the cursor are inputs that an earlier launch of this pair
  // never writes; only the partial buffers below are shared with the previous launch's merge
  if (ROWS || p.cursor != nullptr) pdl_wait();  // the cursor, or the row's q and newest cache row, come from the previous kernel
  const CUtensorMap *map_k = map_k_all, *map_v = map_v_all;
  const float *q_row;
  const uint32_t *table;
  uint32_t context, page_count, y_base;
  if (ROWS) {
    const FusedAttentionRow &r = p.rows[b];
    map_k += r.map_index;
    map_v += r.map_index;
    q_row = r.qkv;
    table = r.page_table;
    context = r.position + 1u;
    page_count = r.page_count;
    y_base = p.layer * r.page_count * kPageTokens;
  } else {
    q_row = p.q + static_cast<uint64_t>(b) * p.heads * D;
    table = p.page_table + static_cast<uint64_t>(b) * p.page_count;
    context = p.cursor != nullptr ? *p.cursor + 1u : p.context;
    page_count = p.page_count;
    y_base = b * p.page_count * kPageTokens;  // row of the [batch * pages * 16][kv_hidden] view
  }
  const uint32_t pages_total = (context + kPageTokens - 1u) / kPageTokens;
  const uint32_t pages_per_split = (pages_total + p.splits - 1u) / p.splits;
  const uint32_t page_begin = split * pages_per_split;
  uint32_t page_end = page_begin + pages_per_split;
  if (page_end > pages_total) page_end = pages_total;

  // q, pre-multiplied by log2(e)/sqrt(d) so that the softmax runs on exp2; rows beyond the group stay zero.
  const float qscale = kLog2e * rsqrtf(static_cast<float>(D));
  const float *q_in = q_row + static_cast<uint64_t>(kvh) * G * D;
  for (uint32_t i = threadIdx.x; i < kMaxGroupHeads * D; i += blockDim.x) q_s[i] = i < G * D ? q_in[i] * qscale : 0.0f;
  if (lane == 0) {
    for (uint32_t s = 0; s < kAttnStages; ++s) mbar_init(&sh.full[warp][s], 1);
    mbar_init_fence();
  }
  __syncthreads();

  uint8_t *ring = rings + warp * L::kWarpBytes;
  // This warp's pages: page_begin + warp, + kAttnWarps, ...
  const uint32_t first = page_begin + warp;
  const uint32_t my_pages = first < page_end ? (page_end - first + kAttnWarps - 1u) / kAttnWarps : 0u;
  auto issue = [&](uint32_t i) {  // lane 0 only
    const uint32_t logical = first + i * kAttnWarps;
    uint32_t phys = table[logical];
    if (phys >= page_count) {
      report_error(p.error_word, kErrPageOutOfRange);
      phys = 0;
    }
    const uint32_t stage = i % kAttnStages;
    uint8_t *dst = ring + stage * L::kStageBytes;
    const uint32_t y = y_base + phys * kPageTokens;
    mbar_arrive_expect_tx(&sh.full[warp][stage], L::kStageBytes);
#pragma unroll
    for (uint32_t h = 0; h < L::kHalves; ++h) {
      tma_load_box(dst + h * L::kBoxBytes, map_k, kvh * D + h * 64u, y, &sh.full[warp][stage]);
      tma_load_box(dst + (L::kHalves + h) * L::kBoxBytes, map_v, kvh * D + h * 64u, y, &sh.full[warp][stage]);
    }
  };
  if (lane == 0) {
    for (uint32_t i = 0; i < kAttnStages && i < my_pages; ++i) issue(i);
  }

  // A fragments of q: thread (g = lane / 4, t = lane % 4) holds, for row g, columns 2t, 2t+1 and
  // 2t+8, 2t+9 of every 16-wide k-step; registers 0 and 2 carry the bf16 rounding (row g), 1 and 3
  // what it lost (row g + 8).
  const uint32_t g = lane >> 2, t = lane & 3u;
  uint32_t qa[kKSteps][4];
#pragma unroll
  for (uint32_t ks = 0; ks < kKSteps; ++ks) {
    const float *src = q_s + g * D + ks * 16u + 2u * t;
    qa[ks][0] = pack_bf16_hi(src[0], src[1]);
    qa[ks][1] = pack_bf16_lo(src[0], src[1]);
    qa[ks][2] = pack_bf16_hi(src[8], src[9]);
    qa[ks][3] = pack_bf16_lo(src[8], src[9]);
  }
  const bool live = g < G;  // threads of rows beyond the group carry zeros through the whole loop

  float m_run = -INFINITY, l_run = 0.0f;
  float o[kNTiles][4];
#pragma unroll
  for (uint32_t n = 0; n < kNTiles; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;

  bool dead = false;
  for (uint32_t i = 0; i < my_pages; ++i) {
    const uint32_t stage = i % kAttnStages;
    if (!dead && !mbar_wait_bounded(&sh.full[warp][stage], (i / kAttnStages) & 1u)) {
      dead = true;
      report_error(p.error_word, kErrTmaWaitTimeout);
    }
    const uint32_t k_base = smem_addr(ring + stage * L::kStageBytes);
    const uint32_t v_base = k_base + L::kHalves * L::kBoxBytes;
    const uint32_t token0 = (first + i * kAttnWarps) * kPageTokens;
    const uint32_t valid = context - token0 < kPageTokens ? context - token0 : kPageTokens;
    if (valid < kPageTokens) {
      // the last page: rows beyond the context hold whatever the pool had; a zero probability times
      // a non-finite value would still poison P.V, so those V rows are cleared first
      uint8_t *v_ptr = ring + stage * L::kStageBytes + L::kHalves * L::kBoxBytes;
      for (uint32_t idx = lane; idx < (kPageTokens - valid) * 8u * L::kHalves; idx += 32u) {
        const uint32_t row = valid + idx / (8u * L::kHalves), rest = idx % (8u * L::kHalves);
        *reinterpret_cast<uint4 *>(v_ptr + (rest / 8u) * L::kBoxBytes + row * 128u + (rest % 8u) * 16u) =
            make_uint4(0u, 0u, 0u, 0u);
      }
      __syncwarp();
    }
    // ---- scores: S[16 x 16 tokens] = Q K^T, two n-tiles of 8 tokens ----
    float s_acc[2][4];
#pragma unroll
    for (uint32_t nt = 0; nt < 2; ++nt) s_acc[nt][0] = s_acc[nt][1] = s_acc[nt][2] = s_acc[nt][3] = 0.0f;
#pragma unroll
    for (uint32_t nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (uint32_t kp = 0; kp < kKSteps / 2u; ++kp) {
        // four 8x8 matrices: tokens nt*8.., dims kp*32 + {0, 8, 16, 24}: B fragments of two k-steps
        const uint32_t row = nt * 8u + (lane & 7u);
        const uint32_t dim_piece = kp * 4u + (lane >> 3);  // 16-byte piece (8 dims) along the whole row
        const uint32_t addr = k_base + (dim_piece / 8u) * L::kBoxBytes + swizzled(row, dim_piece % 8u);
        uint32_t kb[4];
        ldmatrix_x4(kb, addr);
        mma_bf16(s_acc[nt], qa[2u * kp], kb[0], kb[1]);
        mma_bf16(s_acc[nt], qa[2u * kp + 1u], kb[2], kb[3]);
      }
    }
    // this thread's four scores of row g: tokens 2t, 2t+1 (n-tile 0) and 8+2t, 9+2t (n-tile 1)
    float sc[4] = {s_acc[0][0] + s_acc[0][2], s_acc[0][1] + s_acc[0][3], s_acc[1][0] + s_acc[1][2],
                   s_acc[1][1] + s_acc[1][3]};
    const uint32_t tok[4] = {2u * t, 2u * t + 1u, 8u + 2u * t, 9u + 2u * t};
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j)
      if (tok[j] >= valid || !live || dead) sc[j] = -INFINITY;
    // ---- online softmax (base 2) over the page ----
    float m_page = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
    m_page = fmaxf(m_page, __shfl_xor_sync(0xffffffffu, m_page, 1));
    m_page = fmaxf(m_page, __shfl_xor_sync(0xffffffffu, m_page, 2));
    const float m_new = fmaxf(m_run, m_page);
    const float corr = m_new == -INFINITY ? 1.0f : exp2f(m_run - m_new);  // first page: exp2(-inf) = 0
    float pr[4];
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j) pr[j] = m_new == -INFINITY ? 0.0f : exp2f(sc[j] - m_new);
    l_run = l_run * corr + ((pr[0] + pr[1]) + (pr[2] + pr[3]));  // this thread's share; the quad is summed at the end
    m_run = m_new;
#pragma unroll
    for (uint32_t n = 0; n < kNTiles; ++n) {
      o[n][0] *= corr;
      o[n][1] *= corr;
      o[n][2] *= corr;
      o[n][3] *= corr;
    }
    // A fragment of P for the page's 16 tokens: registers 0, 2 the bf16 roundings, 1, 3 what they lost
    uint32_t pa[4];
    pa[0] = pack_bf16_hi(pr[0], pr[1]);
    pa[1] = pack_bf16_lo(pr[0], pr[1]);
    pa[2] = pack_bf16_hi(pr[2], pr[3]);
    pa[3] = pack_bf16_lo(pr[2], pr[3]);
    // ---- O += P V: n-tiles of 8 dims, V fragments transposed on the way out of shared memory ----
#pragma unroll
    for (uint32_t np = 0; np < kNTiles / 2u; ++np) {
      // four 8x8 matrices: (tokens 0..7 | 8..15) x (dims np*16 + 0..7 | 8..15)
      const uint32_t row = ((lane >> 3) & 1u) * 8u + (lane & 7u);
      const uint32_t dim_piece = np * 2u + (lane >> 4);
      const uint32_t addr = v_base + (dim_piece / 8u) * L::kBoxBytes + swizzled(row, dim_piece % 8u);
      uint32_t vb[4];
      ldmatrix_x4_trans(vb, addr);
      mma_bf16(o[2u * np], pa, vb[0], vb[1]);
      mma_bf16(o[2u * np + 1u], pa, vb[2], vb[3]);
    }
    __syncwarp();
    // refill the stage this iteration has finished with
    if (lane == 0 && !dead && i + kAttnStages < my_pages) {
      fence_proxy_async();
      issue(i + kAttnStages);
    }
  }
  if (dead && lane == 0) {
    // give copies still in flight one more bounded chance to land before the memory is reused
    for (uint32_t s = 0; s < kAttnStages; ++s) {
      mbar_wait_bounded(&sh.full[warp][s], 0);
      mbar_wait_bounded(&sh.full[warp][s], 1);
    }
  }
  // the quad holds four shares of the row's l
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  __syncthreads();

  // ---- merge the block's warps (stage memory is free now) ----
  pdl_wait();  // the previous launch's merge may still be reading the partial buffers
  float *merge = reinterpret_cast<float *>(rings);  // [warps][G][D + 2]
  constexpr uint32_t kRec = D + 2u;
  if (live) {
    float *rec = merge + (warp * G + g) * kRec;
#pragma unroll
    for (uint32_t n = 0; n < kNTiles; ++n) {
      rec[n * 8u + 2u * t] = o[n][0] + o[n][2];
      rec[n * 8u + 2u * t + 1u] = o[n][1] + o[n][3];
    }
    if (t == 0) {
      rec[D] = m_run;
      rec[D + 1] = l_run;
    }
  }
  __syncthreads();
  for (uint32_t idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const uint32_t gg = idx / D, d = idx % D;
    float m = -INFINITY;
    for (uint32_t w = 0; w < kAttnWarps; ++w) m = fmaxf(m, merge[(w * G + gg) * kRec + D]);
    float a = 0.0f, l = 0.0f;
    if (m > -INFINITY) {
      for (uint32_t w = 0; w < kAttnWarps; ++w) {
        const float *rec = merge + (w * G + gg) * kRec;
        if (rec[D] == -INFINITY) continue;
        const float wgt = exp2f(rec[D] - m);
        a = fmaf(rec[d], wgt, a);
        l = fmaf(rec[D + 1], wgt, l);
      }
    }
    const uint64_t slot = (static_cast<uint64_t>(b) * p.heads + kvh * G + gg) * p.splits + split;
    p.partial_acc[slot * D + d] = a;
    if (d == 0) {
      p.partial_m[slot] = m;
      p.partial_l[slot] = l;
    }
  }
}

template <uint32_t D>
__global__ void __launch_bounds__(kAttnWarps * 32, kAttnBlocksPerSm)
gqa_decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                  AttentionParams p) {
  gqa_decode_block<D, false>(&map_k, &map_v, p);
}

template <uint32_t D>
__global__ void __launch_bounds__(kAttnWarps * 32, kAttnBlocksPerSm)
gqa_decode_rows_kernel(const __grid_constant__ RowCacheMaps maps, AttentionParams p) {
  gqa_decode_block<D, true>(maps.k, maps.v, p);
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

// out = sum_s acc_s 2^{m_s - M} / sum_s l_s 2^{m_s - M}; one block per (head, batch), blockDim =
// (dims rounded up to 32, groups).  Warp 0 turns the (m, l) pairs of all spans into normalised
// weights in one round trip (a lane per span); then thread (i, g) adds dimension i over the spans
// g, g + groups, ... with eight loads in flight, and the groups' sums are added in group order.
constexpr uint32_t kMergeGroups = 8;
__global__ void gqa_merge_kernel(AttentionParams p) {
  __shared__ float weight[256];  // launch_attention refuses more spans
  __shared__ float part[kMergeGroups][256];
  pdl_trigger();
  pdl_wait();  // the partials come from the launch just before
  const uint32_t head = blockIdx.x, b = blockIdx.y;
  const uint32_t d = p.head_dim, S = p.splits;
  const uint64_t slot0 = (static_cast<uint64_t>(b) * p.heads + head) * S;
  const uint32_t tid = threadIdx.y * blockDim.x + threadIdx.x;
  if (tid < 32u) {
    const uint32_t lane = tid;
    float m = -INFINITY;
    for (uint32_t s = lane; s < S; s += 32u)
      if (__ldcg(p.partial_l + slot0 + s) > 0.0f) m = fmaxf(m, __ldcg(p.partial_m + slot0 + s));
    m = warp_max(m);
    float l = 0.0f;
    for (uint32_t s = lane; s < S; s += 32u) {
      const float ls = __ldcg(p.partial_l + slot0 + s);
      const float w = ls > 0.0f ? exp2f(__ldcg(p.partial_m + slot0 + s) - m) : 0.0f;
      weight[s] = w;
      l = fmaf(ls, w, l);
    }
    l = warp_sum(l);
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    __syncwarp();
    for (uint32_t s = lane; s < S; s += 32u) weight[s] *= inv;
  }
  __syncthreads();
  const uint32_t i = threadIdx.x, g = threadIdx.y, groups = blockDim.y;
  if (i < d) {
    float a = 0.0f;
    uint32_t s = g;
    for (; s + 7u * groups < S; s += 8u * groups) {
      float v[8];
#pragma unroll
      for (uint32_t u = 0; u < 8u; ++u) v[u] = __ldcg(p.partial_acc + (slot0 + s + u * groups) * d + i);
#pragma unroll
      for (uint32_t u = 0; u < 8u; ++u) a = fmaf(v[u], weight[s + u * groups], a);
    }
    for (; s < S; s += groups) a = fmaf(__ldcg(p.partial_acc + (slot0 + s) * d + i), weight[s], a);
    part[g][i] = a;
  }
  __syncthreads();
  if (g == 0 && i < d) {
    float a = part[0][i];
    for (uint32_t k = 1; k < groups; ++k) a += part[k][i];
    const uint64_t o = (static_cast<uint64_t>(b) * p.heads + head) * d + i;
    if (p.out_f32 != nullptr) p.out_f32[o] = a;
    if (p.out_bf16 != nullptr) p.out_bf16[o] = f32_to_bf16_bits(a);
  }
}

// Threads of the merge launch: one per dimension, and as many span groups as the spans can use.
dim3 merge_block(uint32_t head_dim, uint32_t splits) {
  uint32_t x = ((head_dim + 31u) / 32u) * 32u;
  if (x > 256u) x = 256u;
  uint32_t groups = splits >= 64u ? kMergeGroups : (splits >= 16u ? 4u : 1u);
  while (x * groups > 1024u) groups /= 2u;
  return dim3(x, groups);
}

}  // namespace

cudaError_t configure_attention_kernels() {
  cudaError_t err = cudaFuncSetAttribute(gqa_decode_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(paged_smem_bytes<128>()));
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(gqa_decode_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(paged_smem_bytes<64>()));
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(gqa_decode_rows_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(paged_smem_bytes<128>()));
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(gqa_decode_rows_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(paged_smem_bytes<64>()));
  return err;
}

// Spans per (sequence, KV head).  kAttnBlocksPerSm blocks per SM are resident, blocks run in waves
// of that many per SM, and a block's time is its span: the count that minimises waves x pages-per-span is taken, with
// at least one page per warp in a span and at most kMaxSplits spans.
uint32_t attention_default_splits(uint32_t context, uint32_t batch, uint32_t kv_heads,
                                  uint32_t sm_count) {
  const uint32_t pages = (context + kPageTokens - 1u) / kPageTokens;
  const uint32_t units = batch * kv_heads;
  uint32_t most = pages / kAttnWarps;
  if (most > kMaxSplits) most = kMaxSplits;
  if (most == 0) most = 1;
  uint32_t best = 1;
  uint64_t best_cost = UINT64_MAX;
  for (uint32_t s = 1; s <= most; ++s) {
    const uint64_t slots = static_cast<uint64_t>(sm_count) * kAttnBlocksPerSm;
    const uint64_t waves = (static_cast<uint64_t>(units) * s + slots - 1u) / slots;
    const uint64_t span = (pages + s - 1u) / s + 8u;  // + a fixed cost per block (set-up, merge) in page units
    // the second launch merges s spans per head: about a page's time per 16 spans on top of a fixed two
    const uint64_t cost = waves * span + 2u + s / 16u;
    if (cost < best_cost) {
      best_cost = cost;
      best = s;
    }
  }
  return best;
}

cudaError_t launch_attention(cudaStream_t stream, const AttentionParams &p) {
  if (p.splits == 0 || p.splits > 256u) return cudaErrorInvalidValue;  // the merge kernel's weight table
  const uint32_t group = p.heads / p.kv_heads;
  const uint32_t kv_hidden = p.kv_heads * p.head_dim;
  const bool paged = (p.head_dim == 128 || p.head_dim == 64) && group <= kMaxGroupHeads && tensor_map_available() &&
                     reinterpret_cast<uintptr_t>(p.key_pages) % 16u == 0 &&
                     reinterpret_cast<uintptr_t>(p.value_pages) % 16u == 0;
  if (paged) {
    // K and V as 2-D tensors [batch * pages * 16 tokens][kv_hidden]; a box is one page x 64 dims
    alignas(64) CUtensorMap map_k, map_v;
    const uint64_t rows = static_cast<uint64_t>(p.batch) * p.page_count * kPageTokens;
    if (!encode_bf16_map_2d(&map_k, p.key_pages, kv_hidden, rows, 64, kPageTokens) ||
        !encode_bf16_map_2d(&map_v, p.value_pages, kv_hidden, rows, 64, kPageTokens))
      return cudaErrorInvalidValue;
    const dim3 grid(p.splits, p.kv_heads, p.batch);
    cudaError_t launched;
    if (p.head_dim == 128) {
      launched = launch_with_pdl(gqa_decode_kernel<128>, grid, dim3(kAttnWarps * 32), paged_smem_bytes<128>(), stream,
                                 true, map_k, map_v, p);
    } else {
      launched = launch_with_pdl(gqa_decode_kernel<64>, grid, dim3(kAttnWarps * 32), paged_smem_bytes<64>(), stream, true,
                                 map_k, map_v, p);
    }
    if (launched != cudaSuccess) return launched;
  } else {
    if (p.head_dim > 256) return cudaErrorNotSupported;
    gqa_decode_generic_kernel<<<dim3(p.heads, p.batch), 32, 0, stream>>>(p);
  }
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return err;
  return launch_with_pdl(gqa_merge_kernel, dim3(p.heads, p.batch), merge_block(p.head_dim, p.splits), 0, stream, paged, p);
}

bool attention_rows_supported(uint32_t heads, uint32_t kv_heads, uint32_t head_dim) {
  return (head_dim == 128 || head_dim == 64) && kv_heads != 0 && heads % kv_heads == 0 &&
         heads / kv_heads <= kMaxGroupHeads && tensor_map_available();
}

uint32_t attention_rows_splits(uint32_t longest_context, uint32_t rows, uint32_t kv_heads, uint32_t sm_count) {
  const uint32_t splits = attention_default_splits(longest_context, rows, kv_heads, sm_count);
  return splits > 16u ? 16u : splits;  // the block steps keep 16 partial slots per (row, head)
}

cudaError_t launch_attention_rows(cudaStream_t stream, const AttentionParams &p, const TensorMapStorage *k_maps,
                                  const TensorMapStorage *v_maps, uint32_t caches) {
  if (p.rows == nullptr || p.batch == 0 || p.splits == 0 || p.splits > 16u || caches == 0 ||
      caches > kAttentionRowCaches || !attention_rows_supported(p.heads, p.kv_heads, p.head_dim))
    return cudaErrorInvalidValue;
  static_assert(sizeof(TensorMapStorage) == sizeof(CUtensorMap), "a tensor map is 128 bytes");
  RowCacheMaps maps;
  for (uint32_t i = 0; i < kAttentionRowCaches; ++i) {
    const uint32_t from = i < caches ? i : 0;  // unused entries repeat the first pair
    memcpy(&maps.k[i], &k_maps[from], sizeof(CUtensorMap));
    memcpy(&maps.v[i], &v_maps[from], sizeof(CUtensorMap));
  }
  const dim3 grid(p.splits, p.kv_heads, p.batch);
  cudaError_t err;
  if (p.head_dim == 128)
    err = launch_with_pdl(gqa_decode_rows_kernel<128>, grid, dim3(kAttnWarps * 32), paged_smem_bytes<128>(), stream,
                          true, maps, p);
  else
    err = launch_with_pdl(gqa_decode_rows_kernel<64>, grid, dim3(kAttnWarps * 32), paged_smem_bytes<64>(), stream, true,
                          maps, p);
  if (err != cudaSuccess) return err;
  return launch_with_pdl(gqa_merge_kernel, dim3(p.heads, p.batch), merge_block(p.head_dim, p.splits), 0, stream, true, p);
}

}  // namespace nb
