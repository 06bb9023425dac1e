// DeepSeek multi-head latent attention of the resident decode step, absorbed form, for one token.
//
// The reference runs this attention behind a query low-rank stage (hf_decode_sequence/deepseek/
// session_decode_v3_projection.inc.cu:1-624; kernels_v3_mla.inc.cu:1-61 cache row, :196-236 absorbed
// query, :465 attention tile, :890 value projection) with the whole layer's attention of a batch-1
// step in ONE thread block.  Here, after the fused [query; latent + rotary key] projection:
//   mla_prepare_kernel    blocks (head h, 64-wide slice): rotary part of query head h in place, and the
//                         slice of its absorbed query ql[h] = q_nope[h] . W_UK[h] (128 x 512 mat-vec);
//                         last block: cache row of the new token — bf16(RMSNorm(latent) * w) and
//                         bf16(rope(bf16(k_pe))), interleaved rotary pairs — appended to its page
//   mla_attention_kernel  grid = splits: the block's span of cached rows goes through shared memory
//                         once for ALL heads (the latent cache is shared between heads), one warp
//                         per head: s = (ql . c + q_pe . k_pe) * scale, online softmax, acc += p c
//   mla_output_kernel     blocks (head h, 8 output rows): merge of the spans, then out[h] = W_UV[h] . lat[h] -> bf16
// Cache rows are (rank + rope) bf16 values in the session's K pages, addressed through the page
// table like every other cache row (hf_decode_sequence/types.cuh:328-337).
#include <math.h>

#include "common.cuh"
#include "kernels.cuh"
#include "mma_bf16.cuh"

namespace nb {
namespace {

constexpr uint32_t kMlaMaxRank = 512, kMlaMaxRope = 64, kMlaMaxNope = 256;
constexpr uint32_t kMlaTile = 32;       // cached rows per shared-memory tile
constexpr uint32_t kMlaMaxSplits = 64;
constexpr float kLog2e = 1.4426950408889634f;

// Interleaved rotary pair (2i, 2i + 1) of a `dim`-wide vector at `position`:
// hf_decode_sequence/deepseek/kernels_helpers_math.inc.cu:236-262 without frequency scaling.
__device__ __forceinline__ void rope_pair(float &left, float &right, uint32_t pair, uint32_t dim, uint32_t position,
                                          float theta) {
  const float exponent = static_cast<float>(2u * pair) / static_cast<float>(dim);
  const float angle = static_cast<float>(position) * (1.0f / powf(theta, exponent));
  float s, c;
  sincosf(angle, &s, &c);
  const float l = left, r = right;
  left = l * c - r * s;
  right = r * c + l * s;
}

constexpr uint32_t kMlaPrepareSlice = 64;  // absorbed-query elements per block

// Grid: heads * (rank / 64) blocks for the absorbed queries, one more for the cache row.
__global__ void __launch_bounds__(256) mla_prepare_kernel(MlaParams p) {
  __shared__ float q_nope[kMlaMaxNope];
  __shared__ float part[4][kMlaPrepareSlice];
  __shared__ float scratch[40];
  pdl_trigger();
  pdl_wait();  // the fused projection of this step
  const uint32_t position = *p.cursor;
  if (position >= p.max_context) return;
  const uint32_t qdim = p.nope + p.rope, width = p.rank + p.rope;
  const uint32_t slices = p.rank / kMlaPrepareSlice;
  if (blockIdx.x < p.heads * slices) {
    const uint32_t h = blockIdx.x / slices, slice = blockIdx.x % slices;
    float *q = p.qkv + static_cast<uint64_t>(h) * qdim;
    for (uint32_t i = threadIdx.x; i < p.nope; i += blockDim.x) q_nope[i] = q[i];
    if (slice == 0 && p.rope_theta > 0.0f && threadIdx.x < p.rope / 2u) {
      // the head's rotary part, in place, by one of the head's blocks (the others read q_nope only)
      float l = q[p.nope + 2u * threadIdx.x], r = q[p.nope + 2u * threadIdx.x + 1u];
      rope_pair(l, r, threadIdx.x, p.rope, position, p.rope_theta);
      q[p.nope + 2u * threadIdx.x] = l;
      q[p.nope + 2u * threadIdx.x + 1u] = r;
    }
    __syncthreads();
    // ql[r] = sum_n q_nope[n] W_UK[h][n][r] for 64 consecutive r: thread (r, quarter) adds a quarter
    // of the n range (64 consecutive threads read one 128-byte piece of a W_UK row, all of a
    // thread's loads are independent), the quarters are added in order
    const uint16_t *w_uk = p.w_kv_b + static_cast<uint64_t>(h) * (p.nope + p.v_dim) * p.rank;
    const uint32_t r_local = threadIdx.x & (kMlaPrepareSlice - 1u), quarter = threadIdx.x / kMlaPrepareSlice;
    const uint32_t r = slice * kMlaPrepareSlice + r_local;
    const uint32_t per = (p.nope + 3u) / 4u;
    const uint32_t n_begin = quarter * per, n_end = n_begin + per < p.nope ? n_begin + per : p.nope;
    float acc = 0.0f;
#pragma unroll 8
    for (uint32_t n = n_begin; n < n_end; ++n)
      acc = fmaf(q_nope[n], bf16_bits_to_f32(w_uk[static_cast<uint64_t>(n) * p.rank + r]), acc);
    part[quarter][r_local] = acc;
    __syncthreads();
    if (quarter == 0)
      p.ql[static_cast<uint64_t>(h) * p.rank + r] = ((part[0][r_local] + part[1][r_local]) + part[2][r_local]) + part[3][r_local];
    return;
  }
  // the new token's cache row
  const float *kv = p.qkv + static_cast<uint64_t>(p.heads) * qdim;
  float sumsq = 0.0f;
  for (uint32_t i = threadIdx.x; i < p.rank; i += blockDim.x) sumsq += kv[i] * kv[i];
  const float total = block_sum(sumsq, scratch);
  const float scale = rsqrtf(total / static_cast<float>(p.rank) + p.eps);
  uint32_t page = p.page_table[position / NERVA_KV_CACHE_BLOCK_TOKENS];
  if (page >= p.page_count) {
    if (threadIdx.x == 0) report_error(p.error_word, kErrPageOutOfRange);
    return;
  }
  uint16_t *row = p.cache + (static_cast<uint64_t>(page) * NERVA_KV_CACHE_BLOCK_TOKENS +
                             position % NERVA_KV_CACHE_BLOCK_TOKENS) * width;
  for (uint32_t i = threadIdx.x; i < p.rank; i += blockDim.x)
    row[i] = f32_to_bf16_bits(kv[i] * scale * bf16_bits_to_f32(p.kv_a_norm[i]));
  if (threadIdx.x < p.rope / 2u) {
    float l = bf16_round(kv[p.rank + 2u * threadIdx.x]), r = bf16_round(kv[p.rank + 2u * threadIdx.x + 1u]);
    if (p.rope_theta > 0.0f) rope_pair(l, r, threadIdx.x, p.rope, position, p.rope_theta);
    row[p.rank + 2u * threadIdx.x] = f32_to_bf16_bits(l);
    row[p.rank + 2u * threadIdx.x + 1u] = f32_to_bf16_bits(r);
  }
}

// Split attention over the latent cache on the tensor pipe.  The heads are the M dimension of the
// MMA (at most 16 of them: one m16n8k16 tile), so a block of 16 warps handles all heads of its span
// of cached rows, one tile of 32 rows at a time:
//   scores   S[16 heads][32 rows] = Q . C^T over the rank + rope features: warp (n-tile of 8 rows,
//            quarter of the feature range); the four quarters are added in order through shared memory
//   softmax  warp h owns head h (one lane per row): running maximum and sum, p = exp2(s - m)
//   values   acc[16 heads][rank] += P . C: warp w owns rank / 16 consecutive features of all heads,
//            the C fragments come out of shared memory transposed (ldmatrix.trans)
// Q and P are fp32 values split into a bf16 rounding and what it lost (two MMAs each), the cache
// rows are bf16 as stored, accumulation is fp32.
// Shared memory: tile of kMlaTile cache rows | Q roundings | Q remainders (16 rows each, the tile's
// row stride: width * 2 + 16 bytes, which keeps fragment loads free of bank conflicts when
// width * 2 is a multiple of 128) | score quarters | P roundings, remainders | per-head rescale.
constexpr uint32_t kMlaHeadsTile = 16;   // MMA M
constexpr uint32_t kMlaPStride = kMlaTile + 8u;  // bf16 elements per row of P (80 bytes: conflict-free A loads)

__host__ __device__ inline uint32_t mla_row_bytes(uint32_t rank, uint32_t rope) { return (rank + rope) * 2u + 16u; }
__host__ __device__ inline uint32_t mla_attention_smem(uint32_t rank, uint32_t rope) {
  return (kMlaTile + 2u * kMlaHeadsTile) * mla_row_bytes(rank, rope) + 4u * kMlaHeadsTile * kMlaTile * 4u +
         2u * kMlaHeadsTile * kMlaPStride * 2u + kMlaHeadsTile * 4u;
}

template <uint32_t NT>  // n-tiles of 8 features per warp in the value product: rank / 128
__global__ void __launch_bounds__(512) mla_attention_kernel(MlaParams p) {
  constexpr uint32_t RANK = NT * 128u;
  extern __shared__ __align__(16) uint8_t smem[];
  pdl_trigger();
  pdl_wait();
  const uint32_t position = *p.cursor;
  if (position >= p.max_context) return;
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const uint32_t g = lane >> 2, t = lane & 3u;
  const uint32_t width = RANK + p.rope, row_bytes = mla_row_bytes(RANK, p.rope);
  const uint32_t k_steps = (width + 15u) / 16u;
  uint8_t *tile = smem;
  uint8_t *q_hi = tile + kMlaTile * row_bytes;
  uint8_t *q_lo = q_hi + kMlaHeadsTile * row_bytes;
  float *s_part = reinterpret_cast<float *>(q_lo + kMlaHeadsTile * row_bytes);  // [4][16][32]
  uint16_t *p_hi = reinterpret_cast<uint16_t *>(s_part + 4u * kMlaHeadsTile * kMlaTile);
  uint16_t *p_lo = p_hi + kMlaHeadsTile * kMlaPStride;
  float *rescale = reinterpret_cast<float *>(p_lo + kMlaHeadsTile * kMlaPStride);

  const uint32_t context = position + 1u;  // the new token's row was appended by the prepare kernel
  const uint32_t split = blockIdx.x, S = gridDim.x;
  const uint32_t tiles_total = (context + kMlaTile - 1u) / kMlaTile;
  const uint32_t tiles_per_split = (tiles_total + S - 1u) / S;
  const uint32_t tile_begin = split * tiles_per_split;
  uint32_t tile_end = tile_begin + tiles_per_split;
  if (tile_end > tiles_total) tile_end = tiles_total;

  // Q[h] = [absorbed query | rotary query] * scale * log2(e), rows of absent heads and the row
  // padding zero
  if (tile_begin < tile_end) {
    const float qscale = kLog2e * rsqrtf(static_cast<float>(p.nope + p.rope));
    const uint32_t padded = row_bytes / 2u, total = kMlaHeadsTile * padded;
    constexpr uint32_t kBatch = 8;  // loads in flight per thread
    for (uint32_t base = threadIdx.x; base < total; base += blockDim.x * kBatch) {
      float v[kBatch];
#pragma unroll
      for (uint32_t u = 0; u < kBatch; ++u) {
        const uint32_t i = base + u * blockDim.x;
        const uint32_t h = i / padded, k = i % padded;
        v[u] = 0.0f;
        if (i < total && h < p.heads && k < RANK) v[u] = __ldcg(p.ql + static_cast<uint64_t>(h) * RANK + k);
        else if (i < total && h < p.heads && k < width)
          v[u] = __ldcg(p.qkv + static_cast<uint64_t>(h) * (p.nope + p.rope) + p.nope + (k - RANK));
      }
#pragma unroll
      for (uint32_t u = 0; u < kBatch; ++u) {
        const uint32_t i = base + u * blockDim.x;
        if (i >= total) break;
        const uint32_t h = i / padded, k = i % padded;
        const float scaled = v[u] * qscale;
        const uint16_t hi = f32_to_bf16_bits(scaled);
        reinterpret_cast<uint16_t *>(q_hi + h * row_bytes)[k] = hi;
        reinterpret_cast<uint16_t *>(q_lo + h * row_bytes)[k] = f32_to_bf16_bits(scaled - bf16_bits_to_f32(hi));
      }
    }
  }
  // warp h keeps head h's running maximum and sum; every warp its features of all heads
  float m_run = -INFINITY, l_run = 0.0f;
  float acc[NT][4];
#pragma unroll
  for (uint32_t i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;

  for (uint32_t tl = tile_begin; tl < tile_end; ++tl) {
    const uint32_t token0 = tl * kMlaTile;
    const uint32_t valid = context - token0 < kMlaTile ? context - token0 : kMlaTile;
    __syncthreads();  // the previous tile has been consumed
    // the tile's rows in 16-byte pieces (a row is width * 2 bytes, a multiple of 16, then 16 bytes
    // of padding); rows beyond the context and the padding are zero
    const uint32_t pieces = row_bytes / 16u;
    constexpr uint32_t kBatch = 5;  // 32 rows of rank 512 + rope 64 are 4.6 pieces per thread
    for (uint32_t base = threadIdx.x; base < kMlaTile * pieces; base += blockDim.x * kBatch) {
      uint32_t page[kBatch];
      bool fetch[kBatch];
      uint4 v[kBatch];
#pragma unroll
      for (uint32_t u = 0; u < kBatch; ++u) {
        const uint32_t i = base + u * blockDim.x;
        const uint32_t r = i / pieces, piece = i % pieces;
        fetch[u] = i < kMlaTile * pieces && r < valid && piece < width / 8u;
        page[u] = fetch[u] ? p.page_table[(token0 + r) / NERVA_KV_CACHE_BLOCK_TOKENS] : 0u;
      }
#pragma unroll
      for (uint32_t u = 0; u < kBatch; ++u) {
        const uint32_t i = base + u * blockDim.x;
        const uint32_t r = i / pieces, piece = i % pieces;
        v[u] = make_uint4(0u, 0u, 0u, 0u);
        if (!fetch[u]) continue;
        if (page[u] >= p.page_count) {
          report_error(p.error_word, kErrPageOutOfRange);
          page[u] = 0;
        }
        const uint16_t *src = p.cache + (static_cast<uint64_t>(page[u]) * NERVA_KV_CACHE_BLOCK_TOKENS +
                                         (token0 + r) % NERVA_KV_CACHE_BLOCK_TOKENS) * width + piece * 8u;
        v[u] = __ldcg(reinterpret_cast<const uint4 *>(src));
      }
#pragma unroll
      for (uint32_t u = 0; u < kBatch; ++u) {
        const uint32_t i = base + u * blockDim.x;
        if (i >= kMlaTile * pieces) break;
        *reinterpret_cast<uint4 *>(tile + (i / pieces) * row_bytes + (i % pieces) * 16u) = v[u];
      }
    }
    __syncthreads();
    {
      // ---- scores: this warp's 8 rows, its quarter of the features ----
      const uint32_t nt = warp & 3u, quarter = warp >> 2;
      const uint32_t per = (k_steps + 3u) / 4u;
      const uint32_t ks_begin = quarter * per;
      const uint32_t ks_end = ks_begin + per < k_steps ? ks_begin + per : k_steps;
      float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      const uint8_t *b_row = tile + (nt * 8u + g) * row_bytes + 4u * t;
      const uint8_t *a_row = q_hi + g * row_bytes + 4u * t;
      const uint32_t lo_offset = kMlaHeadsTile * row_bytes;  // q_lo - q_hi
      for (uint32_t ks = ks_begin; ks < ks_end; ++ks) {
        const uint32_t at = ks * 32u;  // bytes into a row
        const uint32_t b0 = *reinterpret_cast<const uint32_t *>(b_row + at);
        const uint32_t b1 = *reinterpret_cast<const uint32_t *>(b_row + at + 16u);
        uint32_t a[4];
        a[0] = *reinterpret_cast<const uint32_t *>(a_row + at);
        a[1] = *reinterpret_cast<const uint32_t *>(a_row + 8u * row_bytes + at);
        a[2] = *reinterpret_cast<const uint32_t *>(a_row + at + 16u);
        a[3] = *reinterpret_cast<const uint32_t *>(a_row + 8u * row_bytes + at + 16u);
        mma_bf16(c, a, b0, b1);
        a[0] = *reinterpret_cast<const uint32_t *>(a_row + lo_offset + at);
        a[1] = *reinterpret_cast<const uint32_t *>(a_row + lo_offset + 8u * row_bytes + at);
        a[2] = *reinterpret_cast<const uint32_t *>(a_row + lo_offset + at + 16u);
        a[3] = *reinterpret_cast<const uint32_t *>(a_row + lo_offset + 8u * row_bytes + at + 16u);
        mma_bf16(c, a, b0, b1);
      }
      float *out = s_part + quarter * kMlaHeadsTile * kMlaTile + nt * 8u + 2u * t;
      *reinterpret_cast<float2 *>(out + g * kMlaTile) = make_float2(c[0], c[1]);
      *reinterpret_cast<float2 *>(out + (g + 8u) * kMlaTile) = make_float2(c[2], c[3]);
    }
    __syncthreads();
    {
      // ---- softmax: head = warp, row = lane ----
      const float *sp = s_part + warp * kMlaTile + lane;
      float s = ((sp[0] + sp[kMlaHeadsTile * kMlaTile]) + sp[2u * kMlaHeadsTile * kMlaTile]) +
                sp[3u * kMlaHeadsTile * kMlaTile];
      if (lane >= valid) s = -INFINITY;
      const float m_new = fmaxf(m_run, warp_max(s));
      const float corr = exp2f(m_run - m_new);  // first tile: exp2(-inf) = 0
      const float pr = exp2f(s - m_new);
      l_run = l_run * corr + warp_sum(pr);
      m_run = m_new;
      const uint16_t hi = f32_to_bf16_bits(pr);
      p_hi[warp * kMlaPStride + lane] = hi;
      p_lo[warp * kMlaPStride + lane] = f32_to_bf16_bits(pr - bf16_bits_to_f32(hi));
      if (lane == 0) rescale[warp] = corr;
    }
    __syncthreads();
    {
      // ---- values: acc = acc * corr + P . C for this warp's features ----
      const float corr_a = rescale[g], corr_b = rescale[g + 8u];
#pragma unroll
      for (uint32_t i = 0; i < NT; ++i) {
        acc[i][0] *= corr_a;
        acc[i][1] *= corr_a;
        acc[i][2] *= corr_b;
        acc[i][3] *= corr_b;
      }
#pragma unroll
      for (uint32_t ks = 0; ks < kMlaTile / 16u; ++ks) {
        uint32_t a_hi[4], a_lo[4];
        const uint32_t a0 = g * kMlaPStride + ks * 16u + 2u * t;
        a_hi[0] = *reinterpret_cast<const uint32_t *>(p_hi + a0);
        a_hi[1] = *reinterpret_cast<const uint32_t *>(p_hi + a0 + 8u * kMlaPStride);
        a_hi[2] = *reinterpret_cast<const uint32_t *>(p_hi + a0 + 8u);
        a_hi[3] = *reinterpret_cast<const uint32_t *>(p_hi + a0 + 8u * kMlaPStride + 8u);
        a_lo[0] = *reinterpret_cast<const uint32_t *>(p_lo + a0);
        a_lo[1] = *reinterpret_cast<const uint32_t *>(p_lo + a0 + 8u * kMlaPStride);
        a_lo[2] = *reinterpret_cast<const uint32_t *>(p_lo + a0 + 8u);
        a_lo[3] = *reinterpret_cast<const uint32_t *>(p_lo + a0 + 8u * kMlaPStride + 8u);
        // four 8 x 8 matrices per load: (rows 0..7 | 8..15 of the k-step) x (features of n-tile i | i + 1)
        const uint32_t row = ks * 16u + ((lane >> 3) & 1u) * 8u + (lane & 7u);
        if constexpr (NT >= 2) {
#pragma unroll
          for (uint32_t i = 0; i < NT; i += 2) {
            const uint32_t feature = (warp * NT + i + (lane >> 4)) * 8u;
            uint32_t b[4];
            ldmatrix_x4_trans(b, smem_addr(tile + row * row_bytes + feature * 2u));
            mma_bf16(acc[i], a_hi, b[0], b[1]);
            mma_bf16(acc[i], a_lo, b[0], b[1]);
            mma_bf16(acc[i + 1], a_hi, b[2], b[3]);
            mma_bf16(acc[i + 1], a_lo, b[2], b[3]);
          }
        } else {
          // one n-tile per warp: lanes 16..31 repeat the addresses of lanes 0..15
          const uint32_t feature = warp * 8u;
          uint32_t b[4];
          ldmatrix_x4_trans(b, smem_addr(tile + row * row_bytes + feature * 2u));
          mma_bf16(acc[0], a_hi, b[0], b[1]);
          mma_bf16(acc[0], a_lo, b[0], b[1]);
        }
      }
    }
  }
  // partial results of the span: accumulator rows g and g + 8 are heads, columns features
#pragma unroll
  for (uint32_t i = 0; i < NT; ++i) {
    const uint32_t feature = (warp * NT + i) * 8u + 2u * t;
    if (g < p.heads)
      *reinterpret_cast<float2 *>(p.partial_acc + (static_cast<uint64_t>(g) * S + split) * RANK + feature) =
          make_float2(acc[i][0], acc[i][1]);
    if (g + 8u < p.heads)
      *reinterpret_cast<float2 *>(p.partial_acc + (static_cast<uint64_t>(g + 8u) * S + split) * RANK + feature) =
          make_float2(acc[i][2], acc[i][3]);
  }
  if (warp < p.heads && lane == 0) {
    p.partial_m[static_cast<uint64_t>(warp) * S + split] = m_run;
    p.partial_l[static_cast<uint64_t>(warp) * S + split] = l_run;
  }
}

__global__ void __launch_bounds__(256) mla_output_kernel(MlaParams p, uint32_t slots) {
  __shared__ float lat[kMlaMaxRank];
  __shared__ float weight[kMlaMaxSplits];
  pdl_trigger();
  pdl_wait();
  const uint32_t position = *p.cursor;
  if (position >= p.max_context) return;
  const uint32_t h = blockIdx.x;
  uint32_t splits;  // spans that hold something; `slots` of them were launched and are the stride
  {
    // spans beyond the context's last tile hold nothing (the attention kernel's split arithmetic)
    const uint32_t tiles_total = (position + 1u + kMlaTile - 1u) / kMlaTile;
    const uint32_t tiles_per_split = (tiles_total + slots - 1u) / slots;
    splits = (tiles_total + tiles_per_split - 1u) / tiles_per_split;
    if (splits > slots) splits = slots;
  }
  if (threadIdx.x < 32u) {
    // one lane per span (two when there are more than 32): the (m, l) pairs become normalised weights
    const uint32_t lane = threadIdx.x;
    float m = -INFINITY;
    for (uint32_t s = lane; s < splits; s += 32u)
      if (__ldcg(p.partial_l + h * slots + s) > 0.0f) m = fmaxf(m, __ldcg(p.partial_m + h * slots + s));
    m = warp_max(m);
    float l = 0.0f;
    for (uint32_t s = lane; s < splits; s += 32u) {
      const float ls = __ldcg(p.partial_l + h * slots + s);
      const float w = ls > 0.0f ? exp2f(__ldcg(p.partial_m + h * slots + s) - m) : 0.0f;
      weight[s] = w;
      l = fmaf(ls, w, l);
    }
    l = warp_sum(l);
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    __syncwarp();
    for (uint32_t s = lane; s < splits; s += 32u) weight[s] *= inv;
  }
  __syncthreads();
  for (uint32_t r = threadIdx.x; r < p.rank; r += blockDim.x) {
    float a = 0.0f;
    uint32_t s = 0;
    for (; s + 8u <= splits; s += 8u) {
      float v[8];
#pragma unroll
      for (uint32_t u = 0; u < 8u; ++u) v[u] = __ldcg(p.partial_acc + (static_cast<uint64_t>(h) * slots + s + u) * p.rank + r);
#pragma unroll
      for (uint32_t u = 0; u < 8u; ++u) a = fmaf(v[u], weight[s + u], a);
    }
    for (; s < splits; ++s)
      a = fmaf(__ldcg(p.partial_acc + (static_cast<uint64_t>(h) * slots + s) * p.rank + r), weight[s], a);
    lat[r] = a;
  }
  __syncthreads();
  // out[v] = sum_r lat[r] W_UV[h][v][r]: one warp per output row, 16-byte loads along r; block
  // (h, y) takes rows y * warps .. of the head (the merge above is repeated by the head's blocks:
  // it reads a few KB that stay in L2, the value projection reads the weights)
  const uint16_t *w_uv = p.w_kv_b + (static_cast<uint64_t>(h) * (p.nope + p.v_dim) + p.nope) * p.rank;
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  for (uint32_t v = blockIdx.y * warps + warp; v < p.v_dim; v += gridDim.y * warps) {
    const uint4 *row = reinterpret_cast<const uint4 *>(w_uv + static_cast<uint64_t>(v) * p.rank);
    float acc = 0.0f;
    for (uint32_t i = lane; i < p.rank / 8u; i += 32u) {
      const uint4 w = row[i];
      const float *x = lat + 8u * i;
      acc = fmaf(bf16x2_lo(w.x), x[0], acc);
      acc = fmaf(bf16x2_hi(w.x), x[1], acc);
      acc = fmaf(bf16x2_lo(w.y), x[2], acc);
      acc = fmaf(bf16x2_hi(w.y), x[3], acc);
      acc = fmaf(bf16x2_lo(w.z), x[4], acc);
      acc = fmaf(bf16x2_hi(w.z), x[5], acc);
      acc = fmaf(bf16x2_lo(w.w), x[6], acc);
      acc = fmaf(bf16x2_hi(w.w), x[7], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) p.out_bf16[static_cast<uint64_t>(h) * p.v_dim + v] = f32_to_bf16_bits(acc);
  }
}

}  // namespace

cudaError_t configure_mla_kernels() {
  const int bytes = static_cast<int>(mla_attention_smem(kMlaMaxRank, kMlaMaxRope));
  cudaError_t err = cudaFuncSetAttribute(mla_attention_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(mla_attention_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(mla_attention_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  return err;
}

bool mla_session_supported(uint32_t heads, uint32_t rank, uint32_t nope, uint32_t rope, uint32_t v_dim) {
  return heads != 0 && heads <= 16u && (rank == 128u || rank == 256u || rank == 512u) && nope != 0 &&
         nope <= kMlaMaxNope && rope % 8u == 0 && rope <= kMlaMaxRope && rope != 0 && v_dim != 0;
}

uint32_t mla_attention_splits(uint32_t target_context) {
  const uint32_t tiles = (target_context + kMlaTile - 1u) / kMlaTile;
  uint32_t s = 1;
  while (s < tiles && s < kMlaMaxSplits) s <<= 1;
  return s;
}

cudaError_t launch_mla_attention(cudaStream_t stream, const MlaParams &p, uint32_t splits, bool pdl) {
  if (!mla_session_supported(p.heads, p.rank, p.nope, p.rope, p.v_dim) || splits == 0 || splits > kMlaMaxSplits)
    return cudaErrorInvalidValue;
  cudaError_t err = launch_with_pdl(mla_prepare_kernel, dim3(p.heads * (p.rank / kMlaPrepareSlice) + 1u), dim3(256), 0,
                                    stream, pdl, p);
  if (err != cudaSuccess) return err;
  const uint32_t smem = mla_attention_smem(p.rank, p.rope);
  const dim3 grid(splits), block(512);
  switch (p.rank / 128u) {
#define NERVA_MLA_CASE(N)                                                                            \
  case N:                                                                                            \
    err = launch_with_pdl(mla_attention_kernel<N>, grid, block, smem, stream, pdl, p);               \
    break;
    NERVA_MLA_CASE(1)
    NERVA_MLA_CASE(2)
    NERVA_MLA_CASE(4)
#undef NERVA_MLA_CASE
    default:
      return cudaErrorNotSupported;  // latent ranks 128, 256 and 512
  }
  if (err != cudaSuccess) return err;
  return launch_with_pdl(mla_output_kernel, dim3(p.heads, (p.v_dim + 7u) / 8u), dim3(256), 0, stream, pdl, p, splits);
}

}  // namespace nb
