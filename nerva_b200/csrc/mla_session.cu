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

// Shared memory: one tile of kMlaTile cache rows, bf16, rows padded by 16 bytes.
template <uint32_t RANK_PER_LANE>
__global__ void __launch_bounds__(512) mla_attention_kernel(MlaParams p) {
  constexpr uint32_t RANK = RANK_PER_LANE * 32u;
  extern __shared__ __align__(16) uint8_t tile[];
  pdl_trigger();
  pdl_wait();
  const uint32_t position = *p.cursor;
  if (position >= p.max_context) return;
  const uint32_t lane = threadIdx.x & 31u, h = threadIdx.x >> 5;  // one warp per head
  const uint32_t width = RANK + p.rope, row_bytes = width * 2u + 16u;
  const uint32_t context = position + 1u;  // the new token's row was appended by the prepare kernel
  const uint32_t split = blockIdx.x, S = gridDim.x;
  const uint32_t tiles_total = (context + kMlaTile - 1u) / kMlaTile;
  const uint32_t tiles_per_split = (tiles_total + S - 1u) / S;
  const uint32_t tile_begin = split * tiles_per_split;
  uint32_t tile_end = tile_begin + tiles_per_split;
  if (tile_end > tiles_total) tile_end = tiles_total;

  // this head's absorbed query and rotary query, pre-multiplied by scale * log2(e)
  const float qscale = kLog2e * rsqrtf(static_cast<float>(p.nope + p.rope));
  float ql[RANK_PER_LANE], qr[2] = {0.0f, 0.0f};
  if (h < p.heads) {
#pragma unroll
    for (uint32_t j = 0; j < RANK_PER_LANE; ++j) ql[j] = __ldcg(p.ql + static_cast<uint64_t>(h) * RANK + lane + 32u * j) * qscale;
    const float *q_pe = p.qkv + static_cast<uint64_t>(h) * (p.nope + p.rope) + p.nope;
    if (lane < p.rope) qr[0] = __ldcg(q_pe + lane) * qscale;
    if (lane + 32u < p.rope) qr[1] = __ldcg(q_pe + lane + 32u) * qscale;
  }
  float m_run = -INFINITY, l_run = 0.0f, acc[RANK_PER_LANE];
#pragma unroll
  for (uint32_t j = 0; j < RANK_PER_LANE; ++j) acc[j] = 0.0f;

  for (uint32_t t = tile_begin; t < tile_end; ++t) {
    const uint32_t token0 = t * kMlaTile;
    const uint32_t valid = context - token0 < kMlaTile ? context - token0 : kMlaTile;
    __syncthreads();  // the previous tile has been consumed
    // copy the tile's rows (16-byte pieces; a row is `width * 2` bytes, a multiple of 16)
    const uint32_t pieces = width / 8u;
    for (uint32_t i = threadIdx.x; i < valid * pieces; i += blockDim.x) {
      const uint32_t r = i / pieces, piece = i % pieces;
      const uint32_t token = token0 + r;
      uint32_t page = p.page_table[token / NERVA_KV_CACHE_BLOCK_TOKENS];
      if (page >= p.page_count) {
        report_error(p.error_word, kErrPageOutOfRange);
        page = 0;
      }
      const uint16_t *src = p.cache + (static_cast<uint64_t>(page) * NERVA_KV_CACHE_BLOCK_TOKENS +
                                       token % NERVA_KV_CACHE_BLOCK_TOKENS) * width + piece * 8u;
      *reinterpret_cast<uint4 *>(tile + r * row_bytes + piece * 16u) = __ldcg(reinterpret_cast<const uint4 *>(src));
    }
    __syncthreads();
    if (h >= p.heads) continue;
    for (uint32_t r = 0; r < valid; ++r) {
      const uint16_t *c = reinterpret_cast<const uint16_t *>(tile + r * row_bytes);
      float dot = 0.0f;
#pragma unroll
      for (uint32_t j = 0; j < RANK_PER_LANE; ++j) dot = fmaf(ql[j], bf16_bits_to_f32(c[lane + 32u * j]), dot);
      if (lane < p.rope) dot = fmaf(qr[0], bf16_bits_to_f32(c[RANK + lane]), dot);
      if (lane + 32u < p.rope) dot = fmaf(qr[1], bf16_bits_to_f32(c[RANK + lane + 32u]), dot);
      const float s = warp_sum(dot);
      const float m_new = fmaxf(m_run, s);
      const float corr = exp2f(m_run - m_new);  // first row: exp2(-inf) = 0
      const float pr = exp2f(s - m_new);
      l_run = l_run * corr + pr;
      m_run = m_new;
#pragma unroll
      for (uint32_t j = 0; j < RANK_PER_LANE; ++j) acc[j] = fmaf(pr, bf16_bits_to_f32(c[lane + 32u * j]), acc[j] * corr);
    }
  }
  if (h < p.heads) {
    const uint64_t slot = static_cast<uint64_t>(h) * S + split;
#pragma unroll
    for (uint32_t j = 0; j < RANK_PER_LANE; ++j) p.partial_acc[slot * RANK + lane + 32u * j] = acc[j];
    if (lane == 0) {
      p.partial_m[slot] = m_run;
      p.partial_l[slot] = l_run;
    }
  }
}

__global__ void __launch_bounds__(256) mla_output_kernel(MlaParams p, uint32_t splits) {
  __shared__ float lat[kMlaMaxRank];
  __shared__ float weight[kMlaMaxSplits];
  pdl_trigger();
  pdl_wait();
  const uint32_t position = *p.cursor;
  if (position >= p.max_context) return;
  const uint32_t h = blockIdx.x;
  if (threadIdx.x < 32u) {
    // one lane per span (two when there are more than 32): the (m, l) pairs become normalised weights
    const uint32_t lane = threadIdx.x;
    float m = -INFINITY;
    for (uint32_t s = lane; s < splits; s += 32u)
      if (__ldcg(p.partial_l + h * splits + s) > 0.0f) m = fmaxf(m, __ldcg(p.partial_m + h * splits + s));
    m = warp_max(m);
    float l = 0.0f;
    for (uint32_t s = lane; s < splits; s += 32u) {
      const float ls = __ldcg(p.partial_l + h * splits + s);
      const float w = ls > 0.0f ? exp2f(__ldcg(p.partial_m + h * splits + s) - m) : 0.0f;
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
      for (uint32_t u = 0; u < 8u; ++u) v[u] = __ldcg(p.partial_acc + (static_cast<uint64_t>(h) * splits + s + u) * p.rank + r);
#pragma unroll
      for (uint32_t u = 0; u < 8u; ++u) a = fmaf(v[u], weight[s + u], a);
    }
    for (; s < splits; ++s)
      a = fmaf(__ldcg(p.partial_acc + (static_cast<uint64_t>(h) * splits + s) * p.rank + r), weight[s], a);
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
  const uint32_t smem = kMlaTile * ((p.rank + p.rope) * 2u + 16u);
  const dim3 grid(splits), block(512);
  switch (p.rank / 32u) {
#define NERVA_MLA_CASE(N)                                                                            \
  case N:                                                                                            \
    err = launch_with_pdl(mla_attention_kernel<N>, grid, block, smem, stream, pdl, p);               \
    break;
    NERVA_MLA_CASE(4)
    NERVA_MLA_CASE(8)
    NERVA_MLA_CASE(16)
#undef NERVA_MLA_CASE
    default:
      return cudaErrorNotSupported;  // latent ranks 128, 256 and 512
  }
  if (err != cudaSuccess) return err;
  return launch_with_pdl(mla_output_kernel, dim3(p.heads, (p.v_dim + 7u) / 8u), dim3(256), 0, stream, pdl, p, splits);
}

}  // namespace nb
