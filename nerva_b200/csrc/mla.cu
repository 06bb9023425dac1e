// DeepSeek multi-head latent attention decode for one token, as a per-operator entry
// point.  Replaces the reference's nerva_cuda_deepseek_mla_decode
// (native/cuda/deepseek/nerva_cuda_deepseek_mla.cu:144-227, 660-860), whose kernel runs
// every head and token in one thread.  Same "absorbed" algebra:
//   ql[h][l]  = sum_n q_nope[h][n] * w_uk[(l*heads + h)*nope + n]
//   score[t]  = (ql[h] . kv_c[t] + q_pe[h] . k_pe[t]) * softmax_scale
//   latent[h] = softmax(score) over the kv_c rows;  out[h][v] = sum_l latent[h][l] * w_uv[(l*heads + h)*v_dim + v]
// Three launches:
//   mla_q_latent_kernel   one warp per (head, latent): the absorbed query
//   mla_attend_kernel     grid = spans of the context; a block stages 16-token tiles of the
//                         latent cache (the cache is shared by all heads: it is read once per
//                         block, not once per head), one warp per head keeps its ql and its
//                         latent accumulator in registers (rank <= 1024: 32 values per lane)
//                         and runs the online softmax; partial (acc, m, l) per (head, span)
//   mla_output_kernel     merges the spans and applies w_uv
// All fp32, as the reference interface is.
#include <math.h>
#include <string.h>

#include "common.cuh"
#include "kernels.cuh"
#include "session.h"

using namespace nb;

namespace {

constexpr uint32_t kMaxRank = 1024;       // the reference's kMaxDynamicKvLoraRank
constexpr uint32_t kPerLane = kMaxRank / 32;
constexpr uint32_t kTileTokens = 16;
constexpr uint32_t kMaxHeadsPerBlock = 8;  // 256 threads: the two 32-value register arrays per lane need room
constexpr uint32_t kMaxSpans = 64;

struct MlaArgs {
  const float *q_nope, *q_pe, *kv_c, *k_pe, *w_uk, *w_uv;
  float *ql;         // [heads][rank]
  float *part_acc;   // [heads][spans][rank]
  float *part_m;     // [heads][spans]
  float *part_l;
  float *output;     // [heads][v]
  uint32_t heads, tokens, rank, nope, rope, v, spans;
  float scale;
  int32_t *decode_error;
};

__global__ void mla_q_latent_kernel(MlaArgs a) {
  const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31u;
  if (warp >= a.heads * a.rank) return;
  const uint32_t head = warp / a.rank, latent = warp - head * a.rank;
  const float *q = a.q_nope + head * a.nope;
  const float *w = a.w_uk + (static_cast<uint64_t>(latent) * a.heads + head) * a.nope;
  float sum = 0.0f;
  for (uint32_t n = lane; n < a.nope; n += 32u) sum = fmaf(q[n], w[n], sum);
  sum = warp_sum(sum);
  if (lane == 0) a.ql[head * a.rank + latent] = sum;
}

// grid (spans, head groups); block = heads_in_group warps.  Shared: kv tile [16][rank] + k_pe tile [16][rope].
__global__ void __launch_bounds__(kMaxHeadsPerBlock * 32) mla_attend_kernel(MlaArgs a) {
  extern __shared__ __align__(16) float tile[];
  float *kv_tile = tile;
  float *pe_tile = tile + kTileTokens * a.rank;
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const uint32_t head = blockIdx.y * kMaxHeadsPerBlock + warp;
  const bool active = head < a.heads;
  const uint32_t span = blockIdx.x;
  const uint32_t per_span = (a.tokens + a.spans - 1u) / a.spans;
  const uint32_t begin = span * per_span;
  uint32_t end = begin + per_span;
  if (end > a.tokens) end = a.tokens;

  float ql[kPerLane], acc[kPerLane];
#pragma unroll
  for (uint32_t i = 0; i < kPerLane; ++i) {
    const uint32_t l = lane + 32u * i;
    ql[i] = active && l < a.rank ? a.ql[head * a.rank + l] : 0.0f;
    acc[i] = 0.0f;
  }
  float m = -INFINITY, denom = 0.0f;
  for (uint32_t first = begin; first < end; first += kTileTokens) {
    const uint32_t count = end - first < kTileTokens ? end - first : kTileTokens;
    __syncthreads();  // the previous tile has been consumed
    for (uint32_t i = threadIdx.x; i < count * a.rank; i += blockDim.x) kv_tile[i] = a.kv_c[static_cast<uint64_t>(first) * a.rank + i];
    for (uint32_t i = threadIdx.x; i < count * a.rope; i += blockDim.x) pe_tile[i] = a.k_pe[static_cast<uint64_t>(first) * a.rope + i];
    __syncthreads();
    if (!active) continue;
    for (uint32_t t = 0; t < count; ++t) {
      const float *kv = kv_tile + t * a.rank;
      float dot = 0.0f;
#pragma unroll
      for (uint32_t i = 0; i < kPerLane; ++i) {
        const uint32_t l = lane + 32u * i;
        if (l < a.rank) dot = fmaf(ql[i], kv[l], dot);
      }
      for (uint32_t r = lane; r < a.rope; r += 32u) dot = fmaf(a.q_pe[head * a.rope + r], pe_tile[t * a.rope + r], dot);
      const float score = warp_sum(dot) * a.scale;
      const float next = fmaxf(m, score);
      const float keep = denom == 0.0f ? 0.0f : expf(m - next);
      const float add = expf(score - next);
#pragma unroll
      for (uint32_t i = 0; i < kPerLane; ++i) {
        const uint32_t l = lane + 32u * i;
        if (l < a.rank) acc[i] = acc[i] * keep + kv[l] * add;
      }
      denom = denom * keep + add;
      m = next;
    }
  }
  if (!active) return;
  const uint64_t slot = static_cast<uint64_t>(head) * a.spans + span;
#pragma unroll
  for (uint32_t i = 0; i < kPerLane; ++i) {
    const uint32_t l = lane + 32u * i;
    if (l < a.rank) a.part_acc[slot * a.rank + l] = acc[i];
  }
  if (lane == 0) {
    a.part_m[slot] = m;
    a.part_l[slot] = denom;
  }
}

// One block per head: merge the spans, divide, apply w_uv.
__global__ void mla_output_kernel(MlaArgs a) {
  extern __shared__ __align__(16) float latent[];  // [rank]
  __shared__ float weight[kMaxSpans];
  __shared__ float total_sh;
  const uint32_t head = blockIdx.x;
  if (threadIdx.x == 0) {
    float m = -INFINITY;
    for (uint32_t s = 0; s < a.spans; ++s)
      if (a.part_l[head * a.spans + s] > 0.0f) m = fmaxf(m, a.part_m[head * a.spans + s]);
    float total = 0.0f;
    for (uint32_t s = 0; s < a.spans; ++s) {
      const float l = a.part_l[head * a.spans + s];
      weight[s] = l > 0.0f ? expf(a.part_m[head * a.spans + s] - m) : 0.0f;
      total += l * weight[s];
    }
    total_sh = total;
    if (total == 0.0f) *a.decode_error = -2;
  }
  __syncthreads();
  const float total = total_sh;
  if (total == 0.0f) return;
  for (uint32_t l = threadIdx.x; l < a.rank; l += blockDim.x) {
    float sum = 0.0f;
    for (uint32_t s = 0; s < a.spans; ++s)
      sum = fmaf(a.part_acc[(static_cast<uint64_t>(head) * a.spans + s) * a.rank + l], weight[s], sum);
    latent[l] = sum / total;
  }
  __syncthreads();
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  for (uint32_t v = warp; v < a.v; v += warps) {
    float sum = 0.0f;
    for (uint32_t l = lane; l < a.rank; l += 32u)
      sum = fmaf(latent[l], a.w_uv[(static_cast<uint64_t>(l) * a.heads + head) * a.v + v], sum);
    sum = warp_sum(sum);
    if (lane == 0) a.output[head * a.v + v] = sum;
  }
}

uint64_t hash_f32(const float *values, uint32_t n) {  // nerva_cuda_deepseek_mla.cu:333-343
  uint64_t hash = 1469598103934665603ull;
  for (uint32_t i = 0; i < n; ++i) {
    uint32_t bits;
    memcpy(&bits, &values[i], 4);
    for (uint32_t byte = 0; byte < 4; ++byte) {
      hash ^= (bits >> (byte * 8)) & 0xffu;
      hash *= 1099511628211ull;
    }
  }
  return hash;
}

struct Scratch {
  void *ptr = nullptr;
  ~Scratch() {
    if (ptr != nullptr) cudaFree(ptr);
  }
};

}  // namespace

extern "C" int nerva_cuda_deepseek_mla_decode(const NervaCudaDeepSeekMlaDecodeRequest *request,
                                              NervaCudaDeepSeekMlaDecodeResult *out) {
  if (out == nullptr) return -1;
  memset(out, 0, sizeof(*out));
  out->status = -1;
  out->decode_error = -1;
  if (request != nullptr) {
    out->heads = request->heads;
    out->tokens = request->tokens;
    out->kv_lora_rank = request->kv_lora_rank;
    out->qk_nope_head_dim = request->qk_nope_head_dim;
    out->qk_rope_head_dim = request->qk_rope_head_dim;
    out->v_head_dim = request->v_head_dim;
    out->softmax_scale = request->softmax_scale;
  }
  // nerva_cuda_deepseek_mla.cu:421-430
  if (request == nullptr || request->q_nope == nullptr || request->q_pe == nullptr || request->kv_c == nullptr ||
      request->k_pe == nullptr || request->w_uk == nullptr || request->w_uv == nullptr ||
      request->output == nullptr || request->heads == 0 || request->tokens == 0 || request->kv_lora_rank == 0 ||
      request->kv_lora_rank > kMaxRank || request->qk_nope_head_dim == 0 || request->v_head_dim == 0)
    return -1;
  cudaError_t err = cudaGetDeviceCount(&out->device_count);
  if (err != cudaSuccess || out->device_count <= 0) {
    out->cuda_error = static_cast<int32_t>(err != cudaSuccess ? err : cudaErrorNoDevice);
    cudaGetLastError();
    return -1;
  }
  const uint64_t heads = request->heads, tokens = request->tokens, rank = request->kv_lora_rank;
  const uint64_t nope = request->qk_nope_head_dim, rope = request->qk_rope_head_dim, v = request->v_head_dim;
  uint32_t spans = static_cast<uint32_t>((tokens + 4u * kTileTokens - 1u) / (4u * kTileTokens));
  if (spans > kMaxSpans) spans = kMaxSpans;
  const uint64_t sizes[] = {heads * nope, heads * (rope == 0 ? 1 : rope), tokens * rank, tokens * (rope == 0 ? 1 : rope),
                            rank * heads * nope, rank * heads * v,          // inputs
                            heads * rank, heads * spans * rank, heads * spans, heads * spans, heads * v, 64};
  uint64_t offsets[12], total = 0;
  for (int i = 0; i < 12; ++i) {
    offsets[i] = total;
    total += (sizes[i] * 4u + 255u) & ~uint64_t{255};
  }
  Scratch scratch;
  err = cudaMalloc(&scratch.ptr, total);
  uint8_t *base = static_cast<uint8_t *>(scratch.ptr);
  const void *inputs[] = {request->q_nope, request->q_pe, request->kv_c, request->k_pe, request->w_uk, request->w_uv};
  const uint64_t input_elems[] = {heads * nope, heads * rope, tokens * rank, tokens * rope, rank * heads * nope,
                                  rank * heads * v};
  for (int i = 0; err == cudaSuccess && i < 6; ++i) {
    if (input_elems[i] != 0) err = cudaMemcpy(base + offsets[i], inputs[i], input_elems[i] * 4u, cudaMemcpyHostToDevice);
    out->h2d_bytes += input_elems[i] * 4u;
  }
  if (err == cudaSuccess) err = cudaMemset(base + offsets[11], 0, 4);
  if (err == cudaSuccess) {
    MlaArgs a{};
    a.q_nope = reinterpret_cast<const float *>(base + offsets[0]);
    a.q_pe = reinterpret_cast<const float *>(base + offsets[1]);
    a.kv_c = reinterpret_cast<const float *>(base + offsets[2]);
    a.k_pe = reinterpret_cast<const float *>(base + offsets[3]);
    a.w_uk = reinterpret_cast<const float *>(base + offsets[4]);
    a.w_uv = reinterpret_cast<const float *>(base + offsets[5]);
    a.ql = reinterpret_cast<float *>(base + offsets[6]);
    a.part_acc = reinterpret_cast<float *>(base + offsets[7]);
    a.part_m = reinterpret_cast<float *>(base + offsets[8]);
    a.part_l = reinterpret_cast<float *>(base + offsets[9]);
    a.output = reinterpret_cast<float *>(base + offsets[10]);
    a.decode_error = reinterpret_cast<int32_t *>(base + offsets[11]);
    a.heads = request->heads;
    a.tokens = request->tokens;
    a.rank = request->kv_lora_rank;
    a.nope = request->qk_nope_head_dim;
    a.rope = request->qk_rope_head_dim;
    a.v = request->v_head_dim;
    a.spans = spans;
    a.scale = request->softmax_scale;
    const uint32_t q_warps = request->heads * request->kv_lora_rank;
    mla_q_latent_kernel<<<(q_warps + 7u) / 8u, 256>>>(a);
    const uint32_t groups = (request->heads + kMaxHeadsPerBlock - 1u) / kMaxHeadsPerBlock;
    const uint32_t block_heads = request->heads < kMaxHeadsPerBlock ? request->heads : kMaxHeadsPerBlock;
    const size_t attend_smem = static_cast<size_t>(kTileTokens) * (rank + rope) * 4u;
    err = cudaFuncSetAttribute(mla_attend_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(kTileTokens * (kMaxRank + 1024u) * 4u));
    if (err == cudaSuccess && attend_smem > kTileTokens * (kMaxRank + 1024u) * 4u) err = cudaErrorNotSupported;
    if (err == cudaSuccess) {
      mla_attend_kernel<<<dim3(spans, groups), block_heads * 32u, attend_smem>>>(a);
      mla_output_kernel<<<request->heads, 256, rank * 4u>>>(a);
      err = cudaGetLastError();
      out->kernel_launches = 3;
    }
  }
  if (err == cudaSuccess) err = cudaDeviceSynchronize();
  out->sync_calls = 1;
  int32_t decode_error = -1;
  if (err == cudaSuccess) err = cudaMemcpy(&decode_error, base + offsets[11], 4, cudaMemcpyDeviceToHost);
  if (err == cudaSuccess) err = cudaMemcpy(request->output, base + offsets[10], heads * v * 4u, cudaMemcpyDeviceToHost);
  out->device_arena_bytes = total;
  out->d2h_bytes = heads * v * 4u + 4u;
  out->decode_error = decode_error;
  if (err != cudaSuccess) {
    out->cuda_error = static_cast<int32_t>(err);
    set_last_error(cudaGetErrorString(err));
    return -1;
  }
  if (decode_error != 0) return -1;
  out->output_hash = hash_f32(request->output, static_cast<uint32_t>(heads * v));
  out->status = 0;
  return 0;
}
