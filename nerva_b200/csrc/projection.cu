// Decode projections: bf16 W[rows][cols] times one bf16 activation vector,
// fp32 accumulate.  Replaces the reference's cuBLAS/cuBLASLt calls
// (hf_decode_sequence/projection.cu:63-79,287-353; session_common.inc.cu:1243-1268)
// and folds the neighbouring element-wise kernels into the same launch:
//   prologue  residual add + RMSNorm -> bf16   (kernels.cu:182-217, 577-593, 651-687)
//   epilogue  SwiGLU -> bf16                    (kernels.cu:597-612)
//             per-block greedy arg-max partials (sampler.cu:89-119)
#include "kernels.cuh"
#include "step_device.cuh"
#include "weight_stream.cuh"

namespace nb {
namespace {

struct StoreEpilogue {
  float *out;
  __device__ __forceinline__ void row(uint32_t r, float v) {
    if ((threadIdx.x & 31u) == 0) out[r] = v;
  }
};

// Rows come as (gate_i, up_i) pairs; a warp always owns whole pairs.
struct SwigluEpilogue {
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

// Tie rule of the reference sampler: larger value, then lower index; non-finite
// logits never win (sampler.cu:35-40).
__device__ __forceinline__ bool candidate_better(float v, uint32_t i, float best_v,
                                                 uint32_t best_i) {
  return v > best_v || (v == best_v && i < best_i);
}

struct ArgmaxEpilogue {
  float *out;
  float best_v;
  uint32_t best_i;
  __device__ __forceinline__ void row(uint32_t r, float v) {
    if ((threadIdx.x & 31u) == 0) out[r] = v;
    if (isfinite(v) && candidate_better(v, r, best_v, best_i)) {
      best_v = v;
      best_i = r;
    }
  }
};

constexpr uint32_t kNoIndex = 0xffffffffu;

// Shared memory map of the streaming kernel (dynamic):
//   [0, kRingBytes)                     weight ring
//   [kRingBytes, +cols*2 rounded 16)    activation vector, bf16
//   then 24 mbarriers, 40 floats of reduction scratch, 8+8 arg-max words
__device__ __forceinline__ uint32_t round16(uint32_t v) { return (v + 15u) & ~15u; }

template <uint32_t EPI>
__global__ void __launch_bounds__(kStreamThreads, 1) projection_stream_kernel(ProjectionParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t *ring = smem;
  uint16_t *x = reinterpret_cast<uint16_t *>(smem + kRingBytes);
  uint8_t *tail = smem + kRingBytes + round16(p.cols * 2u);
  uint64_t *bars = reinterpret_cast<uint64_t *>(tail);
  float *scratch = reinterpret_cast<float *>(tail + kStreamWarps * kStreamSlots * 8u);
  float *warp_best_v = scratch + 40;
  uint32_t *warp_best_i = reinterpret_cast<uint32_t *>(scratch + 48);

  WarpStream ws;
  stream_init(ws, ring, bars);

  const bool pairs = EPI == kEpilogueSwiglu;
  const StreamShape shape = make_stream_shape(p.cols, pairs);
  uint32_t row_begin, row_end;
  block_row_range(p.rows, pairs ? 2u : 1u, blockIdx.x, gridDim.x, &row_begin, &row_end);
  const StreamJob job = make_stream_job(p.weight, shape, row_begin, row_end);
  uint32_t next = 0;
  // Weights do not depend on the activations: start streaming before the prologue.
  stream_fill(ws, job, &next);

  if (p.prologue == kProloguePlain) {
    const uint4 *src = reinterpret_cast<const uint4 *>(p.x_bf16);
    uint4 *dst = reinterpret_cast<uint4 *>(x);
    for (uint32_t i = threadIdx.x; i < p.cols / 8u; i += blockDim.x) dst[i] = src[i];
  } else {
    add_norm_to_smem(x, p.add_a, p.add_b, p.add_bias, p.norm_weight, p.eps, p.cols,
                     blockIdx.x == 0 ? p.resid_out : nullptr, scratch);
  }
  __syncthreads();

  if (EPI == kEpilogueStore) {
    StoreEpilogue epi{p.out_f32};
    stream_consume(ws, job, &next, x, epi, p.error_word);
  } else if (EPI == kEpilogueSwiglu) {
    SwigluEpilogue epi{p.out_bf16, 0.0f};
    stream_consume(ws, job, &next, x, epi, p.error_word);
  } else {
    ArgmaxEpilogue epi{p.out_f32, -INFINITY, kNoIndex};
    stream_consume(ws, job, &next, x, epi, p.error_word);
    const uint32_t warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31u) == 0) {
      warp_best_v[warp] = epi.best_v;
      warp_best_i[warp] = epi.best_i;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float bv = -INFINITY;
      uint32_t bi = kNoIndex;
      for (uint32_t w = 0; w < kStreamWarps; ++w) {
        if (warp_best_i[w] != kNoIndex && candidate_better(warp_best_v[w], warp_best_i[w], bv, bi)) {
          bv = warp_best_v[w];
          bi = warp_best_i[w];
        }
      }
      p.best_value[blockIdx.x] = bv;
      p.best_index[blockIdx.x] = bi;
    }
  }
  stream_drain(ws);
}

// Any-shape path (cols not a multiple of 8, or an unaligned matrix): one warp
// per row, scalar loads.  Correctness path for toy shapes only.
__global__ void projection_generic_prologue_kernel(ProjectionParams p, uint16_t *x_out) {
  __shared__ float scratch[40];
  float sumsq = 0.0f;
  for (uint32_t i = threadIdx.x; i < p.cols; i += blockDim.x) {
    float r = p.add_a[i];
    if (p.add_b != nullptr) r += p.add_b[i];
    if (p.add_bias != nullptr) r += bf16_bits_to_f32(p.add_bias[i]);
    sumsq += r * r;
  }
  const float total = block_sum(sumsq, scratch);
  const float scale = rsqrtf(total / static_cast<float>(p.cols) + p.eps);
  for (uint32_t i = threadIdx.x; i < p.cols; i += blockDim.x) {
    float r = p.add_a[i];
    if (p.add_b != nullptr) r += p.add_b[i];
    if (p.add_bias != nullptr) r += bf16_bits_to_f32(p.add_bias[i]);
    if (p.resid_out != nullptr) p.resid_out[i] = r;
    x_out[i] = f32_to_bf16_bits(r * scale * bf16_bits_to_f32(p.norm_weight[i]));
  }
}

__global__ void projection_generic_kernel(ProjectionParams p, const uint16_t *x) {
  // one block, warps stride over rows (pairs stay within one warp)
  __shared__ float warp_best_v[32];
  __shared__ uint32_t warp_best_i[32];
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t warps = blockDim.x >> 5;
  const uint32_t unit = p.epilogue == kEpilogueSwiglu ? 2u : 1u;
  float best_v = -INFINITY;
  uint32_t best_i = kNoIndex;
  for (uint32_t base = warp * unit; base < p.rows; base += warps * unit) {
    float gate = 0.0f;
    for (uint32_t u = 0; u < unit; ++u) {
      const uint32_t r = base + u;
      const uint16_t *w = p.weight + static_cast<uint64_t>(r) * p.cols;
      float acc = 0.0f;
      for (uint32_t k = lane; k < p.cols; k += 32u) {
        acc = fmaf(bf16_bits_to_f32(w[k]), bf16_bits_to_f32(x[k]), acc);
      }
      const float v = warp_sum(acc);
      if (p.epilogue == kEpilogueSwiglu) {
        if (u == 0) {
          gate = v;
        } else if (lane == 0) {
          p.out_bf16[r >> 1] = f32_to_bf16_bits(silu(gate) * v);
        }
      } else {
        if (lane == 0) p.out_f32[r] = v;
        if (p.epilogue == kEpilogueArgmax && isfinite(v) && candidate_better(v, r, best_v, best_i)) {
          best_v = v;
          best_i = r;
        }
      }
    }
  }
  if (p.epilogue == kEpilogueArgmax) {
    if (lane == 0) {
      warp_best_v[warp] = best_v;
      warp_best_i[warp] = best_i;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float bv = -INFINITY;
      uint32_t bi = kNoIndex;
      for (uint32_t w = 0; w < warps; ++w) {
        if (warp_best_i[w] != kNoIndex && candidate_better(warp_best_v[w], warp_best_i[w], bv, bi)) {
          bv = warp_best_v[w];
          bi = warp_best_i[w];
        }
      }
      p.best_value[0] = bv;
      p.best_index[0] = bi;
    }
  }
}

uint32_t stream_smem_bytes(uint32_t cols) {
  return kRingBytes + ((cols * 2u + 15u) & ~15u) + kStreamWarps * kStreamSlots * 8u + 64u * 4u;
}

bool stream_eligible(const ProjectionParams &p) {
  if (p.cols % 8u != 0 || p.cols == 0) return false;
  if (reinterpret_cast<uintptr_t>(p.weight) % 16u != 0) return false;
  if (p.prologue == kProloguePlain && reinterpret_cast<uintptr_t>(p.x_bf16) % 16u != 0) return false;
  if (p.epilogue == kEpilogueSwiglu && p.rows % 2u != 0) return false;
  return stream_smem_bytes(p.cols) <= 227u * 1024u;
}

}  // namespace

cudaError_t configure_projection_kernels() {
  const int max_smem = 227 * 1024;
  cudaError_t err = cudaFuncSetAttribute(projection_stream_kernel<kEpilogueStore>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(projection_stream_kernel<kEpilogueSwiglu>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(projection_stream_kernel<kEpilogueArgmax>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
  return err;
}

uint32_t projection_blocks(const ProjectionParams &p, uint32_t sm_count) {
  if (!stream_eligible(p)) return 1;
  // One block per SM; fewer when the matrix is too small to give every warp a
  // chunk (toy shapes).
  const StreamShape shape = make_stream_shape(p.cols, p.epilogue == kEpilogueSwiglu);
  const uint32_t items = (p.rows + shape.rows_per_item - 1) / shape.rows_per_item;
  uint32_t blocks = (items + kStreamWarps - 1) / kStreamWarps;
  if (blocks > sm_count) blocks = sm_count;
  if (blocks == 0) blocks = 1;
  return blocks;
}

cudaError_t launch_projection(cudaStream_t stream, const ProjectionParams &p, uint32_t sm_count) {
  if (stream_eligible(p)) {
    const uint32_t blocks = projection_blocks(p, sm_count);
    const uint32_t smem = stream_smem_bytes(p.cols);
    if (p.epilogue == kEpilogueStore) {
      projection_stream_kernel<kEpilogueStore><<<blocks, kStreamThreads, smem, stream>>>(p);
    } else if (p.epilogue == kEpilogueSwiglu) {
      projection_stream_kernel<kEpilogueSwiglu><<<blocks, kStreamThreads, smem, stream>>>(p);
    } else {
      projection_stream_kernel<kEpilogueArgmax><<<blocks, kStreamThreads, smem, stream>>>(p);
    }
    return cudaGetLastError();
  }
  // Toy-shape path.  With a fused prologue the caller passes `cols` writable
  // bf16 elements in x_bf16; the normalised vector goes through them.
  const uint16_t *x = p.x_bf16;
  if (p.prologue == kPrologueAddNorm) {
    projection_generic_prologue_kernel<<<1, 256, 0, stream>>>(p, const_cast<uint16_t *>(p.x_bf16));
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return err;
  }
  projection_generic_kernel<<<1, 256, 0, stream>>>(p, x);
  return cudaGetLastError();
}

}  // namespace nb
