// Decode projections: bf16 W[rows][cols] times one bf16 activation vector,
// fp32 accumulate.  Replaces the reference's cuBLAS/cuBLASLt calls
// (hf_decode_sequence/projection.cu:63-79,287-353; session_common.inc.cu:1243-1268)
// and folds the neighbouring element-wise kernels into the same launch:
//   prologue  residual add + RMSNorm -> bf16   (kernels.cu:182-217, 577-593, 651-687)
//   epilogue  SwiGLU -> bf16                    (kernels.cu:597-612)
//             per-block greedy arg-max partials (sampler.cu:89-119)
#include "kernels.cuh"
#include "row_stream.cuh"
#include "step_device.cuh"

namespace nb {
namespace {

constexpr uint32_t kNoIndex = 0xffffffffu;

// Tie rule of the reference sampler: larger value, then lower index; non-finite
// logits never win (sampler.cu:35-40).
__device__ __forceinline__ bool candidate_better(float v, uint32_t i, float best_v,
                                                 uint32_t best_i) {
  return v > best_v || (v == best_v && i < best_i);
}

struct ProjectionShared {
  StreamShared stream;
  JobDesc job;
  float scratch[40];
  float best_v[kStreamWarps];
  uint32_t best_i[kStreamWarps];
};

__host__ __device__ inline uint32_t round128(uint32_t v) { return (v + 127u) & ~127u; }

// Shared memory map (dynamic): weight ring | activation vector (bf16) |
// ProjectionShared | row totals (one float per row of the block).
// The gather of the tensor-parallel prologue, out of line: its register-resident
// batches must not shape the register allocation of the streaming loop.
__device__ __noinline__ void gather_prologue(const ProjectionParams &p, uint16_t *x, float *scratch) {
  const uint32_t tag = static_cast<uint32_t>(*p.gather.epoch) * p.gather.per_epoch + p.gather.offset;
  float *resid = blockIdx.x == 0 ? p.resid_out : nullptr;
  if (p.gather.world == 2 && p.gather.two_stage == 0) {
    // two partials: every block adds them itself (one round trip)
    gather_norm_to_smem<2>(x, p.add_a, p.gather.recv, tag, p.add_bias, p.norm_weight, p.eps, p.cols, resid,
                           scratch, p.error_word);
    return;
  }
  // four or eight partials: each block adds the ranks for its slice of the vector only, then every
  // block gathers the sums (reading all partials in every block costs more than the extra hop)
  if (p.gather.world == 2) {
    reduce_partials_slice<2>(p.gather.recv, p.gather.reduced, tag, p.cols, p.error_word);
  } else if (p.gather.world == 4) {
    reduce_partials_slice<4>(p.gather.recv, p.gather.reduced, tag, p.cols, p.error_word);
  } else {
    reduce_partials_slice<8>(p.gather.recv, p.gather.reduced, tag, p.cols, p.error_word);
  }
  gather_norm_to_smem<1>(x, p.add_a, p.gather.reduced, tag, p.add_bias, p.norm_weight, p.eps, p.cols, resid,
                         scratch, p.error_word);
}

// TP = true adds the tensor-parallel exchange (gather in the AddNorm prologue, push in the
// Store epilogue); the single-GPU instantiations carry none of that code.
// Ring slots a block fills before the dependency wait of a norm prologue; the rest follow the
// prologue's activation loads, which would otherwise queue behind a whole ring of bulk copies
// although they are on the critical path and the ring is not.  Holding back one slot of three
// measured best on the Qwen3-8B shapes (whole ring first: 2-3 % slower per token; two held back:
// about 1 % slower; holding a slot back ahead of the plain vector copy of O/down too: no gain).
// The tensor-parallel gather prologue polls its entries behind the same queue and gains the same
// way (its held-back slot is issued by the first stream_fill of stream_consume).
#ifndef NERVA_PREWAIT_SLOTS
#define NERVA_PREWAIT_SLOTS (NERVA_STREAM_SLOTS - 1)
#endif
constexpr uint32_t kPrewaitSlots = NERVA_PREWAIT_SLOTS;
constexpr uint32_t kPlainL2PrefetchBytes = 16384;  // per warp, after the plain vector copy

template <uint32_t EPI, bool TP>
__global__ void __launch_bounds__(kStreamThreads, 1) projection_stream_kernel(ProjectionParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t *ring = smem;
  uint16_t *x = reinterpret_cast<uint16_t *>(smem + kRingBytes);
  ProjectionShared &sh = *reinterpret_cast<ProjectionShared *>(smem + kRingBytes + round128(p.cols * 2u));
  float *row_total = reinterpret_cast<float *>(smem + kRingBytes + round128(p.cols * 2u) +
                                               round128(sizeof(ProjectionShared)));
  const uint32_t unit = EPI == kEpilogueSwiglu ? 2u : 1u;
  pdl_trigger();
  stamp(p.stamps, kStampEntry);
  if (threadIdx.x == 0) sh.job = JobDesc{p.weight, p.rows, p.cols, unit, 0};
  __syncthreads();

  // A residual stream that arrives already summed needs one vector after the wait; the norm
  // weights come in before it.
  const bool norm_single = p.prologue == kPrologueAddNorm && p.add_b == nullptr && p.add_bias == nullptr &&
                           p.resid_out == nullptr && !(TP && p.gather.world > 1) &&
                           norm_single_eligible(p.add_a, p.norm_weight, p.cols);
  RowStream rs;
  stream_init(rs, ring, sh.stream, &sh.job, 1);
  // Weights do not depend on the activations: start streaming before the prologue.  Ahead of a
  // norm prologue the last ring slot is held back until the activation loads have been issued:
  // they would otherwise queue behind a whole ring of bulk copies.
  const bool gathers = TP && p.prologue == kPrologueAddNorm && p.gather.world > 1 && p.add_b != nullptr;
  stream_fill(rs, norm_single || gathers ? kPrewaitSlots : kStreamSlots);

  uint32_t row_begin, row_end;
  block_row_range(p.rows, unit, blockIdx.x, gridDim.x, &row_begin, &row_end);
  const uint32_t rows_local = row_end - row_begin;
  for (uint32_t r = threadIdx.x; r < rows_local; r += blockDim.x) row_total[r] = 0.0f;
  NormWeightRegs norm_regs;
  if (norm_single) norm_weights_preload(norm_regs, p.norm_weight, p.cols);

  // Everything above is independent of the previous kernel; its output is read below.
  pdl_wait();
  stamp(p.stamps, kStampAfterWait);
  // kEpilogueStore with a fused residual add: this thread's row of the residual, fetched now so
  // that its latency hides behind the weight stream instead of sitting at the kernel's tail.
  float resid_first = 0.0f;
  if (EPI == kEpilogueStore && p.resid_in != nullptr && threadIdx.x < rows_local)
    resid_first = __ldcg(p.resid_in + row_begin + threadIdx.x);
  if (p.prologue == kProloguePlain) {
    const uint4 *src = reinterpret_cast<const uint4 *>(p.x_bf16);
    uint4 *dst = reinterpret_cast<uint4 *>(x);
    for (uint32_t i = threadIdx.x; i < p.cols / 8u; i += blockDim.x) dst[i] = src[i];
    // The ring is full and the block is about to synchronise: let HBM bring the next bytes of every
    // warp's span as far as L2 meanwhile (16 and 32 KiB per warp measured about 1 % faster per token,
    // 64 KiB slower than none; the same behind a norm prologue: no change).
    stream_prefetch_l2(rs, kPlainL2PrefetchBytes);
  } else {
    if (TP && p.gather.world > 1 && p.add_b != nullptr) {
      // the partial sums of the ranks arrive over NVLink while this polls
      gather_prologue(p, x, sh.scratch);
    } else if (norm_single) {
      NormValueRegs loaded;
      norm_single_load(loaded, p.add_a, p.cols);
      stream_fill(rs);  // the slot held back above, now behind the activation loads
      norm_single_finish(x, loaded, norm_regs, p.eps, p.cols, sh.scratch);
    } else {
      add_norm_to_smem(x, p.add_a, p.add_b, p.add_bias, p.norm_weight, p.eps, p.cols,
                       blockIdx.x == 0 ? p.resid_out : nullptr, sh.scratch);
    }
  }
  __syncthreads();
  stamp(p.stamps, kStampAfterPrologue);

  stream_consume(rs, sh.stream, 0, x, row_total, p.error_word);
  __syncthreads();

  // Epilogue over the block's rows, coalesced.
  if (EPI == kEpilogueStore) {
    if (TP && p.push.world > 1) {
      const unsigned long long tag =
          static_cast<unsigned long long>(static_cast<uint32_t>(*p.push.epoch) * p.push.per_epoch + p.push.offset) << 32;
      for (uint32_t r = threadIdx.x; r < rows_local; r += blockDim.x) {
        const float y = stream_row_total(sh.stream, row_total, r);
        const unsigned long long entry = tag | __float_as_uint(y);
        const uint64_t at = static_cast<uint64_t>(p.push.rank) * p.rows + row_begin + r;
        for (uint32_t q = 0; q < p.push.world; ++q) {
          asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p.push.recv[q] + at), "l"(entry) : "memory");
        }
      }
    } else {
      for (uint32_t r = threadIdx.x; r < rows_local; r += blockDim.x) {
        float y = stream_row_total(sh.stream, row_total, r);
        if (p.resid_in != nullptr) y += r == threadIdx.x ? resid_first : __ldcg(p.resid_in + row_begin + r);
        p.out_f32[row_begin + r] = y;
      }
    }
  } else if (EPI == kEpilogueSwiglu) {
    for (uint32_t i = threadIdx.x; i < rows_local / 2u; i += blockDim.x) {
      const float gate = stream_row_total(sh.stream, row_total, 2u * i);
      const float up = stream_row_total(sh.stream, row_total, 2u * i + 1u);
      p.out_bf16[row_begin / 2u + i] = f32_to_bf16_bits(silu(gate) * up);
    }
  } else {
    float bv = -INFINITY;
    uint32_t bi = kNoIndex;
    for (uint32_t r = threadIdx.x; r < rows_local; r += blockDim.x) {
      const float v = stream_row_total(sh.stream, row_total, r);
      p.out_f32[row_begin + r] = v;
      if (isfinite(v) && candidate_better(v, row_begin + r, bv, bi)) {
        bv = v;
        bi = row_begin + r;
      }
    }
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, offset);
      const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, offset);
      if (oi != kNoIndex && candidate_better(ov, oi, bv, bi)) {
        bv = ov;
        bi = oi;
      }
    }
    if ((threadIdx.x & 31u) == 0) {
      sh.best_v[threadIdx.x >> 5] = bv;
      sh.best_i[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      bv = -INFINITY;
      bi = kNoIndex;
      for (uint32_t w = 0; w < kStreamWarps; ++w) {
        if (sh.best_i[w] != kNoIndex && candidate_better(sh.best_v[w], sh.best_i[w], bv, bi)) {
          bv = sh.best_v[w];
          bi = sh.best_i[w];
        }
      }
      p.best_value[blockIdx.x] = bv;
      p.best_index[blockIdx.x] = bi;
    }
  }
  stream_drain(rs);
  stamp(p.stamps, kStampExit);
}

// Any-shape path (cols not a multiple of 8, or an unaligned matrix): one warp
// per row, scalar loads.  Correctness path for toy shapes only.
__global__ void projection_generic_prologue_kernel(ProjectionParams p, uint16_t *x_out) {
  __shared__ float scratch[40];
  float sumsq = 0.0f;
  for (uint32_t i = threadIdx.x; i < p.cols; i += blockDim.x) {
    float r = p.add_b != nullptr ? p.add_b[i] : p.add_a[i];
    if (p.add_bias != nullptr) r += bf16_bits_to_f32(p.add_bias[i]);
    if (p.add_b != nullptr) r += p.add_a[i];
    sumsq += r * r;
  }
  const float total = block_sum(sumsq, scratch);
  const float scale = rsqrtf(total / static_cast<float>(p.cols) + p.eps);
  for (uint32_t i = threadIdx.x; i < p.cols; i += blockDim.x) {
    float r = p.add_b != nullptr ? p.add_b[i] : p.add_a[i];
    if (p.add_bias != nullptr) r += bf16_bits_to_f32(p.add_bias[i]);
    if (p.add_b != nullptr) r += p.add_a[i];
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
  for (uint32_t base = warp * unit; base + unit <= p.rows; base += warps * unit) {
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
        if (lane == 0)
          p.out_f32[r] = p.epilogue == kEpilogueStore && p.resid_in != nullptr ? v + p.resid_in[r] : v;
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

uint32_t blocks_for(const ProjectionParams &p, uint32_t sm_count) {
  // One block per SM; fewer when the matrix is too small to give every warp of
  // every block 4 KiB (toy shapes).
  const uint64_t bytes = static_cast<uint64_t>(p.rows) * p.cols * 2u;
  uint64_t blocks = bytes / (static_cast<uint64_t>(kStreamWarps) * 4096u);
  const uint32_t unit = p.epilogue == kEpilogueSwiglu ? 2u : 1u;
  if (blocks > p.rows / unit) blocks = p.rows / unit;
  if (blocks > sm_count) blocks = sm_count;
  if (blocks == 0) blocks = 1;
  return static_cast<uint32_t>(blocks);
}

uint32_t stream_smem_bytes(const ProjectionParams &p, uint32_t blocks) {
  const uint32_t unit = p.epilogue == kEpilogueSwiglu ? 2u : 1u;
  return kRingBytes + round128(p.cols * 2u) + round128(sizeof(ProjectionShared)) +
         round128(max_rows_per_block(p.rows, unit, blocks) * 4u + 16u);
}

bool stream_eligible(const ProjectionParams &p, uint32_t sm_count) {
  if (p.cols % 8u != 0 || p.cols == 0 || p.rows == 0) return false;
  if (reinterpret_cast<uintptr_t>(p.weight) % 16u != 0) return false;
  if (p.prologue == kProloguePlain && reinterpret_cast<uintptr_t>(p.x_bf16) % 16u != 0) return false;
  if (p.epilogue == kEpilogueSwiglu && p.rows % 2u != 0) return false;
  return stream_smem_bytes(p, blocks_for(p, sm_count)) <= 227u * 1024u;
}

}  // namespace

cudaError_t configure_projection_kernels() {
  const int max_smem = 227 * 1024;
  cudaError_t err = cudaSuccess;
  auto set = [&](void (*kernel)(ProjectionParams)) {
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
  };
  set(projection_stream_kernel<kEpilogueStore, false>);
  set(projection_stream_kernel<kEpilogueSwiglu, false>);
  set(projection_stream_kernel<kEpilogueArgmax, false>);
  set(projection_stream_kernel<kEpilogueStore, true>);
  set(projection_stream_kernel<kEpilogueSwiglu, true>);
  set(projection_stream_kernel<kEpilogueArgmax, true>);
  return err;
}

uint32_t projection_blocks(const ProjectionParams &p, uint32_t sm_count) {
  return stream_eligible(p, sm_count) ? blocks_for(p, sm_count) : 1u;
}

cudaError_t launch_projection(cudaStream_t stream, const ProjectionParams &p, uint32_t sm_count) {
  if (p.gather.world > 1 && (p.cols % 4u != 0 || p.cols / 4u > kNormRegIters * kStreamThreads ||
                             (p.gather.world != 2 && p.gather.world != 4 && p.gather.world != 8)))
    return cudaErrorNotSupported;
  if (stream_eligible(p, sm_count)) {
    const uint32_t blocks = blocks_for(p, sm_count);
    const uint32_t smem = stream_smem_bytes(p, blocks);
    const bool pdl = p.pdl != 0;
    const bool tp = p.push.world > 1 || p.gather.world > 1;
    void (*kernel)(ProjectionParams) = nullptr;
    if (p.epilogue == kEpilogueStore) {
      kernel = tp ? projection_stream_kernel<kEpilogueStore, true> : projection_stream_kernel<kEpilogueStore, false>;
    } else if (p.epilogue == kEpilogueSwiglu) {
      kernel = tp ? projection_stream_kernel<kEpilogueSwiglu, true> : projection_stream_kernel<kEpilogueSwiglu, false>;
    } else {
      kernel = tp ? projection_stream_kernel<kEpilogueArgmax, true> : projection_stream_kernel<kEpilogueArgmax, false>;
    }
    return launch_with_pdl(kernel, dim3(blocks), dim3(kStreamThreads), smem, stream, pdl, p);
  }
  if (p.push.world > 1 || p.gather.world > 1) return cudaErrorNotSupported;  // exchange: streaming path only
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
