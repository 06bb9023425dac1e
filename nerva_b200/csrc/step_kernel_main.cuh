// Second half of step_kernel.cu: the kernel body and its launcher.
#pragma once

namespace nb {
namespace {

struct BlockRows {
  uint32_t begin, count;
};
__device__ __forceinline__ BlockRows block_rows(const JobDesc &d) {
  uint32_t b, e;
  block_row_range(d.rows, d.unit, blockIdx.x, gridDim.x, &b, &e);
  return BlockRows{b, e - b};
}

// Dynamic shared memory: weight ring | activation vector (bf16; the attention
// merge records overlay it) | StepShared | row totals.
template <uint32_t PER>
__global__ void __launch_bounds__(kStreamThreads, 1) decode_step_kernel(StepKernelParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t *ring = smem;
  uint16_t *x = reinterpret_cast<uint16_t *>(smem + kRingBytes);
  StepShared &sh = *reinterpret_cast<StepShared *>(smem + kRingBytes + step_x_bytes(p.x_elems));
  float *row_total = reinterpret_cast<float *>(smem + kRingBytes + step_x_bytes(p.x_elems) +
                                               step_round128(sizeof(StepShared)));

  const uint32_t position = *p.st.cursor;
  if (position >= p.st.max_context) {
    if (blockIdx.x == 0 && threadIdx.x == 0) report_error(p.st.error_word, kErrCursorOutOfRange);
    return;  // uniform over the grid: nobody reaches a barrier
  }
  if (threadIdx.x == 0) sh.dead = 0;
  RowStream rs;
  stream_init(rs, ring, sh.stream, p.jobs, p.job_count);
  __syncthreads();
  stream_fill(rs);

  uint32_t token = position < *p.st.prompt_count ? p.st.prompt[position] : p.st.slots[position - 1].token;
  if (token >= p.st.vocab) {
    if (blockIdx.x == 0 && threadIdx.x == 0) report_error(p.st.error_word, kErrTokenOutOfRange);
    token = 0;
  }
  uint32_t barrier = 0;
  long long mark_last = clock64();
  auto mark = [&](uint32_t phase) {
    if (p.phase_cycles != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
      const long long now = clock64();
      atomicAdd(p.phase_cycles + phase, static_cast<unsigned long long>(now - mark_last));
      mark_last = now;
    }
  };
  // Zeroes the row totals of the job about to run; call before the prologue's
  // closing __syncthreads.
  auto clear_rows = [&](uint32_t job) {
    const uint32_t count = block_rows(p.jobs[job]).count;
    for (uint32_t r = threadIdx.x; r < count; r += blockDim.x) row_total[r] = 0.0f;
  };
  // y[row] = total, coalesced, after the block has synchronised behind the stream.
  auto store_rows = [&](uint32_t job, float *out) {
    const BlockRows br = block_rows(p.jobs[job]);
    for (uint32_t r = threadIdx.x; r < br.count; r += blockDim.x) {
      out[br.begin + r] = stream_row_total(sh.stream, row_total, r);
    }
  };

  for (uint32_t l = 0; l < p.layer_count; ++l) {
    const StepLayerDev &L = p.layers[l];
    // ---- QKV ----
    clear_rows(4u * l);
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
    mark(kPhaseQkvPrologue);
    stream_consume(rs, sh.stream, 4u * l, x, row_total, p.st.error_word);
    __syncthreads();
    store_rows(4u * l, p.qkv);
    mark(kPhaseQkv);
    grid_barrier(p, sh, ++barrier);
    mark(kPhaseBarrierQkv);
    // ---- attention ----
    attention_phase<PER>(p, sh, reinterpret_cast<float *>(x), L, position);
    mark(kPhaseAttention);
    grid_barrier(p, sh, ++barrier);
    mark(kPhaseBarrierAttention);
    // ---- O ----
    clear_rows(4u * l + 1u);
    merge_attention_to_smem(x, sh.weights, p.partial_acc, p.partial_m, p.partial_l, p.heads, p.head_dim,
                            p.attn_splits);
    __syncthreads();
    mark(kPhaseOPrologue);
    stream_consume(rs, sh.stream, 4u * l + 1u, x, row_total, p.st.error_word);
    __syncthreads();
    store_rows(4u * l + 1u, p.o_out);
    mark(kPhaseO);
    grid_barrier(p, sh, ++barrier);
    mark(kPhaseBarrierO);
    // ---- gate/up + SwiGLU ----
    clear_rows(4u * l + 2u);
    add_norm_to_smem(x, p.h_a, p.o_out, L.o_bias, L.rms_mlp, p.eps, p.hidden,
                     blockIdx.x == 0 ? p.h_b : nullptr, sh.scratch);
    __syncthreads();
    mark(kPhaseGateUpPrologue);
    stream_consume(rs, sh.stream, 4u * l + 2u, x, row_total, p.st.error_word);
    __syncthreads();
    {
      const BlockRows br = block_rows(p.jobs[4u * l + 2u]);
      for (uint32_t i = threadIdx.x; i < br.count / 2u; i += blockDim.x) {
        const float gate = stream_row_total(sh.stream, row_total, 2u * i);
        const float up = stream_row_total(sh.stream, row_total, 2u * i + 1u);
        p.ff_bf16[br.begin / 2u + i] = f32_to_bf16_bits(silu(gate) * up);
      }
    }
    mark(kPhaseGateUp);
    grid_barrier(p, sh, ++barrier);
    mark(kPhaseBarrierGateUp);
    // ---- down ----
    clear_rows(4u * l + 3u);
    {
      // all loads of the SwiGLU vector are issued before the first store
      constexpr uint32_t kBatch = 8;
      const uint32_t vecs = p.intermediate / 8u;
      for (uint32_t base = 0; base < vecs; base += kBatch * blockDim.x) {
        uint4 v[kBatch];
#pragma unroll
        for (uint32_t k = 0; k < kBatch; ++k) {
          const uint32_t i = base + k * blockDim.x + threadIdx.x;
          if (i < vecs) v[k] = __ldcg(reinterpret_cast<const uint4 *>(p.ff_bf16) + i);
        }
#pragma unroll
        for (uint32_t k = 0; k < kBatch; ++k) {
          const uint32_t i = base + k * blockDim.x + threadIdx.x;
          if (i < vecs) reinterpret_cast<uint4 *>(x)[i] = v[k];
        }
      }
    }
    __syncthreads();
    mark(kPhaseDownPrologue);
    stream_consume(rs, sh.stream, 4u * l + 3u, x, row_total, p.st.error_word);
    __syncthreads();
    store_rows(4u * l + 3u, p.down);
    mark(kPhaseDown);
    grid_barrier(p, sh, ++barrier);
    mark(kPhaseBarrierDown);
  }
  if (p.sample != 0) {
    const uint32_t job = 4u * p.layer_count;
    clear_rows(job);
    add_norm_to_smem(x, p.h_b, p.down, nullptr, p.final_norm, p.eps, p.hidden,
                     blockIdx.x == 0 ? p.h_a : nullptr, sh.scratch);
    __syncthreads();
    stream_consume(rs, sh.stream, job, x, row_total, p.st.error_word);
    __syncthreads();
    // logits + this block's best (value, lowest index); non-finite logits never win
    const BlockRows br = block_rows(p.jobs[job]);
    float bv = -INFINITY;
    uint32_t bi = kNoIndex;
    for (uint32_t r = threadIdx.x; r < br.count; r += blockDim.x) {
      const float v = stream_row_total(sh.stream, row_total, r);
      p.logits[br.begin + r] = v;
      if (isfinite(v) && better(v, br.begin + r, bv, bi)) {
        bv = v;
        bi = br.begin + r;
      }
    }
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, offset);
      const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, offset);
      if (oi != kNoIndex && better(ov, oi, bv, bi)) {
        bv = ov;
        bi = oi;
      }
    }
    float *wv = sh.scratch;
    uint32_t *wi = reinterpret_cast<uint32_t *>(sh.scratch + 32);
    if ((threadIdx.x & 31u) == 0) {
      wv[threadIdx.x >> 5] = bv;
      wi[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      bv = -INFINITY;
      bi = kNoIndex;
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
    mark(kPhaseLmHead);
  }
  stream_drain(rs);
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

uint32_t step_kernel_smem_bytes(uint32_t x_elems, uint32_t row_elems) {
  return kRingBytes + step_x_bytes(x_elems) + step_round128(sizeof(StepShared)) +
         step_round128(row_elems * 4u + 16u);
}

bool step_kernel_supported(uint32_t hidden, uint32_t heads, uint32_t kv_heads, uint32_t head_dim,
                           uint32_t intermediate, uint32_t x_elems, uint32_t row_elems) {
  return (head_dim == 64 || head_dim == 128) && heads <= kStepMaxHeads && hidden % 8 == 0 &&
         intermediate % 8 == 0 && (heads * head_dim) % 8 == 0 && kv_heads != 0 &&
         heads % kv_heads == 0 && step_kernel_smem_bytes(x_elems, row_elems) <= 227u * 1024u;
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
                                     step_kernel_smem_bytes(p.x_elems, p.row_elems), stream);
}

}  // namespace nb
