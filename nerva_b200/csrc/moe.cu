// Softmax top-k sparse MoE MLP of the resident decode step (Qwen3-MoE / Mixtral
// style).  The reference runs the whole MLP of a layer in ONE thread block
// (run_sparse_moe_mlp, hf_decode_sequence/device_ops.cuh:183-315); here it is two launches:
//   moe_expert_kernel<kGateUp>  residual add + RMSNorm, the router mat-vec, softmax over the
//                       router logits and top-k by (weight descending, index ascending) with
//                       optional renormalisation — by every block for itself —, then the gate
//                       and up projections of the k chosen experts (+ the shared expert) as
//                       ONE weight stream over a job list built from the routing result
//   moe_expert_kernel<kDown>    SwiGLU + down projections of the same experts,
//                       summed with the routing weights in rank order
// Arithmetic follows the reference kernel: the mat-vecs read the UNROUNDED fp32
// normalised hidden state and the unrounded fp32 SwiGLU output (unlike the dense
// path, which rounds both to bf16), accumulate in fp32, and the expert outputs
// are added as down += weight * y in rank order, then the shared expert scaled by
// sigmoid(shared_router . x).
//
// Shape of the expert kernels' weight stream (row_stream.cuh, set for this file only): 16 warps per
// block, each with a ring of two 4 KB slots, where the dense projections run 8 warps with three 8 KB
// slots.  An expert's rows are short (4 KB for gate/up at hidden 2048, 2.8 KB for down at
// intermediate 1408) and the fp32 activations cost two shared loads per weight load, so these
// kernels are bound by the instruction latency of a warp, not by the bytes in flight: twice the
// warps hide twice the latency.
#define NERVA_STREAM_WARPS 16
#define NERVA_CHUNK_BYTES 4096
#define NERVA_STREAM_SLOTS 2
#include "kernels.cuh"
#include "row_stream.cuh"
#include "step_device.cuh"

namespace nb {
namespace {

constexpr uint32_t kMoeMaxTopK = 16;
constexpr uint32_t kMoeMaxJobs = 2u * kMoeMaxTopK + 2u;

// ---- routing ----
__device__ __forceinline__ bool route_precedes(float w, uint32_t e, float best_w, uint32_t best_e) {
  return w > best_w || (w == best_w && e < best_e);
}

// One block of THREADS threads, all of which call.  `logit` is the router logit of expert
// threadIdx.x (anything for threads beyond num_experts).  weights = softmax(logits) with the
// reference's guards (divide only by a finite positive total); the k winners by (weight desc,
// index asc) go to ids_out / weights_out (shared or global memory), written by thread 0.
template <uint32_t THREADS>
__device__ __forceinline__ void moe_route_block(float logit, uint32_t num_experts, uint32_t top_k, uint32_t norm_topk_prob,
                                                uint32_t *ids_out, float *weights_out) {
  __shared__ float w_sh[256];
  __shared__ float scratch[40];
  __shared__ float red_w[THREADS / 32];
  __shared__ uint32_t red_e[THREADS / 32];
  __shared__ uint32_t chosen[kMoeMaxTopK];
  __shared__ float chosen_w[kMoeMaxTopK];
  const uint32_t e = threadIdx.x;
  if (e >= num_experts) logit = -INFINITY;
  // maximum
  float m = logit;
  m = warp_max(m);
  if ((threadIdx.x & 31u) == 0) red_w[threadIdx.x >> 5] = m;
  __syncthreads();
  m = -INFINITY;
  for (uint32_t i = 0; i < THREADS / 32; ++i) m = fmaxf(m, red_w[i]);
  __syncthreads();
  const float ex = e < num_experts ? expf(logit - m) : 0.0f;
  const float total = block_sum(ex, scratch);
  float w = ex;
  if (total > 0.0f && isfinite(total)) w = ex / total;
  if (e < 256u) w_sh[e] = e < num_experts ? w : -INFINITY;
  __syncthreads();
  for (uint32_t rank = 0; rank < top_k; ++rank) {
    float bw = -INFINITY;
    uint32_t be = 0xffffffffu;
    if (e < num_experts) {
      bool taken = false;
      for (uint32_t prev = 0; prev < rank; ++prev) taken = taken || chosen[prev] == e;
      if (!taken) {
        bw = w_sh[e];
        be = e;
      }
    }
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float ow = __shfl_xor_sync(0xffffffffu, bw, offset);
      const uint32_t oe = __shfl_xor_sync(0xffffffffu, be, offset);
      if (oe != 0xffffffffu && (be == 0xffffffffu || route_precedes(ow, oe, bw, be))) {
        bw = ow;
        be = oe;
      }
    }
    if ((threadIdx.x & 31u) == 0) {
      red_w[threadIdx.x >> 5] = bw;
      red_e[threadIdx.x >> 5] = be;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      bw = -INFINITY;
      be = 0xffffffffu;
      for (uint32_t i = 0; i < THREADS / 32; ++i) {
        if (red_e[i] != 0xffffffffu && (be == 0xffffffffu || route_precedes(red_w[i], red_e[i], bw, be))) {
          bw = red_w[i];
          be = red_e[i];
        }
      }
      chosen[rank] = be;
      chosen_w[rank] = bw;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    float sum = 0.0f;
    for (uint32_t rank = 0; rank < top_k; ++rank) sum += chosen_w[rank];
    for (uint32_t rank = 0; rank < top_k; ++rank) {
      float out = chosen_w[rank];
      if (norm_topk_prob != 0 && sum > 0.0f) out /= sum;
      ids_out[rank] = chosen[rank] == 0xffffffffu ? 0u : chosen[rank];
      weights_out[rank] = out;
    }
  }
  __syncthreads();
}

// ---- expert projections ----
enum MoePhase : uint32_t { kGateUp = 0, kDown = 1 };

struct MoeShared {
  StreamShared stream;
  JobDesc jobs[kMoeMaxJobs];       // this block's pieces of the matrices, in order (whole = 1)
  uint32_t piece_job[kMoeMaxJobs]; // the matrix (global job) a piece belongs to
  uint32_t piece_row[kMoeMaxJobs]; // first row of the piece inside its matrix
  uint32_t first[kMoeMaxJobs], end[kMoeMaxJobs];  // this block's rows of every matrix (scratch of the list's construction)
  float scratch[40];
  uint32_t ids[kMoeMaxTopK];       // the chosen experts held by this rank, as local indices, in routing order
  float weights[kMoeMaxTopK + 1];  // their routing weights; [routed] = the shared expert's gate
  uint32_t routed;                 // how many of the top_k experts are held here
  uint32_t route_ids[kMoeMaxTopK]; // kGateUp: the routing result of this block's own routing
  float route_weights[kMoeMaxTopK];
  float logits[256];               // kGateUp: router logits
  uint32_t pieces;
  uint32_t ticket;
};
__host__ __device__ inline uint32_t round128u(uint32_t v) { return (v + 127u) & ~127u; }

// fp32 twin of add_norm_to_smem: x = (r * scale) * w, unrounded.  PLANAR: element i goes to
// xf32_index(i, cols), the layout the fp32 path of the weight stream reads (row_stream.cuh).
template <bool PLANAR>
__device__ void add_norm_to_smem_f32(float *x, const float *a, const float *b, const uint16_t *bias,
                                     const uint16_t *w, float eps, uint32_t cols, float *scratch) {
  float sumsq = 0.0f;
  constexpr uint32_t kBatch = 4;  // elements whose loads are in flight together
  for (uint32_t base = threadIdx.x; base < cols; base += blockDim.x * kBatch) {
    float va[kBatch], vb[kBatch], vbias[kBatch];
#pragma unroll
    for (uint32_t u = 0; u < kBatch; ++u) {
      const uint32_t i = base + u * blockDim.x;
      va[u] = i < cols ? __ldcg(a + i) : 0.0f;
      vb[u] = i < cols && b != nullptr ? __ldcg(b + i) : 0.0f;
      vbias[u] = i < cols && bias != nullptr ? bf16_bits_to_f32(bias[i]) : 0.0f;
    }
#pragma unroll
    for (uint32_t u = 0; u < kBatch; ++u) {
      const uint32_t i = base + u * blockDim.x;
      if (i >= cols) break;
      // the order of the sum: (b or a) + bias, then + a when there are two addends
      float r = b != nullptr ? vb[u] : va[u];
      if (bias != nullptr) r += vbias[u];
      if (b != nullptr) r += va[u];
      x[PLANAR ? xf32_index(i, cols) : i] = r;
      sumsq += r * r;
    }
  }
  const float total = block_sum(sumsq, scratch);
  const float scale = rsqrtf(total / static_cast<float>(cols) + eps);
  for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) {
    const uint32_t at = PLANAR ? xf32_index(i, cols) : i;
    x[at] = x[at] * scale * bf16_bits_to_f32(w[i]);
  }
  __syncthreads();
}

// Matrix `g` of a phase.  kGateUp: gate then up matrix of every chosen expert held here (routing
// order), then of the shared expert; rows = intermediate size, cols = hidden.  kDown: the down matrix
// of the same experts; rows = hidden, cols = intermediate size.
template <uint32_t PHASE>
__device__ __forceinline__ JobDesc moe_matrix(const MoeExpertParams &p, const MoeShared &sh, uint32_t g) {
  const uint32_t r = PHASE == kGateUp ? g / 2u : g;
  const bool is_shared = r >= sh.routed;
  const uint64_t mi = p.moe_intermediate, h = p.hidden;
  JobDesc d{};
  d.unit = 1;
  d.whole = 1;
  if (PHASE == kGateUp) {
    d.cols = p.hidden;
    if (is_shared) {
      d.rows = p.shared_intermediate;
      d.weight = (g & 1u) == 0 ? p.w_shared_gate : p.w_shared_up;
    } else {
      d.rows = p.moe_intermediate;
      d.weight = p.w_expert_gate_up + static_cast<uint64_t>(sh.ids[r]) * p.expert_stride +
                 ((g & 1u) != 0 ? p.expert_up_offset : 0u);
    }
  } else {
    d.rows = p.hidden;
    if (is_shared) {
      d.cols = p.shared_intermediate;
      d.weight = p.w_shared_down;
    } else {
      d.cols = p.moe_intermediate;
      d.weight = p.w_expert_down + static_cast<uint64_t>(sh.ids[r]) * h * mi;
    }
  }
  return d;
}

// One launch per phase.  The matrices of a phase, one after the other, form one long list of rows;
// it is cut into gridDim.x contiguous runs of equal weight-byte count (a row belongs to the block
// in whose run its first byte lies), so a block streams one or two long pieces instead of a sliver
// of every matrix, and the pieces of all matrices stream at the same time.
//   kGateUp  every row's dot product with the normalised hidden state goes to gate_up_out at the
//            row's place in the list: [gate_0 | up_0 | gate_1 | up_1 | ... | shared gate | shared up].
//   kDown    row r of matrix g gives weight_g * (W_g[r] . silu(gate_g) * up_g) into partial[g][r]; the
//            block that draws the last ticket adds the matrices' contributions per row in list order
//            (routing order, then the shared expert: the order of the reference's loop) and writes
//            the MLP output, or pushes it to the other ranks under expert parallel.
// Shared memory: ring | x (fp32, max(hidden, largest intermediate)) | MoeShared | row totals.
template <uint32_t PHASE>
__global__ void __launch_bounds__(kStreamThreads, 1) moe_expert_kernel(MoeExpertParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t x_elems = p.hidden > p.max_intermediate ? p.hidden : p.max_intermediate;
  float *x = reinterpret_cast<float *>(smem + kRingBytes);
  MoeShared &sh = *reinterpret_cast<MoeShared *>(smem + kRingBytes + round128u(x_elems * 4u));
  float *row_total = reinterpret_cast<float *>(smem + kRingBytes + round128u(x_elems * 4u) +
                                               round128u(sizeof(MoeShared)));
  pdl_trigger();
  // Everything depends on the previous kernel: the hidden state, and through it the routing.
  pdl_wait();
  const uint32_t *route_ids = p.expert_ids;
  const float *route_weights = p.route_weights;
  if (PHASE == kGateUp) {
    // Routing.  Every block normalises the hidden state for itself (it needs it for its rows
    // anyway), computes all router logits from it (one warp per expert row; the matrix is small and
    // comes from L2 after the first block has read it) and routes: the same arithmetic in the same
    // order in every block, so all blocks agree.  Block 0 stores the new residual and the routing
    // result for the down launch.
    if (blockIdx.x == 0 && p.resid_out != nullptr) {
      for (uint32_t i = threadIdx.x; i < p.hidden; i += blockDim.x) {
        float r = p.add_b != nullptr ? __ldcg(p.add_b + i) : __ldcg(p.add_a + i);
        if (p.add_bias != nullptr) r += bf16_bits_to_f32(p.add_bias[i]);
        if (p.add_b != nullptr) r += __ldcg(p.add_a + i);
        p.resid_out[i] = r;
      }
    }
    add_norm_to_smem_f32<true>(x, p.add_a, p.add_b, p.add_bias, p.norm_weight, p.eps, p.hidden, sh.scratch);
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const float4 *xa = reinterpret_cast<const float4 *>(x), *xb = xa + p.hidden / 8u;
    for (uint32_t row = warp; row < p.num_experts; row += kStreamWarps) {
      const uint4 *w = reinterpret_cast<const uint4 *>(p.w_router + static_cast<uint64_t>(row) * p.hidden);
      float acc = 0.0f;
      constexpr uint32_t kBatch = 8;  // loads in flight per lane: a 2048-wide row in one round trip
      for (uint32_t base = lane; base < p.hidden / 8u; base += 32u * kBatch) {
        uint4 wv[kBatch];
#pragma unroll
        for (uint32_t u = 0; u < kBatch; ++u) {
          const uint32_t i = base + 32u * u;
          wv[u] = i < p.hidden / 8u ? __ldg(w + i) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (uint32_t u = 0; u < kBatch; ++u) {
          const uint32_t i = base + 32u * u;
          if (i < p.hidden / 8u) acc = dot8_f32(wv[u], xa[i], xb[i], acc);
        }
      }
      acc = warp_sum(acc);
      if (lane == 0) sh.logits[row] = acc;
    }
    __syncthreads();
    moe_route_block<kStreamThreads>(sh.logits[threadIdx.x < 256u ? threadIdx.x : 0u], p.num_experts, p.top_k,
                                    p.norm_topk_prob, sh.route_ids, sh.route_weights);
    route_ids = sh.route_ids;
    route_weights = sh.route_weights;
    if (blockIdx.x == 0 && threadIdx.x < p.top_k) {
      p.expert_ids[threadIdx.x] = sh.route_ids[threadIdx.x];
      p.route_weights[threadIdx.x] = sh.route_weights[threadIdx.x];
    }
  }
  if (threadIdx.x == 0) {
    // routing order is kept; under expert parallel only the experts held here stay in the list
    uint32_t routed = 0;
    for (uint32_t r = 0; r < p.top_k; ++r) {
      const uint32_t local = route_ids[r] - p.expert_base;  // wraps to a large value below the base
      if (p.expert_local == 0 || local < p.expert_local) {
        sh.ids[routed] = local;
        sh.weights[routed] = route_weights[r];
        routed += 1;
      }
    }
    sh.routed = routed;
  }
  __syncthreads();
  const uint32_t routed = sh.routed;
  const uint32_t experts = routed + (p.shared_intermediate != 0 ? 1u : 0u);
  const uint32_t matrices = PHASE == kGateUp ? 2u * experts : experts;
  // this block's rows of every matrix
  uint64_t total = 0;  // weight elements of the whole list
  for (uint32_t g = 0; g < matrices; ++g) {
    const JobDesc d = moe_matrix<PHASE>(p, sh, g);
    total += static_cast<uint64_t>(d.rows) * d.cols;
  }
  const uint64_t run_begin = total * blockIdx.x / gridDim.x, run_end = total * (blockIdx.x + 1ull) / gridDim.x;
  if (threadIdx.x < matrices) {
    uint64_t start = 0;
    for (uint32_t g = 0; g < threadIdx.x; ++g) {
      const JobDesc d = moe_matrix<PHASE>(p, sh, g);
      start += static_cast<uint64_t>(d.rows) * d.cols;
    }
    const JobDesc d = moe_matrix<PHASE>(p, sh, threadIdx.x);
    // first row whose first element lies at or beyond a list position
    auto row_at = [&](uint64_t at) -> uint32_t {
      if (at <= start) return 0u;
      const uint64_t r = (at - start + d.cols - 1u) / d.cols;
      return r > d.rows ? d.rows : static_cast<uint32_t>(r);
    };
    sh.first[threadIdx.x] = row_at(run_begin);
    sh.end[threadIdx.x] = row_at(run_end);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t n = 0;
    for (uint32_t g = 0; g < matrices; ++g) {
      if (sh.end[g] <= sh.first[g]) continue;
      JobDesc d = moe_matrix<PHASE>(p, sh, g);
      d.weight += static_cast<uint64_t>(sh.first[g]) * d.cols;
      d.rows = sh.end[g] - sh.first[g];
      sh.jobs[n] = d;
      sh.piece_job[n] = g;
      sh.piece_row[n] = sh.first[g];
      n += 1;
    }
    sh.pieces = n;
  }
  __syncthreads();
  const uint32_t pieces = sh.pieces;
  RowStream rs;
  stream_init(rs, smem, sh.stream, sh.jobs, pieces);
  stream_fill(rs);
  for (uint32_t i = threadIdx.x; i < p.max_rows_per_block; i += blockDim.x) row_total[i] = 0.0f;

  if (PHASE == kGateUp) {
    if (blockIdx.x == 0 && p.shared_intermediate != 0) {
      // gate of the shared expert: sigmoid(shared_router . x), or 1 for shared experts that are always on
      float dot = 0.0f;
      for (uint32_t i = threadIdx.x; p.w_shared_router != nullptr && i < p.hidden; i += blockDim.x)
        dot += bf16_bits_to_f32(p.w_shared_router[i]) * x[xf32_index(i, p.hidden)];
      const float sum = block_sum(dot, sh.scratch);
      if (threadIdx.x == 0) *p.shared_gate = p.w_shared_router != nullptr ? 1.0f / (1.0f + expf(-sum)) : 1.0f;
    }
  } else if (p.shared_intermediate != 0 && threadIdx.x == 0) {
    sh.weights[routed] = __ldcg(p.shared_gate);
  }
  __syncthreads();

  for (uint32_t j = 0; j < pieces; ++j) {
    const JobDesc &job = sh.jobs[j];
    const uint32_t g = sh.piece_job[j];
    // the matrix's place in the list of rows (kGateUp) / of activations (kDown: gate then up of expert g)
    uint64_t place = 0;
    for (uint32_t k = 0; k < g; ++k) {
      const JobDesc d = moe_matrix<PHASE>(p, sh, k);
      place += PHASE == kGateUp ? d.rows : 2u * d.cols;
    }
    if (PHASE == kDown) {
      // x = silu(gate) * up of expert g, unrounded
      const float *gate = p.gate_up_out + place;
      const float *up = gate + job.cols;
      constexpr uint32_t kBatch = 4;  // elements whose loads are in flight together
      for (uint32_t base = threadIdx.x; base < job.cols; base += blockDim.x * kBatch) {
        float vg[kBatch], vu[kBatch];
#pragma unroll
        for (uint32_t u = 0; u < kBatch; ++u) {
          const uint32_t i = base + u * blockDim.x;
          vg[u] = i < job.cols ? __ldcg(gate + i) : 0.0f;
          vu[u] = i < job.cols ? __ldcg(up + i) : 0.0f;
        }
#pragma unroll
        for (uint32_t u = 0; u < kBatch; ++u) {
          const uint32_t i = base + u * blockDim.x;
          if (i < job.cols) x[xf32_index(i, job.cols)] = silu(vg[u]) * vu[u];
        }
      }
      __syncthreads();
    }
    stream_consume<true>(rs, sh.stream, j, x, row_total, p.error_word);
    __syncthreads();
    if (PHASE == kGateUp) {
      float *out = p.gate_up_out + place + sh.piece_row[j];
      for (uint32_t r = threadIdx.x; r < job.rows; r += blockDim.x) {
        out[r] = stream_row_total(sh.stream, row_total, r);
        row_total[r] = 0.0f;
      }
    } else {
      const float weight = sh.weights[g];
      float *out = p.partial + static_cast<uint64_t>(g) * p.hidden + sh.piece_row[j];
      for (uint32_t r = threadIdx.x; r < job.rows; r += blockDim.x) {
        out[r] = weight * stream_row_total(sh.stream, row_total, r);
        row_total[r] = 0.0f;
      }
    }
    __syncthreads();
  }
  stream_drain(rs);
  if (PHASE == kDown) {
    // the block that sees every other block's rows written adds the matrices' contributions
    if (threadIdx.x == 0) {
      uint32_t drawn;
      asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(drawn) : "l"(p.ticket) : "memory");
      sh.ticket = drawn;
    }
    __syncthreads();
    if (sh.ticket != gridDim.x - 1u) return;
    unsigned long long tag = 0;
    if (p.push.world > 1)
      tag = static_cast<unsigned long long>(static_cast<uint32_t>(*p.push.epoch) * p.push.per_epoch + p.push.offset) << 32;
    for (uint32_t r = threadIdx.x; r < p.hidden; r += blockDim.x) {
      float v[kMoeMaxTopK + 1u];
#pragma unroll
      for (uint32_t g = 0; g < kMoeMaxTopK + 1u; ++g)
        v[g] = g < experts ? __ldcg(p.partial + static_cast<uint64_t>(g) * p.hidden + r) : 0.0f;
      float sum = 0.0f;
#pragma unroll
      for (uint32_t g = 0; g < kMoeMaxTopK + 1u; ++g)
        if (g < experts) sum += v[g];
      if (p.push.world > 1) {
        // expert parallel: this rank's partial sum travels to every rank (projection.cu: the Store epilogue's push)
        const unsigned long long entry = tag | __float_as_uint(sum);
        const uint64_t at = static_cast<uint64_t>(p.push.rank) * p.hidden + r;
        for (uint32_t q = 0; q < p.push.world; ++q)
          asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p.push.recv[q] + at), "l"(entry) : "memory");
      } else {
        p.out_f32[r] = sum;
      }
    }
    if (threadIdx.x == 0) *p.ticket = 0;  // ready for the next launch
  }
}

uint32_t moe_blocks(const MoeExpertParams &p, uint32_t sm_count) {
  uint32_t rows = p.hidden < p.moe_intermediate ? p.hidden : p.moe_intermediate;
  if (p.shared_intermediate != 0 && p.shared_intermediate < rows) rows = p.shared_intermediate;
  uint32_t blocks = rows < sm_count ? rows : sm_count;
  return blocks == 0 ? 1u : blocks;
}

// Most rows a block can get of one matrix: its run of the list (total / blocks weight elements,
// rounded up) divided by the shortest row, plus the rows cut at either end.
uint32_t moe_max_rows(const MoeExpertParams &p, uint32_t blocks) {
  const uint64_t inter = static_cast<uint64_t>(p.top_k) * p.moe_intermediate + p.shared_intermediate;
  const uint64_t gate_up_run = (2u * inter * p.hidden + blocks - 1u) / blocks;
  const uint64_t down_run = (inter * p.hidden + blocks - 1u) / blocks;
  uint32_t narrow = p.moe_intermediate;
  if (p.shared_intermediate != 0 && p.shared_intermediate < narrow) narrow = p.shared_intermediate;
  const uint64_t rows_gate_up = gate_up_run / p.hidden + 2u, rows_down = down_run / narrow + 2u;
  return static_cast<uint32_t>(rows_gate_up > rows_down ? rows_gate_up : rows_down);
}

uint32_t moe_smem_bytes(const MoeExpertParams &p) {
  const uint32_t x_elems = p.hidden > p.max_intermediate ? p.hidden : p.max_intermediate;
  return kRingBytes + round128u(x_elems * 4u) + round128u(sizeof(MoeShared)) + p.max_rows_per_block * 4u + 128u;
}

}  // namespace

bool moe_supported(uint32_t hidden, uint32_t moe_intermediate, uint32_t shared_intermediate,
                   uint32_t num_experts, uint32_t top_k, uint32_t sm_count) {
  if (num_experts == 0 || num_experts > 256 || top_k == 0 || top_k > kMoeMaxTopK || top_k > num_experts) return false;
  if (hidden % 8u != 0 || moe_intermediate % 8u != 0 || shared_intermediate % 8u != 0) return false;
  MoeExpertParams p{};
  p.hidden = hidden;
  p.moe_intermediate = moe_intermediate;
  p.shared_intermediate = shared_intermediate;
  p.max_intermediate = moe_intermediate > shared_intermediate ? moe_intermediate : shared_intermediate;
  p.top_k = top_k;
  p.max_rows_per_block = moe_max_rows(p, moe_blocks(p, sm_count));
  return moe_smem_bytes(p) <= 227u * 1024u - 2048u;
}

// Dynamic shared memory a block may ask for: the 227 KB of an SM less the kernels' static arrays
// (the routing scratch).
constexpr uint32_t kMoeStaticSmemAllowance = 2048;
constexpr uint32_t kMoeMaxDynamicSmem = 227u * 1024u - kMoeStaticSmemAllowance;

cudaError_t configure_moe_kernels() {
  cudaFuncAttributes attr{};
  cudaError_t err = cudaFuncGetAttributes(&attr, moe_expert_kernel<kGateUp>);
  if (err == cudaSuccess && attr.sharedSizeBytes > kMoeStaticSmemAllowance) err = cudaErrorInvalidConfiguration;
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(moe_expert_kernel<kGateUp>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               kMoeMaxDynamicSmem);
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(moe_expert_kernel<kDown>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               kMoeMaxDynamicSmem);
  return err;
}

cudaError_t launch_moe_experts(cudaStream_t stream, const MoeExpertParams &params, uint32_t sm_count, bool pdl) {
  MoeExpertParams p = params;
  p.max_intermediate = p.moe_intermediate > p.shared_intermediate ? p.moe_intermediate : p.shared_intermediate;
  const uint32_t blocks = moe_blocks(p, sm_count);
  p.max_rows_per_block = moe_max_rows(p, blocks);
  const uint32_t smem = moe_smem_bytes(p);
  if (smem > kMoeMaxDynamicSmem || p.partial == nullptr || p.ticket == nullptr || p.w_router == nullptr ||
      p.num_experts == 0 || p.num_experts > 256 || p.top_k == 0 || p.top_k > kMoeMaxTopK || p.hidden % 8u != 0)
    return cudaErrorNotSupported;
  cudaError_t err = launch_with_pdl(moe_expert_kernel<kGateUp>, dim3(blocks), dim3(kStreamThreads), smem, stream,
                                    pdl, p);
  if (err != cudaSuccess) return err;
  return launch_with_pdl(moe_expert_kernel<kDown>, dim3(blocks), dim3(kStreamThreads), smem, stream, pdl, p);
}

}  // namespace nb
