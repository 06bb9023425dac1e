// Softmax top-k sparse MoE MLP of the resident decode step (Qwen3-MoE / Mixtral
// style).  The reference runs the whole MLP of a layer in ONE thread block
// (run_sparse_moe_mlp, hf_decode_sequence/device_ops.cuh:183-315); here it is
//   moe_router_logits_kernel  residual add + RMSNorm + router mat-vec (small matrix)
//   moe_route_kernel    softmax over the router logits, top-k by (weight
//                       descending, index ascending), optional renormalisation
//   moe_expert_kernel<kGateUp>  gate and up projections of the k chosen experts
//                       (+ the shared expert) as ONE weight stream over a job list
//                       built on the device from the routing result
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
// warps hide twice the latency (DeepSeek-V2-Lite step 3.23 -> 2.94 ms; 12, 20 and 24 warps and a
// third slot measured slower).
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
constexpr uint32_t kRouteThreads = 256;

// ---- routing ----
__device__ __forceinline__ bool route_precedes(float w, uint32_t e, float best_w, uint32_t best_e) {
  return w > best_w || (w == best_w && e < best_e);
}

// One block.  weights = softmax(logits) with the reference's guards (divide only
// by a finite positive total); the k winners by (weight desc, index asc).
__device__ __forceinline__ void moe_route_block(const MoeRouteParams &p) {
  __shared__ float w_sh[256];
  __shared__ float scratch[40];
  __shared__ float red_w[kRouteThreads / 32];
  __shared__ uint32_t red_e[kRouteThreads / 32];
  __shared__ uint32_t chosen[kMoeMaxTopK];
  __shared__ float chosen_w[kMoeMaxTopK];
  const uint32_t e = threadIdx.x;
  const float logit = e < p.num_experts ? __ldcg(p.logits + e) : -INFINITY;
  // maximum
  float m = logit;
  m = warp_max(m);
  if ((threadIdx.x & 31u) == 0) red_w[threadIdx.x >> 5] = m;
  __syncthreads();
  m = -INFINITY;
  for (uint32_t i = 0; i < kRouteThreads / 32; ++i) m = fmaxf(m, red_w[i]);
  __syncthreads();
  const float ex = e < p.num_experts ? expf(logit - m) : 0.0f;
  const float total = block_sum(ex, scratch);
  float w = ex;
  if (total > 0.0f && isfinite(total)) w = ex / total;
  w_sh[e] = e < p.num_experts ? w : -INFINITY;
  __syncthreads();
  for (uint32_t rank = 0; rank < p.top_k; ++rank) {
    float bw = -INFINITY;
    uint32_t be = 0xffffffffu;
    if (e < p.num_experts) {
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
      for (uint32_t i = 0; i < kRouteThreads / 32; ++i) {
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
    for (uint32_t rank = 0; rank < p.top_k; ++rank) sum += chosen_w[rank];
    for (uint32_t rank = 0; rank < p.top_k; ++rank) {
      float out = chosen_w[rank];
      if (p.norm_topk_prob != 0 && sum > 0.0f) out /= sum;
      p.expert_ids[rank] = chosen[rank] == 0xffffffffu ? 0u : chosen[rank];
      p.weights[rank] = out;
    }
  }
}
__global__ void __launch_bounds__(kRouteThreads) moe_route_kernel(MoeRouteParams p) {
  pdl_trigger();
  pdl_wait();
  moe_route_block(p);
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
  for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) {
    float r = b != nullptr ? __ldcg(b + i) : __ldcg(a + i);
    if (bias != nullptr) r += bf16_bits_to_f32(bias[i]);
    if (b != nullptr) r += __ldcg(a + i);
    x[PLANAR ? xf32_index(i, cols) : i] = r;
    sumsq += r * r;
  }
  const float total = block_sum(sumsq, scratch);
  const float scale = rsqrtf(total / static_cast<float>(cols) + eps);
  for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) {
    const uint32_t at = PLANAR ? xf32_index(i, cols) : i;
    x[at] = x[at] * scale * bf16_bits_to_f32(w[i]);
  }
  __syncthreads();
}

// Router logits: logits[e] = W_router[e] . x with x the unrounded fp32 normalised hidden state
// (residual add + RMSNorm in front, block 0 stores the new residual).  The matrix is small
// (experts x hidden), so plain 16-byte loads, one warp per row.
__global__ void __launch_bounds__(256) moe_router_logits_kernel(ProjectionParams p) {
  extern __shared__ __align__(16) float xr[];  // [cols]
  __shared__ float scratch[40];
  pdl_trigger();
  pdl_wait();
  if (blockIdx.x == 0 && p.resid_out != nullptr) {
    for (uint32_t i = threadIdx.x; i < p.cols; i += blockDim.x) {
      float r = p.add_b != nullptr ? __ldcg(p.add_b + i) : __ldcg(p.add_a + i);
      if (p.add_bias != nullptr) r += bf16_bits_to_f32(p.add_bias[i]);
      if (p.add_b != nullptr) r += __ldcg(p.add_a + i);
      p.resid_out[i] = r;
    }
  }
  add_norm_to_smem_f32<false>(xr, p.add_a, p.add_b, p.add_bias, p.norm_weight, p.eps, p.cols, scratch);
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  for (uint32_t row = blockIdx.x * warps + warp; row < p.rows; row += gridDim.x * warps) {
    const uint4 *w = reinterpret_cast<const uint4 *>(p.weight + static_cast<uint64_t>(row) * p.cols);
    float acc = 0.0f;
    for (uint32_t i = lane; i < p.cols / 8u; i += 32u) {
      const uint4 wv = w[i];
      const float4 xa = *reinterpret_cast<const float4 *>(xr + 8u * i);
      const float4 xb = *reinterpret_cast<const float4 *>(xr + 8u * i + 4u);
      acc = dot8_f32(wv, xa, xb, acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) p.out_f32[row] = acc;
  }
}

// Router logits and routing in one launch: block e computes logit e (every block normalises the
// hidden state for itself; the eight warps split the row), and the block that draws the last
// ticket — it sees every logit — runs the routing.  Block 0 stores the new residual.
__global__ void __launch_bounds__(kRouteThreads) moe_router_route_kernel(ProjectionParams p, MoeRouteParams route,
                                                                          uint32_t *ticket) {
  extern __shared__ __align__(16) float xr[];  // [cols]
  __shared__ float scratch[40];
  __shared__ uint32_t drawn_sh;
  pdl_trigger();
  pdl_wait();
  if (blockIdx.x == 0 && p.resid_out != nullptr) {
    for (uint32_t i = threadIdx.x; i < p.cols; i += blockDim.x) {
      float r = p.add_b != nullptr ? __ldcg(p.add_b + i) : __ldcg(p.add_a + i);
      if (p.add_bias != nullptr) r += bf16_bits_to_f32(p.add_bias[i]);
      if (p.add_b != nullptr) r += __ldcg(p.add_a + i);
      p.resid_out[i] = r;
    }
  }
  add_norm_to_smem_f32<false>(xr, p.add_a, p.add_b, p.add_bias, p.norm_weight, p.eps, p.cols, scratch);
  for (uint32_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const uint4 *w = reinterpret_cast<const uint4 *>(p.weight + static_cast<uint64_t>(row) * p.cols);
    float acc = 0.0f;
    for (uint32_t i = threadIdx.x; i < p.cols / 8u; i += blockDim.x) {
      const uint4 wv = w[i];
      const float4 xa = *reinterpret_cast<const float4 *>(xr + 8u * i);
      const float4 xb = *reinterpret_cast<const float4 *>(xr + 8u * i + 4u);
      acc = dot8_f32(wv, xa, xb, 0.0f) + acc;
    }
    const float total = block_sum(acc, scratch);
    if (threadIdx.x == 0) p.out_f32[row] = total;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t drawn;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(drawn) : "l"(ticket) : "memory");
    drawn_sh = drawn;
  }
  __syncthreads();
  if (drawn_sh != gridDim.x - 1u) return;
  moe_route_block(route);
  if (threadIdx.x == 0) *ticket = 0;  // ready for the next launch
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
  // The list depends on the routing result of this step.
  pdl_wait();
  if (threadIdx.x == 0) {
    // routing order is kept; under expert parallel only the experts held here stay in the list
    uint32_t routed = 0;
    for (uint32_t r = 0; r < p.top_k; ++r) {
      const uint32_t local = p.expert_ids[r] - p.expert_base;  // wraps to a large value below the base
      if (p.expert_local == 0 || local < p.expert_local) {
        sh.ids[routed] = local;
        sh.weights[routed] = p.route_weights[r];
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
    add_norm_to_smem_f32<true>(x, p.add_a, p.add_b, p.add_bias, p.norm_weight, p.eps, p.hidden, sh.scratch);
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
      for (uint32_t i = threadIdx.x; i < job.cols; i += blockDim.x)
        x[xf32_index(i, job.cols)] = silu(__ldcg(gate + i)) * __ldcg(up + i);
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
  if (hidden * 4u > 48u * 1024u) return false;  // the router kernel keeps the fp32 hidden state in 48 KB
  MoeExpertParams p{};
  p.hidden = hidden;
  p.moe_intermediate = moe_intermediate;
  p.shared_intermediate = shared_intermediate;
  p.max_intermediate = moe_intermediate > shared_intermediate ? moe_intermediate : shared_intermediate;
  p.top_k = top_k;
  p.max_rows_per_block = moe_max_rows(p, moe_blocks(p, sm_count));
  return moe_smem_bytes(p) <= 227u * 1024u;
}

cudaError_t configure_moe_kernels() {
  cudaError_t err = cudaFuncSetAttribute(moe_expert_kernel<kGateUp>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         227 * 1024);
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(moe_expert_kernel<kDown>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  return err;
}

cudaError_t launch_router_logits_f32(cudaStream_t stream, const ProjectionParams &p, uint32_t sm_count) {
  if (p.cols % 8u != 0 || p.cols * 4u > 48u * 1024u || p.rows == 0) return cudaErrorNotSupported;
  uint32_t blocks = (p.rows + 7u) / 8u;
  if (blocks > sm_count) blocks = sm_count;
  return launch_with_pdl(moe_router_logits_kernel, dim3(blocks), dim3(256), p.cols * 4u, stream, p.pdl != 0, p);
}

cudaError_t launch_moe_router_route(cudaStream_t stream, const ProjectionParams &p, const MoeRouteParams &route,
                                    uint32_t *ticket, uint32_t sm_count) {
  if (p.cols % 8u != 0 || p.cols * 4u > 48u * 1024u || p.rows == 0 || ticket == nullptr) return cudaErrorNotSupported;
  if (route.num_experts == 0 || route.num_experts > 256 || route.top_k == 0 || route.top_k > kMoeMaxTopK ||
      route.num_experts != p.rows)
    return cudaErrorInvalidValue;
  const uint32_t blocks = p.rows < sm_count ? p.rows : sm_count;
  return launch_with_pdl(moe_router_route_kernel, dim3(blocks), dim3(kRouteThreads), p.cols * 4u, stream, p.pdl != 0,
                         p, route, ticket);
}

cudaError_t launch_moe_route(cudaStream_t stream, const MoeRouteParams &p, bool pdl) {
  if (p.num_experts == 0 || p.num_experts > 256 || p.top_k == 0 || p.top_k > kMoeMaxTopK) return cudaErrorInvalidValue;
  return launch_with_pdl(moe_route_kernel, dim3(1), dim3(kRouteThreads), 0, stream, pdl, p);
}

cudaError_t launch_moe_experts(cudaStream_t stream, const MoeExpertParams &params, uint32_t sm_count, bool pdl) {
  MoeExpertParams p = params;
  p.max_intermediate = p.moe_intermediate > p.shared_intermediate ? p.moe_intermediate : p.shared_intermediate;
  const uint32_t blocks = moe_blocks(p, sm_count);
  p.max_rows_per_block = moe_max_rows(p, blocks);
  const uint32_t smem = moe_smem_bytes(p);
  if (smem > 227u * 1024u || p.partial == nullptr || p.ticket == nullptr) return cudaErrorNotSupported;
  cudaError_t err = launch_with_pdl(moe_expert_kernel<kGateUp>, dim3(blocks), dim3(kStreamThreads), smem, stream,
                                    pdl, p);
  if (err != cudaSuccess) return err;
  return launch_with_pdl(moe_expert_kernel<kDown>, dim3(blocks), dim3(kStreamThreads), smem, stream, pdl, p);
}

}  // namespace nb
