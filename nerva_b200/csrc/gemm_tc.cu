// Block projection on the tensor pipe: bf16 W[rows][cols] times a block of bf16 activation rows
// X[tokens][cols], fp32 accumulate, for 2..256 tokens at once.  The weights are streamed from HBM
// once for the whole block.  Replaces the reference's cublasLtMatmul of the packed block step and
// of the chunked prefill (hf_decode_sequence/projection.cu:192-262 launch_lt_gemm_tokens_plan,
// session_api_batch_fork_destroy.inc.cu:1-310, session_decode_prefill.inc.cu:1879-2245).
//
// Shape of the work.  The operands are swapped so that the weight rows are the M dimension of the
// MMA: D[128 weight rows][N tokens] += W_tile[128][64] * X_tile[N][64]^T per 64-wide slice of the
// inner dimension, `tcgen05.mma.cta_group::1.kind::f16` (M = 128, N = tokens rounded up to 16,
// K = 16 per instruction) with both operands in shared memory and the fp32 accumulator in tensor
// memory.  A 64-element slice of a row is 128 bytes, i.e. one 128-byte swizzle atom, so a weight
// tile and an activation tile arrive by ONE 2-D `cp.async.bulk.tensor` each (SWIZZLE_128B) in the
// canonical K-major layout the MMA descriptors describe.  No cluster, no multicast.
//
// Decomposition ("stream-K").  The sequence of (row tile, 64-wide slice) pairs is cut into one
// contiguous, equally long run per thread block, so every SM streams the same number of weight
// bytes whatever the shape (QKV has 48 row tiles, lm_head 1187).  A run that starts or ends in the
// middle of a row tile leaves a partial accumulator in a workspace slot (fp32, token-major: a warp's
// 32 rows of one token are one line); a small second launch (gemm_fixup_kernel, one block per split
// tile and 16 tokens) adds the partials of every split tile in ascending block order and runs the
// epilogue for it.  A matrix with between one and two row tiles per SM gets one block per tile
// instead: nothing is split and no second launch follows.  Summing inside the projection kernel by
// the last block to arrive was measured first: that one block reads every partial of its tile with
// 128 threads while the rest of the grid has left, which cost more than the launch.  The partition
// depends on the shape only, so a token's result does not depend on which other tokens share its
// block, and results are bit-stable run to run.
//
// Roles inside a block (192 threads): warp 0 issues the TMA copies into an mbarrier ring, warp 1
// allocates tensor memory and issues the MMAs (one elected lane), warps 2..5 read the accumulator
// with `tcgen05.ld` (each warp its own 32-lane quarter) and run the epilogue; two accumulator
// buffers let the epilogue of one tile overlap the MMAs of the next.  Every wait is bounded; a
// wait that gives up sets the error word and an abort flag that all roles poll, the block drains
// and frees its tensor memory before it returns.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <mutex>

#include "common.cuh"
#include "kernels.cuh"

namespace nb {
namespace {

constexpr uint32_t kTileRows = 128;   // MMA M
constexpr uint32_t kSliceK = 64;      // bf16 elements per ring stage along the inner dimension (128 bytes)
constexpr uint32_t kUmmaK = 16;       // inner elements per MMA instruction
constexpr uint32_t kATileBytes = kTileRows * kSliceK * 2u;
constexpr uint32_t kMaxStages = 8;
constexpr uint32_t kGemmThreads = 192;
constexpr uint32_t kEpilogueThreads = 128;
constexpr uint32_t kGroup = 16;         // tokens per tcgen05.ld
// Blocks of up to kSmallBlockTokens tokens run two thread blocks per SM (half the shared memory and
// a quarter of the tensor memory each): while one block of a launch drains its last tile, writes
// its results and leaves, the block that takes its place — of this launch or, with programmatic
// dependent launch, of the next one — is already filling its ring, so the SM keeps weights in
// flight across the hand-over.  Larger blocks (prefill chunks) take the SM alone.
constexpr uint32_t kSmallBlockTokens = 64;

struct GemmShared {
  uint64_t full[kMaxStages], empty[kMaxStages];
  uint64_t acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  uint32_t abort;
};

struct GemmKernelParams {
  uint32_t rows, cols, tokens, n_pad;  // n_pad: tokens rounded up to 16 (the MMA N)
  uint32_t stages;
  uint32_t tmem_columns;  // allocation: two accumulator buffers of tmem_columns / 2 fp32 columns
  uint32_t epilogue;
  const float *resid_in;
  float *out_f32;
  uint16_t *out_bf16;
  float *workspace;
  uint32_t *tickets;
  uint32_t *error_word;
  unsigned long long *stamps;
};

// Timeline stamp by an arbitrary thread of the first or the last block (common.cuh stamp() is thread 0 only).
__device__ __forceinline__ void stamp_any(unsigned long long *stamps, uint32_t slot) {
  if (stamps == nullptr) return;
  const uint32_t last = gridDim.x - 1u;
  if (blockIdx.x != 0 && blockIdx.x != last) return;
  unsigned long long now;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
  if (blockIdx.x == 0) stamps[slot] = now;
  if (blockIdx.x == last) stamps[4u + slot] = now;
}

// ---- static partition, computed identically by every role and by the fix-up ----
struct Partition {
  uint32_t tiles, slices, blocks;
  uint64_t total;
  __device__ __host__ uint64_t begin(uint32_t b) const { return total * b / blocks; }
  __device__ __host__ uint64_t end(uint32_t b) const { return total * (b + 1ull) / blocks; }
};
__device__ __host__ inline Partition make_partition(uint32_t rows, uint32_t cols, uint32_t blocks) {
  Partition p;
  p.tiles = (rows + kTileRows - 1u) / kTileRows;
  p.slices = cols / kSliceK;
  p.total = static_cast<uint64_t>(p.tiles) * p.slices;
  p.blocks = blocks;
  return p;
}
// First block whose run touches tile t.
__device__ __host__ inline uint32_t first_block_of_tile(const Partition &p, uint32_t t) {
  const uint64_t at = static_cast<uint64_t>(t) * p.slices;
  uint32_t b = static_cast<uint32_t>(at * p.blocks / p.total);
  while (b + 1u < p.blocks && p.end(b) <= at) ++b;
  while (b > 0 && p.end(b - 1u) > at) --b;
  return b;
}
// Last block whose run touches tile t.
__device__ __host__ inline uint32_t last_block_of_tile(const Partition &p, uint32_t t) {
  const uint64_t last_slice = static_cast<uint64_t>(t + 1u) * p.slices - 1u;
  uint32_t hi = static_cast<uint32_t>(last_slice * p.blocks / p.total);
  while (hi + 1u < p.blocks && p.end(hi) <= last_slice) ++hi;
  while (hi > 0 && p.begin(hi) > last_slice) --hi;
  return hi;
}
// Workspace slot of block b's partial accumulator of tile t: slot 0 when the tile is where the
// block's run begins, slot 1 when it is where the run ends in another tile.
__device__ __host__ inline uint32_t partial_slot(const Partition &p, uint32_t b, uint32_t t) {
  return 2u * b + (static_cast<uint32_t>(p.begin(b) / p.slices) == t ? 0u : 1u);
}

struct Segment {
  uint32_t tile, slice_begin, slice_end;
};
// Walks the segments of this block's run.
struct SegmentWalk {
  uint64_t pos, end;
  uint32_t slices;
  __device__ bool next(Segment *s) {
    if (pos >= end) return false;
    s->tile = static_cast<uint32_t>(pos / slices);
    s->slice_begin = static_cast<uint32_t>(pos % slices);
    const uint64_t left = end - pos;
    const uint32_t room = slices - s->slice_begin;
    s->slice_end = s->slice_begin + (left < room ? static_cast<uint32_t>(left) : room);
    pos += s->slice_end - s->slice_begin;
    return true;
  }
};

// ---- PTX wrappers ----
__device__ __forceinline__ bool abortable_wait(uint64_t *bar, uint32_t parity, volatile uint32_t *abort,
                                               uint32_t *error_word) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  for (;;) {
#pragma unroll 1
    for (uint32_t spin = 0; spin < 64; ++spin) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (*abort != 0u) return false;
    if (clock64() - start > kWaitCycleLimit) {
      *abort = 1u;
      report_error(error_word, kErrTmaWaitTimeout);
      return false;
    }
  }
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, uint32_t x, uint32_t y, uint64_t *bar,
                                            uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%2, %3}], [%4], %5;" ::"r"(smem_addr(dst)),
      "l"(map), "r"(x), "r"(y), "r"(smem_addr(bar)), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t l2_evict_last_policy() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar))
               : "memory");
}
__device__ __forceinline__ void tcgen05_mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_load16(uint32_t taddr, float *v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (uint32_t i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (one swizzle atom):
// start address, 8-row groups 1024 bytes apart, SWIZZLE_128B, descriptor version 1.
__device__ __forceinline__ uint64_t kmajor_sw128_desc(const void *tile) {
  const uint64_t addr = smem_addr(tile);
  return ((addr & 0x3ffffull) >> 4) | (1ull << 16) | (static_cast<uint64_t>(1024u >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}
// Instruction descriptor: fp32 accumulator, bf16 A and B, both K-major, N = n, M = 128.
__device__ __forceinline__ uint32_t instr_desc_bf16(uint32_t n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((kTileRows >> 4) << 24);
}

// Epilogue of 16 tokens (g .. g + 15) of accumulator row `row`, values in v.  Called by all 32 lanes
// of a warp whose lanes hold 32 consecutive rows.
__device__ __forceinline__ void tile_epilogue(const GemmKernelParams &p, const float (&v)[kGroup], uint32_t row,
                                              uint32_t g, uint32_t lane) {
  if (p.epilogue == kEpilogueSwiglu) {
    // rows interleaved (gate, up): the neighbouring lane holds the other half of the pair
#pragma unroll
    for (uint32_t j = 0; j < kGroup; ++j) {
      const float other = __shfl_xor_sync(0xffffffffu, v[j], 1);
      const uint32_t m = g + j;
      if ((lane & 1u) == 0 && row + 1u < p.rows && m < p.tokens)
        p.out_bf16[static_cast<uint64_t>(m) * (p.rows / 2u) + row / 2u] = f32_to_bf16_bits(silu(v[j]) * other);
    }
  } else if (row < p.rows) {
#pragma unroll
    for (uint32_t j = 0; j < kGroup; ++j) {
      const uint32_t m = g + j;
      if (m < p.tokens) {
        const uint64_t at = static_cast<uint64_t>(m) * p.rows + row;
        p.out_f32[at] = p.resid_in != nullptr ? v[j] + __ldcg(p.resid_in + at) : v[j];
      }
    }
  }
}

// Finishes the row tiles that more than one block of gemm_tc_kernel contributed to.  Grid (row
// tiles, n_pad / 16), block (128 rows, 4 groups of 4 tokens): a thread adds the partials of its four
// values in ascending block order (bit-stable) with the loads of up to eight contributors in flight
// together, and runs the epilogue.  Blocks of tiles that one projection block covered alone (it has
// written them itself) leave at once.
constexpr uint32_t kFixupMaxListed = 320;  // contributors whose slots are looked up once, in shared memory
constexpr uint32_t kFixupBatch = 8;

__device__ __forceinline__ void fixup_epilogue(const GemmKernelParams &p, const float4 &v, uint32_t row, uint32_t m0) {
  const float vals[4] = {v.x, v.y, v.z, v.w};
  if (p.epilogue == kEpilogueSwiglu) {
    // rows interleaved (gate, up): the neighbouring lane holds the other half of the pair
#pragma unroll
    for (uint32_t j = 0; j < 4u; ++j) {
      const float other = __shfl_xor_sync(0xffffffffu, vals[j], 1);
      const uint32_t m = m0 + j;
      if ((threadIdx.x & 1u) == 0 && row + 1u < p.rows && m < p.tokens)
        p.out_bf16[static_cast<uint64_t>(m) * (p.rows / 2u) + row / 2u] = f32_to_bf16_bits(silu(vals[j]) * other);
    }
  } else if (row < p.rows) {
#pragma unroll
    for (uint32_t j = 0; j < 4u; ++j) {
      const uint32_t m = m0 + j;
      if (m < p.tokens) {
        const uint64_t at = static_cast<uint64_t>(m) * p.rows + row;
        p.out_f32[at] = p.resid_in != nullptr ? vals[j] + __ldcg(p.resid_in + at) : vals[j];
      }
    }
  }
}

__global__ void __launch_bounds__(4 * kTileRows) gemm_fixup_kernel(GemmKernelParams p, uint32_t gemm_blocks) {
  __shared__ uint32_t range[2];
  __shared__ uint32_t slots[kFixupMaxListed];
  pdl_trigger();
  const Partition part = make_partition(p.rows, p.cols, gemm_blocks);
  const uint32_t tile = blockIdx.x;
  const uint32_t tid = threadIdx.y * blockDim.x + threadIdx.x;
  if (tid == 0) {
    range[0] = first_block_of_tile(part, tile);
    range[1] = last_block_of_tile(part, tile);
  }
  __syncthreads();
  const uint32_t lo = range[0], hi = range[1];
  if (lo == hi) return;  // one block covered the tile: nothing to add
  const uint32_t count = hi - lo + 1u;
  const bool listed = count <= kFixupMaxListed;
  if (listed) {
    for (uint32_t i = tid; i < count; i += blockDim.x * blockDim.y) slots[i] = partial_slot(part, lo + i, tile);
  }
  __syncthreads();
  pdl_wait();  // the partials come from the projection launch just before
  const uint32_t row_in_tile = threadIdx.x;
  const uint32_t m0 = blockIdx.y * kGroup + 4u * threadIdx.y;
  const uint64_t slot_floats = static_cast<uint64_t>(p.n_pad) * kTileRows;
  const float *base = p.workspace + static_cast<uint64_t>(m0) * kTileRows + row_in_tile;
  float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  for (uint32_t q = 0; q < count; q += kFixupBatch) {
    float4 x[kFixupBatch];
#pragma unroll
    for (uint32_t u = 0; u < kFixupBatch; ++u) {
      const uint32_t i = q + u < count ? q + u : count - 1u;
      const uint32_t slot = listed ? slots[i] : partial_slot(part, lo + i, tile);
      const float *src = base + slot * slot_floats;  // four tokens of this row: 128 rows apart
      x[u] = make_float4(__ldcg(src), __ldcg(src + kTileRows), __ldcg(src + 2u * kTileRows), __ldcg(src + 3u * kTileRows));
    }
#pragma unroll
    for (uint32_t u = 0; u < kFixupBatch; ++u) {
      if (q + u >= count) break;
      if (q + u == 0) {
        v = x[u];
      } else {
        v.x += x[u].x;
        v.y += x[u].y;
        v.z += x[u].z;
        v.w += x[u].w;
      }
    }
  }
  fixup_epilogue(p, v, tile * kTileRows + row_in_tile, m0);
}

__global__ void __launch_bounds__(kGemmThreads, 2)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               GemmKernelParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // the ring must start on a 1024-byte boundary (the swizzle pattern is a function of the address)
  uint8_t *ring = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t{1023});
  const uint32_t x_tile_bytes = p.n_pad * kSliceK * 2u;
  const uint32_t stage_bytes = kATileBytes + x_tile_bytes;
  GemmShared &sh = *reinterpret_cast<GemmShared *>(ring + p.stages * stage_bytes);
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  volatile uint32_t *abort = &sh.abort;

  pdl_trigger();
  const Partition part = make_partition(p.rows, p.cols, gridDim.x);
  const uint64_t run_begin = part.begin(blockIdx.x), run_end = part.end(blockIdx.x);
  // The weights do not depend on the previous kernel: the first ring-full of weight tiles is
  // requested by thread 0 as soon as its barriers exist — before the block's set-up barrier and
  // before the dependency wait; the activation tiles of the same stages follow after that wait.
  const uint64_t run_len = run_end - run_begin;
  const uint32_t head = run_len < p.stages ? static_cast<uint32_t>(run_len) : p.stages;
  if (threadIdx.x == 0) {
    stamp_any(p.stamps, kStampEntry);
    for (uint32_t s = 0; s < p.stages; ++s) {
      mbar_init(&sh.full[s], 1);
      mbar_init(&sh.empty[s], 1);
    }
    for (uint32_t a = 0; a < 2; ++a) {
      mbar_init(&sh.acc_full[a], 1);
      mbar_init(&sh.acc_empty[a], kEpilogueThreads);
    }
    sh.abort = 0;
    mbar_init_fence();
    const uint64_t w_policy = l2_evict_first_policy();  // weights are read once
    SegmentWalk walk{run_begin, run_end, part.slices};
    Segment seg;
    uint32_t i = 0;
    while (i < head && walk.next(&seg)) {
      for (uint32_t c = seg.slice_begin; c < seg.slice_end && i < head; ++c, ++i) {
        mbar_arrive_expect_tx(&sh.full[i], stage_bytes);
        tma_load_2d(ring + i * stage_bytes, &map_w, c * kSliceK, seg.tile * kTileRows, &sh.full[i], w_policy);
      }
    }
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&sh.tmem_base)),
                 "r"(p.tmem_columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = sh.tmem_base;
  const uint32_t acc_stride = p.tmem_columns / 2u;

  if (warp == 0) {
    // ---------------- producer ----------------
    if (lane == 0) {
      const uint64_t w_policy = l2_evict_first_policy();  // weights are read once
      const uint64_t x_policy = l2_evict_last_policy();   // every block re-reads the activation block
      SegmentWalk walk{run_begin, run_end, part.slices};
      Segment seg;
      uint32_t issued = 0;
      pdl_wait();
      bool ok = true;
      while (ok && walk.next(&seg)) {
        for (uint32_t c = seg.slice_begin; c < seg.slice_end; ++c, ++issued) {
          const uint32_t s = issued % p.stages;
          uint8_t *stage = ring + s * stage_bytes;
          if (issued >= head) {
            if (!abortable_wait(&sh.empty[s], ((issued / p.stages) & 1u) ^ 1u, abort, p.error_word)) {
              ok = false;
              break;
            }
            mbar_arrive_expect_tx(&sh.full[s], stage_bytes);
            tma_load_2d(stage, &map_w, c * kSliceK, seg.tile * kTileRows, &sh.full[s], w_policy);
          }
          tma_load_2d(stage + kATileBytes, &map_x, c * kSliceK, 0, &sh.full[s], x_policy);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    pdl_wait();
    if (lane == 0) {
      const uint32_t idesc = instr_desc_bf16(p.n_pad);
      SegmentWalk walk{run_begin, run_end, part.slices};
      Segment seg;
      uint32_t consumed = 0, segment_index = 0;
      bool ok = true;
      while (ok && walk.next(&seg)) {
        const uint32_t acc = segment_index & 1u;
        // the epilogue must have drained this accumulator buffer (two segments ago)
        if (!abortable_wait(&sh.acc_empty[acc], ((segment_index >> 1) & 1u) ^ 1u, abort, p.error_word)) break;
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + acc * acc_stride;
        for (uint32_t c = seg.slice_begin; c < seg.slice_end; ++c, ++consumed) {
          const uint32_t s = consumed % p.stages;
          if (!abortable_wait(&sh.full[s], (consumed / p.stages) & 1u, abort, p.error_word)) {
            ok = false;
            break;
          }
          if (consumed == 0) stamp_any(p.stamps, kStampAfterWait);
          tcgen05_fence_after();
          const uint8_t *stage = ring + s * stage_bytes;
          const uint64_t desc_a = kmajor_sw128_desc(stage);
          const uint64_t desc_b = kmajor_sw128_desc(stage + kATileBytes);
#pragma unroll
          for (uint32_t k = 0; k < kSliceK / kUmmaK; ++k) {
            // 16 bf16 = 32 bytes further along the row: +2 in the 16-byte units of the descriptor
            tcgen05_mma_f16(tmem_d, desc_a + 2ull * k, desc_b + 2ull * k, idesc, (c != seg.slice_begin || k != 0) ? 1u : 0u);
          }
          tcgen05_commit(&sh.empty[s]);  // the stage is free once these MMAs have read it
        }
        if (ok) tcgen05_commit(&sh.acc_full[acc]);
        ++segment_index;
      }
      stamp_any(p.stamps, kStampAfterPrologue);  // every MMA of this block issued and committed
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    pdl_wait();
    const uint32_t quarter = warp & 3u;                 // the TMEM lanes this warp may read
    const uint32_t row_in_tile = quarter * 32u + lane;  // accumulator row = TMEM lane
    SegmentWalk walk{run_begin, run_end, part.slices};
    Segment seg;
    uint32_t segment_index = 0;
    const uint64_t slot_floats = static_cast<uint64_t>(p.n_pad) * kTileRows;
    while (walk.next(&seg)) {
      const uint32_t acc = segment_index & 1u;
      if (!abortable_wait(&sh.acc_full[acc], (segment_index >> 1) & 1u, abort, p.error_word)) break;
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + acc * acc_stride + ((quarter * 32u) << 16);
      const bool whole = seg.slice_begin == 0 && seg.slice_end == part.slices;
      if (!whole) {
        // partial accumulator -> this block's workspace slot, [token][row] (a warp's 32 rows of one token
        // are one 128-byte line); gemm_fixup_kernel, or the caller's next kernel, finishes the tile
        float *slot = p.workspace + partial_slot(part, blockIdx.x, seg.tile) * slot_floats + row_in_tile;
        for (uint32_t g = 0; g < p.n_pad; g += kGroup) {
          float v[kGroup];
          tmem_load16(taddr + g, v);
#pragma unroll
          for (uint32_t j = 0; j < kGroup; ++j) slot[static_cast<uint64_t>(g + j) * kTileRows] = v[j];
        }
      } else {
        const uint32_t row = seg.tile * kTileRows + row_in_tile;
        for (uint32_t g = 0; g < p.n_pad; g += kGroup) {
          float v[kGroup];
          tmem_load16(taddr + g, v);
          tile_epilogue(p, v, row, g, lane);
        }
      }
      tcgen05_fence_before();
      mbar_arrive(&sh.acc_empty[acc]);
      ++segment_index;
    }
  }
  // ---- teardown: nothing of this block may still be in flight when its memory is released ----
  tcgen05_fence_before();
  __syncthreads();
  if (sh.abort != 0u && threadIdx.x == 0) {
    // a wait gave up: give the copies that were issued one more bounded chance to land
    for (uint32_t s = 0; s < p.stages; ++s) {
      mbar_wait_bounded(&sh.full[s], 0);
      mbar_wait_bounded(&sh.full[s], 1);
    }
  }
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_columns) : "memory");
    if (lane == 0) stamp_any(p.stamps, kStampExit);
  }
}

// ---- host side ----
PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *entry = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &status) == cudaSuccess &&
        status == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(entry);
  });
  return fn;
}

// bf16 [outer][inner] row-major, boxes of 64 x box_outer elements, 128-byte swizzle; rows beyond
// `outer` read as zero.
bool make_map(CUtensorMap *map, const uint16_t *base, uint64_t inner, uint64_t outer, uint32_t box_outer) {
  PFN_cuTensorMapEncodeTiled_v12000 encode = tensor_map_encoder();
  if (encode == nullptr) return false;
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {inner * 2u};
  const cuuint32_t box[2] = {kSliceK, box_outer};
  const cuuint32_t elem_strides[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t *>(base), dims, strides, box,
                elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

uint32_t padded_tokens(uint32_t tokens) { return (tokens + 15u) & ~15u; }

bool two_blocks_per_sm(uint32_t n_pad) { return n_pad <= kSmallBlockTokens; }

uint32_t stages_for(uint32_t n_pad) {
  const uint32_t stage_bytes = kATileBytes + n_pad * kSliceK * 2u;
  const uint32_t budget = two_blocks_per_sm(n_pad) ? 108u * 1024u : 200u * 1024u;
  uint32_t stages = budget / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  return stages;
}

uint32_t tmem_columns_for(uint32_t n_pad) { return two_blocks_per_sm(n_pad) ? 128u : 512u; }

uint32_t gemm_smem_bytes(uint32_t n_pad, uint32_t stages) {
  return 1024u + stages * (kATileBytes + n_pad * kSliceK * 2u) + static_cast<uint32_t>(sizeof(GemmShared)) + 64u;
}

// Two runs per SM whatever the block size, so that the split points — and with them the order in
// which a row's partial sums are added — depend on the matrix shape alone: a token gets the same
// bits in a block of 2 and in a block of 256.  Blocks too large for two per SM run the grid in two waves.
uint32_t gemm_blocks(uint32_t rows, uint32_t cols, uint32_t sm_count) {
  const Partition p = make_partition(rows, cols, 1);
  const uint32_t want = 2u * sm_count;
  // Between one and two row tiles per SM (gate/up of the 8B shapes: 192 tiles): one block per tile.
  // Nothing is split, so no fix-up launch follows; the SMs that hold two blocks stream twice the
  // bytes of the others, which the memory system evens out better than a second launch costs.
  if (p.tiles >= sm_count && p.tiles <= want) return p.tiles;
  return p.total < want ? static_cast<uint32_t>(p.total) : want;
}

}  // namespace

bool tensor_map_available() { return tensor_map_encoder() != nullptr; }

bool encode_bf16_map_2d(void *map, const uint16_t *base, uint64_t inner, uint64_t outer, uint32_t box_inner,
                        uint32_t box_outer) {
  PFN_cuTensorMapEncodeTiled_v12000 encode = tensor_map_encoder();
  if (encode == nullptr || box_inner != kSliceK) return false;
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {inner * 2u};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t elem_strides[2] = {1, 1};
  return encode(static_cast<CUtensorMap *>(map), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t *>(base), dims,
                strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool gemm_tc_eligible(const GemmParams &g) {
  return g.tokens >= 1 && g.tokens <= kGemmMaxTokens && g.cols % kSliceK == 0 && g.cols != 0 && g.rows != 0 &&
         reinterpret_cast<uintptr_t>(g.weight) % 16u == 0 && reinterpret_cast<uintptr_t>(g.x) % 16u == 0 &&
         (g.epilogue != kEpilogueSwiglu || g.rows % 2u == 0) &&
         (g.epilogue == kEpilogueStore || g.epilogue == kEpilogueSwiglu);
}

uint64_t gemm_tc_workspace_bytes(uint32_t tokens, uint32_t sm_count) {
  // two partial accumulators per thread block of the 2 x sm_count grid
  return 2ull * (2ull * sm_count) * padded_tokens(tokens) * kTileRows * sizeof(float);
}

uint32_t gemm_tc_ticket_count(uint32_t rows) { return (rows + kTileRows - 1u) / kTileRows; }

cudaError_t configure_gemm_tc_kernel() {
  return cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
}

cudaError_t launch_gemm_tc(cudaStream_t stream, const GemmParams &g, uint32_t sm_count) {
  if (!gemm_tc_eligible(g) || g.workspace == nullptr) return cudaErrorInvalidValue;
  GemmKernelParams p{};
  p.rows = g.rows;
  p.cols = g.cols;
  p.tokens = g.tokens;
  p.n_pad = padded_tokens(g.tokens);
  p.stages = stages_for(p.n_pad);
  p.tmem_columns = tmem_columns_for(p.n_pad);
  p.epilogue = g.epilogue;
  p.resid_in = g.resid_in;
  p.out_f32 = g.out_f32;
  p.out_bf16 = g.out_bf16;
  p.workspace = g.workspace;
  p.tickets = g.tickets;
  p.error_word = g.error_word;
  p.stamps = g.stamps;
  CUtensorMap map_w, map_x;
  if (!make_map(&map_w, g.weight, g.cols, g.rows, kTileRows) || !make_map(&map_x, g.x, g.cols, g.tokens, p.n_pad))
    return cudaErrorNotSupported;
  const uint32_t blocks = gemm_blocks(g.rows, g.cols, sm_count);
  cudaError_t err = launch_with_pdl(gemm_tc_kernel, dim3(blocks), dim3(kGemmThreads), gemm_smem_bytes(p.n_pad, p.stages),
                                    stream, g.pdl != 0, map_w, map_x, p);
  if (err != cudaSuccess) return err;
  // the fix-up launch follows only when some tile is shared between blocks (a block whose run
  // begins inside a tile)
  const Partition part = make_partition(g.rows, g.cols, blocks);
  bool split = false;
  for (uint32_t b = 0; b < blocks && !split; ++b) split = part.begin(b) % part.slices != 0;
  if (!split) return cudaSuccess;
  return launch_with_pdl(gemm_fixup_kernel, dim3(part.tiles, p.n_pad / kGroup), dim3(kTileRows, 4), 0, stream, true, p,
                         blocks);
}

}  // namespace nb
