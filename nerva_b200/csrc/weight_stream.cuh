// Weight-streaming matrix-vector core.
//
// A projection y[n] = sum_k W[n][k] * x[k] at one token is pure HBM streaming:
// every weight byte is read once and used once.  Each warp therefore owns a
// private ring of shared-memory slots that it keeps filled with 8 KiB pieces
// ("chunks") of its own rows through 1-D bulk TMA copies, and drains them with
// 128-bit shared loads, fp32 FMAs and one warp-shuffle reduction per row.  There
// is no block-level synchronisation in the loop: a warp waits only on the
// mbarrier of the slot it is about to read, and refills that slot as soon as it
// has read it.  With 8 warps x 3 slots x 8 KiB an SM keeps up to 192 KiB of
// weight reads in flight.
//
// Rows are not split across warps, the chunk order inside a row is fixed and
// the lane->column map is fixed, so results are bit-identical run to run.
#pragma once

#include "common.cuh"

namespace nb {

constexpr uint32_t kStreamWarps = 8;
constexpr uint32_t kStreamThreads = kStreamWarps * 32;
constexpr uint32_t kStreamSlots = 3;
constexpr uint32_t kChunkBytes = 8192;
constexpr uint32_t kChunkElems = kChunkBytes / 2;
constexpr uint32_t kRingBytes = kStreamWarps * kStreamSlots * kChunkBytes;

// How the rows of one projection are cut into chunks.
struct StreamShape {
  uint32_t cols;             // K, a multiple of 8
  uint32_t rows_per_chunk;   // whole rows per chunk (cols <= kChunkElems), else 1
  uint32_t chunks_per_row;   // pieces of one row (cols > kChunkElems), else 1
  uint32_t rows_per_item;    // consecutive rows owned by one warp (2 keeps gate/up pairs together)
  uint32_t chunks_per_item;
};

__host__ __device__ inline StreamShape make_stream_shape(uint32_t cols, bool row_pairs) {
  StreamShape s;
  s.cols = cols;
  if (cols <= kChunkElems) {
    uint32_t rpc = kChunkElems / cols;
    if (row_pairs && rpc > 1) rpc &= ~1u;
    s.rows_per_chunk = rpc;
    s.chunks_per_row = 1;
    s.rows_per_item = rpc > 1 ? rpc : (row_pairs ? 2u : 1u);
    s.chunks_per_item = s.rows_per_item / rpc;
  } else {
    s.rows_per_chunk = 1;
    s.chunks_per_row = (cols + kChunkElems - 1) / kChunkElems;
    s.rows_per_item = row_pairs ? 2u : 1u;
    s.chunks_per_item = s.rows_per_item * s.chunks_per_row;
  }
  return s;
}

// Rows [begin, end) of block `block` out of `blocks`, in units of `unit` rows.
__host__ __device__ inline void block_row_range(uint32_t rows, uint32_t unit, uint32_t block,
                                                uint32_t blocks, uint32_t *begin, uint32_t *end) {
  const uint64_t units = rows / unit;
  *begin = static_cast<uint32_t>(units * block / blocks) * unit;
  *end = static_cast<uint32_t>(units * (block + 1) / blocks) * unit;
}

// Per-warp ring state.  Every field is warp-uniform.
struct WarpStream {
  uint8_t *ring;     // kStreamSlots * kChunkBytes of shared memory
  uint64_t *bars;    // kStreamSlots mbarriers
  uint32_t issued;   // chunks issued since the barriers were initialised
  uint32_t consumed; // chunks consumed
  bool dead;         // a wait timed out: stop issuing and waiting, finish the loop
  uint32_t drain_from, drain_to;  // chunks that were in flight when the wait timed out
};

// Call with all threads of the block; `bars` points at kStreamWarps*kStreamSlots barriers.
__device__ inline void stream_init(WarpStream &ws, uint8_t *ring_base, uint64_t *bars) {
  const uint32_t warp = threadIdx.x >> 5;
  ws.ring = ring_base + warp * kStreamSlots * kChunkBytes;
  ws.bars = bars + warp * kStreamSlots;
  ws.issued = 0;
  ws.consumed = 0;
  ws.dead = false;
  ws.drain_from = 0;
  ws.drain_to = 0;
  if ((threadIdx.x & 31u) == 0) {
    for (uint32_t s = 0; s < kStreamSlots; ++s) mbar_init(&ws.bars[s], 1);
    mbar_init_fence();
  }
  __syncwarp();
}

// One projection's work list for one warp.
struct StreamJob {
  const uint16_t *weight;  // row-major [rows][cols] bf16
  StreamShape shape;
  uint32_t row_begin, row_end;  // this block's rows
  uint32_t chunks;              // chunk slots this warp walks (some at the tail may be empty)
};

__device__ inline StreamJob make_stream_job(const uint16_t *weight, StreamShape shape,
                                            uint32_t row_begin, uint32_t row_end) {
  StreamJob job;
  job.weight = weight;
  job.shape = shape;
  job.row_begin = row_begin;
  job.row_end = row_end;
  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t rows = row_end - row_begin;
  const uint32_t items = (rows + shape.rows_per_item - 1) / shape.rows_per_item;
  const uint32_t mine = items > warp ? (items - warp + kStreamWarps - 1) / kStreamWarps : 0;
  job.chunks = mine * shape.chunks_per_item;
  return job;
}

struct ChunkDesc {
  uint32_t row0, rows, k0, klen;
  bool last_of_row;
};

// Chunk `j` of this warp's list.  Returns false for an empty tail chunk.
__device__ __forceinline__ bool stream_chunk(const StreamJob &job, uint32_t j, ChunkDesc &d) {
  const StreamShape &s = job.shape;
  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t item_local = j / s.chunks_per_item;
  const uint32_t c = j - item_local * s.chunks_per_item;
  const uint32_t base_row = job.row_begin + (warp + item_local * kStreamWarps) * s.rows_per_item;
  if (s.chunks_per_row == 1) {
    d.row0 = base_row + c * s.rows_per_chunk;
    d.k0 = 0;
    d.klen = s.cols;
    d.last_of_row = true;
    if (d.row0 >= job.row_end) return false;
    const uint32_t left = job.row_end - d.row0;
    d.rows = left < s.rows_per_chunk ? left : s.rows_per_chunk;
  } else {
    const uint32_t r = c / s.chunks_per_row;
    const uint32_t kc = c - r * s.chunks_per_row;
    d.row0 = base_row + r;
    d.k0 = kc * kChunkElems;
    d.klen = s.cols - d.k0 < kChunkElems ? s.cols - d.k0 : kChunkElems;
    d.last_of_row = kc + 1 == s.chunks_per_row;
    d.rows = 1;
    if (d.row0 >= job.row_end) return false;
  }
  return true;
}

// Issues chunks from cursor `*next` while ring slots are free.
__device__ __forceinline__ void stream_fill(WarpStream &ws, const StreamJob &job, uint32_t *next) {
  if (ws.dead) return;
  while (*next < job.chunks && ws.issued - ws.consumed < kStreamSlots) {
    ChunkDesc d;
    const uint32_t j = (*next)++;
    if (!stream_chunk(job, j, d)) continue;
    const uint32_t slot = ws.issued % kStreamSlots;
    if ((threadIdx.x & 31u) == 0) {
      const uint32_t bytes = d.rows * d.klen * 2u;
      const uint16_t *src = job.weight + static_cast<uint64_t>(d.row0) * job.shape.cols + d.k0;
      fence_proxy_async();
      mbar_arrive_expect_tx(&ws.bars[slot], bytes);
      tma_load_1d(ws.ring + slot * kChunkBytes, src, bytes, &ws.bars[slot]);
    }
    ws.issued += 1;
  }
}

// dot of 8 bf16 weights with 8 bf16 activations, fp32.
__device__ __forceinline__ float dot8(const uint4 &w, const uint4 &x, float acc) {
  acc = fmaf(bf16x2_lo(w.x), bf16x2_lo(x.x), acc);
  acc = fmaf(bf16x2_hi(w.x), bf16x2_hi(x.x), acc);
  acc = fmaf(bf16x2_lo(w.y), bf16x2_lo(x.y), acc);
  acc = fmaf(bf16x2_hi(w.y), bf16x2_hi(x.y), acc);
  acc = fmaf(bf16x2_lo(w.z), bf16x2_lo(x.z), acc);
  acc = fmaf(bf16x2_hi(w.z), bf16x2_hi(x.z), acc);
  acc = fmaf(bf16x2_lo(w.w), bf16x2_lo(x.w), acc);
  acc = fmaf(bf16x2_hi(w.w), bf16x2_hi(x.w), acc);
  return acc;
}

// Streams one job.  `x` is the bf16 activation vector in shared memory
// (16-byte aligned, job.shape.cols elements).  `epi.row(row, value)` is called
// by every lane of the warp (value is the full dot product in all lanes) once
// per finished row, rows in ascending order within the warp.
// `next`/`carry` let a caller that pre-issued chunks (before its activations
// were ready) continue the same job.
template <class Epilogue>
__device__ __forceinline__ void stream_consume(WarpStream &ws, const StreamJob &job,
                                               uint32_t *next, const uint16_t *x, Epilogue &epi,
                                               uint32_t *error_word) {
  const uint32_t lane = threadIdx.x & 31u;
  float acc0 = 0.0f, acc1 = 0.0f, acc2 = 0.0f, acc3 = 0.0f;
  for (uint32_t j = 0; j < job.chunks; ++j) {
    ChunkDesc d;
    if (!stream_chunk(job, j, d)) continue;
    stream_fill(ws, job, next);
    const uint32_t slot = ws.consumed % kStreamSlots;
    const uint32_t parity = (ws.consumed / kStreamSlots) & 1u;
    if (!ws.dead && !mbar_wait_bounded(&ws.bars[slot], parity)) {
      ws.dead = true;
      ws.drain_from = ws.consumed;
      ws.drain_to = ws.issued;
      report_error(error_word, kErrTmaWaitTimeout);
    }
    const uint8_t *chunk = ws.ring + slot * kChunkBytes;
    const uint8_t *xk = reinterpret_cast<const uint8_t *>(x) + d.k0 * 2u;
    const uint32_t row_bytes = d.klen * 2u;
    for (uint32_t r = 0; r < d.rows; ++r) {
      const uint8_t *wrow = chunk + r * row_bytes;
      uint32_t off = lane * 16u;
      // four independent accumulators, 1024 B of the row per step
      for (; off + 3u * 512u < row_bytes; off += 4u * 512u) {
        const uint4 w0 = lds128(wrow + off), x0 = lds128(xk + off);
        const uint4 w1 = lds128(wrow + off + 512u), x1 = lds128(xk + off + 512u);
        const uint4 w2 = lds128(wrow + off + 1024u), x2 = lds128(xk + off + 1024u);
        const uint4 w3 = lds128(wrow + off + 1536u), x3 = lds128(xk + off + 1536u);
        acc0 = dot8(w0, x0, acc0);
        acc1 = dot8(w1, x1, acc1);
        acc2 = dot8(w2, x2, acc2);
        acc3 = dot8(w3, x3, acc3);
      }
      for (; off < row_bytes; off += 512u) {
        acc0 = dot8(lds128(wrow + off), lds128(xk + off), acc0);
      }
      if (d.last_of_row) {
        const float total = warp_sum((acc0 + acc1) + (acc2 + acc3));
        epi.row(d.row0 + r, total);
        acc0 = acc1 = acc2 = acc3 = 0.0f;
      }
    }
    __syncwarp();
    ws.consumed += 1;
  }
}

// After a timeout: give copies still in flight one more bounded chance to land
// before the block's shared memory is released.
__device__ inline void stream_drain(WarpStream &ws) {
  if (!ws.dead) return;
  for (uint32_t c = ws.drain_from; c < ws.drain_to; ++c) {
    mbar_wait_bounded(&ws.bars[c % kStreamSlots], (c / kStreamSlots) & 1u);
  }
}

}  // namespace nb
