// Weight-streaming matrix-vector core.
//
// A projection y[n] = sum_k W[n][k] * x[k] at one token is pure HBM streaming:
// every weight byte is read once and used once.  The rows of a projection are
// dealt to thread blocks as equal contiguous row ranges, and inside a block the
// BYTES of that range are dealt to the warps as equal contiguous byte ranges
// (cut at 512-byte lane sweeps, not at row boundaries), so every warp of the
// grid streams the same amount of memory whatever the shape.  Each warp owns a
// private ring of shared-memory slots that it keeps filled with pieces ("chunks",
// at most kChunkBytes, never crossing a row end) of its range through 1-D bulk
// TMA copies, and drains them with 128-bit shared loads and fp32 FMAs.  There is
// no block-level synchronisation in the loop: a warp waits only on the mbarrier
// of the slot it is about to read and refills that slot as soon as it has read it.
//
// The chunk list runs ACROSS projections (a job list): weights do not depend on
// activations, so the issue side of a ring runs ahead into the next projection
// while the block is still normalising, attending or waiting at a grid barrier.
//
// A row that lies inside one warp's range is reduced by that warp and its total
// goes to the block's row-total buffer in shared memory.  A row cut by a range
// boundary leaves one partial per warp in that warp's two "edge" records.  After
// the block has synchronised, stream_finish() adds the edge partials to the
// totals in ascending warp order, so results do not depend on timing and are
// bit-identical run to run.
#pragma once

#include "common.cuh"

namespace nb {

#ifndef NERVA_STREAM_WARPS
#define NERVA_STREAM_WARPS 8
#endif
#ifndef NERVA_STREAM_SLOTS
#define NERVA_STREAM_SLOTS 3
#endif
#ifndef NERVA_CHUNK_BYTES
#define NERVA_CHUNK_BYTES 8192
#endif
constexpr uint32_t kStreamWarps = NERVA_STREAM_WARPS;
constexpr uint32_t kStreamThreads = kStreamWarps * 32;
constexpr uint32_t kStreamSlots = NERVA_STREAM_SLOTS;
constexpr uint32_t kChunkBytes = NERVA_CHUNK_BYTES;
constexpr uint32_t kRingBytes = kStreamWarps * kStreamSlots * kChunkBytes;
constexpr uint32_t kSweepBytes = 512;  // 32 lanes x 16 bytes
static_assert(kChunkBytes % (4 * kSweepBytes) == 0, "a chunk is a whole number of 4-sweep steps");
constexpr uint32_t kNoRow = 0xffffffffu;

struct JobDesc {
  const uint16_t *weight;  // [rows][cols] bf16 row-major, 16-byte aligned, cols % 8 == 0
  uint32_t rows, cols;
  uint32_t unit;           // rows are dealt to blocks in multiples of `unit` (2 keeps gate/up pairs together)
  uint32_t whole;          // non-zero: the job belongs to this block alone (its list was built per block):
                           // all `rows` are this block's, nothing is dealt
};

// Rows [begin, end) of block `block` out of `blocks`, in units of `unit` rows.
__host__ __device__ inline void block_row_range(uint32_t rows, uint32_t unit, uint32_t block,
                                                uint32_t blocks, uint32_t *begin, uint32_t *end) {
  const uint64_t units = rows / unit;
  *begin = static_cast<uint32_t>(units * block / blocks) * unit;
  *end = static_cast<uint32_t>(units * (block + 1) / blocks) * unit;
}
__host__ __device__ inline uint32_t max_rows_per_block(uint32_t rows, uint32_t unit, uint32_t blocks) {
  const uint32_t units = rows / unit;
  return ((units + blocks - 1) / blocks) * unit;
}

// One warp's share of one job: bytes [begin, end) of the block's row range,
// offsets relative to the first byte of the block's first row.
struct WarpJob {
  const uint8_t *base;   // first byte of the block's first row
  uint32_t row_bytes;
  uint32_t begin, end;
};

__device__ __forceinline__ WarpJob warp_job(const JobDesc &d) {
  uint32_t row_begin = 0, row_end = d.rows;
  if (d.whole == 0) block_row_range(d.rows, d.unit, blockIdx.x, gridDim.x, &row_begin, &row_end);
  WarpJob j;
  j.row_bytes = d.cols * 2u;
  j.base = reinterpret_cast<const uint8_t *>(d.weight) + static_cast<uint64_t>(row_begin) * j.row_bytes;
  const uint32_t warp = threadIdx.x >> 5;
  if (j.row_bytes % kSweepBytes == 0) {
    // cut the block's bytes into equal runs of whole 512-byte lane sweeps
    const uint32_t sweeps = (row_end - row_begin) * (j.row_bytes / kSweepBytes);
    j.begin = static_cast<uint32_t>(static_cast<uint64_t>(sweeps) * warp / kStreamWarps) * kSweepBytes;
    j.end = static_cast<uint32_t>(static_cast<uint64_t>(sweeps) * (warp + 1) / kStreamWarps) * kSweepBytes;
  } else {
    // rows that are not a whole number of sweeps are dealt whole
    const uint32_t rows = row_end - row_begin;
    j.begin = static_cast<uint32_t>(static_cast<uint64_t>(rows) * warp / kStreamWarps) * j.row_bytes;
    j.end = static_cast<uint32_t>(static_cast<uint64_t>(rows) * (warp + 1) / kStreamWarps) * j.row_bytes;
  }
  return j;
}

// A cursor walks a WarpJob chunk by chunk.
struct StreamCursor {
  uint32_t pos;      // byte offset of the next chunk
  uint32_t row_end;  // end byte of the row that contains pos
  uint32_t row;      // block-local index of that row
};
__device__ __forceinline__ StreamCursor cursor_at_start(const WarpJob &j) {
  StreamCursor c;
  c.pos = j.begin;
  c.row = j.begin / j.row_bytes;
  c.row_end = (c.row + 1u) * j.row_bytes;
  return c;
}
// Length of the chunk at the cursor, its position, the end of its row and the row's index;
// advances the cursor.
__device__ __forceinline__ uint32_t cursor_next(const WarpJob &j, StreamCursor &c, uint32_t *pos,
                                                uint32_t *row_end, uint32_t *row = nullptr) {
  uint32_t len = kChunkBytes;
  if (c.row_end - c.pos < len) len = c.row_end - c.pos;
  if (j.end - c.pos < len) len = j.end - c.pos;
  *pos = c.pos;
  *row_end = c.row_end;
  if (row != nullptr) *row = c.row;
  c.pos += len;
  if (c.pos == c.row_end) {
    c.row_end += j.row_bytes;
    c.row += 1u;
  }
  return len;
}

struct EdgeRecord {
  uint32_t row;  // block-local row, kNoRow when unused
  float value;
};

// Shared-memory bookkeeping of a block's streams.
struct StreamShared {
  uint64_t bars[kStreamWarps * kStreamSlots];
  EdgeRecord edge[kStreamWarps][2];
};

// Per-warp state.  Every field is warp-uniform.
struct RowStream {
  uint8_t *ring;
  uint64_t *bars;
  const JobDesc *jobs;
  uint32_t job_count;
  uint32_t issued, consumed;  // chunks
  bool dead;
  uint32_t drain_from, drain_to;
  uint32_t issue_job;
  WarpJob issue;
  StreamCursor issue_cursor;
  uint64_t policy;  // L2 evict-first: weights are read once per step
};

__device__ inline void stream_init(RowStream &rs, uint8_t *ring_base, StreamShared &sh,
                                   const JobDesc *jobs, uint32_t job_count) {
  const uint32_t warp = threadIdx.x >> 5;
  rs.ring = ring_base + warp * kStreamSlots * kChunkBytes;
  rs.bars = sh.bars + warp * kStreamSlots;
  rs.jobs = jobs;
  rs.job_count = job_count;
  rs.issued = rs.consumed = 0;
  rs.dead = false;
  rs.drain_from = rs.drain_to = 0;
  rs.policy = l2_evict_first_policy();
  rs.issue_job = 0;
  if (job_count != 0) {
    rs.issue = warp_job(jobs[0]);
    rs.issue_cursor = cursor_at_start(rs.issue);
  }
  if ((threadIdx.x & 31u) == 0) {
    for (uint32_t s = 0; s < kStreamSlots; ++s) mbar_init(&rs.bars[s], 1);
    mbar_init_fence();
  }
  __syncwarp();
}

// Issues chunks, crossing into later jobs, while ring slots are free (at most `depth` in flight).
__device__ __forceinline__ void stream_fill(RowStream &rs, uint32_t depth = kStreamSlots) {
  if (rs.dead) return;
  while (rs.issue_job < rs.job_count && rs.issued - rs.consumed < depth) {
    if (rs.issue_cursor.pos >= rs.issue.end) {
      rs.issue_job += 1;
      if (rs.issue_job < rs.job_count) {
        rs.issue = warp_job(rs.jobs[rs.issue_job]);
        rs.issue_cursor = cursor_at_start(rs.issue);
      }
      continue;
    }
    uint32_t pos, row_end;
    const uint32_t len = cursor_next(rs.issue, rs.issue_cursor, &pos, &row_end);
    const uint32_t slot = rs.issued % kStreamSlots;
    if ((threadIdx.x & 31u) == 0) {
      mbar_arrive_expect_tx(&rs.bars[slot], len);
      tma_load_1d_hint(rs.ring + slot * kChunkBytes, rs.issue.base + pos, len, &rs.bars[slot], rs.policy);
    }
    rs.issued += 1;
  }
}

// Asks L2 for the `bytes` that follow the chunks already issued (the warp's own span of the
// current job only): the ring cannot hold more, but HBM can keep working while the block is
// busy with its prologue.
__device__ __forceinline__ void stream_prefetch_l2(const RowStream &rs, uint32_t bytes) {
  if (rs.dead || bytes == 0 || rs.issue_job >= rs.job_count || (threadIdx.x & 31u) != 0) return;
  const uint32_t pos = rs.issue_cursor.pos;
  if (pos >= rs.issue.end) return;
  uint32_t size = rs.issue.end - pos;
  if (size > bytes) size = bytes;
  size &= ~15u;
  if (size == 0) return;
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(rs.issue.base + pos), "r"(size) : "memory");
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

// Packed fp32 multiply-add (two lanes per instruction).
__device__ __forceinline__ float2 fma2(float a0, float a1, float b0, float b1, float2 c) {
  uint64_t a, b, cc, d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(a0), "f"(a1));
  asm("mov.b64 %0, {%1, %2};" : "=l"(b) : "f"(b0), "f"(b1));
  asm("mov.b64 %0, {%1, %2};" : "=l"(cc) : "f"(c.x), "f"(c.y));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(cc));
  float2 r;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(d));
  return r;
}
// dot of 8 bf16 weights with 8 fp32 activations, even elements into acc.x and odd ones into acc.y.
__device__ __forceinline__ float2 dot8_f32x2(const uint4 &w, const float4 &xa, const float4 &xb, float2 acc) {
  acc = fma2(bf16x2_lo(w.x), bf16x2_hi(w.x), xa.x, xa.y, acc);
  acc = fma2(bf16x2_lo(w.y), bf16x2_hi(w.y), xa.z, xa.w, acc);
  acc = fma2(bf16x2_lo(w.z), bf16x2_hi(w.z), xb.x, xb.y, acc);
  acc = fma2(bf16x2_lo(w.w), bf16x2_hi(w.w), xb.z, xb.w, acc);
  return acc;
}

// dot of 8 bf16 weights with 8 fp32 activations (the sparse-MoE path of the
// reference feeds unrounded activations to its mat-vec).
__device__ __forceinline__ float dot8_f32(const uint4 &w, const float4 &xa, const float4 &xb, float acc) {
  acc = fmaf(bf16x2_lo(w.x), xa.x, acc);
  acc = fmaf(bf16x2_hi(w.x), xa.y, acc);
  acc = fmaf(bf16x2_lo(w.y), xa.z, acc);
  acc = fmaf(bf16x2_hi(w.y), xa.w, acc);
  acc = fmaf(bf16x2_lo(w.z), xb.x, acc);
  acc = fmaf(bf16x2_hi(w.z), xb.y, acc);
  acc = fmaf(bf16x2_lo(w.w), xb.z, acc);
  acc = fmaf(bf16x2_hi(w.w), xb.w, acc);
  return acc;
}
// fp32 activations (XF32) sit in shared memory in two planes, so that the lanes of a warp read
// consecutive 16-byte pieces (a plain [cols] array would put a lane's two float4 32 bytes from the
// next lane's: a two-way bank conflict on every load): element i of a `cols`-wide vector is at
// xf32_index(i, cols) — the first four of every eight elements in plane A, the last four in plane B.
__host__ __device__ inline uint32_t xf32_index(uint32_t i, uint32_t cols) {
  return ((i & 4u) != 0 ? cols / 2u : 0u) + ((i >> 3) << 2) + (i & 3u);
}
// One 16-byte piece of weights at `wp + off` times the matching activations: bf16 at byte offset
// `off` of xp, or (XF32) the piece's two float4 at index off / 16 of the planes xa and xb.
template <bool XF32>
__device__ __forceinline__ float dot_piece(const uint8_t *wp, const uint8_t *xp, const float4 *xa, const float4 *xb,
                                           uint32_t off, float acc) {
  if (XF32) return dot8_f32(lds128(wp + off), xa[off / 16u], xb[off / 16u], acc);
  return dot8(lds128(wp + off), lds128(xp + off), acc);
}
__device__ __forceinline__ float2 dot_piece_x2(const uint8_t *wp, const float4 *xa, const float4 *xb, uint32_t off,
                                               float2 acc) {
  return dot8_f32x2(lds128(wp + off), xa[off / 16u], xb[off / 16u], acc);
}

// Consumes job `index` (jobs are consumed in order, each exactly once, by every
// warp of the block).  `x` is the bf16 activation vector in shared memory;
// row_total[r] (shared, one float per block-local row, zeroed by the caller
// before the block's previous synchronisation) receives the total of every row
// that lies wholly inside this warp's range; partial rows go to sh.edge.
// XF32: `x` points at fp32 activations instead of bf16 ones.
template <bool XF32 = false>
__device__ __forceinline__ void stream_consume(RowStream &rs, StreamShared &sh, uint32_t index,
                                               const void *x, float *row_total,
                                               uint32_t *error_word) {
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const WarpJob job = warp_job(rs.jobs[index]);
  StreamCursor cur = cursor_at_start(job);
  if (lane == 0) {
    sh.edge[warp][0].row = kNoRow;
    sh.edge[warp][1].row = kNoRow;
  }
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  uint32_t edges = 0;
  bool row_from_start = job.begin % job.row_bytes == 0;  // this warp has seen the current row from byte 0
  while (cur.pos < job.end) {
    uint32_t pos, row_end, row;
    const uint32_t len = cursor_next(job, cur, &pos, &row_end, &row);
    stream_fill(rs);
    const uint32_t slot = rs.consumed % kStreamSlots;
    const uint32_t parity = (rs.consumed / kStreamSlots) & 1u;
    if (!rs.dead && !mbar_wait_bounded(&rs.bars[slot], parity)) {
      rs.dead = true;
      rs.drain_from = rs.consumed;
      rs.drain_to = rs.issued;
      report_error(error_word, kErrTmaWaitTimeout);
    }
    const uint8_t *wp = rs.ring + slot * kChunkBytes + lane * 16u;
    const uint32_t row_offset = pos - (row_end - job.row_bytes);  // bytes into the row
    const uint8_t *xp = reinterpret_cast<const uint8_t *>(x) + row_offset + lane * 16u;
    if (XF32) {
      // planes A and B of the fp32 vector (xf32_index), at this lane's first piece of the chunk
      const float4 *xa = reinterpret_cast<const float4 *>(x) + row_offset / 16u + lane;
      const float4 *xb = xa + job.row_bytes / 16u;
      // packed multiply-adds: every accumulator splits into an even and an odd half for the chunk
      float2 a2[4] = {make_float2(acc[0], 0.0f), make_float2(acc[1], 0.0f), make_float2(acc[2], 0.0f),
                      make_float2(acc[3], 0.0f)};
      uint32_t off = 0;
      if (len == kChunkBytes) {
#pragma unroll
        for (uint32_t i = 0; i < kChunkBytes / kSweepBytes; i += 4) {
          a2[0] = dot_piece_x2(wp, xa, xb, (i + 0) * kSweepBytes, a2[0]);
          a2[1] = dot_piece_x2(wp, xa, xb, (i + 1) * kSweepBytes, a2[1]);
          a2[2] = dot_piece_x2(wp, xa, xb, (i + 2) * kSweepBytes, a2[2]);
          a2[3] = dot_piece_x2(wp, xa, xb, (i + 3) * kSweepBytes, a2[3]);
        }
        off = kChunkBytes;
      } else if (len == kChunkBytes / 2u) {
#pragma unroll
        for (uint32_t i = 0; i < kChunkBytes / kSweepBytes / 2u; i += 4) {
          a2[0] = dot_piece_x2(wp, xa, xb, (i + 0) * kSweepBytes, a2[0]);
          a2[1] = dot_piece_x2(wp, xa, xb, (i + 1) * kSweepBytes, a2[1]);
          a2[2] = dot_piece_x2(wp, xa, xb, (i + 2) * kSweepBytes, a2[2]);
          a2[3] = dot_piece_x2(wp, xa, xb, (i + 3) * kSweepBytes, a2[3]);
        }
        off = kChunkBytes / 2u;
      }
      for (; off + 4u * kSweepBytes <= len; off += 4u * kSweepBytes) {
        a2[0] = dot_piece_x2(wp, xa, xb, off, a2[0]);
        a2[1] = dot_piece_x2(wp, xa, xb, off + kSweepBytes, a2[1]);
        a2[2] = dot_piece_x2(wp, xa, xb, off + 2u * kSweepBytes, a2[2]);
        a2[3] = dot_piece_x2(wp, xa, xb, off + 3u * kSweepBytes, a2[3]);
      }
      for (; off + lane * 16u < len; off += kSweepBytes) a2[0] = dot_piece_x2(wp, xa, xb, off, a2[0]);
#pragma unroll
      for (uint32_t i = 0; i < 4; ++i) acc[i] = a2[i].x + a2[i].y;
    } else if (len == kChunkBytes) {
#pragma unroll
      for (uint32_t i = 0; i < kChunkBytes / kSweepBytes; i += 4) {
        const uint4 w0 = lds128(wp + (i + 0) * kSweepBytes), x0 = lds128(xp + (i + 0) * kSweepBytes);
        const uint4 w1 = lds128(wp + (i + 1) * kSweepBytes), x1 = lds128(xp + (i + 1) * kSweepBytes);
        const uint4 w2 = lds128(wp + (i + 2) * kSweepBytes), x2 = lds128(xp + (i + 2) * kSweepBytes);
        const uint4 w3 = lds128(wp + (i + 3) * kSweepBytes), x3 = lds128(xp + (i + 3) * kSweepBytes);
        acc[0] = dot8(w0, x0, acc[0]);
        acc[1] = dot8(w1, x1, acc[1]);
        acc[2] = dot8(w2, x2, acc[2]);
        acc[3] = dot8(w3, x3, acc[3]);
      }
    } else {
      uint32_t off = 0;
      for (; off + 4u * kSweepBytes <= len; off += 4u * kSweepBytes) {
        const uint4 w0 = lds128(wp + off), x0 = lds128(xp + off);
        const uint4 w1 = lds128(wp + off + kSweepBytes), x1 = lds128(xp + off + kSweepBytes);
        const uint4 w2 = lds128(wp + off + 2u * kSweepBytes), x2 = lds128(xp + off + 2u * kSweepBytes);
        const uint4 w3 = lds128(wp + off + 3u * kSweepBytes), x3 = lds128(xp + off + 3u * kSweepBytes);
        acc[0] = dot8(w0, x0, acc[0]);
        acc[1] = dot8(w1, x1, acc[1]);
        acc[2] = dot8(w2, x2, acc[2]);
        acc[3] = dot8(w3, x3, acc[3]);
      }
      // tail: whole sweeps, then (rows that are not a multiple of 512 bytes) the lanes that still have data
      for (; off + lane * 16u < len; off += kSweepBytes) {
        acc[0] = dot8(lds128(wp + off), lds128(xp + off), acc[0]);
      }
    }
    const bool row_done = pos + len == row_end;
    const bool range_done = pos + len == job.end;
    if (row_done || range_done) {
      const float total = warp_sum((acc[0] + acc[1]) + (acc[2] + acc[3]));
      if (lane == 0) {
        if (row_done && row_from_start) {
          row_total[row] = total;
        } else {
          sh.edge[warp][edges].row = row;
          sh.edge[warp][edges].value = total;
        }
      }
      if (!(row_done && row_from_start)) edges += 1;
      acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
      row_from_start = true;
    }
    __syncwarp();
    rs.consumed += 1;
  }
  // keep the ring full while the block goes on to its next phase
  stream_fill(rs);
}

// After the block has synchronised behind stream_consume: row r's total with
// the partials of cut rows added in ascending warp order.
__device__ __forceinline__ float stream_row_total(const StreamShared &sh, const float *row_total,
                                                  uint32_t r) {
  float total = row_total[r];
#pragma unroll
  for (uint32_t w = 0; w < kStreamWarps; ++w) {
    if (sh.edge[w][0].row == r) total += sh.edge[w][0].value;
    if (sh.edge[w][1].row == r) total += sh.edge[w][1].value;
  }
  return total;
}

// After a timeout: give copies still in flight one more bounded chance to land
// before the block's shared memory is released.
__device__ inline void stream_drain(RowStream &rs) {
  if (!rs.dead) return;
  for (uint32_t c = rs.drain_from; c < rs.drain_to; ++c) {
    mbar_wait_bounded(&rs.bars[c % kStreamSlots], (c / kStreamSlots) & 1u);
  }
}

}  // namespace nb
