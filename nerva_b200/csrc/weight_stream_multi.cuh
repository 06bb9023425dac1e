// Weight stream that runs across projections.
//
// In the whole-step kernel every warp walks one long list of chunks: its rows
// of the QKV matrix of layer 0, then of the O matrix, gate/up, down, the next
// layer, ... and finally lm_head.  Weights do not depend on activations, so the
// issue side of the ring simply runs ahead into the next projection while the
// block is still normalising, attending, or waiting at a grid barrier: up to
// kStreamSlots chunks per warp are in flight at any time, and HBM keeps
// streaming through every phase boundary.
#pragma once

#include "weight_stream.cuh"

namespace nb {

struct JobDesc {
  const uint16_t *weight;  // [rows][cols] bf16
  uint32_t rows, cols;
  uint32_t pairs;          // rows interleaved (gate, up): keep pairs in one warp
  uint32_t reserved;
};

struct MultiStream {
  WarpStream ws;
  const JobDesc *jobs;
  uint32_t job_count;
  uint32_t issue_job;   // job the issue cursor is in
  uint32_t issue_next;  // next chunk slot of that job
  StreamJob issue;      // work list of issue_job for this warp
};

__device__ __forceinline__ StreamJob job_for_block(const JobDesc &d) {
  const bool pairs = d.pairs != 0;
  const StreamShape shape = make_stream_shape(d.cols, pairs);
  uint32_t row_begin, row_end;
  block_row_range(d.rows, pairs ? 2u : 1u, blockIdx.x, gridDim.x, &row_begin, &row_end);
  return make_stream_job(d.weight, shape, row_begin, row_end);
}

__device__ inline void multi_init(MultiStream &ms, uint8_t *ring_base, uint64_t *bars,
                                  const JobDesc *jobs, uint32_t job_count) {
  stream_init(ms.ws, ring_base, bars);
  ms.jobs = jobs;
  ms.job_count = job_count;
  ms.issue_job = 0;
  ms.issue_next = 0;
  if (job_count != 0) ms.issue = job_for_block(jobs[0]);
}

// Issues chunks, crossing into later jobs, while ring slots are free.
__device__ __forceinline__ void multi_fill(MultiStream &ms) {
  WarpStream &ws = ms.ws;
  if (ws.dead) return;
  while (ms.issue_job < ms.job_count && ws.issued - ws.consumed < kStreamSlots) {
    if (ms.issue_next >= ms.issue.chunks) {
      ms.issue_job += 1;
      ms.issue_next = 0;
      if (ms.issue_job < ms.job_count) ms.issue = job_for_block(ms.jobs[ms.issue_job]);
      continue;
    }
    ChunkDesc d;
    const uint32_t j = ms.issue_next++;
    if (!stream_chunk(ms.issue, j, d)) continue;
    const uint32_t slot = ws.issued % kStreamSlots;
    if ((threadIdx.x & 31u) == 0) {
      const uint32_t bytes = d.rows * d.klen * 2u;
      const uint16_t *src =
          ms.issue.weight + static_cast<uint64_t>(d.row0) * ms.issue.shape.cols + d.k0;
      fence_proxy_async();
      mbar_arrive_expect_tx(&ws.bars[slot], bytes);
      tma_load_1d(ws.ring + slot * kChunkBytes, src, bytes, &ws.bars[slot]);
    }
    ws.issued += 1;
  }
}

// Consumes job `index` (jobs must be consumed in order, each exactly once).
template <class Epilogue>
__device__ __forceinline__ void multi_consume(MultiStream &ms, uint32_t index, const uint16_t *x,
                                              Epilogue &epi, uint32_t *error_word) {
  WarpStream &ws = ms.ws;
  const StreamJob job = job_for_block(ms.jobs[index]);
  const uint32_t lane = threadIdx.x & 31u;
  float acc0 = 0.0f, acc1 = 0.0f, acc2 = 0.0f, acc3 = 0.0f;
  for (uint32_t j = 0; j < job.chunks; ++j) {
    ChunkDesc d;
    if (!stream_chunk(job, j, d)) continue;
    multi_fill(ms);
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
  // keep the ring full while the block goes on to its next phase
  multi_fill(ms);
}

}  // namespace nb
