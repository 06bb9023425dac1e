// Per-operator C ABI: isolated projection (and the reference's projection bench
// entry point), isolated GQA decode attention, greedy arg-max, and the host
// synthetic-checkpoint generator.  Host pointers in, host pointers out.
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <string>
#include <vector>

#include "../../include/nerva_synth.h"
#include "kernels.cuh"
#include "session.h"

using namespace nb;

namespace {

struct DeviceBuffers {
  std::vector<void *> ptrs;
  ~DeviceBuffers() {
    for (void *p : ptrs) cudaFree(p);
  }
  template <class T>
  cudaError_t alloc(T **out, uint64_t count) {
    void *p = nullptr;
    const cudaError_t err = cudaMalloc(&p, (count == 0 ? 1 : count) * sizeof(T));
    if (err == cudaSuccess) ptrs.push_back(p);
    *out = static_cast<T *>(p);
    return err;
  }
};

struct Timing {
  cudaEvent_t a = nullptr, b = nullptr;
  ~Timing() {
    if (a != nullptr) cudaEventDestroy(a);
    if (b != nullptr) cudaEventDestroy(b);
  }
  cudaError_t init() {
    cudaError_t err = cudaEventCreate(&a);
    if (err == cudaSuccess) err = cudaEventCreate(&b);
    return err;
  }
};

// Times `iterations` calls of launch(i) (i counts on from `first`) between two events on `stream`.
// The calls are captured into one CUDA graph and replayed (once untimed, once timed), so that the
// host's launch cost is not part of the figure; where capture is not possible they are issued directly.
template <class Launch>
cudaError_t time_launch_train(cudaStream_t stream, Timing &t, uint32_t first, uint32_t iterations, Launch launch,
                              float *ms) {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  cudaError_t err = cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal);
  if (err == cudaSuccess) {
    cudaError_t launched = cudaSuccess;
    for (uint32_t i = 0; launched == cudaSuccess && i < iterations; ++i) launched = launch(first + i);
    err = cudaStreamEndCapture(stream, &graph);
    if (err == cudaSuccess) err = launched;
    if (err == cudaSuccess) err = cudaGraphInstantiate(&exec, graph, 0);
  }
  if (err == cudaSuccess) {
    err = cudaGraphLaunch(exec, stream);  // untimed replay: the caches and the clocks see the same train
    if (err == cudaSuccess) err = cudaEventRecord(t.a, stream);
    if (err == cudaSuccess) err = cudaGraphLaunch(exec, stream);
    if (err == cudaSuccess) err = cudaEventRecord(t.b, stream);
  } else {
    cudaGetLastError();
    err = cudaEventRecord(t.a, stream);
    for (uint32_t i = 0; err == cudaSuccess && i < iterations; ++i) err = launch(first + i);
    if (err == cudaSuccess) err = cudaEventRecord(t.b, stream);
  }
  if (err == cudaSuccess) err = cudaEventSynchronize(t.b);
  if (err == cudaSuccess) err = cudaEventElapsedTime(ms, t.a, t.b);
  if (exec != nullptr) cudaGraphExecDestroy(exec);
  if (graph != nullptr) cudaGraphDestroy(graph);
  return err;
}

cudaError_t device_sm_count(uint32_t *sms, int *major, int *minor, int *ordinal) {
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  cudaDeviceProp prop{};
  if (err == cudaSuccess) err = cudaGetDeviceProperties(&prop, device);
  if (err == cudaSuccess) {
    *sms = static_cast<uint32_t>(prop.multiProcessorCount);
    if (major != nullptr) *major = prop.major;
    if (minor != nullptr) *minor = prop.minor;
    if (ordinal != nullptr) *ordinal = device;
  }
  return err;
}

// L2 flush between timed launches: a write larger than the 126 MB L2.
constexpr uint64_t kFlushBytes = 192ull << 20;

}  // namespace

extern "C" int nerva_b200_projection(const uint16_t *weight, const uint16_t *x, float *y,
                                     uint32_t rows, uint32_t cols, uint32_t tokens,
                                     uint32_t warmup, uint32_t iterations, uint64_t *avg_ns) {
  set_last_error("");
  if (weight == nullptr || x == nullptr || y == nullptr || rows == 0 || cols == 0 || tokens == 0) return -1;
  uint32_t sms = 0;
  cudaError_t err = device_sm_count(&sms, nullptr, nullptr, nullptr);
  if (err == cudaSuccess) err = configure_projection_kernels();
  DeviceBuffers buf;
  Timing t;
  uint16_t *d_w = nullptr, *d_x = nullptr;
  float *d_y = nullptr;
  uint8_t *d_flush = nullptr;
  const uint64_t w_elems = static_cast<uint64_t>(rows) * cols;
  if (err == cudaSuccess) err = buf.alloc(&d_w, w_elems);
  if (err == cudaSuccess) err = buf.alloc(&d_x, static_cast<uint64_t>(tokens) * cols);
  if (err == cudaSuccess) err = buf.alloc(&d_y, static_cast<uint64_t>(tokens) * rows);
  if (err == cudaSuccess && iterations > 1) err = buf.alloc(&d_flush, kFlushBytes);
  if (err == cudaSuccess) err = t.init();
  if (err == cudaSuccess) err = cudaMemcpy(d_w, weight, w_elems * 2u, cudaMemcpyHostToDevice);
  if (err == cudaSuccess)
    err = cudaMemcpy(d_x, x, static_cast<uint64_t>(tokens) * cols * 2u, cudaMemcpyHostToDevice);
  // More than one token: the block kernel on the tensor pipe streams the weights once for all of them.
  GemmParams g{};
  g.weight = d_w;
  g.rows = rows;
  g.cols = cols;
  g.x = d_x;
  g.tokens = tokens;
  g.epilogue = kEpilogueStore;
  g.out_f32 = d_y;
  const bool block = tokens > 1 && gemm_tc_eligible(g);
  uint32_t *d_error = nullptr;
  if (block) {
    float *d_ws = nullptr;
    uint32_t *d_tickets = nullptr;
    if (err == cudaSuccess) err = configure_gemm_tc_kernel();
    if (err == cudaSuccess) err = buf.alloc(&d_ws, gemm_tc_workspace_bytes(tokens, sms) / sizeof(float));
    if (err == cudaSuccess) err = buf.alloc(&d_tickets, static_cast<uint64_t>(gemm_tc_ticket_count(rows)) + 1u);
    if (err == cudaSuccess)
      err = cudaMemset(d_tickets, 0, (static_cast<uint64_t>(gemm_tc_ticket_count(rows)) + 1u) * sizeof(uint32_t));
    g.workspace = d_ws;
    g.tickets = d_tickets;
    d_error = d_tickets + gemm_tc_ticket_count(rows);
    g.error_word = d_error;
  }
  double total_ms = 0.0;
  for (uint32_t it = 0; err == cudaSuccess && it < warmup + iterations; ++it) {
    if (d_flush != nullptr) err = cudaMemsetAsync(d_flush, it & 0xff, kFlushBytes, nullptr);
    if (err == cudaSuccess) err = cudaEventRecord(t.a, nullptr);
    if (block && err == cudaSuccess) err = launch_gemm_tc(nullptr, g, sms);
    for (uint32_t m = 0; !block && err == cudaSuccess && m < tokens; ++m) {
      ProjectionParams p{};
      p.weight = d_w;
      p.rows = rows;
      p.cols = cols;
      p.prologue = kProloguePlain;
      p.x_bf16 = d_x + static_cast<uint64_t>(m) * cols;
      p.epilogue = kEpilogueStore;
      p.out_f32 = d_y + static_cast<uint64_t>(m) * rows;
      err = launch_projection(nullptr, p, sms);
    }
    if (err == cudaSuccess) err = cudaEventRecord(t.b, nullptr);
    if (err == cudaSuccess) err = cudaEventSynchronize(t.b);
    float ms = 0.0f;
    if (err == cudaSuccess) err = cudaEventElapsedTime(&ms, t.a, t.b);
    if (it >= warmup) total_ms += ms;
  }
  if (err == cudaSuccess)
    err = cudaMemcpy(y, d_y, static_cast<uint64_t>(tokens) * rows * 4u, cudaMemcpyDeviceToHost);
  uint32_t device_error = 0;
  if (err == cudaSuccess && d_error != nullptr)
    err = cudaMemcpy(&device_error, d_error, sizeof(uint32_t), cudaMemcpyDeviceToHost);
  if (err != cudaSuccess) {
    set_last_error(cudaGetErrorString(err));
    return -1;
  }
  if (device_error != 0) {
    set_last_error("block projection kernel gave up a bounded wait (device error code " + std::to_string(device_error) + ")");
    return -1;
  }
  if (avg_ns != nullptr) *avg_ns = iterations == 0 ? 0 : static_cast<uint64_t>(total_ms * 1.0e6 / iterations);
  return 0;
}

// Sustained form of the same measurement: `copies` device copies of the matrix (together larger
// than the L2, so no launch finds its weights cached) are projected back to back, each launch
// allowed to start while its predecessor drains (programmatic dependent launch), the way the
// projections of consecutive layers follow each other inside a decode step.  avg_ns is the time
// per launch over `iterations` launches after `warmup`; y receives the last launch's output.
extern "C" int nerva_b200_projection_sustained(const uint16_t *weight, const uint16_t *x, float *y, uint32_t rows,
                                               uint32_t cols, uint32_t tokens, uint32_t copies, uint32_t warmup,
                                               uint32_t iterations, uint64_t *avg_ns) {
  set_last_error("");
  if (weight == nullptr || x == nullptr || y == nullptr || rows == 0 || cols == 0 || tokens == 0 || copies == 0 ||
      iterations == 0)
    return -1;
  uint32_t sms = 0;
  cudaError_t err = device_sm_count(&sms, nullptr, nullptr, nullptr);
  if (err == cudaSuccess) err = configure_projection_kernels();
  if (err == cudaSuccess) err = configure_gemm_tc_kernel();
  DeviceBuffers buf;
  Timing t;
  const uint64_t w_elems = static_cast<uint64_t>(rows) * cols;
  std::vector<uint16_t *> d_w(copies, nullptr);
  uint16_t *d_x = nullptr;
  float *d_y = nullptr, *d_ws = nullptr;
  uint32_t *d_tickets = nullptr;
  for (uint32_t c = 0; err == cudaSuccess && c < copies; ++c) {
    err = buf.alloc(&d_w[c], w_elems);
    if (err == cudaSuccess) err = cudaMemcpy(d_w[c], weight, w_elems * 2u, cudaMemcpyHostToDevice);
  }
  if (err == cudaSuccess) err = buf.alloc(&d_x, static_cast<uint64_t>(tokens) * cols);
  if (err == cudaSuccess) err = buf.alloc(&d_y, static_cast<uint64_t>(tokens) * rows);
  if (err == cudaSuccess) err = buf.alloc(&d_ws, gemm_tc_workspace_bytes(tokens, sms) / sizeof(float));
  if (err == cudaSuccess) err = buf.alloc(&d_tickets, static_cast<uint64_t>(gemm_tc_ticket_count(rows)) + 1u);
  if (err == cudaSuccess)
    err = cudaMemset(d_tickets, 0, (static_cast<uint64_t>(gemm_tc_ticket_count(rows)) + 1u) * sizeof(uint32_t));
  if (err == cudaSuccess) err = cudaMemcpy(d_x, x, static_cast<uint64_t>(tokens) * cols * 2u, cudaMemcpyHostToDevice);
  if (err == cudaSuccess) err = t.init();
  cudaStream_t stream = nullptr;
  if (err == cudaSuccess) err = cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
  uint32_t *d_error = d_tickets != nullptr ? d_tickets + gemm_tc_ticket_count(rows) : nullptr;
  GemmParams g{};
  g.rows = rows;
  g.cols = cols;
  g.x = d_x;
  g.tokens = tokens;
  g.epilogue = kEpilogueStore;
  g.out_f32 = d_y;
  g.workspace = d_ws;
  g.tickets = d_tickets;
  g.error_word = d_error;
  g.pdl = 1;
  g.weight = d_w.empty() ? nullptr : d_w[0];
  const bool block = tokens > 1 && err == cudaSuccess && gemm_tc_eligible(g);
  if (tokens > 1 && err == cudaSuccess && !block) err = cudaErrorNotSupported;
  auto launch = [&](uint32_t i) {
    if (block) {
      g.weight = d_w[i % copies];
      return launch_gemm_tc(stream, g, sms);
    }
    ProjectionParams p{};
    p.weight = d_w[i % copies];
    p.rows = rows;
    p.cols = cols;
    p.prologue = kProloguePlain;
    p.x_bf16 = d_x;
    p.epilogue = kEpilogueStore;
    p.out_f32 = d_y;
    p.error_word = d_error;
    p.pdl = 1;
    return launch_projection(stream, p, sms);
  };
  // NERVA_B200_GEMM_TIMELINE=1 (tuning aid): kernel-written %globaltimer stamps of two consecutive
  // block launches in the middle of the run go to stderr, in nanoseconds after the first stamp.
  const char *timeline_env = getenv("NERVA_B200_GEMM_TIMELINE");
  unsigned long long *d_stamps = nullptr;
  if (block && timeline_env != nullptr && timeline_env[0] == '1' && err == cudaSuccess) {
    err = buf.alloc(&d_stamps, uint64_t{2} * kTimelineSlots);
    if (err == cudaSuccess) err = cudaMemset(d_stamps, 0, 2 * kTimelineSlots * sizeof(unsigned long long));
  }
  for (uint32_t i = 0; err == cudaSuccess && i < warmup; ++i) err = launch(i);
  float ms = 0.0f;
  if (err == cudaSuccess)
    err = time_launch_train(
        stream, t, warmup, iterations,
        [&](uint32_t i) {
          const uint32_t at = i - warmup;
          if (d_stamps != nullptr)
            g.stamps = at == iterations / 2 ? d_stamps : (at == iterations / 2 + 1 ? d_stamps + kTimelineSlots : nullptr);
          return launch(i);
        },
        &ms);
  if (err == cudaSuccess) err = cudaMemcpy(y, d_y, static_cast<uint64_t>(tokens) * rows * 4u, cudaMemcpyDeviceToHost);
  uint32_t device_error = 0;
  if (err == cudaSuccess) err = cudaMemcpy(&device_error, d_error, sizeof(uint32_t), cudaMemcpyDeviceToHost);
  if (err == cudaSuccess && d_stamps != nullptr) {
    unsigned long long h[2 * kTimelineSlots] = {};
    err = cudaMemcpy(h, d_stamps, sizeof(h), cudaMemcpyDeviceToHost);
    const char *names[4] = {"entry", "first_tile_ready", "last_mma_committed", "exit"};
    for (uint32_t launch_index = 0; launch_index < 2; ++launch_index)
      for (uint32_t which = 0; which < 2; ++which)
        for (uint32_t k = 0; k < 4; ++k)
          fprintf(stderr, "gemm timeline rows=%u cols=%u tokens=%u launch %u %s block %s: %lld ns\n", rows, cols, tokens,
                  launch_index, which == 0 ? "first" : "last", names[k],
                  static_cast<long long>(h[launch_index * kTimelineSlots + which * 4 + k]) - static_cast<long long>(h[0]));
  }
  if (stream != nullptr) cudaStreamDestroy(stream);
  if (err != cudaSuccess) {
    set_last_error(cudaGetErrorString(err));
    return -1;
  }
  if (device_error != 0) {
    set_last_error("projection kernel gave up a bounded wait (device error code " + std::to_string(device_error) + ")");
    return -1;
  }
  if (avg_ns != nullptr) *avg_ns = static_cast<uint64_t>(static_cast<double>(ms) * 1.0e6 / iterations);
  return 0;
}

// Reference: native/cuda/nerva_cuda_projection_bench.cu.  Same deterministic
// inputs (((17 i + 13) mod 127) - 63) / 128 for the matrix and the vector
// (:38-41,84-101).  `custom_*` time this library's projection kernel as single
// launches and as graph replays; the `cublaslt_*` fields stay zero.
extern "C" int nerva_cuda_projection_bench(const NervaCudaProjectionBenchRequest *request,
                                           NervaCudaProjectionBenchResult *out) {
  if (out == nullptr) return -1;
  memset(out, 0, sizeof(*out));
  out->status = -1;
  if (request == nullptr || request->rows == 0 || request->cols == 0 || request->iterations == 0 ||
      request->dtype > NERVA_DTYPE_BF16)
    return -1;
  set_last_error("");
  int count = 0;
  cudaError_t err = cudaGetDeviceCount(&count);
  if (err != cudaSuccess || count == 0) {
    out->cuda_error = static_cast<int32_t>(err != cudaSuccess ? err : cudaErrorNoDevice);
    cudaGetLastError();
    return -1;
  }
  out->device_count = count;
  if (request->dtype != NERVA_DTYPE_BF16) {
    out->cuda_error = static_cast<int32_t>(cudaErrorNotSupported);
    return -1;
  }
  uint32_t sms = 0;
  err = device_sm_count(&sms, &out->compute_capability_major, &out->compute_capability_minor,
                        &out->device_ordinal);
  if (err == cudaSuccess) err = configure_projection_kernels();
  const uint32_t rows = request->rows, cols = request->cols;
  const uint32_t tokens = request->block_tokens == 0 ? 1u : request->block_tokens;
  out->dtype = request->dtype;
  out->rows = rows;
  out->cols = cols;
  out->block_tokens = request->block_tokens;
  out->iterations = request->iterations;
  out->warmup_iterations = request->warmup_iterations;
  const uint64_t w_elems = static_cast<uint64_t>(rows) * cols;
  out->matrix_bytes = w_elems * 2u;
  out->input_bytes = static_cast<uint64_t>(cols) * 2u;
  out->output_bytes = static_cast<uint64_t>(rows) * 4u;

  auto value_at = [](uint64_t i) { return (static_cast<float>((17u * i + 13u) % 127u) - 63.0f) / 128.0f; };
  std::vector<uint16_t> h_w(w_elems), h_x(cols);
  for (uint64_t i = 0; i < w_elems; ++i) h_w[i] = nerva_synth_f32_to_bf16(value_at(i));
  for (uint32_t i = 0; i < cols; ++i) h_x[i] = nerva_synth_f32_to_bf16(value_at(i));

  DeviceBuffers buf;
  Timing t;
  uint16_t *d_w = nullptr, *d_x = nullptr;
  float *d_y = nullptr;
  if (err == cudaSuccess) err = buf.alloc(&d_w, w_elems);
  if (err == cudaSuccess) err = buf.alloc(&d_x, static_cast<uint64_t>(cols));
  if (err == cudaSuccess) err = buf.alloc(&d_y, static_cast<uint64_t>(rows));
  out->device_allocations = 3;
  out->device_arena_bytes = w_elems * 2u + cols * 2u + rows * 4u;
  if (err == cudaSuccess) err = t.init();
  cudaStream_t stream = nullptr;
  if (err == cudaSuccess) err = cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
  if (err == cudaSuccess) err = cudaMemcpy(d_w, h_w.data(), w_elems * 2u, cudaMemcpyHostToDevice);
  if (err == cudaSuccess) err = cudaMemcpy(d_x, h_x.data(), cols * 2u, cudaMemcpyHostToDevice);
  ProjectionParams p{};
  p.weight = d_w;
  p.rows = rows;
  p.cols = cols;
  p.prologue = kProloguePlain;
  p.x_bf16 = d_x;
  p.epilogue = kEpilogueStore;
  p.out_f32 = d_y;
  // single-token kernel: stream launches
  for (uint32_t i = 0; err == cudaSuccess && i < request->warmup_iterations; ++i)
    err = launch_projection(stream, p, sms);
  if (err == cudaSuccess) err = cudaEventRecord(t.a, stream);
  for (uint32_t i = 0; err == cudaSuccess && i < request->iterations; ++i) {
    err = launch_projection(stream, p, sms);
    out->kernel_launches += 1;
  }
  if (err == cudaSuccess) err = cudaEventRecord(t.b, stream);
  if (err == cudaSuccess) err = cudaEventSynchronize(t.b);
  out->sync_calls += 1;
  float ms = 0.0f;
  if (err == cudaSuccess) err = cudaEventElapsedTime(&ms, t.a, t.b);
  out->custom_total_ns = static_cast<uint64_t>(ms * 1.0e6f);
  out->custom_avg_ns = out->custom_total_ns / request->iterations;
  // single-token kernel: graph replays
  auto time_graph = [&](auto &&enqueue, uint64_t *total_ns, uint64_t *avg_ns, uint64_t *nodes_out) {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    if (err == cudaSuccess) err = cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal);
    if (err == cudaSuccess) {
      err = enqueue();
      const cudaError_t end_err = cudaStreamEndCapture(stream, &graph);
      if (err == cudaSuccess) err = end_err;
    }
    if (err == cudaSuccess) err = cudaGraphInstantiate(&exec, graph, 0);
    if (err == cudaSuccess) {
      size_t nodes = 0;
      cudaGraphGetNodes(graph, nullptr, &nodes);
      *nodes_out = nodes;
      out->graph_captures += 1;
    }
    for (uint32_t i = 0; err == cudaSuccess && i < request->warmup_iterations; ++i) err = cudaGraphLaunch(exec, stream);
    if (err == cudaSuccess) err = cudaEventRecord(t.a, stream);
    for (uint32_t i = 0; err == cudaSuccess && i < request->iterations; ++i) {
      err = cudaGraphLaunch(exec, stream);
      out->graph_replays += 1;
    }
    if (err == cudaSuccess) err = cudaEventRecord(t.b, stream);
    if (err == cudaSuccess) err = cudaEventSynchronize(t.b);
    out->sync_calls += 1;
    float graph_ms = 0.0f;
    if (err == cudaSuccess) err = cudaEventElapsedTime(&graph_ms, t.a, t.b);
    *total_ns = static_cast<uint64_t>(graph_ms * 1.0e6f);
    *avg_ns = *total_ns / request->iterations;
    if (exec != nullptr) cudaGraphExecDestroy(exec);
    if (graph != nullptr) cudaGraphDestroy(graph);
  };
  time_graph([&] { return launch_projection(stream, p, sms); }, &out->custom_graph_total_ns,
             &out->custom_graph_avg_ns, &out->custom_graph_nodes);
  if (out->custom_graph_avg_ns != 0) {
    const uint64_t bytes = out->matrix_bytes + out->input_bytes + out->output_bytes;
    out->custom_effective_bandwidth_bps = bytes * 1000000000ull / out->custom_graph_avg_ns;
  }
  // block_tokens > 1: the block kernel on the tensor pipe (weights streamed once for the block), in
  // the result fields the reference uses for its block path (nerva_cuda_projection_bench.cu:791-830).
  uint16_t *d_xb = nullptr;
  float *d_yb = nullptr;
  std::vector<uint16_t> h_xb;
  uint32_t *d_block_error = nullptr;
  if (tokens > 1) {
    h_xb.resize(static_cast<uint64_t>(tokens) * cols);
    for (uint64_t i = 0; i < h_xb.size(); ++i) h_xb[i] = nerva_synth_f32_to_bf16(value_at(i));
    float *d_ws = nullptr;
    uint32_t *d_tickets = nullptr;
    if (err == cudaSuccess) err = buf.alloc(&d_xb, h_xb.size());
    if (err == cudaSuccess) err = buf.alloc(&d_yb, static_cast<uint64_t>(tokens) * rows);
    if (err == cudaSuccess) err = buf.alloc(&d_ws, gemm_tc_workspace_bytes(tokens, sms) / sizeof(float));
    if (err == cudaSuccess) err = buf.alloc(&d_tickets, static_cast<uint64_t>(gemm_tc_ticket_count(rows)) + 1u);
    if (err == cudaSuccess)
      err = cudaMemset(d_tickets, 0, (static_cast<uint64_t>(gemm_tc_ticket_count(rows)) + 1u) * sizeof(uint32_t));
    if (err == cudaSuccess) err = cudaMemcpy(d_xb, h_xb.data(), h_xb.size() * 2u, cudaMemcpyHostToDevice);
    if (err == cudaSuccess) err = configure_gemm_tc_kernel();
    out->device_allocations += 4;
    GemmParams g{};
    g.weight = d_w;
    g.rows = rows;
    g.cols = cols;
    g.x = d_xb;
    g.tokens = tokens;
    g.epilogue = kEpilogueStore;
    g.out_f32 = d_yb;
    g.workspace = d_ws;
    g.tickets = d_tickets;
    d_block_error = d_tickets + gemm_tc_ticket_count(rows);
    g.error_word = d_block_error;
    if (err == cudaSuccess && !gemm_tc_eligible(g)) err = cudaErrorNotSupported;
    for (uint32_t i = 0; err == cudaSuccess && i < request->warmup_iterations; ++i) err = launch_gemm_tc(stream, g, sms);
    if (err == cudaSuccess) err = cudaEventRecord(t.a, stream);
    for (uint32_t i = 0; err == cudaSuccess && i < request->iterations; ++i) {
      err = launch_gemm_tc(stream, g, sms);
      out->kernel_launches += 1;
    }
    if (err == cudaSuccess) err = cudaEventRecord(t.b, stream);
    if (err == cudaSuccess) err = cudaEventSynchronize(t.b);
    out->sync_calls += 1;
    if (err == cudaSuccess) err = cudaEventElapsedTime(&ms, t.a, t.b);
    out->block_cublaslt_total_ns = static_cast<uint64_t>(ms * 1.0e6f);
    out->block_cublaslt_avg_ns = out->block_cublaslt_total_ns / request->iterations;
    out->block_cublaslt_per_token_ns = out->block_cublaslt_avg_ns / tokens;
    time_graph([&] { return launch_gemm_tc(stream, g, sms); }, &out->block_cublaslt_graph_total_ns,
               &out->block_cublaslt_graph_avg_ns, &out->block_cublaslt_graph_nodes);
    out->block_cublaslt_graph_per_token_ns = out->block_cublaslt_graph_avg_ns / tokens;
    if (out->block_cublaslt_per_token_ns != 0)
      out->block_cublaslt_speedup_x1000 = out->custom_avg_ns * 1000ull / out->block_cublaslt_per_token_ns;
    if (out->block_cublaslt_graph_per_token_ns != 0)
      out->block_cublaslt_graph_speedup_x1000 = out->custom_graph_avg_ns * 1000ull / out->block_cublaslt_graph_per_token_ns;
    if (out->block_cublaslt_graph_avg_ns != 0) {
      const uint64_t bytes = out->matrix_bytes + tokens * (out->input_bytes + out->output_bytes);
      out->block_cublaslt_effective_bandwidth_bps = bytes * 1000000000ull / out->block_cublaslt_graph_avg_ns;
    }
  }
  // check against an fp64 host dot product of the same bf16 inputs on a row sample
  std::vector<float> h_y(rows);
  if (err == cudaSuccess) err = cudaMemcpy(h_y.data(), d_y, rows * 4u, cudaMemcpyDeviceToHost);
  if (err == cudaSuccess) {
    const uint32_t stride = rows > 4096 ? rows / 4096 : 1;
    for (uint32_t r = 0; r < rows; r += stride) {
      double acc = 0.0;
      for (uint32_t k = 0; k < cols; ++k) {
        const float w = __builtin_bit_cast(float, static_cast<uint32_t>(h_w[static_cast<uint64_t>(r) * cols + k]) << 16);
        const float xv = __builtin_bit_cast(float, static_cast<uint32_t>(h_x[k]) << 16);
        acc += static_cast<double>(w) * xv;
      }
      const float diff = fabsf(h_y[r] - static_cast<float>(acc));
      if (diff > out->max_abs_diff) out->max_abs_diff = diff;
      if (diff > 0.25f) out->mismatch_count += 1;  // the reference's tolerance (:843-845)
    }
  }
  if (err == cudaSuccess && tokens > 1) {
    // every token of the block on a sparser row sample, and the kernel's own error word
    std::vector<float> h_yb(static_cast<uint64_t>(tokens) * rows);
    uint32_t device_error = 0;
    err = cudaMemcpy(h_yb.data(), d_yb, h_yb.size() * 4u, cudaMemcpyDeviceToHost);
    if (err == cudaSuccess) err = cudaMemcpy(&device_error, d_block_error, sizeof(uint32_t), cudaMemcpyDeviceToHost);
    if (device_error != 0) out->mismatch_count += 1;
    const uint32_t stride = rows > 512 ? rows / 512 : 1;
    for (uint32_t m = 0; err == cudaSuccess && m < tokens; ++m) {
      for (uint32_t r = m % stride; r < rows; r += stride) {
        double acc = 0.0;
        for (uint32_t k = 0; k < cols; ++k) {
          const float w = __builtin_bit_cast(float, static_cast<uint32_t>(h_w[static_cast<uint64_t>(r) * cols + k]) << 16);
          const float xv = __builtin_bit_cast(float, static_cast<uint32_t>(h_xb[static_cast<uint64_t>(m) * cols + k]) << 16);
          acc += static_cast<double>(w) * xv;
        }
        const float diff = fabsf(h_yb[static_cast<uint64_t>(m) * rows + r] - static_cast<float>(acc));
        if (diff > out->max_abs_diff) out->max_abs_diff = diff;
        if (!(diff <= 0.25f)) out->mismatch_count += 1;
      }
    }
  }
  if (stream != nullptr) cudaStreamDestroy(stream);
  out->device_frees = out->device_allocations;
  out->selected_strategy = 1;        // custom kernel
  out->selected_graph_strategy = 1;
  out->hot_path_allocations = 0;
  if (err != cudaSuccess) {
    out->cuda_error = static_cast<int32_t>(err);
    set_last_error(cudaGetErrorString(err));
    return -1;
  }
  out->status = out->mismatch_count == 0 ? 0 : -1;
  return out->status;
}

// Sustained form: `copies` device copies of the K and V pages (the caches of `copies` layers,
// together larger than the L2) are attended over one after the other, back to back on one stream,
// as the attention launches of the layers of a decode step follow each other.  avg_ns: time per
// launch pair (attention + merge) over `iterations` after `warmup`; out: the last launch's output.
extern "C" int nerva_b200_gqa_decode_attention_sustained(const float *q, const uint16_t *key_pages,
                                                         const uint16_t *value_pages, const uint32_t *page_table,
                                                         float *out, uint32_t batch, uint32_t context, uint32_t heads,
                                                         uint32_t kv_heads, uint32_t head_dim, uint32_t copies,
                                                         uint32_t warmup, uint32_t iterations, uint64_t *avg_ns) {
  set_last_error("");
  if (q == nullptr || key_pages == nullptr || value_pages == nullptr || page_table == nullptr || out == nullptr ||
      batch == 0 || context == 0 || heads == 0 || kv_heads == 0 || heads % kv_heads != 0 || head_dim == 0 ||
      head_dim > 256 || copies == 0 || iterations == 0)
    return -1;
  uint32_t sms = 0;
  cudaError_t err = device_sm_count(&sms, nullptr, nullptr, nullptr);
  if (err == cudaSuccess) err = configure_attention_kernels();
  const uint32_t pages = (context + NERVA_KV_CACHE_BLOCK_TOKENS - 1) / NERVA_KV_CACHE_BLOCK_TOKENS;
  const uint64_t kv_hidden = static_cast<uint64_t>(kv_heads) * head_dim;
  const uint64_t kv_elems = static_cast<uint64_t>(batch) * pages * NERVA_KV_CACHE_BLOCK_TOKENS * kv_hidden;
  const uint64_t q_elems = static_cast<uint64_t>(batch) * heads * head_dim;
  const uint32_t splits = attention_default_splits(context, batch, kv_heads, sms);
  DeviceBuffers buf;
  Timing t;
  float *d_q = nullptr, *d_out = nullptr, *d_acc = nullptr, *d_m = nullptr, *d_l = nullptr;
  std::vector<uint16_t *> d_k(copies, nullptr), d_v(copies, nullptr);
  uint32_t *d_table = nullptr, *d_err = nullptr;
  if (err == cudaSuccess) err = buf.alloc(&d_q, q_elems);
  if (err == cudaSuccess) err = buf.alloc(&d_out, q_elems);
  for (uint32_t c = 0; err == cudaSuccess && c < copies; ++c) {
    err = buf.alloc(&d_k[c], kv_elems);
    if (err == cudaSuccess) err = buf.alloc(&d_v[c], kv_elems);
    if (err == cudaSuccess) err = cudaMemcpy(d_k[c], key_pages, kv_elems * 2u, cudaMemcpyHostToDevice);
    if (err == cudaSuccess) err = cudaMemcpy(d_v[c], value_pages, kv_elems * 2u, cudaMemcpyHostToDevice);
  }
  if (err == cudaSuccess) err = buf.alloc(&d_table, static_cast<uint64_t>(batch) * pages);
  if (err == cudaSuccess) err = buf.alloc(&d_acc, q_elems * splits);
  if (err == cudaSuccess) err = buf.alloc(&d_m, static_cast<uint64_t>(batch) * heads * splits);
  if (err == cudaSuccess) err = buf.alloc(&d_l, static_cast<uint64_t>(batch) * heads * splits);
  if (err == cudaSuccess) err = buf.alloc(&d_err, uint64_t{1});
  if (err == cudaSuccess) err = t.init();
  if (err == cudaSuccess) err = cudaMemset(d_err, 0, 4);
  if (err == cudaSuccess) err = cudaMemcpy(d_q, q, q_elems * 4u, cudaMemcpyHostToDevice);
  if (err == cudaSuccess)
    err = cudaMemcpy(d_table, page_table, static_cast<uint64_t>(batch) * pages * 4u, cudaMemcpyHostToDevice);
  cudaStream_t stream = nullptr;
  if (err == cudaSuccess) err = cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
  AttentionParams p{};
  p.q = d_q;
  p.page_table = d_table;
  p.batch = batch;
  p.heads = heads;
  p.kv_heads = kv_heads;
  p.head_dim = head_dim;
  p.page_count = pages;
  p.context = context;
  p.splits = splits;
  p.partial_acc = d_acc;
  p.partial_m = d_m;
  p.partial_l = d_l;
  p.out_f32 = d_out;
  p.error_word = d_err;
  auto launch = [&](uint32_t i) {
    p.key_pages = d_k[i % copies];
    p.value_pages = d_v[i % copies];
    return launch_attention(stream, p);
  };
  for (uint32_t i = 0; err == cudaSuccess && i < warmup; ++i) err = launch(i);
  float ms = 0.0f;
  if (err == cudaSuccess) err = time_launch_train(stream, t, warmup, iterations, launch, &ms);
  uint32_t device_error = 0;
  if (err == cudaSuccess) err = cudaMemcpy(&device_error, d_err, 4, cudaMemcpyDeviceToHost);
  if (err == cudaSuccess) err = cudaMemcpy(out, d_out, q_elems * 4u, cudaMemcpyDeviceToHost);
  if (stream != nullptr) cudaStreamDestroy(stream);
  if (err != cudaSuccess) {
    set_last_error(cudaGetErrorString(err));
    return -1;
  }
  if (device_error != 0) {
    set_last_error("attention kernel reported device error code " + std::to_string(device_error));
    return -1;
  }
  if (avg_ns != nullptr) *avg_ns = static_cast<uint64_t>(static_cast<double>(ms) * 1.0e6 / iterations);
  return 0;
}

extern "C" int nerva_b200_gqa_decode_attention(const float *q, const uint16_t *key_pages,
                                               const uint16_t *value_pages,
                                               const uint32_t *page_table, float *out,
                                               uint32_t batch, uint32_t context, uint32_t heads,
                                               uint32_t kv_heads, uint32_t head_dim,
                                               uint32_t warmup, uint32_t iterations,
                                               uint64_t *avg_ns) {
  set_last_error("");
  if (q == nullptr || key_pages == nullptr || value_pages == nullptr || page_table == nullptr ||
      out == nullptr || batch == 0 || context == 0 || heads == 0 || kv_heads == 0 ||
      heads % kv_heads != 0 || head_dim == 0 || head_dim > 256)
    return -1;
  uint32_t sms = 0;
  cudaError_t err = device_sm_count(&sms, nullptr, nullptr, nullptr);
  if (err == cudaSuccess) err = configure_attention_kernels();
  const uint32_t pages = (context + NERVA_KV_CACHE_BLOCK_TOKENS - 1) / NERVA_KV_CACHE_BLOCK_TOKENS;
  const uint64_t kv_hidden = static_cast<uint64_t>(kv_heads) * head_dim;
  const uint64_t kv_elems = static_cast<uint64_t>(batch) * pages * NERVA_KV_CACHE_BLOCK_TOKENS * kv_hidden;
  const uint64_t q_elems = static_cast<uint64_t>(batch) * heads * head_dim;
  const uint32_t splits = attention_default_splits(context, batch, kv_heads, sms);
  DeviceBuffers buf;
  Timing t;
  AttentionParams p{};
  float *d_q = nullptr, *d_out = nullptr, *d_acc = nullptr, *d_m = nullptr, *d_l = nullptr;
  uint16_t *d_k = nullptr, *d_v = nullptr;
  uint32_t *d_table = nullptr, *d_err = nullptr;
  uint8_t *d_flush = nullptr;
  if (err == cudaSuccess) err = buf.alloc(&d_q, q_elems);
  if (err == cudaSuccess) err = buf.alloc(&d_out, q_elems);
  if (err == cudaSuccess) err = buf.alloc(&d_k, kv_elems);
  if (err == cudaSuccess) err = buf.alloc(&d_v, kv_elems);
  if (err == cudaSuccess) err = buf.alloc(&d_table, static_cast<uint64_t>(batch) * pages);
  if (err == cudaSuccess) err = buf.alloc(&d_acc, q_elems * splits);
  if (err == cudaSuccess) err = buf.alloc(&d_m, static_cast<uint64_t>(batch) * heads * splits);
  if (err == cudaSuccess) err = buf.alloc(&d_l, static_cast<uint64_t>(batch) * heads * splits);
  if (err == cudaSuccess) err = buf.alloc(&d_err, uint64_t{1});
  if (err == cudaSuccess && iterations > 1) err = buf.alloc(&d_flush, kFlushBytes);
  if (err == cudaSuccess) err = t.init();
  if (err == cudaSuccess) err = cudaMemset(d_err, 0, 4);
  if (err == cudaSuccess) err = cudaMemcpy(d_q, q, q_elems * 4u, cudaMemcpyHostToDevice);
  if (err == cudaSuccess) err = cudaMemcpy(d_k, key_pages, kv_elems * 2u, cudaMemcpyHostToDevice);
  if (err == cudaSuccess) err = cudaMemcpy(d_v, value_pages, kv_elems * 2u, cudaMemcpyHostToDevice);
  if (err == cudaSuccess)
    err = cudaMemcpy(d_table, page_table, static_cast<uint64_t>(batch) * pages * 4u, cudaMemcpyHostToDevice);
  p.q = d_q;
  p.key_pages = d_k;
  p.value_pages = d_v;
  p.page_table = d_table;
  p.batch = batch;
  p.heads = heads;
  p.kv_heads = kv_heads;
  p.head_dim = head_dim;
  p.page_count = pages;
  p.cursor = nullptr;
  p.context = context;
  p.splits = splits;
  p.partial_acc = d_acc;
  p.partial_m = d_m;
  p.partial_l = d_l;
  p.out_f32 = d_out;
  p.error_word = d_err;
  double total_ms = 0.0;
  for (uint32_t it = 0; err == cudaSuccess && it < warmup + iterations; ++it) {
    if (d_flush != nullptr) err = cudaMemsetAsync(d_flush, it & 0xff, kFlushBytes, nullptr);
    if (err == cudaSuccess) err = cudaEventRecord(t.a, nullptr);
    if (err == cudaSuccess) err = launch_attention(nullptr, p);
    if (err == cudaSuccess) err = cudaEventRecord(t.b, nullptr);
    if (err == cudaSuccess) err = cudaEventSynchronize(t.b);
    float ms = 0.0f;
    if (err == cudaSuccess) err = cudaEventElapsedTime(&ms, t.a, t.b);
    if (it >= warmup) total_ms += ms;
  }
  uint32_t device_error = 0;
  if (err == cudaSuccess) err = cudaMemcpy(&device_error, d_err, 4, cudaMemcpyDeviceToHost);
  if (err == cudaSuccess) err = cudaMemcpy(out, d_out, q_elems * 4u, cudaMemcpyDeviceToHost);
  if (err != cudaSuccess) {
    set_last_error(cudaGetErrorString(err));
    return -1;
  }
  if (device_error != 0) {
    set_last_error("attention kernel reported a page index outside the page table");
    return -1;
  }
  if (avg_ns != nullptr) *avg_ns = iterations == 0 ? 0 : static_cast<uint64_t>(total_ms * 1.0e6 / iterations);
  return 0;
}

extern "C" int nerva_b200_greedy_argmax(const float *logits, uint32_t count, uint32_t *token) {
  set_last_error("");
  if (logits == nullptr || token == nullptr || count == 0) return -1;
  DeviceBuffers buf;
  float *d_logits = nullptr;
  uint32_t *d_token = nullptr;
  cudaError_t err = buf.alloc(&d_logits, static_cast<uint64_t>(count));
  if (err == cudaSuccess) err = buf.alloc(&d_token, uint64_t{1});
  if (err == cudaSuccess) err = cudaMemcpy(d_logits, logits, static_cast<uint64_t>(count) * 4u, cudaMemcpyHostToDevice);
  if (err == cudaSuccess) err = launch_argmax(nullptr, d_logits, count, d_token);
  if (err == cudaSuccess) err = cudaMemcpy(token, d_token, 4, cudaMemcpyDeviceToHost);
  if (err != cudaSuccess) {
    set_last_error(cudaGetErrorString(err));
    return -1;
  }
  return 0;
}

// One token from host logits at `position` with the step's temperature / top-k / top-p sampler
// (the configuration is normalised and the arg-max cases are taken as in the session).
extern "C" int nerva_b200_sample_token(const float *logits, uint32_t count, uint32_t position, float temperature,
                                       float top_p, uint32_t top_k, uint64_t seed, uint32_t *token) {
  set_last_error("");
  if (logits == nullptr || token == nullptr || count == 0 || position == UINT32_MAX || !isfinite(temperature) ||
      temperature < 0.0f || !isfinite(top_p) || top_p <= 0.0f || top_p > 1.0f)
    return -1;
  DeviceBuffers buf;
  float *d_logits = nullptr;
  uint32_t *d_word = nullptr;
  SamplerParams *d_params = nullptr;
  NervaCudaSyntheticTokenSlot *d_slots = nullptr;
  cudaError_t err = buf.alloc(&d_logits, static_cast<uint64_t>(count));
  if (err == cudaSuccess) err = buf.alloc(&d_word, uint64_t{2});
  if (err == cudaSuccess) err = buf.alloc(&d_params, uint64_t{1});
  if (err == cudaSuccess) err = buf.alloc(&d_slots, static_cast<uint64_t>(position) + 1u);
  if (err == cudaSuccess) err = cudaMemcpy(d_logits, logits, static_cast<uint64_t>(count) * 4u, cudaMemcpyHostToDevice);
  if (err == cudaSuccess) err = cudaMemcpy(d_word, &position, 4, cudaMemcpyHostToDevice);
  if (err != cudaSuccess) {
    set_last_error(cudaGetErrorString(err));
    return -1;
  }
  if (!(temperature > 0.0f) || top_k == 1) {
    err = launch_argmax(nullptr, d_logits, count, d_word + 1);
    if (err == cudaSuccess) err = cudaMemcpy(token, d_word + 1, 4, cudaMemcpyDeviceToHost);
  } else {
    const SamplerParams params{temperature, top_p, top_k, 0u, seed};
    StepState st{};
    st.cursor = d_word;
    st.slots = d_slots;
    st.max_context = position + 1u;
    st.vocab = count;
    err = cudaMemcpy(d_params, &params, sizeof(params), cudaMemcpyHostToDevice);
    if (err == cudaSuccess) err = launch_sample_general(nullptr, st, d_logits, d_params, false);
    NervaCudaSyntheticTokenSlot slot{};
    if (err == cudaSuccess) err = cudaMemcpy(&slot, d_slots + position, sizeof(slot), cudaMemcpyDeviceToHost);
    if (err == cudaSuccess) *token = slot.token;
  }
  if (err != cudaSuccess) {
    set_last_error(cudaGetErrorString(err));
    return -1;
  }
  return 0;
}

// A rectangular block of a row-major tensor with `full_cols` columns: the shard
// generator of the tensor-parallel tests and bench (same bits as the whole tensor).
extern "C" void nerva_b200_synth_normal_bf16_block(uint64_t seed, uint64_t tensor_id, uint64_t full_cols,
                                                   uint64_t row_begin, uint64_t rows, uint64_t col_begin,
                                                   uint64_t cols, float std, uint16_t *out) {
  const uint64_t key = nerva_synth_key(seed, tensor_id);
  const float scale = std * (1.0f / 65536.0f);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < static_cast<int64_t>(rows); ++r) {
    const uint64_t base = (row_begin + static_cast<uint64_t>(r)) * full_cols + col_begin;
    uint16_t *dst = out + static_cast<uint64_t>(r) * cols;
    for (uint64_t c = 0; c < cols; ++c) dst[c] = nerva_synth_normal_bf16(key, base + c, scale);
  }
}

extern "C" void nerva_b200_synth_normal_bf16(uint64_t seed, uint64_t tensor_id, uint64_t count,
                                             float std, uint16_t *out) {
  const uint64_t key = nerva_synth_key(seed, tensor_id);
  const float scale = std * (1.0f / 65536.0f);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < static_cast<int64_t>(count); ++i) {
    out[i] = nerva_synth_normal_bf16(key, static_cast<uint64_t>(i), scale);
  }
}
