// DeepSeek expert MLP of one token as a per-operator entry point (fp32 weights and
// activations): out = sum_rank weight[rank] * W_down[e] . swiglu(W_gate[e] . x, W_up[e] . x).
// Replaces the reference's nerva_cuda_deepseek_moe_forward
// (native/cuda/deepseek/nerva_cuda_deepseek_moe.cu:456-510, 779-960), whose kernel runs in
// one thread.  Two launches: one warp per (rank, intermediate row) for gate, up and the
// (optionally clamped, :118-127) SwiGLU; then one warp per output row, the experts added in
// rank order.  Only the chosen experts' matrices are copied to the device.
#include <math.h>
#include <string.h>

#include <vector>

#include "common.cuh"
#include "kernels.cuh"
#include "session.h"

using namespace nb;

namespace {

struct ForwardArgs {
  const float *input, *weights;
  const float *w_gate, *w_up, *w_down;  // [top_k] experts, already gathered
  float *activation;                     // [top_k][intermediate]
  float *output;                         // [hidden]
  uint32_t hidden, intermediate, top_k, clamp;
  float limit;
};

__device__ __forceinline__ float warp_dot(const float *a, const float *b, uint32_t n) {
  float sum = 0.0f;
  for (uint32_t i = threadIdx.x & 31u; i < n; i += 32u) sum = fmaf(a[i], b[i], sum);
  return warp_sum(sum);
}

__global__ void moe_forward_activation_kernel(ForwardArgs a) {
  const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (warp >= a.top_k * a.intermediate) return;
  const float *gate_row = a.w_gate + static_cast<uint64_t>(warp) * a.hidden;
  const float *up_row = a.w_up + static_cast<uint64_t>(warp) * a.hidden;
  float gate = warp_dot(gate_row, a.input, a.hidden);
  float up = warp_dot(up_row, a.input, a.hidden);
  if (a.clamp != 0) {
    gate = fminf(gate, a.limit);
    up = fminf(fmaxf(up, -a.limit), a.limit);
  }
  if ((threadIdx.x & 31u) == 0) a.activation[warp] = silu(gate) * up;
}

__global__ void moe_forward_down_kernel(ForwardArgs a) {
  const uint32_t row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (row >= a.hidden) return;
  float total = 0.0f;
  for (uint32_t rank = 0; rank < a.top_k; ++rank) {
    const float *w = a.w_down + (static_cast<uint64_t>(rank) * a.hidden + row) * a.intermediate;
    total += a.weights[rank] * warp_dot(w, a.activation + static_cast<uint64_t>(rank) * a.intermediate, a.intermediate);
  }
  if ((threadIdx.x & 31u) == 0) a.output[row] = total;
}

uint64_t hash_f32_values(const float *values, uint64_t n) {
  uint64_t hash = 1469598103934665603ull;
  for (uint64_t i = 0; i < n; ++i) {
    uint32_t bits;
    memcpy(&bits, &values[i], 4);
    for (uint32_t byte = 0; byte < 4; ++byte) {
      hash ^= (bits >> (byte * 8)) & 0xffu;
      hash *= 1099511628211ull;
    }
  }
  return hash;
}

struct DeviceBlock {
  void *ptr = nullptr;
  ~DeviceBlock() {
    if (ptr != nullptr) cudaFree(ptr);
  }
};

}  // namespace

extern "C" int nerva_cuda_deepseek_moe_forward(const NervaCudaDeepSeekMoeForwardRequest *request,
                                               NervaCudaDeepSeekMoeForwardResult *out) {
  if (out == nullptr) return -1;
  memset(out, 0, sizeof(*out));
  out->status = -1;
  out->moe_error = -1;
  if (request != nullptr) {
    out->hidden_size = request->hidden_size;
    out->intermediate_size = request->intermediate_size;
    out->num_experts = request->num_experts;
    out->top_k = request->top_k;
    out->clamp_swiglu = request->clamp_swiglu;
    out->swiglu_limit = request->swiglu_limit;
  }
  // nerva_cuda_deepseek_moe.cu:647-654
  if (request == nullptr || request->input == nullptr || request->expert_ids == nullptr ||
      request->expert_weights == nullptr || request->w_gate == nullptr || request->w_up == nullptr ||
      request->w_down == nullptr || request->output == nullptr || request->hidden_size == 0 ||
      request->intermediate_size == 0 || request->num_experts == 0 || request->top_k == 0)
    return -1;
  for (uint32_t rank = 0; rank < request->top_k; ++rank) {
    if (request->expert_ids[rank] >= request->num_experts) {
      out->moe_error = -2;  // the reference's kernel reports the same code (:488-491)
      return -1;
    }
  }
  cudaError_t err = cudaGetDeviceCount(&out->device_count);
  if (err != cudaSuccess || out->device_count <= 0) {
    out->cuda_error = static_cast<int32_t>(err != cudaSuccess ? err : cudaErrorNoDevice);
    cudaGetLastError();
    return -1;
  }
  const uint64_t h = request->hidden_size, inter = request->intermediate_size, k = request->top_k;
  const uint64_t matrix = inter * h;
  auto align = [](uint64_t v) { return (v + 63u) & ~uint64_t{63}; };  // floats
  const uint64_t o_input = 0, o_weights = o_input + align(h), o_gate = o_weights + align(k);
  const uint64_t o_up = o_gate + align(k * matrix), o_down = o_up + align(k * matrix);
  const uint64_t o_act = o_down + align(k * matrix), o_out = o_act + align(k * inter), total = o_out + align(h);
  DeviceBlock block;
  err = cudaMalloc(&block.ptr, total * 4u);
  float *base = static_cast<float *>(block.ptr);
  if (err == cudaSuccess) err = cudaMemcpy(base + o_input, request->input, h * 4u, cudaMemcpyHostToDevice);
  if (err == cudaSuccess) err = cudaMemcpy(base + o_weights, request->expert_weights, k * 4u, cudaMemcpyHostToDevice);
  for (uint32_t rank = 0; err == cudaSuccess && rank < k; ++rank) {
    const uint64_t e = request->expert_ids[rank];
    err = cudaMemcpy(base + o_gate + rank * matrix, request->w_gate + e * matrix, matrix * 4u, cudaMemcpyHostToDevice);
    if (err == cudaSuccess)
      err = cudaMemcpy(base + o_up + rank * matrix, request->w_up + e * matrix, matrix * 4u, cudaMemcpyHostToDevice);
    if (err == cudaSuccess)
      err = cudaMemcpy(base + o_down + rank * matrix, request->w_down + e * matrix, matrix * 4u, cudaMemcpyHostToDevice);
  }
  out->h2d_bytes = (h + k + 3u * k * matrix) * 4u;
  if (err == cudaSuccess) {
    ForwardArgs a{};
    a.input = base + o_input;
    a.weights = base + o_weights;
    a.w_gate = base + o_gate;
    a.w_up = base + o_up;
    a.w_down = base + o_down;
    a.activation = base + o_act;
    a.output = base + o_out;
    a.hidden = request->hidden_size;
    a.intermediate = request->intermediate_size;
    a.top_k = request->top_k;
    a.clamp = request->clamp_swiglu;
    a.limit = request->swiglu_limit;
    const uint64_t act_warps = k * inter;
    moe_forward_activation_kernel<<<static_cast<uint32_t>((act_warps + 7u) / 8u), 256>>>(a);
    moe_forward_down_kernel<<<static_cast<uint32_t>((h + 7u) / 8u), 256>>>(a);
    err = cudaGetLastError();
    out->kernel_launches = 2;
  }
  if (err == cudaSuccess) err = cudaDeviceSynchronize();
  out->sync_calls = 1;
  if (err == cudaSuccess) err = cudaMemcpy(request->output, base + o_out, h * 4u, cudaMemcpyDeviceToHost);
  out->device_arena_bytes = total * 4u;
  out->d2h_bytes = h * 4u;
  if (err != cudaSuccess) {
    out->cuda_error = static_cast<int32_t>(err);
    set_last_error(cudaGetErrorString(err));
    return -1;
  }
  out->moe_error = 0;
  out->output_hash = hash_f32_values(request->output, h);
  out->status = 0;
  return 0;
}
