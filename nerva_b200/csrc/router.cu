// DeepSeek expert routing as a per-operator entry point: V3 grouped sigmoid,
// V4 sqrt-softplus and V4 hash-table routes.  Replaces the reference's
// nerva_cuda_deepseek_router_route (native/cuda/deepseek/nerva_cuda_deepseek_router.cu:396-560),
// whose kernel runs the whole route in one thread (<<<1, 1>>>, :83-143).
//
// Here the transcendental part (one biased score per expert) is computed by the
// whole block into shared memory, the per-group top-2 sums by one thread per
// group, and only the ordered insertion (expert ids are integer results that
// must not depend on the schedule) is left to one thread, which replays the
// reference's insertion order (deepseek_router.cuh:45-61) over the scores in
// shared memory.  Selection rule: higher biased score first, equal scores by
// lower id; weights are the unbiased scores of the selected experts scaled by
// route_scale (deepseek_router.cuh:63-70).
#include <math.h>
#include <string.h>

#include "common.cuh"
#include "kernels.cuh"
#include "session.h"

using namespace nb;

namespace {

constexpr uint32_t kKindV3GroupedSigmoid = 1, kKindV4SqrtSoftplus = 2, kKindV4Hash = 3;
constexpr uint32_t kMaxTopK = 16, kMaxGroups = 64;
constexpr uint32_t kRouterThreads = 256;
constexpr uint32_t kMaxExperts = 12288;  // biased scores of all experts live in 48 KB of shared memory

__device__ __forceinline__ float score_sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float score_sqrtsoftplus(float v) {
  float sp;
  if (v > 20.0f) {
    sp = v;
  } else if (v < -20.0f) {
    sp = expf(v);
  } else {
    sp = log1pf(expf(v));
  }
  return sqrtf(sp);
}
__device__ __forceinline__ bool precedes(float a, uint32_t a_id, float b, uint32_t b_id) {
  return a > b || (a == b && a_id < b_id);
}
__device__ void keep_best(float score, uint32_t id, float *scores, uint32_t *ids, uint32_t k) {
  uint32_t at = k;
  for (uint32_t slot = 0; slot < k; ++slot) {
    if (precedes(score, id, scores[slot], ids[slot])) {
      at = slot;
      break;
    }
  }
  if (at == k) return;
  for (uint32_t move = k - 1; move > at; --move) {
    scores[move] = scores[move - 1];
    ids[move] = ids[move - 1];
  }
  scores[at] = score;
  ids[at] = id;
}

struct RouteArgs {
  uint32_t kind, num_experts, num_groups, top_k_groups, top_k, norm_topk_prob, route_token;
  float routed_scaling_factor;
  const float *logits, *bias;
  const uint32_t *table;
  uint32_t table_len;
  uint32_t *expert_ids;
  float *weights;
  int32_t *route_error;
};

__global__ void __launch_bounds__(kRouterThreads) router_route_kernel(RouteArgs a) {
  extern __shared__ float choice[];          // [num_experts] biased scores
  __shared__ float group_score[kMaxGroups];
  const bool sigmoid = a.kind == kKindV3GroupedSigmoid;
  if (a.kind != kKindV4Hash) {
    for (uint32_t e = threadIdx.x; e < a.num_experts; e += blockDim.x) {
      const float raw = sigmoid ? score_sigmoid(a.logits[e]) : score_sqrtsoftplus(a.logits[e]);
      choice[e] = raw + (a.bias != nullptr ? a.bias[e] : 0.0f);
    }
  }
  __syncthreads();
  const uint32_t per_group = sigmoid ? a.num_experts / a.num_groups : 0;
  if (sigmoid && threadIdx.x < a.num_groups) {
    // sum of the two best biased scores of the group (deepseek_router.cuh:150-170)
    float first = -INFINITY, second = -INFINITY;
    for (uint32_t i = 0; i < per_group; ++i) {
      const float c = choice[threadIdx.x * per_group + i];
      if (c > first) {
        second = first;
        first = c;
      } else if (c > second) {
        second = c;
      }
    }
    group_score[threadIdx.x] = first + second;
  }
  __syncthreads();
  if (threadIdx.x != 0) return;

  float scores[kMaxTopK];
  uint32_t ids[kMaxTopK];
  float weight_sum = 0.0f;
  if (a.kind == kKindV4Hash) {
    const uint64_t first = static_cast<uint64_t>(a.route_token) * a.top_k;
    if (first + a.top_k > a.table_len) {
      *a.route_error = -2;
      return;
    }
    for (uint32_t r = 0; r < a.top_k; ++r) {
      const uint32_t e = a.table[first + r];
      if (e >= a.num_experts) {
        *a.route_error = -3;
        return;
      }
      ids[r] = e;
    }
  } else {
    for (uint32_t i = 0; i < a.top_k; ++i) {
      scores[i] = -INFINITY;
      ids[i] = i;
    }
    if (sigmoid) {
      float best_group[kMaxGroups];
      uint32_t best_group_id[kMaxGroups];
      for (uint32_t i = 0; i < a.top_k_groups; ++i) {
        best_group[i] = -INFINITY;
        best_group_id[i] = i;
      }
      for (uint32_t g = 0; g < a.num_groups; ++g)
        keep_best(group_score[g], g, best_group, best_group_id, a.top_k_groups);
      for (uint32_t g = 0; g < a.num_groups; ++g) {
        bool chosen = false;
        for (uint32_t i = 0; i < a.top_k_groups; ++i) chosen = chosen || best_group_id[i] == g;
        if (!chosen) continue;
        for (uint32_t i = 0; i < per_group; ++i) keep_best(choice[g * per_group + i], g * per_group + i, scores, ids, a.top_k);
      }
    } else {
      for (uint32_t e = 0; e < a.num_experts; ++e) keep_best(choice[e], e, scores, ids, a.top_k);
    }
  }
  for (uint32_t r = 0; r < a.top_k; ++r) {
    const float w = sigmoid ? score_sigmoid(a.logits[ids[r]]) : score_sqrtsoftplus(a.logits[ids[r]]);
    a.weights[r] = w;
    weight_sum += w;
  }
  float scale = a.routed_scaling_factor;
  if (a.norm_topk_prob != 0) scale = weight_sum == 0.0f ? 0.0f : a.routed_scaling_factor / weight_sum;
  for (uint32_t r = 0; r < a.top_k; ++r) {
    a.expert_ids[r] = ids[r];
    a.weights[r] *= scale;
  }
  *a.route_error = 0;
}

// nerva_cuda_deepseek_router.cu:145-160
uint64_t mix_u32(uint64_t hash, uint32_t value) {
  for (uint32_t byte = 0; byte < 4; ++byte) {
    hash ^= (value >> (byte * 8)) & 0xffu;
    hash *= 1099511628211ull;
  }
  return hash;
}
uint64_t hash_route(const uint32_t *ids, const float *weights, uint32_t n) {
  uint64_t hash = 1469598103934665603ull;
  for (uint32_t i = 0; i < n; ++i) {
    uint32_t bits;
    memcpy(&bits, &weights[i], 4);
    hash = mix_u32(hash, ids[i]);
    hash = mix_u32(hash, bits);
  }
  return hash;
}

// nerva_cuda_deepseek_router.cu:253-279
bool valid_route_request(const NervaCudaDeepSeekRouterRouteRequest *r) {
  if (r == nullptr || r->logits == nullptr || r->expert_ids == nullptr || r->weights == nullptr ||
      r->num_experts == 0 || r->top_k == 0 || r->top_k > kMaxTopK || r->top_k > r->num_experts)
    return false;
  if (r->router_kind == kKindV3GroupedSigmoid)
    return r->num_groups > 0 && r->num_groups <= kMaxGroups && r->top_k_groups > 0 &&
           r->top_k_groups <= r->num_groups && r->num_experts % r->num_groups == 0;
  if (r->router_kind == kKindV4SqrtSoftplus) return true;
  if (r->router_kind == kKindV4Hash) {
    const uint64_t end = static_cast<uint64_t>(r->route_token) * r->top_k + r->top_k;
    return r->hash_route_table != nullptr && end <= r->hash_route_table_len;
  }
  return false;
}

struct DeviceScratch {
  void *ptr = nullptr;
  ~DeviceScratch() {
    if (ptr != nullptr) cudaFree(ptr);
  }
};

}  // namespace

extern "C" int nerva_cuda_deepseek_router_route(const NervaCudaDeepSeekRouterRouteRequest *request,
                                                NervaCudaDeepSeekRouterRouteResult *out) {
  if (out == nullptr) return -1;
  memset(out, 0, sizeof(*out));
  out->status = -1;
  out->route_error = -1;
  if (request != nullptr) {
    out->router_kind = request->router_kind;
    out->num_experts = request->num_experts;
    out->num_groups = request->num_groups;
    out->top_k_groups = request->top_k_groups;
    out->top_k = request->top_k;
  }
  if (!valid_route_request(request)) return -1;
  cudaError_t err = cudaGetDeviceCount(&out->device_count);
  if (err != cudaSuccess || out->device_count <= 0) {
    out->cuda_error = static_cast<int32_t>(err != cudaSuccess ? err : cudaErrorNoDevice);
    cudaGetLastError();
    return -1;
  }
  if (request->num_experts > kMaxExperts) {
    out->cuda_error = static_cast<int32_t>(cudaErrorNotSupported);
    set_last_error("router: more than 12288 experts");
    return -1;
  }
  // one device block: logits | bias | table | ids | weights | error
  const uint64_t e = request->num_experts, k = request->top_k;
  const uint64_t logits_bytes = e * 4u, bias_bytes = request->correction_bias != nullptr ? e * 4u : 0u;
  const uint64_t table_bytes =
      request->hash_route_table != nullptr ? static_cast<uint64_t>(request->hash_route_table_len) * 4u : 0u;
  auto align = [](uint64_t v) { return (v + 255u) & ~uint64_t{255}; };
  const uint64_t o_bias = align(logits_bytes), o_table = o_bias + align(bias_bytes);
  const uint64_t o_ids = o_table + align(table_bytes), o_weights = o_ids + align(k * 4u);
  const uint64_t o_error = o_weights + align(k * 4u), total = o_error + 256u;
  DeviceScratch scratch;
  err = cudaMalloc(&scratch.ptr, total);
  uint8_t *base = static_cast<uint8_t *>(scratch.ptr);
  if (err == cudaSuccess) err = cudaMemcpy(base, request->logits, logits_bytes, cudaMemcpyHostToDevice);
  if (err == cudaSuccess && bias_bytes != 0)
    err = cudaMemcpy(base + o_bias, request->correction_bias, bias_bytes, cudaMemcpyHostToDevice);
  if (err == cudaSuccess && table_bytes != 0)
    err = cudaMemcpy(base + o_table, request->hash_route_table, table_bytes, cudaMemcpyHostToDevice);
  const int32_t unset = -1;
  if (err == cudaSuccess) err = cudaMemcpy(base + o_error, &unset, 4, cudaMemcpyHostToDevice);
  if (err == cudaSuccess) {
    RouteArgs a{};
    a.kind = request->router_kind;
    a.num_experts = request->num_experts;
    a.num_groups = request->num_groups;
    a.top_k_groups = request->top_k_groups;
    a.top_k = request->top_k;
    a.norm_topk_prob = request->norm_topk_prob;
    a.route_token = request->route_token;
    a.routed_scaling_factor = request->routed_scaling_factor;
    a.logits = reinterpret_cast<const float *>(base);
    a.bias = bias_bytes != 0 ? reinterpret_cast<const float *>(base + o_bias) : nullptr;
    a.table = table_bytes != 0 ? reinterpret_cast<const uint32_t *>(base + o_table) : nullptr;
    a.table_len = request->hash_route_table_len;
    a.expert_ids = reinterpret_cast<uint32_t *>(base + o_ids);
    a.weights = reinterpret_cast<float *>(base + o_weights);
    a.route_error = reinterpret_cast<int32_t *>(base + o_error);
    router_route_kernel<<<1, kRouterThreads, request->num_experts * 4u>>>(a);
    err = cudaGetLastError();
    out->kernel_launches = 1;
  }
  if (err == cudaSuccess) err = cudaDeviceSynchronize();
  out->sync_calls = 1;
  int32_t route_error = -1;
  if (err == cudaSuccess) err = cudaMemcpy(&route_error, base + o_error, 4, cudaMemcpyDeviceToHost);
  if (err == cudaSuccess) err = cudaMemcpy(request->expert_ids, base + o_ids, k * 4u, cudaMemcpyDeviceToHost);
  if (err == cudaSuccess) err = cudaMemcpy(request->weights, base + o_weights, k * 4u, cudaMemcpyDeviceToHost);
  out->device_arena_bytes = total;
  out->h2d_bytes = logits_bytes + bias_bytes + table_bytes + 4u;
  out->d2h_bytes = 4u + 2u * k * 4u;
  out->route_error = route_error;
  if (err != cudaSuccess) {
    out->cuda_error = static_cast<int32_t>(err);
    set_last_error(cudaGetErrorString(err));
    return -1;
  }
  if (route_error != 0) return -1;
  out->output_hash = hash_route(request->expert_ids, request->weights, request->top_k);
  out->hot_path_allocations = 0;
  out->status = 0;
  return 0;
}
