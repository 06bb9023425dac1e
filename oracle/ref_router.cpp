// Test infrastructure: exposes the REFERENCE's own router header
// (native/cuda/deepseek/deepseek_router.cuh, every function `__host__ __device__
// inline`) to the tests, compiled for the host from the reference checkout where it
// lies.  Built only where that checkout exists (see the Makefile's `ref` target);
// the resulting library is what the oracle's restatement is checked against.
#define __host__
#define __device__
#include "deepseek/deepseek_router.cuh"

namespace dsr = nerva::deepseek::router;

extern "C" int ref_route_v3_grouped_sigmoid(const float *logits, const float *bias, uint32_t num_experts,
                                            uint32_t num_groups, uint32_t top_k_groups, uint32_t top_k,
                                            uint32_t norm_topk_prob, float routed_scaling_factor,
                                            uint32_t *expert_ids, float *weights) {
  return dsr::route_v3_grouped_sigmoid(logits, bias, num_experts, num_groups, top_k_groups, top_k,
                                       norm_topk_prob, routed_scaling_factor, expert_ids, weights);
}

extern "C" int ref_route_v4_sqrtsoftplus(const float *logits, const float *bias, uint32_t num_experts,
                                         uint32_t top_k, uint32_t norm_topk_prob,
                                         float routed_scaling_factor, uint32_t *expert_ids,
                                         float *weights) {
  return dsr::route_v4_sqrtsoftplus(logits, bias, num_experts, top_k, norm_topk_prob,
                                    routed_scaling_factor, expert_ids, weights);
}

extern "C" int ref_route_v4_hash(const float *logits, const uint32_t *table, uint32_t table_len,
                                 uint32_t route_token, uint32_t num_experts, uint32_t top_k,
                                 uint32_t norm_topk_prob, float routed_scaling_factor,
                                 uint32_t *expert_ids, float *weights) {
  return dsr::route_v4_hash(logits, table, table_len, route_token, num_experts, top_k, norm_topk_prob,
                            routed_scaling_factor, expert_ids, weights);
}
