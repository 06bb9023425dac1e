/* CPU oracle (test infrastructure): the DeepSeek expert routers of the reference,
 * restated from native/cuda/deepseek/deepseek_router.cuh.
 *
 *   V3 grouped sigmoid   deepseek_router.cuh:190-252 (group score = sum of the two best
 *                        biased sigmoid scores of the group, :150-170)
 *   V4 sqrt-softplus     deepseek_router.cuh:78-116
 *   V4 hash table        deepseek_router.cuh:118-148
 *
 * Selection rule everywhere (better_score, :37-43; insert_topk, :45-61): higher
 * biased score first, equal scores by lower id; a score that compares false
 * against everything (NaN) is never selected and leaves the placeholder id of
 * its rank.  Weights are the UNBIASED scores of the selected experts times
 * route_scale (:63-70).  Same libm calls as the reference (expf, log1pf, sqrtf),
 * so on one machine the results are bit-identical to the reference header
 * compiled for the host. */
#include <math.h>
#include <stdint.h>

#define ROUTER_MAX_TOPK 16u
#define ROUTER_MAX_GROUPS 64u

static float score_sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }

static float score_sqrtsoftplus(float v) {
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

static int precedes(float a_score, uint32_t a_id, float b_score, uint32_t b_id) {
  return a_score > b_score || (a_score == b_score && a_id < b_id);
}

/* Keeps the k best (score, id) pairs seen so far in order. */
static void keep_best(float score, uint32_t id, float *scores, uint32_t *ids, uint32_t k) {
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

static void placeholders(float *scores, uint32_t *ids, uint32_t k) {
  for (uint32_t i = 0; i < k; ++i) {
    scores[i] = -INFINITY;
    ids[i] = i;
  }
}

static float scale_for(float sum, uint32_t norm_topk_prob, float routed_scaling_factor) {
  if (norm_topk_prob == 0) return routed_scaling_factor;
  return sum == 0.0f ? 0.0f : routed_scaling_factor / sum;
}

static int common_ok(uint32_t num_experts, uint32_t top_k) {
  return num_experts > 0 && top_k > 0 && top_k <= ROUTER_MAX_TOPK && top_k <= num_experts;
}

int oracle_route_v4_sqrtsoftplus(const float *logits, const float *bias, uint32_t num_experts,
                                 uint32_t top_k, uint32_t norm_topk_prob,
                                 float routed_scaling_factor, uint32_t *expert_ids, float *weights) {
  if (!logits || !expert_ids || !weights || !common_ok(num_experts, top_k)) return -1;
  float scores[ROUTER_MAX_TOPK];
  uint32_t ids[ROUTER_MAX_TOPK];
  placeholders(scores, ids, top_k);
  for (uint32_t e = 0; e < num_experts; ++e) {
    const float choice = score_sqrtsoftplus(logits[e]) + (bias ? bias[e] : 0.0f);
    keep_best(choice, e, scores, ids, top_k);
  }
  float sum = 0.0f;
  for (uint32_t r = 0; r < top_k; ++r) {
    weights[r] = score_sqrtsoftplus(logits[ids[r]]);
    sum += weights[r];
  }
  const float scale = scale_for(sum, norm_topk_prob, routed_scaling_factor);
  for (uint32_t r = 0; r < top_k; ++r) {
    expert_ids[r] = ids[r];
    weights[r] *= scale;
  }
  return 0;
}

int oracle_route_v4_hash(const float *logits, const uint32_t *table, uint32_t table_len,
                         uint32_t route_token, uint32_t num_experts, uint32_t top_k,
                         uint32_t norm_topk_prob, float routed_scaling_factor,
                         uint32_t *expert_ids, float *weights) {
  if (!logits || !table || !expert_ids || !weights || !common_ok(num_experts, top_k)) return -1;
  const uint64_t first = (uint64_t)route_token * top_k;
  if (first + top_k > table_len) return -2;
  float sum = 0.0f;
  for (uint32_t r = 0; r < top_k; ++r) {
    const uint32_t e = table[first + r];
    if (e >= num_experts) return -3;
    expert_ids[r] = e;
    weights[r] = score_sqrtsoftplus(logits[e]);
    sum += weights[r];
  }
  const float scale = scale_for(sum, norm_topk_prob, routed_scaling_factor);
  for (uint32_t r = 0; r < top_k; ++r) weights[r] *= scale;
  return 0;
}

int oracle_route_v3_grouped_sigmoid(const float *logits, const float *bias, uint32_t num_experts,
                                    uint32_t num_groups, uint32_t top_k_groups, uint32_t top_k,
                                    uint32_t norm_topk_prob, float routed_scaling_factor,
                                    uint32_t *expert_ids, float *weights) {
  if (!logits || !expert_ids || !weights || !common_ok(num_experts, top_k) || num_groups == 0 ||
      num_groups > ROUTER_MAX_GROUPS || top_k_groups == 0 || top_k_groups > num_groups ||
      num_experts % num_groups != 0)
    return -1;
  const uint32_t per_group = num_experts / num_groups;
  float group_scores[ROUTER_MAX_GROUPS];
  uint32_t group_ids[ROUTER_MAX_GROUPS];
  placeholders(group_scores, group_ids, top_k_groups);
  for (uint32_t g = 0; g < num_groups; ++g) {
    float first = -INFINITY, second = -INFINITY;
    for (uint32_t i = 0; i < per_group; ++i) {
      const uint32_t e = g * per_group + i;
      const float choice = score_sigmoid(logits[e]) + (bias ? bias[e] : 0.0f);
      if (choice > first) {
        second = first;
        first = choice;
      } else if (choice > second) {
        second = choice;
      }
    }
    keep_best(first + second, g, group_scores, group_ids, top_k_groups);
  }
  float scores[ROUTER_MAX_TOPK];
  uint32_t ids[ROUTER_MAX_TOPK];
  placeholders(scores, ids, top_k);
  for (uint32_t g = 0; g < num_groups; ++g) {
    int chosen = 0;
    for (uint32_t i = 0; i < top_k_groups; ++i) chosen |= group_ids[i] == g;
    if (!chosen) continue;
    for (uint32_t i = 0; i < per_group; ++i) {
      const uint32_t e = g * per_group + i;
      const float choice = score_sigmoid(logits[e]) + (bias ? bias[e] : 0.0f);
      keep_best(choice, e, scores, ids, top_k);
    }
  }
  float sum = 0.0f;
  for (uint32_t r = 0; r < top_k; ++r) {
    weights[r] = score_sigmoid(logits[ids[r]]);
    sum += weights[r];
  }
  const float scale = scale_for(sum, norm_topk_prob, routed_scaling_factor);
  for (uint32_t r = 0; r < top_k; ++r) {
    expert_ids[r] = ids[r];
    weights[r] *= scale;
  }
  return 0;
}
