/* CPU oracle (test infrastructure): DeepSeek multi-head latent attention decode for one
 * token in its "absorbed" form, restated from the reference's per-operator kernel
 * (native/cuda/deepseek/nerva_cuda_deepseek_mla.cu:144-227; CPU twin
 * crates/nerva-model/src/attention/exact/mla.rs:162-253).
 *
 *   ql[head][latent]  = sum_nope q_nope[head][nope] * w_uk[(latent*heads + head)*nope_dim + nope]
 *   score[token]      = (ql . kv_c[token] + q_pe[head] . k_pe[token]) * softmax_scale
 *   latent[head]      = softmax(score) applied to the kv_c rows (online, tokens in order)
 *   out[head][v]      = sum_latent latent[head][latent] * w_uv[(latent*heads + head)*v_dim + v]
 *
 * All fp32, every sum serial in index order, online softmax with the reference's update
 * (old_scale is 0 while the running sum is 0).  Returns 0, -1 (bad shape) or -2 (the
 * running sum stayed 0). */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

int oracle_mla_decode(const float *q_nope, const float *q_pe, const float *kv_c, const float *k_pe,
                      const float *w_uk, const float *w_uv, float *output, uint32_t heads,
                      uint32_t tokens, uint32_t kv_lora_rank, uint32_t qk_nope_head_dim,
                      uint32_t qk_rope_head_dim, uint32_t v_head_dim, float softmax_scale) {
  if (heads == 0 || tokens == 0 || kv_lora_rank == 0 || kv_lora_rank > 1024 || qk_nope_head_dim == 0 ||
      v_head_dim == 0)
    return -1;
  float *ql = (float *)malloc(sizeof(float) * kv_lora_rank);
  float *latent = (float *)malloc(sizeof(float) * kv_lora_rank);
  if (!ql || !latent) {
    free(ql);
    free(latent);
    return -1;
  }
  int status = 0;
  for (uint32_t i = 0; i < heads * v_head_dim; ++i) output[i] = 0.0f;
  for (uint32_t head = 0; head < heads && status == 0; ++head) {
    for (uint32_t l = 0; l < kv_lora_rank; ++l) {
      float sum = 0.0f;
      for (uint32_t n = 0; n < qk_nope_head_dim; ++n)
        sum += q_nope[head * qk_nope_head_dim + n] * w_uk[((uint64_t)l * heads + head) * qk_nope_head_dim + n];
      ql[l] = sum;
      latent[l] = 0.0f;
    }
    float m = -INFINITY, denom = 0.0f;
    for (uint32_t t = 0; t < tokens; ++t) {
      const float *kv = kv_c + (uint64_t)t * kv_lora_rank;
      float a = 0.0f, b = 0.0f;
      for (uint32_t l = 0; l < kv_lora_rank; ++l) a += ql[l] * kv[l];
      for (uint32_t r = 0; r < qk_rope_head_dim; ++r)
        b += q_pe[head * qk_rope_head_dim + r] * k_pe[(uint64_t)t * qk_rope_head_dim + r];
      const float score = (a + b) * softmax_scale;
      const float next = fmaxf(m, score);
      const float keep = denom == 0.0f ? 0.0f : expf(m - next);
      const float add = expf(score - next);
      for (uint32_t l = 0; l < kv_lora_rank; ++l) latent[l] = latent[l] * keep + kv[l] * add;
      denom = denom * keep + add;
      m = next;
    }
    if (denom == 0.0f) {
      status = -2;
      break;
    }
    for (uint32_t l = 0; l < kv_lora_rank; ++l) latent[l] /= denom;
    for (uint32_t v = 0; v < v_head_dim; ++v) {
      float sum = 0.0f;
      for (uint32_t l = 0; l < kv_lora_rank; ++l)
        sum += latent[l] * w_uv[((uint64_t)l * heads + head) * v_head_dim + v];
      output[head * v_head_dim + v] = sum;
    }
  }
  free(ql);
  free(latent);
  return status;
}

/* DeepSeek expert MLP of one token, fp32 (native/cuda/deepseek/nerva_cuda_deepseek_moe.cu:456-510;
 * SwiGLU with the optional clamp of :118-127: gate = min(gate, limit), up clamped to +-limit).
 * Experts are added in rank order: out += weight[rank] * W_down[e] . act.  Returns 0, -1, or -2 when
 * an expert id is out of range. */
static float mlp_dot(const float *a, const float *b, uint32_t n) {
  float sum = 0.0f;
  for (uint32_t i = 0; i < n; ++i) sum += a[i] * b[i];
  return sum;
}

int oracle_moe_forward(const float *input, const uint32_t *expert_ids, const float *expert_weights,
                       const float *w_gate, const float *w_up, const float *w_down, float *output,
                       uint32_t hidden, uint32_t intermediate, uint32_t num_experts, uint32_t top_k,
                       uint32_t clamp_swiglu, float swiglu_limit) {
  if (hidden == 0 || intermediate == 0 || num_experts == 0 || top_k == 0) return -1;
  float *act = (float *)malloc(sizeof(float) * intermediate);
  if (!act) return -1;
  for (uint32_t i = 0; i < hidden; ++i) output[i] = 0.0f;
  for (uint32_t rank = 0; rank < top_k; ++rank) {
    const uint32_t e = expert_ids[rank];
    if (e >= num_experts) {
      free(act);
      return -2;
    }
    const uint64_t base = (uint64_t)e * intermediate * hidden;
    for (uint32_t row = 0; row < intermediate; ++row) {
      float gate = mlp_dot(w_gate + base + (uint64_t)row * hidden, input, hidden);
      float up = mlp_dot(w_up + base + (uint64_t)row * hidden, input, hidden);
      if (clamp_swiglu != 0) {
        gate = fminf(gate, swiglu_limit);
        up = fminf(fmaxf(up, -swiglu_limit), swiglu_limit);
      }
      act[row] = gate / (1.0f + expf(-gate)) * up;
    }
    for (uint32_t i = 0; i < hidden; ++i)
      output[i] += expert_weights[rank] * mlp_dot(w_down + base + (uint64_t)i * intermediate, act, intermediate);
  }
  free(act);
  return 0;
}
