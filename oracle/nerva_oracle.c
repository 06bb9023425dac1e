/*
 * TEST INFRASTRUCTURE — NOT A PRODUCT CODE PATH.  See nerva_oracle.h.
 *
 * Build with -ffp-contract=off: the reference CPU path is Rust, which never
 * fuses a multiply and an add, and every sum below is a serial ascending f32
 * accumulation exactly as the reference's iterator sums are.
 */
#include "nerva_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

static int g_threads = 0;

void oracle_set_threads(int threads) {
  g_threads = threads;
  if (threads > 0) {
    omp_set_num_threads(threads); /* parallel regions without a num_threads clause (the synthetic fill) */
  }
}

int oracle_get_threads(void) {
#ifdef _OPENMP
  return g_threads > 0 ? g_threads : omp_get_max_threads();
#else
  return 1;
#endif
}

/* ---- codecs: crates/nerva-model/src/precision/bits.rs:4-18 ---- */

static inline float bits_to_f32(uint32_t bits) {
  float out;
  memcpy(&out, &bits, sizeof(out));
  return out;
}

static inline uint32_t f32_to_bits(float value) {
  uint32_t out;
  memcpy(&out, &value, sizeof(out));
  return out;
}

float oracle_bf16_to_f32(uint16_t bits) { return bits_to_f32((uint32_t)bits << 16); }

uint16_t oracle_f32_to_bf16(float value) {
  const uint32_t bits = f32_to_bits(value);
  const uint32_t exponent = bits & 0x7f800000u;
  const uint32_t mantissa = bits & 0x007fffffu;
  if (exponent == 0x7f800000u && mantissa != 0u) {
    return (uint16_t)((bits >> 16) | 1u);
  }
  const uint32_t lsb = (bits >> 16) & 1u;
  return (uint16_t)((bits + 0x7fffu + lsb) >> 16);
}

/* bits.rs:20-46 */
float oracle_f16_to_f32(uint16_t bits) {
  const uint32_t sign = ((uint32_t)(bits & 0x8000u)) << 16;
  const uint32_t exp = (bits >> 10) & 0x1fu;
  uint32_t frac = bits & 0x03ffu;
  if (exp == 0) {
    if (frac == 0) {
      return bits_to_f32(sign);
    }
    int32_t exponent = -14;
    while ((frac & 0x0400u) == 0) {
      frac <<= 1;
      exponent -= 1;
    }
    frac &= 0x03ffu;
    return bits_to_f32(sign | ((uint32_t)(exponent + 127) << 23) | (frac << 13));
  }
  if (exp == 0x1f) {
    return bits_to_f32(sign | 0x7f800000u | (frac << 13));
  }
  return bits_to_f32(sign | ((exp + 112u) << 23) | (frac << 13));
}

/* bits.rs:48-85 */
uint16_t oracle_f32_to_f16(float value) {
  const uint32_t bits = f32_to_bits(value);
  const uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
  const int32_t exp = (int32_t)((bits >> 23) & 0xffu);
  const uint32_t mant = bits & 0x007fffffu;
  if (exp == 255) {
    return (uint16_t)(sign | 0x7c00u | (mant != 0 ? 0x0200u : 0u));
  }
  const int32_t half_exp = exp - 127 + 15;
  if (half_exp >= 31) {
    return (uint16_t)(sign | 0x7c00u);
  }
  if (half_exp <= 0) {
    if (half_exp < -10) {
      return sign;
    }
    const uint32_t mantissa = mant | 0x00800000u;
    const uint32_t shift = (uint32_t)(14 - half_exp);
    uint16_t half = (uint16_t)(mantissa >> shift);
    const uint32_t round_bit = 1u << (shift - 1);
    const uint32_t remainder = mantissa & (round_bit | (round_bit - 1));
    if (remainder > round_bit || (remainder == round_bit && (half & 1u) != 0)) {
      half = (uint16_t)(half + 1);
    }
    return (uint16_t)(sign | half);
  }
  uint16_t half = (uint16_t)(((uint16_t)half_exp << 10) | (uint16_t)(mant >> 13));
  const uint32_t remainder = mant & 0x1fffu;
  if (remainder > 0x1000u || (remainder == 0x1000u && (half & 1u) != 0)) {
    half = (uint16_t)(half + 1);
  }
  return (uint16_t)(sign | half);
}

static inline float decode(uint32_t dtype, uint16_t bits) {
  return dtype == ORACLE_DTYPE_BF16 ? oracle_bf16_to_f32(bits) : oracle_f16_to_f32(bits);
}

static inline uint16_t encode(uint32_t dtype, float value) {
  return dtype == ORACLE_DTYPE_BF16 ? oracle_f32_to_bf16(value) : oracle_f32_to_f16(value);
}

static inline float round_to_dtype(uint32_t dtype, float value) {
  return decode(dtype, encode(dtype, value));
}

/* ---- primitive ops ---- */

/* precision/block/ops.rs:32-52 */
void oracle_rms_norm(uint32_t dtype, const float *input, const uint16_t *weight,
                     uint32_t n, float eps, float *output) {
  float sum = 0.0f;
  for (uint32_t i = 0; i < n; ++i) {
    sum += input[i] * input[i];
  }
  const float mean_square = sum / (float)n;
  const float scale = 1.0f / sqrtf(mean_square + eps);
  for (uint32_t i = 0; i < n; ++i) {
    output[i] = input[i] * scale * decode(dtype, weight[i]);
  }
}

/* precision/block/ops.rs:54-76: values[i] *= (scale * weight[i]) */
void oracle_per_head_rms_norm(uint32_t dtype, const uint16_t *weight, uint32_t head_dim,
                              float *values, uint32_t n, float eps) {
  for (uint32_t base = 0; base + head_dim <= n; base += head_dim) {
    float sum = 0.0f;
    for (uint32_t i = 0; i < head_dim; ++i) {
      sum += values[base + i] * values[base + i];
    }
    const float mean_square = sum / (float)head_dim;
    const float scale = 1.0f / sqrtf(mean_square + eps);
    for (uint32_t i = 0; i < head_dim; ++i) {
      values[base + i] *= scale * decode(dtype, weight[i]);
    }
  }
}

/* precision/block/ops.rs:78-93: one serial ascending f32 sum per row.  Rows are
 * independent, so distributing them over threads does not change any bit. */
/* Summation-order probe (NOT the reference order): with lanes > 1 every row is
 * summed in `lanes` interleaved fp32 partial sums that are added at the end.
 * Tests use it to measure how far two equally valid fp32 evaluations of the
 * same contract drift apart (the floor under any logit tolerance). */
static int g_sum_lanes = 1;
void oracle_set_sum_lanes(int lanes) { g_sum_lanes = lanes < 1 ? 1 : (lanes > 16 ? 16 : lanes); }

static void matvec_lanes(uint32_t dtype, const uint16_t *matrix, const float *input,
                         uint32_t rows, uint32_t cols, float *output, int lanes) {
  const int threads = oracle_get_threads();
  (void)threads;
#pragma omp parallel for schedule(static) num_threads(threads) if (rows >= 64)
  for (int64_t row = 0; row < (int64_t)rows; ++row) {
    const uint16_t *w = matrix + (uint64_t)row * cols;
    float part[16] = {0};
    for (uint32_t col = 0; col < cols; ++col) {
      part[col % (uint32_t)lanes] += decode(dtype, w[col]) * input[col];
    }
    float sum = 0.0f;
    for (int l = 0; l < lanes; ++l) {
      sum += part[l];
    }
    output[row] = sum;
  }
}

void oracle_matvec(uint32_t dtype, const uint16_t *matrix, const float *input,
                   uint32_t rows, uint32_t cols, float *output) {
  const int threads = oracle_get_threads();
  (void)threads;
  if (g_sum_lanes > 1) {
    matvec_lanes(dtype, matrix, input, rows, cols, output, g_sum_lanes);
    return;
  }
  /* Eight rows advance together so that their eight independent add chains
   * overlap in the pipeline; each row's own sum is still col = 0, 1, 2, ... */
  const int64_t blocks = ((int64_t)rows + 7) / 8;
#pragma omp parallel for schedule(static) num_threads(threads) if (rows >= 64)
  for (int64_t block = 0; block < blocks; ++block) {
    const uint32_t row0 = (uint32_t)block * 8u;
    const uint32_t count = rows - row0 < 8u ? rows - row0 : 8u;
    if (count == 8u && dtype == ORACLE_DTYPE_BF16) {
      const uint16_t *w = matrix + (uint64_t)row0 * cols;
      float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
      float s4 = 0.0f, s5 = 0.0f, s6 = 0.0f, s7 = 0.0f;
      for (uint32_t col = 0; col < cols; ++col) {
        const float x = input[col];
        s0 += oracle_bf16_to_f32(w[col]) * x;
        s1 += oracle_bf16_to_f32(w[(uint64_t)cols + col]) * x;
        s2 += oracle_bf16_to_f32(w[(uint64_t)cols * 2 + col]) * x;
        s3 += oracle_bf16_to_f32(w[(uint64_t)cols * 3 + col]) * x;
        s4 += oracle_bf16_to_f32(w[(uint64_t)cols * 4 + col]) * x;
        s5 += oracle_bf16_to_f32(w[(uint64_t)cols * 5 + col]) * x;
        s6 += oracle_bf16_to_f32(w[(uint64_t)cols * 6 + col]) * x;
        s7 += oracle_bf16_to_f32(w[(uint64_t)cols * 7 + col]) * x;
      }
      float *out = output + row0;
      out[0] = s0; out[1] = s1; out[2] = s2; out[3] = s3;
      out[4] = s4; out[5] = s5; out[6] = s6; out[7] = s7;
      continue;
    }
    for (uint32_t r = 0; r < count; ++r) {
      const uint16_t *w = matrix + (uint64_t)(row0 + r) * cols;
      float sum = 0.0f;
      for (uint32_t col = 0; col < cols; ++col) {
        sum += decode(dtype, w[col]) * input[col];
      }
      output[row0 + r] = sum;
    }
  }
}

static void add_bias(uint32_t dtype, const uint16_t *bias, float *values, uint32_t n) {
  if (bias == NULL) {
    return;
  }
  for (uint32_t i = 0; i < n; ++i) {
    values[i] += decode(dtype, bias[i]);
  }
}

/* common/rope.rs:54-79: pairs (i, i + d/2), angle = pos / theta^(2i/d). */
void oracle_rope(float *values, uint32_t heads, uint32_t head_dim, uint32_t position,
                 float theta) {
  const uint32_t half = head_dim / 2;
  for (uint32_t head = 0; head < heads; ++head) {
    float *base = values + (uint64_t)head * head_dim;
    for (uint32_t offset = 0; offset < half; ++offset) {
      const float exponent = (float)(2 * offset) / (float)head_dim;
      const float angle = (float)position / powf(theta, exponent);
      const float s = sinf(angle);
      const float c = cosf(angle);
      const float left = base[offset];
      const float right = base[offset + half];
      base[offset] = left * c - right * s;
      base[offset + half] = right * c + left * s;
    }
  }
}

/* common/math.rs:76-78 */
float oracle_silu(float value) { return value / (1.0f + expf(-value)); }

static float oracle_sigmoid(float value) { return 1.0f / (1.0f + expf(-value)); }

/* attention/exact/run.rs:56-120 for one block holding every visible token:
 * the block-local pass is a token-serial online softmax; merging it into the
 * empty global accumulator multiplies by exp(0) = 1, then the output is divided
 * by the normaliser. */
static int attention_head(const float *q, uint32_t head_dim, uint32_t tokens,
                          const float *keys, const float *values, uint64_t token_stride,
                          float *local) {
  const float scale = 1.0f / sqrtf((float)head_dim);
  float local_m = -INFINITY;
  float local_l = 0.0f;
  for (uint32_t i = 0; i < head_dim; ++i) {
    local[i] = 0.0f;
  }
  for (uint32_t token = 0; token < tokens; ++token) {
    const float *k = keys + (uint64_t)token * token_stride;
    const float *v = values + (uint64_t)token * token_stride;
    float dot = 0.0f;
    for (uint32_t i = 0; i < head_dim; ++i) {
      dot += q[i] * k[i];
    }
    const float score = dot * scale;
    const float next_m = fmaxf(local_m, score);
    const float old_scale = local_l == 0.0f ? 0.0f : expf(local_m - next_m);
    const float new_scale = expf(score - next_m);
    for (uint32_t i = 0; i < head_dim; ++i) {
      local[i] = local[i] * old_scale + v[i] * new_scale;
    }
    local_l = local_l * old_scale + new_scale;
    local_m = next_m;
  }
  /* global merge: global_l == 0 -> global_scale = 0, local_scale = exp(0) */
  const float local_scale = expf(local_m - local_m);
  const float normalizer = 0.0f * 0.0f + local_l * local_scale;
  if (normalizer == 0.0f || !isfinite(normalizer)) {
    return -1;
  }
  for (uint32_t i = 0; i < head_dim; ++i) {
    const float merged = 0.0f * 0.0f + local[i] * local_scale;
    local[i] = merged / normalizer;
  }
  return 0;
}

int oracle_attention(const float *query, const float *keys, const float *values,
                     uint32_t tokens, uint32_t heads, uint32_t kv_heads, uint32_t head_dim,
                     float *output) {
  if (tokens == 0 || kv_heads == 0 || heads % kv_heads != 0) {
    return -1;
  }
  const uint32_t groups = heads / kv_heads;
  const uint64_t kv_hidden = (uint64_t)kv_heads * head_dim;
  int status = 0;
  const int threads = oracle_get_threads();
  (void)threads;
#pragma omp parallel for schedule(static) num_threads(threads) if (tokens >= 256)
  for (int64_t head = 0; head < (int64_t)heads; ++head) {
    const uint32_t kv_head = (uint32_t)head / groups; /* common/shape.rs:98-100 */
    const int rc = attention_head(query + (uint64_t)head * head_dim, head_dim, tokens,
                                  keys + (uint64_t)kv_head * head_dim,
                                  values + (uint64_t)kv_head * head_dim, kv_hidden,
                                  output + (uint64_t)head * head_dim);
    if (rc != 0) {
#pragma omp atomic write
      status = -1;
    }
  }
  return status;
}

int oracle_attention_paged(uint32_t dtype, const float *query, const uint16_t *key_pages,
                           const uint16_t *value_pages, const uint32_t *page_table,
                           uint32_t tokens, uint32_t heads, uint32_t kv_heads,
                           uint32_t head_dim, float *output) {
  if (tokens == 0 || kv_heads == 0 || heads % kv_heads != 0) {
    return -1;
  }
  const uint64_t kv_hidden = (uint64_t)kv_heads * head_dim;
  float *keys = (float *)malloc(sizeof(float) * tokens * kv_hidden);
  float *values = (float *)malloc(sizeof(float) * tokens * kv_hidden);
  if (keys == NULL || values == NULL) {
    free(keys);
    free(values);
    return -1;
  }
  for (uint32_t token = 0; token < tokens; ++token) {
    /* types.cuh:328-337 with layer_index = 0 */
    const uint64_t base = ((uint64_t)page_table[token / 16u] * 16u + token % 16u) * kv_hidden;
    for (uint64_t i = 0; i < kv_hidden; ++i) {
      keys[(uint64_t)token * kv_hidden + i] = decode(dtype, key_pages[base + i]);
      values[(uint64_t)token * kv_hidden + i] = decode(dtype, value_pages[base + i]);
    }
  }
  const int rc = oracle_attention(query, keys, values, tokens, heads, kv_heads, head_dim, output);
  free(keys);
  free(values);
  return rc;
}

int64_t oracle_argmax(const float *logits, uint32_t n, int mode) {
  if (n == 0) {
    return -1;
  }
  if (mode == ORACLE_MODE_CPU) {
    /* common/token.rs:33-58: first maximum wins, any non-finite value is an error */
    uint32_t best = 0;
    float best_value = logits[0];
    if (!isfinite(best_value)) {
      return -1;
    }
    for (uint32_t i = 1; i < n; ++i) {
      if (!isfinite(logits[i])) {
        return -1;
      }
      if (logits[i] > best_value) {
        best = i;
        best_value = logits[i];
      }
    }
    return best;
  }
  /* sampler.cu:35-40,89-119 */
  uint32_t best = 0;
  float best_value = -INFINITY;
  for (uint32_t i = 0; i < n; ++i) {
    const float v = logits[i];
    if (isfinite(v) && (v > best_value || (v == best_value && i < best))) {
      best = i;
      best_value = v;
    }
  }
  return best;
}

void oracle_route_softmax_topk(const float *router_logits, uint32_t num_experts,
                               uint32_t top_k, uint32_t norm_topk_prob,
                               uint32_t *experts, float *weights) {
  float max_logit = -INFINITY;
  for (uint32_t e = 0; e < num_experts; ++e) {
    max_logit = fmaxf(max_logit, router_logits[e]);
  }
  float total = 0.0f;
  for (uint32_t e = 0; e < num_experts; ++e) {
    total += expf(router_logits[e] - max_logit);
  }
  for (uint32_t rank = 0; rank < top_k; ++rank) {
    uint32_t best = UINT32_MAX;
    float best_weight = -INFINITY;
    for (uint32_t e = 0; e < num_experts; ++e) {
      int taken = 0;
      for (uint32_t prev = 0; prev < rank; ++prev) {
        taken |= experts[prev] == e;
      }
      if (taken) {
        continue;
      }
      float w = expf(router_logits[e] - max_logit);
      if (total > 0.0f && isfinite(total)) {
        w /= total;
      }
      if (w > best_weight || (w == best_weight && e < best)) {
        best_weight = w;
        best = e;
      }
    }
    experts[rank] = best;
    weights[rank] = best_weight;
  }
  if (norm_topk_prob != 0) {
    float sum = 0.0f;
    for (uint32_t rank = 0; rank < top_k; ++rank) {
      sum += weights[rank];
    }
    if (sum > 0.0f) {
      for (uint32_t rank = 0; rank < top_k; ++rank) {
        weights[rank] /= sum;
      }
    }
  }
}

uint64_t oracle_hash_tokens(const uint32_t *tokens, uint32_t count) {
  uint64_t hash = 0xcbf29ce484222325ull;
  for (uint32_t i = 0; i < count; ++i) {
    for (uint32_t byte = 0; byte < 4; ++byte) {
      hash ^= (uint64_t)((tokens[i] >> (8u * byte)) & 0xffu);
      hash *= 0x00000100000001b3ull;
    }
  }
  return hash;
}

/* ---- decoder ---- */

struct OracleCtx {
  OracleModel model;
  OracleLayer *layers;
  uint32_t max_context;
  int mode;
  uint32_t len;
  float *keys;   /* [layers][max_context][kv_hidden] */
  float *values;
  float *input, *attn_norm, *q, *k, *v, *attn, *residual, *mlp_norm;
  float *gate, *up, *ff, *down, *tmp, *hidden_f32, *router;
  uint16_t *hidden_bits, *next_bits;
  float *mla_q, *mla_kv, *mla_ql, *mla_lat, *mla_scores;  /* latent-attention scratch (attention_kind 2) */
};

static float *alloc_f32(uint64_t n) { return (float *)calloc(n ? n : 1, sizeof(float)); }

OracleCtx *oracle_create(const OracleModel *model, uint32_t max_context, int mode) {
  if (model == NULL || max_context == 0 || model->layers == 0 || model->kv_heads == 0 ||
      model->heads % model->kv_heads != 0 || model->dtype > ORACLE_DTYPE_BF16) {
    return NULL;
  }
  OracleCtx *ctx = (OracleCtx *)calloc(1, sizeof(OracleCtx));
  if (ctx == NULL) {
    return NULL;
  }
  ctx->model = *model;
  ctx->layers = (OracleLayer *)malloc(sizeof(OracleLayer) * model->layers);
  memcpy(ctx->layers, model->layer, sizeof(OracleLayer) * model->layers);
  ctx->model.layer = ctx->layers;
  ctx->max_context = max_context;
  ctx->mode = mode;
  const uint64_t hidden = model->hidden;
  const uint64_t attention_hidden = (uint64_t)model->heads * model->head_dim;
  const uint64_t kv_hidden = (uint64_t)model->kv_heads * model->head_dim;
  uint64_t inter = model->intermediate;
  uint32_t experts = 1;
  for (uint32_t l = 0; l < model->layers; ++l) {
    if (model->layer[l].num_experts > experts) {
      experts = model->layer[l].num_experts;
    }
  }
  ctx->keys = alloc_f32((uint64_t)model->layers * max_context * kv_hidden);
  ctx->values = alloc_f32((uint64_t)model->layers * max_context * kv_hidden);
  ctx->input = alloc_f32(hidden);
  ctx->attn_norm = alloc_f32(hidden);
  ctx->q = alloc_f32(attention_hidden);
  ctx->k = alloc_f32(kv_hidden);
  ctx->v = alloc_f32(kv_hidden);
  ctx->attn = alloc_f32(attention_hidden);
  ctx->residual = alloc_f32(hidden);
  ctx->mlp_norm = alloc_f32(hidden);
  ctx->gate = alloc_f32(inter);
  ctx->up = alloc_f32(inter);
  ctx->ff = alloc_f32(inter);
  ctx->down = alloc_f32(hidden);
  ctx->tmp = alloc_f32(hidden);
  ctx->hidden_f32 = alloc_f32(hidden);
  ctx->router = alloc_f32(experts);
  ctx->hidden_bits = (uint16_t *)calloc(hidden, sizeof(uint16_t));
  ctx->next_bits = (uint16_t *)calloc(hidden, sizeof(uint16_t));
  uint64_t mla_q = 0, mla_width = 0, mla_rank = 0;
  for (uint32_t l = 0; l < model->layers; ++l) {
    const OracleLayer *layer = &model->layer[l];
    if (layer->attention_kind != 2u) {
      continue;
    }
    const uint64_t q = (uint64_t)model->heads * (layer->qk_nope_head_dim + layer->qk_rope_head_dim);
    const uint64_t w = (uint64_t)layer->kv_lora_rank + layer->qk_rope_head_dim;
    mla_q = q > mla_q ? q : mla_q;
    mla_width = w > mla_width ? w : mla_width;
    mla_rank = layer->kv_lora_rank > mla_rank ? layer->kv_lora_rank : mla_rank;
  }
  if (mla_q != 0) {
    ctx->mla_q = alloc_f32(mla_q);
    ctx->mla_kv = alloc_f32(mla_width);
    ctx->mla_ql = alloc_f32((uint64_t)model->heads * mla_rank);
    ctx->mla_lat = alloc_f32((uint64_t)model->heads * mla_rank);
    ctx->mla_scores = alloc_f32(max_context);
  }
  return ctx;
}

void oracle_destroy(OracleCtx *ctx) {
  if (ctx == NULL) {
    return;
  }
  free(ctx->layers);
  free(ctx->keys);
  free(ctx->values);
  free(ctx->input);
  free(ctx->attn_norm);
  free(ctx->q);
  free(ctx->k);
  free(ctx->v);
  free(ctx->attn);
  free(ctx->residual);
  free(ctx->mlp_norm);
  free(ctx->gate);
  free(ctx->up);
  free(ctx->ff);
  free(ctx->down);
  free(ctx->tmp);
  free(ctx->hidden_f32);
  free(ctx->router);
  free(ctx->mla_q);
  free(ctx->mla_kv);
  free(ctx->mla_ql);
  free(ctx->mla_lat);
  free(ctx->mla_scores);
  free(ctx->hidden_bits);
  free(ctx->next_bits);
  free(ctx);
}

void oracle_reset(OracleCtx *ctx) { ctx->len = 0; }

uint32_t oracle_position(const OracleCtx *ctx) { return ctx->len; }

/* Timing aid of the CPU baseline: makes `position` the next position without running the
 * prompt, the cache rows in between filled with a fixed pattern.  A decode step at context n
 * does the same arithmetic whatever the cached values are, so the steps that follow cost what
 * they cost after a real n-token prefill; their tokens mean nothing. */
int oracle_seek_for_timing(OracleCtx *ctx, uint32_t position) {
  if (ctx == NULL || position > ctx->max_context || position < ctx->len) {
    return -1;
  }
  const OracleModel *m = &ctx->model;
  const uint64_t kv_hidden = (uint64_t)m->kv_heads * m->head_dim;
  for (uint32_t l = 0; l < m->layers; ++l) {
    for (uint64_t t = ctx->len; t < position; ++t) {
      float *k = ctx->keys + ((uint64_t)l * ctx->max_context + t) * kv_hidden;
      float *v = ctx->values + ((uint64_t)l * ctx->max_context + t) * kv_hidden;
      for (uint64_t i = 0; i < kv_hidden; ++i) {
        k[i] = 0.03125f * (float)((t + i) % 7) - 0.09375f;
        v[i] = 0.0625f * (float)((t + 3 * i) % 5) - 0.125f;
      }
    }
  }
  ctx->len = position;
  return 0;
}

const float *oracle_hidden_state(const OracleCtx *ctx) { return ctx->hidden_f32; }

static void round_vec(uint32_t dtype, float *values, uint64_t n) {
  for (uint64_t i = 0; i < n; ++i) {
    values[i] = round_to_dtype(dtype, values[i]);
  }
}

/* Dense SwiGLU MLP: precision/block/model/kv_finish.rs:39-65 (CPU) and
 * hf_decode_sequence/kernels.cu:597-612 (CUDA: ff rounded before down). */
static void dense_mlp(OracleCtx *ctx, const OracleLayer *layer, const float *x, float *down) {
  const OracleModel *m = &ctx->model;
  oracle_matvec(m->dtype, layer->w_gate, x, m->intermediate, m->hidden, ctx->gate);
  oracle_matvec(m->dtype, layer->w_up, x, m->intermediate, m->hidden, ctx->up);
  for (uint32_t i = 0; i < m->intermediate; ++i) {
    ctx->ff[i] = oracle_silu(ctx->gate[i]) * ctx->up[i];
  }
  if (ctx->mode == ORACLE_MODE_CUDA) {
    round_vec(m->dtype, ctx->ff, m->intermediate);
  }
  oracle_matvec(m->dtype, layer->w_down, ctx->ff, m->hidden, m->intermediate, down);
}

/* Softmax top-k sparse MoE: hf_decode_sequence/device_ops.cuh:183-315.  The
 * reference kernel feeds the f32 (unrounded) mlp_norm and ff to its mat_vec. */
static void sparse_moe_mlp(OracleCtx *ctx, const OracleLayer *layer, const float *x,
                           float *down) {
  const OracleModel *m = &ctx->model;
  const uint32_t hidden = m->hidden;
  const uint32_t mi = layer->moe_intermediate;
  uint32_t experts[16];
  float weights[16];
  for (uint32_t i = 0; i < hidden; ++i) {
    down[i] = 0.0f;
  }
  oracle_matvec(m->dtype, layer->w_router, x, layer->num_experts, hidden, ctx->router);
  oracle_route_softmax_topk(ctx->router, layer->num_experts, layer->top_k,
                            layer->norm_topk_prob, experts, weights);
  for (uint32_t rank = 0; rank < layer->top_k; ++rank) {
    const uint16_t *gate_w = layer->w_expert_gate_up + (uint64_t)experts[rank] * mi * 2u * hidden;
    const uint16_t *up_w = gate_w + (uint64_t)mi * hidden;
    const uint16_t *down_w = layer->w_expert_down + (uint64_t)experts[rank] * hidden * mi;
    oracle_matvec(m->dtype, gate_w, x, mi, hidden, ctx->gate);
    oracle_matvec(m->dtype, up_w, x, mi, hidden, ctx->up);
    for (uint32_t i = 0; i < mi; ++i) {
      ctx->ff[i] = oracle_silu(ctx->gate[i]) * ctx->up[i];
    }
    oracle_matvec(m->dtype, down_w, ctx->ff, hidden, mi, ctx->tmp);
    for (uint32_t i = 0; i < hidden; ++i) {
      down[i] += weights[rank] * ctx->tmp[i];
    }
  }
  if (layer->shared_intermediate != 0) {
    const uint32_t si = layer->shared_intermediate;
    float gate_weight = 0.0f;
    for (uint32_t i = 0; layer->w_shared_router != NULL && i < hidden; ++i) {
      gate_weight += decode(m->dtype, layer->w_shared_router[i]) * x[i];
    }
    oracle_matvec(m->dtype, layer->w_shared_gate, x, si, hidden, ctx->gate);
    oracle_matvec(m->dtype, layer->w_shared_up, x, si, hidden, ctx->up);
    for (uint32_t i = 0; i < si; ++i) {
      ctx->ff[i] = oracle_silu(ctx->gate[i]) * ctx->up[i];
    }
    oracle_matvec(m->dtype, layer->w_shared_down, ctx->ff, hidden, si, ctx->tmp);
    /* DeepSeek shared experts are always on: no router, scale 1 */
    const float shared_scale = layer->w_shared_router != NULL ? oracle_sigmoid(gate_weight) : 1.0f;
    for (uint32_t i = 0; i < hidden; ++i) {
      down[i] += shared_scale * ctx->tmp[i];
    }
  }
}

/* DeepSeek multi-head latent attention in its absorbed form, for one token (CUDA numeric contract:
 * bf16 mat-vec inputs, bf16 latent cache).  The reference has this attention only behind a query
 * low-rank stage and grouped-sigmoid routing (hf_decode_sequence/deepseek/
 * session_decode_v3_projection.inc.cu:1-624); the pieces restated here are its cache row
 * (kernels_v3_mla.inc.cu:1-61: normalised latent, then the rotary key with interleaved pairs on
 * inputs rounded to the model dtype), its rotary helper (kernels_helpers_math.inc.cu:236-262,
 * no YaRN scaling), its softmax scale rsqrt(nope + rope) (:166-180) and the absorbed algebra of
 * the stand-alone operator (native/cuda/deepseek/nerva_cuda_deepseek_mla.cu:144-227):
 *   ql[h] = q_nope[h] . W_UK[h];  s[h][t] = (ql[h] . c[t] + q_pe[h] . k_pe[t]) * scale;
 *   lat[h] = sum_t softmax(s)[t] c[t];  out[h] = W_UV[h] . lat[h].
 * Writes heads * head_dim values to ctx->attn. */
static void rope_interleaved(float *values, uint32_t dim, uint32_t position, float theta) {
  if (!(theta > 0.0f) || dim < 2) {
    return;
  }
  for (uint32_t pair = 0; pair < dim / 2u; ++pair) {
    const float exponent = (float)(2u * pair) / (float)dim;
    const float angle = (float)position * (1.0f / powf(theta, exponent));
    const float s = sinf(angle), c = cosf(angle);
    const float left = values[2u * pair], right = values[2u * pair + 1u];
    values[2u * pair] = left * c - right * s;
    values[2u * pair + 1u] = right * c + left * s;
  }
}

static int mla_attention(OracleCtx *ctx, const OracleLayer *layer, uint32_t layer_index,
                         uint32_t position) {
  const OracleModel *m = &ctx->model;
  const uint32_t dtype = m->dtype, hidden = m->hidden, heads = m->heads;
  const uint32_t rank = layer->kv_lora_rank, nope = layer->qk_nope_head_dim;
  const uint32_t rope = layer->qk_rope_head_dim, vdim = m->head_dim;
  const uint32_t width = rank + rope, qdim = nope + rope;
  const uint64_t stride = (uint64_t)m->kv_heads * m->head_dim;  /* cache row stride of this context */
  if (width > stride) {
    return -1;
  }
  oracle_matvec(dtype, layer->w_q, ctx->attn_norm, heads * qdim, hidden, ctx->mla_q);
  oracle_matvec(dtype, layer->w_kv_a, ctx->attn_norm, width, hidden, ctx->mla_kv);
  /* cache row: bf16(rmsnorm(latent) * w) | bf16(rope(bf16(k_pe))) */
  float *row = ctx->keys + ((uint64_t)layer_index * ctx->max_context + position) * stride;
  oracle_rms_norm(dtype, ctx->mla_kv, layer->kv_a_norm, rank, m->rms_eps, row);
  for (uint32_t i = 0; i < rope; ++i) {
    row[rank + i] = round_to_dtype(dtype, ctx->mla_kv[rank + i]);
  }
  rope_interleaved(row + rank, rope, position, m->rope_theta);
  round_vec(dtype, row, width);
  const float scale = 1.0f / sqrtf((float)qdim);
  for (uint32_t h = 0; h < heads; ++h) {
    float *q = ctx->mla_q + (uint64_t)h * qdim;
    rope_interleaved(q + nope, rope, position, m->rope_theta);
    /* absorbed query: ql[r] = sum_n q[n] W_UK[h][n][r] */
    float *ql = ctx->mla_ql + (uint64_t)h * rank;
    const uint16_t *w_uk = layer->w_kv_b + (uint64_t)h * (nope + vdim) * rank;
    for (uint32_t r = 0; r < rank; ++r) {
      ql[r] = 0.0f;
    }
    for (uint32_t n = 0; n < nope; ++n) {
      const float qn = q[n];
      for (uint32_t r = 0; r < rank; ++r) {
        ql[r] += qn * decode(dtype, w_uk[(uint64_t)n * rank + r]);
      }
    }
    float top = -INFINITY;
    for (uint32_t t = 0; t <= position; ++t) {
      const float *c = ctx->keys + ((uint64_t)layer_index * ctx->max_context + t) * stride;
      float s = 0.0f;
      for (uint32_t r = 0; r < rank; ++r) {
        s += ql[r] * c[r];
      }
      for (uint32_t i = 0; i < rope; ++i) {
        s += q[nope + i] * c[rank + i];
      }
      ctx->mla_scores[t] = s * scale;
      if (ctx->mla_scores[t] > top) {
        top = ctx->mla_scores[t];
      }
    }
    float total = 0.0f;
    float *lat = ctx->mla_lat + (uint64_t)h * rank;
    for (uint32_t r = 0; r < rank; ++r) {
      lat[r] = 0.0f;
    }
    for (uint32_t t = 0; t <= position; ++t) {
      const float p = expf(ctx->mla_scores[t] - top);
      const float *c = ctx->keys + ((uint64_t)layer_index * ctx->max_context + t) * stride;
      total += p;
      for (uint32_t r = 0; r < rank; ++r) {
        lat[r] += p * c[r];
      }
    }
    const uint16_t *w_uv = w_uk + (uint64_t)nope * rank;
    for (uint32_t v = 0; v < vdim; ++v) {
      float acc = 0.0f;
      for (uint32_t r = 0; r < rank; ++r) {
        acc += (lat[r] / total) * decode(dtype, w_uv[(uint64_t)v * rank + r]);
      }
      ctx->attn[(uint64_t)h * vdim + v] = acc;
    }
  }
  return 0;
}

/* One layer for one token at `position`.
 * CPU : precision/block/model/kv.rs:94-205 + kv_finish.rs:10-75.
 * CUDA: hf_decode_sequence/session_decode_prefill.inc.cu:74-372 (K1..K9). */
static int layer_forward(OracleCtx *ctx, uint32_t layer_index, uint32_t position) {
  const OracleModel *m = &ctx->model;
  const OracleLayer *layer = &ctx->layers[layer_index];
  const uint32_t dtype = m->dtype;
  const uint32_t hidden = m->hidden;
  const uint32_t attention_hidden = m->heads * m->head_dim;
  const uint32_t kv_hidden = m->kv_heads * m->head_dim;
  const int cuda = ctx->mode == ORACLE_MODE_CUDA;

  oracle_rms_norm(dtype, ctx->input, layer->rms_attn, hidden, m->rms_eps, ctx->attn_norm);
  if (cuda) {
    round_vec(dtype, ctx->attn_norm, hidden);
  }
  if (layer->attention_kind == 2u) {
    if (mla_attention(ctx, layer, layer_index, position) != 0) {
      return -1;
    }
    goto attention_done;
  }
  /* K: mat-vec, bias, k-norm, (V: mat-vec, bias), RoPE on K  — kv.rs:113-141 */
  oracle_matvec(dtype, layer->w_k, ctx->attn_norm, kv_hidden, hidden, ctx->k);
  add_bias(dtype, layer->k_bias, ctx->k, kv_hidden);
  if (layer->k_norm != NULL) {
    oracle_per_head_rms_norm(dtype, layer->k_norm, m->head_dim, ctx->k, kv_hidden, m->rms_eps);
  }
  oracle_matvec(dtype, layer->w_v, ctx->attn_norm, kv_hidden, hidden, ctx->v);
  add_bias(dtype, layer->v_bias, ctx->v, kv_hidden);
  if (m->rope_theta > 0.0f) {
    oracle_rope(ctx->k, m->kv_heads, m->head_dim, position, m->rope_theta);
  }
  if (cuda || ctx->mode == ORACLE_MODE_CPU_KV16) {
    round_vec(dtype, ctx->k, kv_hidden);
    round_vec(dtype, ctx->v, kv_hidden);
  }
  float *layer_keys = ctx->keys + (uint64_t)layer_index * ctx->max_context * kv_hidden;
  float *layer_values = ctx->values + (uint64_t)layer_index * ctx->max_context * kv_hidden;
  memcpy(layer_keys + (uint64_t)position * kv_hidden, ctx->k, sizeof(float) * kv_hidden);
  memcpy(layer_values + (uint64_t)position * kv_hidden, ctx->v, sizeof(float) * kv_hidden);

  /* Q: kv.rs:160-175 */
  oracle_matvec(dtype, layer->w_q, ctx->attn_norm, attention_hidden, hidden, ctx->q);
  add_bias(dtype, layer->q_bias, ctx->q, attention_hidden);
  if (layer->q_norm != NULL) {
    oracle_per_head_rms_norm(dtype, layer->q_norm, m->head_dim, ctx->q, attention_hidden,
                             m->rms_eps);
  }
  if (m->rope_theta > 0.0f) {
    oracle_rope(ctx->q, m->heads, m->head_dim, position, m->rope_theta);
  }
  if (oracle_attention(ctx->q, layer_keys, layer_values, position + 1, m->heads, m->kv_heads,
                       m->head_dim, ctx->attn) != 0) {
    return -1;
  }
attention_done:
  if (cuda) {
    round_vec(dtype, ctx->attn, attention_hidden);
  }
  /* kv_finish.rs:15-38 */
  oracle_matvec(dtype, layer->w_o, ctx->attn, hidden, attention_hidden, ctx->residual);
  add_bias(dtype, layer->o_bias, ctx->residual, hidden);
  for (uint32_t i = 0; i < hidden; ++i) {
    ctx->residual[i] += ctx->input[i];
  }
  oracle_rms_norm(dtype, ctx->residual, layer->rms_mlp, hidden, m->rms_eps, ctx->mlp_norm);
  if (cuda && layer->mlp_kind == 0) {
    round_vec(dtype, ctx->mlp_norm, hidden);
  }
  if (layer->mlp_kind == 0) {
    dense_mlp(ctx, layer, ctx->mlp_norm, ctx->down);
  } else {
    sparse_moe_mlp(ctx, layer, ctx->mlp_norm, ctx->down);
  }
  for (uint32_t i = 0; i < hidden; ++i) {
    ctx->residual[i] += ctx->down[i];
  }
  if (cuda) {
    /* kernels.cu:651-668: the stream stays f32 */
    memcpy(ctx->input, ctx->residual, sizeof(float) * hidden);
  } else {
    /* kv_finish.rs:74: re-encode between layers */
    for (uint32_t i = 0; i < hidden; ++i) {
      ctx->next_bits[i] = encode(dtype, ctx->residual[i]);
      ctx->input[i] = decode(dtype, ctx->next_bits[i]);
    }
  }
  return 0;
}

int oracle_step(OracleCtx *ctx, uint32_t token, float *logits) {
  const OracleModel *m = &ctx->model;
  if (token >= m->vocab || ctx->len >= ctx->max_context) {
    return -1;
  }
  const uint32_t position = ctx->len;
  /* causal_lm/decode.rs: copy_embedding_into + decode_vec_into */
  for (uint32_t i = 0; i < m->hidden; ++i) {
    ctx->input[i] = decode(m->dtype, m->embeddings[(uint64_t)token * m->hidden + i]);
  }
  for (uint32_t l = 0; l < m->layers; ++l) {
    if (layer_forward(ctx, l, position) != 0) {
      return -1;
    }
  }
  memcpy(ctx->hidden_f32, ctx->input, sizeof(float) * m->hidden);
  ctx->len = position + 1;
  if (logits != NULL) {
    /* causal_lm/decode.rs:82-101 (sample_current_hidden) */
    oracle_rms_norm(m->dtype, ctx->input, m->final_norm, m->hidden, m->rms_eps, ctx->attn_norm);
    if (ctx->mode == ORACLE_MODE_CUDA) {
      round_vec(m->dtype, ctx->attn_norm, m->hidden);
    }
    oracle_matvec(m->dtype, m->lm_head, ctx->attn_norm, m->vocab, m->hidden, logits);
  }
  return 0;
}

int oracle_decode_greedy(OracleCtx *ctx, const uint32_t *prompt, uint32_t prompt_count,
                         uint32_t steps, uint32_t *tokens_out, float *logits_out) {
  const OracleModel *m = &ctx->model;
  if (prompt == NULL || prompt_count == 0 || steps == 0 || tokens_out == NULL ||
      (uint64_t)prompt_count + steps - 1 > ctx->max_context) {
    return -1;
  }
  for (uint32_t i = 0; i < prompt_count; ++i) {
    if (prompt[i] >= m->vocab) {
      return -1;
    }
  }
  float *scratch_logits = logits_out != NULL ? NULL : alloc_f32(m->vocab);
  oracle_reset(ctx);
  int produced = 0;
  uint32_t current = 0;
  for (uint32_t i = 0; i + 1 < prompt_count; ++i) {
    if (oracle_step(ctx, prompt[i], NULL) != 0) {
      produced = -1;
      goto done;
    }
  }
  current = prompt[prompt_count - 1];
  for (uint32_t step = 0; step < steps; ++step) {
    float *logits = logits_out != NULL ? logits_out + (uint64_t)step * m->vocab : scratch_logits;
    if (oracle_step(ctx, current, logits) != 0) {
      produced = -1;
      goto done;
    }
    const int64_t next = oracle_argmax(logits, m->vocab, ctx->mode);
    if (next < 0) {
      produced = -1;
      goto done;
    }
    current = (uint32_t)next;
    tokens_out[step] = current;
    produced = (int)(step + 1);
  }
done:
  free(scratch_logits);
  return produced;
}
