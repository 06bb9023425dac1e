/* CPU oracle (test infrastructure): the temperature / top-k / top-p token sampler of the
 * resident decode step, restated from the reference's device sampler
 * (native/cuda/hf_decode_sequence/sampler.cu:18-33 randomness, :88-160 arg-max and
 * Gumbel-max, :161-392 top-k / top-p).
 *
 * Pinning: the reference holds no known-answer test for this sampler and has no CPU twin of
 * it, so this restatement is checked, on a GPU, against the reference's own kernel compiled
 * from its source (oracle/ref_sampler.cu -> oracle/_ref/libnerva_ref_sampler.so).  logf and
 * expf here are glibc's and the device's differ from them in the last place, so a decision
 * that hangs on the last bits can fall the other way: oracle_sample_token reports how close
 * the decision was, and the tests compare tokens wherever it was not a near tie.
 *
 *   greedy       !(temperature > 0) or top_k == 1: largest finite logit, lowest index on ties,
 *                token 0 when nothing is finite
 *   Gumbel-max   top_k == 0 and top_p >= 0.999999: arg-max over finite logits of
 *                fma(logit, 1/temperature, -log(-log(u(seed, position, index, 0))))
 *                (the device compiler contracts the multiply-add, hence fmaf here)
 *   top-k/top-p  c = min(top_k or 128, 128, vocab) best finite logits by (value descending,
 *                index ascending); w_r = exp((v_r - v_0) / temperature) summed in rank order;
 *                the shortest prefix with mass / total >= top_p (all of them when
 *                top_p >= 0.999999); draw = u(seed, position, 0, 1) * kept mass; the first rank
 *                whose running sum reaches the draw, else the last kept rank
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

#define SAMPLER_TOP_K_MAX 128u

static uint64_t mix64(uint64_t v) {
  v += 0x9e3779b97f4a7c15ull;
  v = (v ^ (v >> 30)) * 0xbf58476d1ce4e5b9ull;
  v = (v ^ (v >> 27)) * 0x94d049bb133111ebull;
  return v ^ (v >> 31);
}

/* Uniform in (0, 1) from 24 bits of the mixed counter (sampler.cu:25-33). */
float oracle_sampler_uniform(uint64_t seed, uint32_t position, uint32_t token, uint32_t salt) {
  const uint64_t v = mix64(seed ^ ((uint64_t)position << 32) ^ (uint64_t)token ^ ((uint64_t)salt << 48));
  const uint32_t mantissa = (uint32_t)((v >> 40) & 0x00ffffffu);
  return ((float)mantissa + 1.0f) / 16777217.0f;
}

typedef struct {
  float value;
  uint32_t index;
} Candidate;

static int better(float v, uint32_t i, float bv, uint32_t bi) { return v > bv || (v == bv && i < bi); }

static int by_rank(const void *a, const void *b) {
  const Candidate *x = (const Candidate *)a, *y = (const Candidate *)b;
  if (better(x->value, x->index, y->value, y->index)) return -1;
  if (better(y->value, y->index, x->value, x->index)) return 1;
  return 0;
}

/* Returns the token.  *margin (nullable) receives the relative distance of the closest
 * comparison the choice depended on (INFINITY for the arg-max branch). */
uint32_t oracle_sample_token(const float *logits, uint32_t vocab, uint32_t position, float temperature,
                             float top_p, uint32_t top_k, uint64_t seed, float *margin) {
  float closest = INFINITY;
  uint32_t token = 0;
  if (!(temperature > 0.0f) || top_k == 1) {
    float bv = -INFINITY;
    uint32_t bi = 0;
    for (uint32_t i = 0; i < vocab; ++i)
      if (isfinite(logits[i]) && better(logits[i], i, bv, bi)) {
        bv = logits[i];
        bi = i;
      }
    token = bi;
  } else if (top_k == 0 && top_p >= 0.999999f) {
    const float inv_temperature = 1.0f / temperature;
    float bv = -INFINITY, second = -INFINITY;
    uint32_t bi = 0;
    for (uint32_t i = 0; i < vocab; ++i) {
      if (!isfinite(logits[i])) continue;
      const float gumbel = -logf(-logf(oracle_sampler_uniform(seed, position, i, 0)));
      const float noisy = fmaf(logits[i], inv_temperature, gumbel);
      if (better(noisy, i, bv, bi)) {
        second = bv;
        bv = noisy;
        bi = i;
      } else if (noisy > second) {
        second = noisy;
      }
    }
    token = bi;
    if (isfinite(second)) closest = (bv - second) / fmaxf(1.0f, fabsf(bv));
  } else {
    Candidate *all = (Candidate *)malloc(sizeof(Candidate) * (vocab ? vocab : 1u));
    if (all == NULL) return 0;
    uint32_t finite = 0;
    for (uint32_t i = 0; i < vocab; ++i)
      if (isfinite(logits[i])) {
        all[finite].value = logits[i];
        all[finite].index = i;
        ++finite;
      }
    qsort(all, finite, sizeof(Candidate), by_rank);
    uint32_t want = top_k == 0 ? SAMPLER_TOP_K_MAX : (top_k < SAMPLER_TOP_K_MAX ? top_k : SAMPLER_TOP_K_MAX);
    if (want > vocab) want = vocab;
    const uint32_t selected = finite < want ? finite : want;
    if (selected != 0) {
      const float inv_temperature = 1.0f / temperature;
      float weight[SAMPLER_TOP_K_MAX];
      float total = 0.0f;
      for (uint32_t r = 0; r < selected; ++r) {
        weight[r] = expf((all[r].value - all[0].value) * inv_temperature);
        total += weight[r];
      }
      float kept_mass = total;
      uint32_t kept = selected;
      if (top_p < 0.999999f) {
        kept_mass = 0.0f;
        kept = 0;
        for (uint32_t r = 0; r < selected; ++r) {
          const float before = kept_mass;
          kept_mass += weight[r];
          kept = r + 1;
          if (total > 0.0f && kept_mass / total >= top_p) {
            closest = fminf(closest, fabsf(kept_mass / total - top_p));
            if (r != 0) closest = fminf(closest, fabsf(before / total - top_p));
            break;
          }
        }
      }
      token = all[0].index;
      if (kept_mass > 0.0f && kept != 0) {
        const float draw = oracle_sampler_uniform(seed, position, 0, 1) * kept_mass;
        float running = 0.0f;
        uint32_t r = 0;
        for (; r + 1 < kept; ++r) {
          running += weight[r];
          if (draw <= running) break;
        }
        token = all[r].index;
        /* distance of the draw from the two boundaries of the chosen rank */
        const float upper = r + 1 < kept ? running : kept_mass;
        const float lower = r + 1 < kept ? running - weight[r] : running;
        if (r + 1 < kept) closest = fminf(closest, fabsf(upper - draw) / kept_mass);
        if (r != 0) closest = fminf(closest, fabsf(draw - lower) / kept_mass);
      }
    }
    free(all);
  }
  if (margin != NULL) *margin = closest;
  return token;
}
