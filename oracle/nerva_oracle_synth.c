/*
 * TEST INFRASTRUCTURE — NOT A PRODUCT CODE PATH.
 *
 * Multi-threaded fill of synthetic bf16 tensors with the counter-based
 * generator of include/nerva_synth.h, so that the oracle, the golden-vector
 * script and the CPU arm of the benchmark can build the full-size synthetic
 * checkpoints (random-init BF16 ~N(0, 0.02), seed 0) without loading the CUDA
 * library.  Same bits as nerva_b200.synth.normal_bf16 and the device fill.
 */
#include <stdint.h>

#include "nerva_synth.h"

static float synth_scale(float std) { return std * (1.0f / 65536.0f); }

void oracle_synth_normal_bf16(uint64_t seed, uint64_t tensor_id, uint64_t count, float std,
                              uint16_t *out) {
  const uint64_t key = nerva_synth_key(seed, tensor_id);
  const float scale = synth_scale(std);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)count; ++i) {
    out[i] = nerva_synth_normal_bf16(key, (uint64_t)i, scale);
  }
}

/* Rows [row_begin, row_begin + rows) x columns [col_begin, col_begin + cols) of the
 * row-major tensor with `full_cols` columns: the slice one tensor-parallel rank holds. */
void oracle_synth_normal_bf16_block(uint64_t seed, uint64_t tensor_id, uint64_t full_cols,
                                    uint64_t row_begin, uint64_t rows, uint64_t col_begin,
                                    uint64_t cols, float std, uint16_t *out) {
  const uint64_t key = nerva_synth_key(seed, tensor_id);
  const float scale = synth_scale(std);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < (int64_t)rows; ++r) {
    const uint64_t base = (row_begin + (uint64_t)r) * full_cols + col_begin;
    uint16_t *dst = out + (uint64_t)r * cols;
    for (uint64_t c = 0; c < cols; ++c) dst[c] = nerva_synth_normal_bf16(key, base + c, scale);
  }
}
