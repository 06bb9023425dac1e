/*
 * Counter-based synthetic input generator shared by the CUDA library, the CPU
 * oracle and the Python harness.
 *
 * The reference ships no checkpoint and no dataset for the decode path; its
 * benchmark configurations are "random-init BF16 weights ~N(0, 0.02), seed 0;
 * prompt ids uniform over [0, vocab), seed 1".  To let a C program, a CUDA
 * kernel and numpy produce the *same bits* without sharing a library RNG, every
 * value is a pure function of (seed, tensor id, element index) computed with
 * integer arithmetic only, followed by exactly one IEEE float multiply and one
 * round-to-nearest-even narrowing:
 *
 *   key   = mix64(seed * GAMMA + tensor_id)
 *   h_j   = mix64(key + (3 * index + j + 1) * GAMMA)            j = 0, 1, 2
 *   s     = sum of the twelve 16-bit fields of h_0, h_1, h_2     (Irwin-Hall, n = 12)
 *   z     = (s - 6 * 65535)                                      integer, sd = 65536 (to 1e-10)
 *   value = (float)z * (std * 2^-16)                             one f32 multiply
 *   bits  = bf16_rne(value)
 *
 * Irwin-Hall with n = 12 has unit variance after the 2^-16 scaling, zero skew,
 * excess kurtosis -0.1 and support +-6 sd.
 */
#ifndef NERVA_SYNTH_H_
#define NERVA_SYNTH_H_

#include <stdint.h>

#if defined(__CUDACC__)
#define NERVA_SYNTH_FN static __host__ __device__ __forceinline__
#else
#define NERVA_SYNTH_FN static inline
#endif

#define NERVA_SYNTH_GAMMA 0x9E3779B97F4A7C15ull

NERVA_SYNTH_FN uint64_t nerva_synth_mix64(uint64_t z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

NERVA_SYNTH_FN uint64_t nerva_synth_key(uint64_t seed, uint64_t tensor_id) {
  return nerva_synth_mix64(seed * NERVA_SYNTH_GAMMA + tensor_id);
}

NERVA_SYNTH_FN uint64_t nerva_synth_u64(uint64_t key, uint64_t counter) {
  return nerva_synth_mix64(key + (counter + 1ull) * NERVA_SYNTH_GAMMA);
}

NERVA_SYNTH_FN uint32_t nerva_synth_fields16(uint64_t h) {
  return (uint32_t)(h & 0xffffu) + (uint32_t)((h >> 16) & 0xffffu) +
         (uint32_t)((h >> 32) & 0xffffu) + (uint32_t)(h >> 48);
}

/* Integer approximately N(0, 65536^2). */
NERVA_SYNTH_FN int32_t nerva_synth_normal_i32(uint64_t key, uint64_t index) {
  const uint64_t c = 3ull * index;
  const uint32_t s = nerva_synth_fields16(nerva_synth_u64(key, c)) +
                     nerva_synth_fields16(nerva_synth_u64(key, c + 1ull)) +
                     nerva_synth_fields16(nerva_synth_u64(key, c + 2ull));
  return (int32_t)s - 6 * 65535;
}

NERVA_SYNTH_FN uint16_t nerva_synth_f32_to_bf16(float value) {
  union { float f; uint32_t u; } v;
  v.f = value;
  const uint32_t bits = v.u;
  if ((bits & 0x7f800000u) == 0x7f800000u && (bits & 0x007fffffu) != 0u) {
    return (uint16_t)((bits >> 16) | 1u);
  }
  const uint32_t lsb = (bits >> 16) & 1u;
  return (uint16_t)((bits + 0x7fffu + lsb) >> 16);
}

/* scale must be (float)std * 2^-16, computed once by the caller. */
NERVA_SYNTH_FN float nerva_synth_normal_f32(uint64_t key, uint64_t index, float scale) {
  return (float)nerva_synth_normal_i32(key, index) * scale;
}

NERVA_SYNTH_FN uint16_t nerva_synth_normal_bf16(uint64_t key, uint64_t index, float scale) {
  return nerva_synth_f32_to_bf16(nerva_synth_normal_f32(key, index, scale));
}

NERVA_SYNTH_FN uint32_t nerva_synth_uniform_u32(uint64_t key, uint64_t index, uint32_t bound) {
  return (uint32_t)(nerva_synth_u64(key, index) % (uint64_t)bound);
}

/* Tensor ids of the synthetic decoder checkpoints. */
enum {
  NERVA_SYNTH_T_EMBEDDINGS = 1,
  NERVA_SYNTH_T_LM_HEAD = 2,
  NERVA_SYNTH_T_PROMPT = 3,
  NERVA_SYNTH_T_PAGE_TABLE = 4,
  NERVA_SYNTH_T_ACTIVATION = 5,
  NERVA_SYNTH_T_LAYER_BASE = 1000, /* + layer * 64 + slot */
  NERVA_SYNTH_L_WQ = 0,
  NERVA_SYNTH_L_WK = 1,
  NERVA_SYNTH_L_WV = 2,
  NERVA_SYNTH_L_WO = 3,
  NERVA_SYNTH_L_WGATE = 4,
  NERVA_SYNTH_L_WUP = 5,
  NERVA_SYNTH_L_WDOWN = 6,
  NERVA_SYNTH_L_ROUTER = 7,
  NERVA_SYNTH_L_EXPERT_GATE_UP = 8,
  NERVA_SYNTH_L_EXPERT_DOWN = 9,
  NERVA_SYNTH_L_SHARED_GATE = 10,
  NERVA_SYNTH_L_SHARED_UP = 11,
  NERVA_SYNTH_L_SHARED_DOWN = 12,
  NERVA_SYNTH_L_Q_A = 13,
  NERVA_SYNTH_L_Q_B = 14,
  NERVA_SYNTH_L_KV_A = 15,
  NERVA_SYNTH_L_KV_B = 16,
  NERVA_SYNTH_L_K = 17,
  NERVA_SYNTH_L_V = 18,
  NERVA_SYNTH_L_Q = 19,
  NERVA_SYNTH_L_SHARED_ROUTER = 20
};

#endif /* NERVA_SYNTH_H_ */
