// Warp-level tensor-pipe helpers shared by the attention kernels: mma.sync m16n8k16 (bf16 in, fp32
// accumulate), ldmatrix, and the split of fp32 values into a bf16 rounding and what it lost.
//
// Fragment layout of m16n8k16 with g = lane / 4, t = lane % 4:
//   A (16 x 16, row-major)  a[0] = A[g][2t, 2t+1]   a[1] = A[g+8][2t, 2t+1]
//                           a[2] = A[g][2t+8, +9]   a[3] = A[g+8][2t+8, +9]
//   B (16 x 8, "col")       b0 = B[2t, 2t+1][g]     b1 = B[2t+8, 2t+9][g]
//   C/D (16 x 8, fp32)      c[0], c[1] = C[g][2t, 2t+1]   c[2], c[3] = C[g+8][2t, 2t+1]
#pragma once

#include "common.cuh"

namespace nb {

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
// Four 8 x 8 matrices (row addresses from lanes 0-7, 8-15, 16-23, 24-31), each transposed on the way:
// lane (g, t) receives rows 2t, 2t+1 of column g, the B fragment of a matrix stored [k][n].
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Two fp32 values -> one register of two bf16 roundings (low half first), and what the rounding lost.
__device__ __forceinline__ uint32_t pack_bf16_hi(float x, float y) {
  return static_cast<uint32_t>(f32_to_bf16_bits(x)) | (static_cast<uint32_t>(f32_to_bf16_bits(y)) << 16);
}
__device__ __forceinline__ uint32_t pack_bf16_lo(float x, float y) {
  return pack_bf16_hi(x - bf16_round(x), y - bf16_round(y));
}

}  // namespace nb
