// Device-side building blocks shared by every kernel of the decode step:
// bf16 codecs, warp/block reductions, mbarrier + bulk-TMA wrappers with bounded
// waits, and the device error word.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace nb {

constexpr uint32_t kWarp = 32;

// Device error codes written (atomicMax) to the session's error word.  A
// kernel that gives up a wait records where and returns; it never traps.
enum DeviceError : uint32_t {
  kErrNone = 0,
  kErrTmaWaitTimeout = 1,
  kErrGridBarrierTimeout = 2,
  kErrPageOutOfRange = 3,
  kErrTokenOutOfRange = 4,
  kErrCursorOutOfRange = 5,
  kErrPeerWaitTimeout = 6,
};

// ---- bf16 ----
// Same rounding as the reference's device codec (hf_decode_sequence/device_ops.cuh:24-31).
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float value) {
  const uint32_t bits = __float_as_uint(value);
  const uint32_t lsb = (bits >> 16) & 1u;
  return static_cast<uint16_t>((bits + 0x7fffu + lsb) >> 16);
}
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t bits) {
  return __uint_as_float(static_cast<uint32_t>(bits) << 16);
}
__device__ __forceinline__ float bf16_round(float value) {
  return bf16_bits_to_f32(f32_to_bf16_bits(value));
}
// A 32-bit word holding two bf16 values (element 0 in the low half).
__device__ __forceinline__ float bf16x2_lo(uint32_t word) { return __uint_as_float(word << 16); }
__device__ __forceinline__ float bf16x2_hi(uint32_t word) {
  return __uint_as_float(word & 0xffff0000u);
}

// ---- reductions ----
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1)
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
  return v;
}
// Block-wide sum; `scratch` holds >= 33 floats of shared memory.  All threads
// of the block must call it; every thread receives the total.
__device__ __forceinline__ float block_sum(float v, float *scratch) {
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t warps = (blockDim.x + 31u) >> 5;
  v = warp_sum(v);
  __syncthreads();  // protects scratch from the previous use
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < warps ? scratch[lane] : 0.0f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// ---- shared-memory address / mbarrier / bulk TMA ----
__device__ __forceinline__ uint32_t smem_addr(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals)
               : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  // Makes the initialised barriers visible to the async (TMA) proxy.
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
// Bounded wait: polls until the phase completes or ~kWaitCycleLimit SM cycles
// (about a second) have passed.  Returns false on timeout.
constexpr long long kWaitCycleLimit = 2000000000ll;
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  for (;;) {
#pragma unroll 1
    for (uint32_t spin = 0; spin < 64; ++spin) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (clock64() - start > kWaitCycleLimit) return false;
  }
}
// Generic-proxy accesses (the reads that just consumed a slot) are ordered
// before the async-proxy write that refills it.
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// 1-D bulk copy global -> shared, completion counted on `bar`.  Both addresses
// 16-byte aligned, `bytes` a multiple of 16.  No multicast.
__device__ __forceinline__ void tma_load_1d(void *smem_dst, const void *gmem_src, uint32_t bytes,
                                            uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(smem_addr(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
      : "memory");
}
// L2 policy for data that is read once per step (the weights): first in line for
// eviction, so that 15 GB of weight traffic per token does not push the small
// per-token working set (KV pages, norm weights, page table, activations) out
// of the 126 MB L2.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ void tma_load_1d_hint(void *smem_dst, const void *gmem_src, uint32_t bytes,
                                                 uint64_t *bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1], %2, [%3], %4;" ::"r"(smem_addr(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar)), "l"(policy)
      : "memory");
}

// ---- programmatic dependent launch ----
// A kernel launched with the programmatic-serialization attribute may start
// while its predecessor in the stream is still running.  Everything it does
// before pdl_wait() must be independent of the predecessor (set-up, weight
// prefetch); pdl_wait() returns once the predecessor has completed and its
// writes are visible.  pdl_trigger() lets the successor start launching.  Both
// are no-ops for a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---- waits on other GPUs (tensor-parallel exchange) ----
// A wait on a peer gives up after kPeerWaitCycleLimit SM cycles (about a second: ranks are separate
// processes, so the limit has to cover launch skew between them) and records kErrPeerWaitTimeout.
// The error word stays set until the next request starts, and a wait whose first poll misses
// looks at it before it looks at the clock: once one exchange has failed, the steps already
// queued behind it run through without waiting again, so a rank that died costs the others one
// limit, not one per exchange.  A wait whose data is already there never reads the word.
constexpr long long kPeerWaitCycleLimit = kWaitCycleLimit;
__device__ __forceinline__ bool step_already_failed(const uint32_t *error_word) {
  return error_word != nullptr && *reinterpret_cast<const volatile uint32_t *>(error_word) != 0u;
}

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
// Bounded wait until *counter >= expected; false on timeout.
__device__ __forceinline__ bool wait_counter_bounded(const unsigned long long *counter,
                                                     unsigned long long expected) {
  if (ld_acquire_sys(counter) >= expected) return true;
  const long long start = clock64();
  for (;;) {
#pragma unroll 1
    for (uint32_t spin = 0; spin < 32; ++spin) {
      if (ld_acquire_sys(counter) >= expected) return true;
    }
    if (clock64() - start > kPeerWaitCycleLimit) return false;
  }
}

// Timeline stamps of one launch (tuning aid, off unless the session asks for it):
// the first block writes slots 0..3, the last block slots 4..7, of
//   +0 kernel entry   +1 after pdl_wait   +2 after the prologue   +3 before exit
// in nanoseconds of %globaltimer.
constexpr uint32_t kStampEntry = 0, kStampAfterWait = 1, kStampAfterPrologue = 2, kStampExit = 3;
__device__ __forceinline__ void stamp(unsigned long long *stamps, uint32_t slot) {
  if (stamps == nullptr || threadIdx.x != 0) return;
  const uint32_t last = gridDim.x * gridDim.y * gridDim.z - 1u;
  const uint32_t block = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
  if (block != 0 && block != last) return;
  unsigned long long now;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
  if (block == 0) stamps[slot] = now;
  if (block == last) stamps[4u + slot] = now;
}

__device__ __forceinline__ void report_error(uint32_t *error_word, uint32_t code) {
  if (error_word != nullptr) atomicMax(error_word, code);
}

// 16-byte shared-memory load.
__device__ __forceinline__ uint4 lds128(const void *p) {
  return *reinterpret_cast<const uint4 *>(p);
}

__device__ __forceinline__ float silu(float v) { return v / (1.0f + expf(-v)); }

}  // namespace nb
