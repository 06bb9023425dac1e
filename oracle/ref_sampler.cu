// Test infrastructure: runs the REFERENCE's own final-head sampler kernel
// (native/cuda/hf_decode_sequence/sampler.cu, included below from the reference checkout
// where it lies) on logits given by the caller, so that the tests can compare this
// repository's sampler with it token for token on the same GPU.  Built only where the
// checkout exists (the Makefile's `ref` target); the built library travels with the tree.
#include "hf_decode_sequence/sampler.cu"

// Samples one token at `position` from host logits.  Returns 0, or a CUDA error code.
extern "C" int ref_sample_token(const float *host_logits, uint32_t vocab, uint32_t position, float temperature,
                                float top_p, uint32_t top_k, uint64_t seed, uint32_t *token) {
  float *scores = nullptr;
  uint32_t *cursor = nullptr;
  NervaCudaSyntheticTokenSlot *slots = nullptr;
  const size_t slot_bytes = sizeof(NervaCudaSyntheticTokenSlot) * (static_cast<size_t>(position) + 1u);
  cudaError_t err = cudaMalloc(&scores, sizeof(float) * vocab);
  if (err == cudaSuccess) err = cudaMalloc(&cursor, sizeof(uint32_t));
  if (err == cudaSuccess) err = cudaMalloc(&slots, slot_bytes);
  if (err == cudaSuccess) err = cudaMemset(slots, 0, slot_bytes);
  if (err == cudaSuccess) err = cudaMemcpy(scores, host_logits, sizeof(float) * vocab, cudaMemcpyHostToDevice);
  if (err == cudaSuccess) err = cudaMemcpy(cursor, &position, sizeof(uint32_t), cudaMemcpyHostToDevice);
  if (err == cudaSuccess) {
    NervaCudaHfDecodeSamplerConfig config{};
    config.temperature = temperature;
    config.top_p = top_p;
    config.top_k = top_k;
    config.seed = seed;
    err = launch_hf_decode_final_head_sampler(nullptr, cursor, position + 1u, 0, 0, scores, vocab, slots,
                                              normalize_hf_decode_sampler_config(config));
  }
  if (err == cudaSuccess) err = cudaDeviceSynchronize();
  NervaCudaSyntheticTokenSlot slot{};
  if (err == cudaSuccess) err = cudaMemcpy(&slot, slots + position, sizeof(slot), cudaMemcpyDeviceToHost);
  if (err == cudaSuccess) *token = slot.token;
  cudaFree(scores);
  cudaFree(cursor);
  cudaFree(slots);
  return static_cast<int>(err);
}
