// GQA paged split-KV decode attention that allocates nothing.
//
// The isolated attention entry point (ops_api.cu) stages host buffers and takes
// its split partials from cudaMalloc.  This variant is for callers that have
// already handed the whole device to an arena of their own, or that sit inside a
// decode loop whose residency contract counts hot-path allocations and requires
// zero: they pass DEVICE inputs and outputs, and the split partials live in a
// file-scope device array of fixed size.  No cudaMalloc, cudaFree, event, stream
// or library allocation happens here, and no host heap allocation on the
// success path (an error message longer than a few characters is the exception).
//
// Limits and rules of use
//  * batch * heads * splits * (head_dim + 2) <= kScratchFloats (1 Mi floats,
//    4 MiB).  The split count is lowered until the partials fit; a shape that does
//    not fit even unsplit is rejected with an error text that names the limit.
//  * Every call on one device shares the one array and it keeps its last
//    contents.  The kernels write every (m, l) slot they later read and skip the
//    accumulator of a slot whose l is 0, so only the error word has to start at
//    zero; the call clears it on the caller's stream.  Two calls that overlap on
//    one device (two streams, two threads) race on the array: serialise them.
//  * The first call on each device does the set-up (address of the array, SM
//    count, shared-memory attributes of the kernels) with that device current.
//  * The call returns after `stream` has finished the work, because it reads the
//    kernel's error word back.
#include <mutex>

#include "kernels.cuh"
#include "session.h"

using namespace nb;

static constexpr uint64_t kScratchFloats = 1ull << 20;  // partial acc + m + l of one call
static constexpr uint32_t kErrorWordFloats = 64;        // the error word keeps 256 bytes to itself
static constexpr int kMaxDevices = 64;

// One instance per device; host code only ever uses the address that
// cudaGetSymbolAddress returned for the current device.
static __device__ __align__(256) float g_attention_scratch[kScratchFloats + kErrorWordFloats];

namespace {

struct DeviceSetup {
  bool ready = false;
  float *scratch = nullptr;
  uint32_t sm_count = 0;
};
DeviceSetup g_setup[kMaxDevices];
std::mutex g_setup_mutex;

// Once per device, with that device current.
cudaError_t setup_current_device(const DeviceSetup **out) {
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return err;
  if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  DeviceSetup &d = g_setup[device];
  if (!d.ready) {
    float *ptr = nullptr;
    err = cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_attention_scratch);
    if (err != cudaSuccess) return err;
    int sms = 0;
    err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (err != cudaSuccess) return err;
    err = configure_attention_kernels();
    if (err != cudaSuccess) return err;
    d.scratch = ptr;
    d.sm_count = static_cast<uint32_t>(sms);
    d.ready = true;
  }
  *out = &d;
  return cudaSuccess;
}

}  // namespace

extern "C" int nerva_b200_gqa_decode_attention_static_scratch(
    const float *q, const uint16_t *key_pages, const uint16_t *value_pages,
    const uint32_t *page_table, float *out, uint32_t batch, uint32_t context, uint32_t heads,
    uint32_t kv_heads, uint32_t head_dim, void *stream_handle) {
  set_last_error("");
  if (q == nullptr || key_pages == nullptr || value_pages == nullptr || page_table == nullptr ||
      out == nullptr || batch == 0 || context == 0 || heads == 0 || kv_heads == 0 ||
      heads % kv_heads != 0 || head_dim == 0 || head_dim > 256) {
    set_last_error("invalid argument");
    return -1;
  }
  // The tiled kernels fetch K and V in 16-byte pieces: a view that starts in the middle of such a
  // piece would fault the device instead of failing the call, so it is refused here.
  if (reinterpret_cast<uintptr_t>(key_pages) % 16u != 0 || reinterpret_cast<uintptr_t>(value_pages) % 16u != 0 ||
      reinterpret_cast<uintptr_t>(q) % 16u != 0 || reinterpret_cast<uintptr_t>(out) % 4u != 0 ||
      reinterpret_cast<uintptr_t>(page_table) % 4u != 0) {
    set_last_error("misaligned buffer: q, key_pages and value_pages must start on a 16-byte boundary");
    return -1;
  }
  const DeviceSetup *setup = nullptr;
  cudaError_t err = setup_current_device(&setup);
  if (err != cudaSuccess) {
    set_last_error(cudaGetErrorString(err));
    return -1;
  }
  const uint64_t per_split = static_cast<uint64_t>(batch) * heads * (static_cast<uint64_t>(head_dim) + 2u);
  if (per_split > kScratchFloats) {
    set_last_error(
        "static scratch too small: batch * heads * (head_dim + 2) exceeds 1048576 floats (4 MiB)");
    return -1;
  }
  uint32_t splits = attention_default_splits(context, batch, kv_heads, setup->sm_count);
  const uint64_t fit = kScratchFloats / per_split;
  if (splits > fit) splits = static_cast<uint32_t>(fit);

  const uint64_t slots = static_cast<uint64_t>(batch) * heads * splits;
  float *scratch = setup->scratch;
  uint32_t *error_word = reinterpret_cast<uint32_t *>(scratch + kScratchFloats);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);

  AttentionParams p{};
  p.q = q;
  p.key_pages = key_pages;
  p.value_pages = value_pages;
  p.page_table = page_table;
  p.batch = batch;
  p.heads = heads;
  p.kv_heads = kv_heads;
  p.head_dim = head_dim;
  p.page_count = (context + NERVA_KV_CACHE_BLOCK_TOKENS - 1) / NERVA_KV_CACHE_BLOCK_TOKENS;
  p.cursor = nullptr;
  p.context = context;
  p.splits = splits;
  p.partial_acc = scratch;                       // [batch][heads][splits][head_dim]
  p.partial_m = scratch + slots * head_dim;      // [batch][heads][splits]
  p.partial_l = scratch + slots * head_dim + slots;
  p.out_f32 = out;
  p.error_word = error_word;

  err = cudaMemsetAsync(error_word, 0, sizeof(uint32_t), stream);
  if (err == cudaSuccess) err = launch_attention(stream, p);
  uint32_t device_error = 0;
  if (err == cudaSuccess)
    err = cudaMemcpyAsync(&device_error, error_word, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream);
  if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
  if (err != cudaSuccess) {
    set_last_error(cudaGetErrorString(err));
    return -1;
  }
  if (device_error != 0) {
    set_last_error("attention kernel reported a page index outside the page table");
    return -1;
  }
  return 0;
}
