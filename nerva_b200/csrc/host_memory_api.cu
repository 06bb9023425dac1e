// C exports of the host-side memory bookkeeping (StaticArena, KvPagePool) so
// the integer behaviour of host_memory.h can be checked from outside the
// library with the scenarios of the reference's own tests
// (crates/nerva-memory/src/tests/arena.rs, tests/kv.rs).  Host only: no call
// here touches a device.
#include <string.h>

#include "../../include/nerva_b200_api.h"
#include "host_memory.h"

using namespace nb;

struct NervaB200StaticArena {
  StaticArena arena;
  explicit NervaB200StaticArena(uint64_t capacity) : arena(capacity) {}
};

struct NervaB200KvPagePool {
  KvPagePool pool;
};

namespace {
KvPrefixKey make_key(const uint8_t *hash32, uint32_t group_id) {
  KvPrefixKey key;
  memcpy(key.hash.data(), hash32, 32);
  key.group_id = group_id;
  return key;
}
}  // namespace

extern "C" NervaB200StaticArena *nerva_b200_static_arena_new(uint64_t capacity_bytes) {
  return new NervaB200StaticArena(capacity_bytes);
}

extern "C" void nerva_b200_static_arena_free(NervaB200StaticArena *arena) { delete arena; }

extern "C" int nerva_b200_static_arena_reserve(NervaB200StaticArena *arena, uint64_t bytes,
                                               uint64_t align, uint32_t phase,
                                               uint64_t *offset_out) {
  if (arena == nullptr || phase > 2) return -1;
  ArenaRegion region;
  if (!arena->arena.reserve(bytes, align, static_cast<AllocationPhase>(phase), &region)) return -1;
  if (offset_out != nullptr) *offset_out = region.offset;
  return 0;
}

extern "C" uint64_t nerva_b200_static_arena_used(const NervaB200StaticArena *arena) {
  return arena == nullptr ? 0 : arena->arena.used();
}

extern "C" uint64_t nerva_b200_static_arena_remaining(const NervaB200StaticArena *arena) {
  return arena == nullptr ? 0 : arena->arena.remaining();
}

extern "C" int nerva_b200_static_arena_restore(NervaB200StaticArena *arena, uint64_t cursor) {
  return arena != nullptr && arena->arena.restore(cursor) ? 0 : -1;
}

extern "C" NervaB200KvPagePool *nerva_b200_kv_page_pool_new(NervaB200StaticArena *arena,
                                                            uint32_t num_pages,
                                                            uint32_t block_size_tokens,
                                                            uint64_t page_bytes, uint64_t align) {
  if (arena == nullptr) return nullptr;
  NervaB200KvPagePool *pool = new NervaB200KvPagePool();
  if (!pool->pool.preallocate(arena->arena, num_pages, block_size_tokens, page_bytes, align)) {
    delete pool;
    return nullptr;
  }
  return pool;
}

extern "C" void nerva_b200_kv_page_pool_free(NervaB200KvPagePool *pool) { delete pool; }

extern "C" uint32_t nerva_b200_kv_page_pool_len(const NervaB200KvPagePool *pool) {
  return pool == nullptr ? 0 : static_cast<uint32_t>(pool->pool.size());
}

extern "C" uint32_t nerva_b200_kv_page_pool_free_pages(const NervaB200KvPagePool *pool) {
  return pool == nullptr ? 0 : static_cast<uint32_t>(pool->pool.free_pages());
}

extern "C" int64_t nerva_b200_kv_page_pool_allocate(NervaB200KvPagePool *pool, uint32_t token_start,
                                                    uint32_t token_count, uint64_t step) {
  return pool == nullptr ? -1 : pool->pool.allocate_page(token_start, token_count, step);
}

extern "C" int nerva_b200_kv_page_pool_retain(NervaB200KvPagePool *pool, uint32_t page, uint64_t step) {
  return pool != nullptr && pool->pool.retain_page(page, step) ? 0 : -1;
}

extern "C" int nerva_b200_kv_page_pool_release(NervaB200KvPagePool *pool, uint32_t page, uint64_t step) {
  return pool != nullptr && pool->pool.release_page(page, step) ? 0 : -1;
}

extern "C" int nerva_b200_kv_page_pool_cache(NervaB200KvPagePool *pool, uint32_t page,
                                             const uint8_t *hash32, uint32_t group_id,
                                             uint32_t prefix_tokens) {
  if (pool == nullptr || hash32 == nullptr) return -1;
  return pool->pool.cache_page(page, make_key(hash32, group_id), prefix_tokens) ? 0 : -1;
}

extern "C" int64_t nerva_b200_kv_page_pool_lookup_cached(const NervaB200KvPagePool *pool,
                                                         const uint8_t *hash32, uint32_t group_id) {
  if (pool == nullptr || hash32 == nullptr) return -1;
  return pool->pool.lookup_cached(make_key(hash32, group_id));
}

extern "C" int64_t nerva_b200_kv_page_pool_retain_cached(NervaB200KvPagePool *pool,
                                                         const uint8_t *hash32, uint32_t group_id,
                                                         uint64_t step) {
  if (pool == nullptr || hash32 == nullptr) return -1;
  return pool->pool.retain_cached(make_key(hash32, group_id), step);
}

extern "C" int nerva_b200_kv_page_pool_evict_cached(NervaB200KvPagePool *pool, uint32_t page) {
  return pool == nullptr ? -1 : pool->pool.evict_cached_page(page);
}

extern "C" int nerva_b200_kv_page_pool_page(const NervaB200KvPagePool *pool, uint32_t page,
                                            NervaB200KvPageInfo *out) {
  if (pool == nullptr || out == nullptr) return -1;
  const KvPageDescriptor *d = pool->pool.page(page);
  if (d == nullptr) return -1;
  out->arena_offset = d->arena_offset;
  out->page_bytes = d->page_bytes;
  out->last_use = d->last_use;
  out->token_start = d->token_start;
  out->token_count = d->token_count;
  out->ref_count = d->ref_count;
  out->prefix_tokens = d->prefix_tokens;
  out->is_free = d->is_free ? 1u : 0u;
  out->has_prefix = d->has_prefix ? 1u : 0u;
  return 0;
}
