// Host-side memory bookkeeping of a resident session.  The reference keeps these
// in Rust (crates/nerva-memory); there is no Rust toolchain in this build, so
// they are C++ with the same integer semantics:
//   StaticArena : crates/nerva-memory/src/arena/static_arena.rs:71-112
//   KvPagePool  : crates/nerva-memory/src/kv/pool/{preallocate.rs:14-67,
//                 allocation.rs:7-88, cache.rs:7-50}, kv/page.rs
#pragma once

#include <stdint.h>

#include <array>
#include <deque>
#include <map>
#include <string>
#include <vector>

namespace nb {

enum class AllocationPhase : uint32_t { Initialization = 0, Warmup = 1, HotPath = 2 };

struct ArenaRegion {
  uint64_t offset = 0;
  uint64_t bytes = 0;
  uint64_t align = 1;
};

// Bump allocator over one pre-made allocation.  It never frees, and it refuses
// to hand out memory once the hot path has started.
class StaticArena {
 public:
  explicit StaticArena(uint64_t capacity_bytes = 0) : capacity_(capacity_bytes) {}
  uint64_t capacity() const { return capacity_; }
  uint64_t used() const { return used_; }
  uint64_t remaining() const { return capacity_ > used_ ? capacity_ - used_ : 0; }
  uint64_t checkpoint() const { return used_; }
  bool restore(uint64_t cursor) {
    if (cursor > used_) return false;
    used_ = cursor;
    return true;
  }
  // Returns false (and leaves the arena unchanged) on a hot-path request,
  // offset overflow or exhaustion.
  bool reserve(uint64_t bytes, uint64_t align, AllocationPhase phase, ArenaRegion *out,
               std::string *why = nullptr) {
    if (phase == AllocationPhase::HotPath) {
      if (why) *why = "static arena allocation attempted during hot path";
      hot_path_rejections_ += 1;
      return false;
    }
    if (align == 0) align = 1;
    const uint64_t rem = used_ % align;
    uint64_t offset = used_;
    if (rem != 0) {
      if (offset > UINT64_MAX - (align - rem)) {
        if (why) *why = "static arena offset overflow";
        return false;
      }
      offset += align - rem;
    }
    if (offset > UINT64_MAX - bytes) {
      if (why) *why = "static arena offset overflow";
      return false;
    }
    const uint64_t end = offset + bytes;
    if (end > capacity_) {
      if (why) *why = "static arena exhausted";
      return false;
    }
    used_ = end;
    if (out) *out = ArenaRegion{offset, bytes, align};
    return true;
  }
  uint64_t hot_path_rejections() const { return hot_path_rejections_; }

 private:
  uint64_t capacity_;
  uint64_t used_ = 0;
  uint64_t hot_path_rejections_ = 0;
};

struct KvPrefixKey {
  std::array<uint8_t, 32> hash{};
  uint32_t group_id = 0;
  bool operator<(const KvPrefixKey &o) const {
    return hash != o.hash ? hash < o.hash : group_id < o.group_id;
  }
  bool operator==(const KvPrefixKey &o) const { return hash == o.hash && group_id == o.group_id; }
};

struct KvPageDescriptor {
  uint32_t page_index = 0;
  uint64_t arena_offset = 0;
  uint32_t token_start = 0;
  uint32_t token_count = 0;
  uint32_t block_size_tokens = 0;
  uint64_t page_bytes = 0;
  uint32_t ref_count = 0;
  bool has_prefix = false;
  KvPrefixKey prefix_key;
  uint32_t prefix_tokens = 0;
  uint64_t last_use = 0;
  bool has_next_use = false;
  uint64_t next_use = 0;
  bool is_free = true;
};

// Pre-allocated page pool: FIFO free list (pop front / push back), reference
// counts, prefix-key cache.
class KvPagePool {
 public:
  // Reserves num_pages * page_bytes in `arena`.  Returns false when the arena
  // cannot hold them or block_size_tokens == 0.
  bool preallocate(StaticArena &arena, uint32_t num_pages, uint32_t block_size_tokens,
                   uint64_t page_bytes, uint64_t align) {
    if (block_size_tokens == 0) return false;
    pages_.clear();
    free_.clear();
    cache_.clear();
    for (uint32_t i = 0; i < num_pages; ++i) {
      ArenaRegion region;
      if (!arena.reserve(page_bytes, align, AllocationPhase::Initialization, &region)) return false;
      KvPageDescriptor page;
      page.page_index = i;
      page.arena_offset = region.offset;
      page.block_size_tokens = block_size_tokens;
      page.page_bytes = page_bytes;
      pages_.push_back(page);
      free_.push_back(i);
    }
    return true;
  }
  size_t size() const { return pages_.size(); }
  size_t free_pages() const { return free_.size(); }
  const KvPageDescriptor *page(uint32_t index) const {
    return index < pages_.size() ? &pages_[index] : nullptr;
  }
  // -1 pool exhausted, -2 token_count exceeds the page size (page returned to the front).
  int64_t allocate_page(uint32_t token_start, uint32_t token_count, uint64_t step) {
    if (free_.empty()) return -1;
    const uint32_t index = free_.front();
    free_.pop_front();
    KvPageDescriptor &page = pages_[index];
    if (token_count > page.block_size_tokens) {
      free_.push_front(index);
      return -2;
    }
    page.token_start = token_start;
    page.token_count = token_count;
    page.ref_count = 1;
    page.last_use = step;
    page.has_next_use = false;
    page.is_free = false;
    return index;
  }
  bool retain_page(uint32_t index, uint64_t step) {
    if (index >= pages_.size()) return false;
    KvPageDescriptor &page = pages_[index];
    if (page.is_free) {
      for (auto it = free_.begin(); it != free_.end();) it = *it == index ? free_.erase(it) : it + 1;
    }
    if (page.ref_count == UINT32_MAX) return false;
    page.is_free = false;
    page.ref_count += 1;
    page.last_use = step;
    return true;
  }
  bool release_page(uint32_t index, uint64_t step) {
    if (index >= pages_.size()) return false;
    KvPageDescriptor &page = pages_[index];
    if (page.ref_count == 0) return false;
    page.ref_count -= 1;
    page.last_use = step;
    if (page.ref_count == 0 && !page.is_free) {
      page.is_free = true;
      if (!page.has_prefix) page.token_count = 0;
      free_.push_back(index);
    }
    return true;
  }
  bool set_next_use(uint32_t index, bool has, uint64_t next_use) {
    if (index >= pages_.size()) return false;
    pages_[index].has_next_use = has;
    pages_[index].next_use = next_use;
    return true;
  }
  bool cache_page(uint32_t index, const KvPrefixKey &key, uint32_t prefix_tokens) {
    if (index >= pages_.size() || prefix_tokens == 0) return false;
    KvPageDescriptor &page = pages_[index];
    if (page.has_prefix) cache_.erase(page.prefix_key);
    page.has_prefix = true;
    page.prefix_key = key;
    page.prefix_tokens = prefix_tokens;
    cache_[key] = index;
    return true;
  }
  int64_t lookup_cached(const KvPrefixKey &key) const {
    auto it = cache_.find(key);
    return it == cache_.end() ? -1 : static_cast<int64_t>(it->second);
  }
  int64_t retain_cached(const KvPrefixKey &key, uint64_t step) {
    const int64_t index = lookup_cached(key);
    if (index < 0) return -1;
    return retain_page(static_cast<uint32_t>(index), step) ? index : -2;
  }
  // Returns 1 when a key was evicted, 0 when the page had none, -1 on a bad index.
  int evict_cached_page(uint32_t index) {
    if (index >= pages_.size()) return -1;
    KvPageDescriptor &page = pages_[index];
    if (!page.has_prefix) return 0;
    cache_.erase(page.prefix_key);
    page.has_prefix = false;
    page.prefix_tokens = 0;
    return 1;
  }

 private:
  std::vector<KvPageDescriptor> pages_;
  std::deque<uint32_t> free_;
  std::map<KvPrefixKey, uint32_t> cache_;
};

}  // namespace nb
