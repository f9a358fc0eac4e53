// Stream-ordered caching memory pool, generic over the raw allocator (device memory, pinned host memory, or
// plain malloc for host-only tests).
//
// Role of the reference's size-class device / pinned pools, allocation statistics, pressure levels and defragmentation
// (crates/torsh-backend/src/cuda/memory/{memory_pools,memory_pools_pinned,manager,allocation}.rs), laid out for a
// 180 GB part: requests below 1 MiB are rounded to 512 B and carved out of 2 MiB segments; larger requests are rounded
// to 2 MiB and take a best-fit free block of the same stream, split when the remainder is at least 1 MiB. A freed block
// merges with free neighbours of its segment and is reused only by the stream that last used it, so reuse never needs
// an event. When the raw allocator fails, fully free segments are returned to it and the request is retried once.
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>
#include <mutex>
#include <set>
#include <unordered_map>
#include <vector>

namespace tbpool {

struct RawAllocator {
  void* (*alloc)(size_t bytes, void* ctx);
  void (*release)(void* ptr, size_t bytes, void* ctx);
  void* ctx;
};

struct Stats {
  uint64_t allocated_bytes, reserved_bytes, peak_allocated_bytes, peak_reserved_bytes;
  uint64_t alloc_calls, free_calls, cache_hits, raw_allocs, raw_frees, splits, merges, oom_retries, segments;
};

enum Pressure { PRESSURE_LOW = 0, PRESSURE_MODERATE = 1, PRESSURE_HIGH = 2, PRESSURE_CRITICAL = 3 };

class Pool {
 public:
  static constexpr size_t kSmallLimit = 1u << 20;      // requests below this come from small segments
  static constexpr size_t kSmallSegment = 2u << 20;
  static constexpr size_t kSmallRound = 512;
  static constexpr size_t kLargeRound = 2u << 20;
  static constexpr size_t kSplitRemainder = 1u << 20;

  explicit Pool(RawAllocator raw, uint64_t limit_bytes = 0) : raw_(raw), limit_(limit_bytes) {}
  ~Pool() { release_all(); }
  Pool(const Pool&) = delete;
  Pool& operator=(const Pool&) = delete;

  static size_t round_size(size_t n) {
    if (n == 0) n = 1;
    if (n < kSmallLimit) return (n + kSmallRound - 1) / kSmallRound * kSmallRound;
    return (n + kLargeRound - 1) / kLargeRound * kLargeRound;
  }

  void* allocate(size_t bytes, uint64_t stream) {
    std::lock_guard<std::mutex> g(mu_);
    const size_t size = round_size(bytes);
    const bool small = size < kSmallLimit;
    ++st_.alloc_calls;
    Block* b = take_free(size, stream, small);
    if (b) {
      ++st_.cache_hits;
    } else {
      size_t seg = small ? kSmallSegment : size;
      if (limit_ && st_.reserved_bytes + seg > limit_) {
        release_cached_locked();
        if (st_.reserved_bytes + seg > limit_) return nullptr;
      }
      void* p = raw_.alloc(seg, raw_.ctx);
      if (!p) {
        ++st_.oom_retries;
        release_cached_locked();
        p = raw_.alloc(seg, raw_.ctx);
        if (!p) return nullptr;
      }
      ++st_.raw_allocs;
      ++st_.segments;
      st_.reserved_bytes += seg;
      if (st_.reserved_bytes > st_.peak_reserved_bytes) st_.peak_reserved_bytes = st_.reserved_bytes;
      b = new Block{(char*)p, seg, stream, small, false, nullptr, nullptr, (char*)p, seg};
    }
    const size_t rem = b->size - size;
    if ((small && rem >= kSmallRound) || (!small && rem >= kSplitRemainder)) {
      Block* r = new Block{b->ptr + size, rem, b->stream, small, false, b, b->next, b->seg_base, b->seg_size};
      if (b->next) b->next->prev = r;
      b->next = r;
      b->size = size;
      free_.insert(r);
      ++st_.splits;
    }
    b->in_use = true;
    b->stream = stream;
    live_[b->ptr] = b;
    st_.allocated_bytes += b->size;
    if (st_.allocated_bytes > st_.peak_allocated_bytes) st_.peak_allocated_bytes = st_.allocated_bytes;
    return b->ptr;
  }

  // Returns false when ptr was not handed out by this pool.
  bool deallocate(void* ptr) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = live_.find((char*)ptr);
    if (it == live_.end()) return false;
    Block* b = it->second;
    live_.erase(it);
    ++st_.free_calls;
    st_.allocated_bytes -= b->size;
    b->in_use = false;
    b = merge(b, b->prev);
    b = merge(b, b->next);
    free_.insert(b);
    return true;
  }

  size_t size_of(void* ptr) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = live_.find((char*)ptr);
    return it == live_.end() ? 0 : it->second->size;
  }

  // Give every fully free segment back to the raw allocator; returns the bytes released.
  uint64_t release_cached() {
    std::lock_guard<std::mutex> g(mu_);
    return release_cached_locked();
  }

  Stats stats() {
    std::lock_guard<std::mutex> g(mu_);
    return st_;
  }
  void reset_peaks() {
    std::lock_guard<std::mutex> g(mu_);
    st_.peak_allocated_bytes = st_.allocated_bytes;
    st_.peak_reserved_bytes = st_.reserved_bytes;
  }
  void set_limit(uint64_t bytes) {
    std::lock_guard<std::mutex> g(mu_);
    limit_ = bytes;
  }

  // Pressure against `capacity` bytes (the device's total memory): <70 % low, <85 % moderate, <95 % high, else critical.
  Pressure pressure(uint64_t capacity) {
    std::lock_guard<std::mutex> g(mu_);
    if (!capacity) return PRESSURE_LOW;
    double f = (double)st_.reserved_bytes / (double)capacity;
    return f < 0.70 ? PRESSURE_LOW : f < 0.85 ? PRESSURE_MODERATE : f < 0.95 ? PRESSURE_HIGH : PRESSURE_CRITICAL;
  }

  // Cached (free) bytes that cannot be returned because their segment still has live blocks, over all cached bytes.
  double fragmentation() {
    std::lock_guard<std::mutex> g(mu_);
    uint64_t cached = 0, stuck = 0;
    for (Block* b : free_) {
      cached += b->size;
      if (b->size != b->seg_size) stuck += b->size;
    }
    return cached ? (double)stuck / (double)cached : 0.0;
  }

 private:
  struct Block {
    char* ptr;
    size_t size;
    uint64_t stream;
    bool small, in_use;
    Block *prev, *next;
    char* seg_base;
    size_t seg_size;
  };
  struct Less {
    bool operator()(const Block* a, const Block* b) const {
      if (a->small != b->small) return a->small < b->small;
      if (a->stream != b->stream) return a->stream < b->stream;
      if (a->size != b->size) return a->size < b->size;
      return a->ptr < b->ptr;
    }
  };

  Block* take_free(size_t size, uint64_t stream, bool small) {
    Block key{nullptr, size, stream, small, false, nullptr, nullptr, nullptr, 0};
    auto it = free_.lower_bound(&key);
    if (it == free_.end() || (*it)->stream != stream || (*it)->small != small) return nullptr;
    Block* b = *it;
    free_.erase(it);
    return b;
  }

  Block* merge(Block* b, Block* nb) {
    if (!nb || nb->in_use || nb->stream != b->stream) return b;
    free_.erase(nb);
    Block* lo = nb->ptr < b->ptr ? nb : b;
    Block* hi = lo == nb ? b : nb;
    lo->size += hi->size;
    lo->next = hi->next;
    if (hi->next) hi->next->prev = lo;
    delete hi;
    ++st_.merges;
    return lo;
  }

  uint64_t release_cached_locked() {
    uint64_t freed = 0;
    for (auto it = free_.begin(); it != free_.end();) {
      Block* b = *it;
      if (!b->prev && !b->next && b->size == b->seg_size) {
        raw_.release(b->seg_base, b->seg_size, raw_.ctx);
        ++st_.raw_frees;
        --st_.segments;
        st_.reserved_bytes -= b->seg_size;
        freed += b->seg_size;
        it = free_.erase(it);
        delete b;
      } else {
        ++it;
      }
    }
    return freed;
  }

  void release_all() {
    // live blocks are abandoned with their segments still reserved: the owner tears the context down afterwards
    release_cached_locked();
  }

  RawAllocator raw_;
  uint64_t limit_;
  std::mutex mu_;
  std::set<Block*, Less> free_;
  std::unordered_map<char*, Block*> live_;
  Stats st_{};
};

}  // namespace tbpool
