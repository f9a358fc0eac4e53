// Host-memory instance of the caching pool (64-byte aligned malloc underneath): staging buffers for the TRSH codec
// and the data loader, and the way the pool logic is exercised without a GPU. The device and pinned-memory instances
// live in the CUDA library (csrc/kernels/runtime.cu) and share the same template.
#include <cstdlib>

#include "host_api.h"
#include "tb_pool.h"

namespace {
struct HostCtx {
  uint64_t budget;   // raw allocator refuses beyond this many bytes (0 = unlimited); lets tests drive the OOM path
  uint64_t in_use;
};
void* host_alloc(size_t n, void* c) {
  auto* h = (HostCtx*)c;
  if (h->budget && h->in_use + n > h->budget) return nullptr;
  void* p = nullptr;
  if (posix_memalign(&p, 64, n) != 0) return nullptr;
  h->in_use += n;
  return p;
}
void host_release(void* p, size_t n, void* c) {
  ((HostCtx*)c)->in_use -= n;
  free(p);
}
struct HostPool {
  HostCtx ctx;
  tbpool::Pool pool;
  explicit HostPool(uint64_t budget, uint64_t limit)
      : ctx{budget, 0}, pool(tbpool::RawAllocator{host_alloc, host_release, &ctx}, limit) {}
};
}  // namespace

TSH_EXPORT void* tsh_pool_create(uint64_t raw_budget_bytes, uint64_t limit_bytes) {
  return new HostPool(raw_budget_bytes, limit_bytes);
}
TSH_EXPORT void tsh_pool_destroy(void* h) { delete (HostPool*)h; }
TSH_EXPORT void* tsh_pool_alloc(void* h, uint64_t bytes, uint64_t stream) {
  return ((HostPool*)h)->pool.allocate(bytes, stream);
}
TSH_EXPORT int tsh_pool_free(void* h, void* p) { return ((HostPool*)h)->pool.deallocate(p) ? 0 : -1; }
TSH_EXPORT uint64_t tsh_pool_release_cached(void* h) { return ((HostPool*)h)->pool.release_cached(); }
TSH_EXPORT uint64_t tsh_pool_round_size(uint64_t n) { return tbpool::Pool::round_size(n); }
TSH_EXPORT uint64_t tsh_pool_size_of(void* h, void* p) { return ((HostPool*)h)->pool.size_of(p); }
TSH_EXPORT void tsh_pool_stats(void* h, uint64_t* out13) {
  tbpool::Stats s = ((HostPool*)h)->pool.stats();
  const uint64_t v[13] = {s.allocated_bytes, s.reserved_bytes, s.peak_allocated_bytes, s.peak_reserved_bytes,
                          s.alloc_calls, s.free_calls, s.cache_hits, s.raw_allocs, s.raw_frees, s.splits, s.merges,
                          s.oom_retries, s.segments};
  for (int i = 0; i < 13; ++i) out13[i] = v[i];
}
TSH_EXPORT int tsh_pool_pressure(void* h, uint64_t capacity) { return (int)((HostPool*)h)->pool.pressure(capacity); }
TSH_EXPORT double tsh_pool_fragmentation(void* h) { return ((HostPool*)h)->pool.fragmentation(); }
