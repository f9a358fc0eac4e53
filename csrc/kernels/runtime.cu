// Device runtime layer: per-device properties, caching device / pinned-host memory pools, a priority stream pool,
// an event pool, and a cache of instantiated CUDA graphs.
//
// Role of the reference's CudaDevice / CudaStream / StreamPool / EventPool / CUDA-graph cache / memory manager
// (crates/torsh-backend/src/cuda/{device,stream,event_coordination,graph}.rs, src/cuda/memory/*). One instance per
// device lives inside this library; Python drives it through the extern "C" calls below
// (torsh_b200/core/runtime.py). tb_torch_alloc / tb_torch_free have the signature PyTorch's pluggable-allocator hook
// expects, so the same pool can back torch tensors.
#include <list>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "host_util.h"
#include "tb_pool.h"

namespace tb {
namespace {

constexpr int kMaxDev = 16;

void* dev_alloc(size_t n, void*) {
  void* p = nullptr;
  if (cudaMalloc(&p, n) != cudaSuccess) {
    cudaGetLastError();  // clear the sticky-free allocation error so later launches are not blamed for it
    return nullptr;
  }
  return p;
}
void dev_release(void* p, size_t, void*) { cudaFree(p); }
void* pin_alloc(size_t n, void*) {
  void* p = nullptr;
  if (cudaHostAlloc(&p, n, cudaHostAllocPortable) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return p;
}
void pin_release(void* p, size_t, void*) { cudaFreeHost(p); }

struct GraphEntry {
  cudaGraphExec_t exec;
  cudaGraph_t graph;
  uint64_t launches;
};

struct DeviceRuntime {
  tbpool::Pool dev_pool{tbpool::RawAllocator{dev_alloc, dev_release, nullptr}};
  std::mutex mu;
  std::vector<cudaStream_t> streams[3];  // 0 = high priority (communication), 1 = normal, 2 = low (prefetch, copies)
  size_t next_stream[3] = {0, 0, 0};
  std::vector<cudaEvent_t> free_events[2];  // [timing?]
  uint64_t events_created = 0, events_reused = 0;
  std::unordered_map<uint64_t, std::pair<GraphEntry, std::list<uint64_t>::iterator>> graphs;
  std::list<uint64_t> lru;  // front = most recent
  size_t graph_capacity = 64;
  uint64_t graph_hits = 0, graph_misses = 0, graph_evictions = 0;
};

DeviceRuntime* rt(int dev) {
  static DeviceRuntime* table[kMaxDev] = {nullptr};
  static std::mutex mu;
  if (dev < 0 || dev >= kMaxDev) return nullptr;
  std::lock_guard<std::mutex> g(mu);
  if (!table[dev]) table[dev] = new DeviceRuntime();
  return table[dev];
}
tbpool::Pool& pinned_pool() {
  static tbpool::Pool* p = new tbpool::Pool(tbpool::RawAllocator{pin_alloc, pin_release, nullptr});
  return *p;
}
int cur_dev() { return g_device().load(std::memory_order_relaxed); }

void fill_stats(const tbpool::Stats& s, uint64_t* out13) {
  const uint64_t v[13] = {s.allocated_bytes, s.reserved_bytes, s.peak_allocated_bytes, s.peak_reserved_bytes,
                          s.alloc_calls, s.free_calls, s.cache_hits, s.raw_allocs, s.raw_frees, s.splits, s.merges,
                          s.oom_retries, s.segments};
  for (int i = 0; i < 13; ++i) out13[i] = v[i];
}

}  // namespace
}  // namespace tb
using namespace tb;

// ---------------------------------------------------------------------------------------------- device
// out[0..15]: SMs, max smem/block (opt-in), smem/SM, L2 bytes, total global bytes, free bytes, cc major, cc minor,
// SM clock kHz, memory clock kHz, bus width bits, max threads/SM, regs/SM, cluster launch supported, warp size,
// tensor-memory columns per SM (512 on compute capability 10.x, else 0).
TB_EXPORT int tb_rt_device_info(int dev, uint64_t* out, char* name64) {
  int count = 0;
  TB_CUDA_CHECK(cudaGetDeviceCount(&count));
  if (dev < 0 || dev >= count) TB_FAIL(TB_E_ARG, "device %d out of range (%d devices)", dev, count);
  cudaDeviceProp p;
  TB_CUDA_CHECK(cudaGetDeviceProperties(&p, dev));
  int clk = 0, mclk = 0, cluster = 0;
  cudaDeviceGetAttribute(&clk, cudaDevAttrClockRate, dev);
  cudaDeviceGetAttribute(&mclk, cudaDevAttrMemoryClockRate, dev);
  cudaDeviceGetAttribute(&cluster, cudaDevAttrClusterLaunch, dev);
  size_t fr = 0, tot = 0;
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(dev);
  cudaMemGetInfo(&fr, &tot);
  cudaSetDevice(prev);
  out[0] = p.multiProcessorCount; out[1] = p.sharedMemPerBlockOptin; out[2] = p.sharedMemPerMultiprocessor;
  out[3] = p.l2CacheSize; out[4] = p.totalGlobalMem; out[5] = fr; out[6] = p.major; out[7] = p.minor;
  out[8] = clk; out[9] = mclk; out[10] = p.memoryBusWidth; out[11] = p.maxThreadsPerMultiProcessor;
  out[12] = p.regsPerMultiprocessor; out[13] = cluster; out[14] = p.warpSize; out[15] = p.major == 10 ? 512 : 0;
  if (name64) snprintf(name64, 64, "%s", p.name);
  return 0;
}
TB_EXPORT int tb_rt_device_count() {
  int n = 0;
  return cudaGetDeviceCount(&n) == cudaSuccess ? n : 0;
}
TB_EXPORT int tb_rt_can_access_peer(int a, int b) {
  int ok = 0;
  return cudaDeviceCanAccessPeer(&ok, a, b) == cudaSuccess ? ok : 0;
}

// ---------------------------------------------------------------------------------------------- memory
TB_EXPORT void* tb_rt_malloc(uint64_t bytes, cudaStream_t stream) {
  if (ensure_device()) return nullptr;
  void* p = rt(cur_dev())->dev_pool.allocate(bytes, (uint64_t)(uintptr_t)stream);
  if (!p) snprintf(last_error_buf(), 512, "device pool: out of memory allocating %llu bytes", (unsigned long long)bytes);
  return p;
}
TB_EXPORT int tb_rt_free(void* p) {
  if (!p) return 0;
  TB_ENSURE_DEVICE();
  if (!rt(cur_dev())->dev_pool.deallocate(p)) TB_FAIL(TB_E_ARG, "pointer %p is not owned by the device pool", p);
  return 0;
}
TB_EXPORT int tb_rt_mem_stats(uint64_t* out13) {
  fill_stats(rt(cur_dev())->dev_pool.stats(), out13);
  return 0;
}
TB_EXPORT uint64_t tb_rt_empty_cache() {
  if (ensure_device()) return 0;
  return rt(cur_dev())->dev_pool.release_cached();
}
TB_EXPORT void tb_rt_set_mem_limit(uint64_t bytes) { rt(cur_dev())->dev_pool.set_limit(bytes); }
TB_EXPORT void tb_rt_reset_peak() { rt(cur_dev())->dev_pool.reset_peaks(); }
TB_EXPORT int tb_rt_mem_pressure() {
  size_t fr = 0, tot = 0;
  if (ensure_device() || cudaMemGetInfo(&fr, &tot) != cudaSuccess) return 0;
  return (int)rt(cur_dev())->dev_pool.pressure(tot);
}
TB_EXPORT double tb_rt_fragmentation() { return rt(cur_dev())->dev_pool.fragmentation(); }

TB_EXPORT void* tb_rt_pinned_alloc(uint64_t bytes) {
  if (ensure_device()) return nullptr;
  return pinned_pool().allocate(bytes, 0);
}
TB_EXPORT int tb_rt_pinned_free(void* p) { return pinned_pool().deallocate(p) ? 0 : TB_E_ARG; }
TB_EXPORT int tb_rt_pinned_stats(uint64_t* out13) {
  fill_stats(pinned_pool().stats(), out13);
  return 0;
}
TB_EXPORT int tb_rt_memcpy_async(void* dst, const void* src, uint64_t bytes, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  TB_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, st));
  return 0;
}
// Unified (managed) memory: one pointer valid on host and device; pages migrate on demand, or ahead of use with
// tb_rt_managed_prefetch. device < 0 means the host.
TB_EXPORT void* tb_rt_managed_alloc(uint64_t bytes) {
  if (ensure_device()) return nullptr;
  void* p = nullptr;
  if (cudaMallocManaged(&p, bytes, cudaMemAttachGlobal) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return p;
}
TB_EXPORT int tb_rt_managed_free(void* p) {
  TB_CUDA_CHECK(cudaFree(p));
  return 0;
}
TB_EXPORT int tb_rt_managed_prefetch(const void* p, uint64_t bytes, int device, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  cudaMemLocation loc{};
  loc.type = device < 0 ? cudaMemLocationTypeHost : cudaMemLocationTypeDevice;
  loc.id = device < 0 ? 0 : device;
  TB_CUDA_CHECK(cudaMemPrefetchAsync_v2(p, bytes, loc, 0, st));
  return 0;
}
// advice: 0 = read-mostly, 1 = preferred location, 2 = accessed by (the device, or the host when device < 0)
TB_EXPORT int tb_rt_managed_advise(const void* p, uint64_t bytes, int advice, int device) {
  TB_ENSURE_DEVICE();
  cudaMemLocation loc{};
  loc.type = device < 0 ? cudaMemLocationTypeHost : cudaMemLocationTypeDevice;
  loc.id = device < 0 ? 0 : device;
  const cudaMemoryAdvise a = advice == 0 ? cudaMemAdviseSetReadMostly
                             : advice == 1 ? cudaMemAdviseSetPreferredLocation : cudaMemAdviseSetAccessedBy;
  TB_CUDA_CHECK(cudaMemAdvise_v2(p, bytes, a, loc));
  return 0;
}
TB_EXPORT int tb_rt_memset_async(void* dst, int value, uint64_t bytes, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  TB_CUDA_CHECK(cudaMemsetAsync(dst, value, bytes, st));
  return 0;
}

// PyTorch pluggable-allocator hooks (torch.cuda.memory.CUDAPluggableAllocator). Blocks are reused in stream order,
// so a tensor that other streams still read when it is freed must be kept alive by its owner until they finish.
TB_EXPORT void* tb_torch_alloc(ssize_t size, int device, cudaStream_t stream) {
  int prev = -1;
  cudaGetDevice(&prev);
  if (prev != device) cudaSetDevice(device);
  void* p = rt(device)->dev_pool.allocate((size_t)size, (uint64_t)(uintptr_t)stream);
  if (prev != device && prev >= 0) cudaSetDevice(prev);
  return p;
}
TB_EXPORT void tb_torch_free(void* ptr, ssize_t, int device, cudaStream_t) {
  if (ptr) rt(device)->dev_pool.deallocate(ptr);
}

// ---------------------------------------------------------------------------------------------- streams
// cls: 0 high priority, 1 normal, 2 low. Streams are created on first use (non-blocking) and handed out round-robin
// from a pool of `pool_size` per class.
TB_EXPORT cudaStream_t tb_rt_stream_get(int cls, int pool_size) {
  if (ensure_device() || cls < 0 || cls > 2) return nullptr;
  DeviceRuntime* r = rt(cur_dev());
  std::lock_guard<std::mutex> g(r->mu);
  if (pool_size < 1) pool_size = 1;
  auto& v = r->streams[cls];
  if ((int)v.size() < pool_size) {
    int lo = 0, hi = 0;  // numerically lowest value = highest priority
    cudaDeviceGetStreamPriorityRange(&lo, &hi);
    int prio = cls == 0 ? hi : (cls == 2 ? lo : (lo + hi) / 2);
    cudaStream_t s = nullptr;
    if (cudaStreamCreateWithPriority(&s, cudaStreamNonBlocking, prio) != cudaSuccess) return nullptr;
    v.push_back(s);
    return s;
  }
  cudaStream_t s = v[r->next_stream[cls] % v.size()];
  r->next_stream[cls]++;
  return s;
}
TB_EXPORT int tb_rt_stream_priority(cudaStream_t s) {
  int p = 0;
  return cudaStreamGetPriority(s, &p) == cudaSuccess ? p : 0;
}
TB_EXPORT int tb_rt_stream_sync(cudaStream_t s) {
  TB_ENSURE_DEVICE();
  TB_CUDA_CHECK(cudaStreamSynchronize(s));
  return 0;
}
TB_EXPORT int tb_rt_stream_query(cudaStream_t s) {  // 1 = idle, 0 = busy, <0 = error
  TB_ENSURE_DEVICE();
  cudaError_t e = cudaStreamQuery(s);
  if (e == cudaSuccess) return 1;
  if (e == cudaErrorNotReady) return 0;
  TB_FAIL(TB_E_CUDA, "cudaStreamQuery: %s", cudaGetErrorString(e));
}
TB_EXPORT int tb_rt_stream_count(int cls) { return cls < 0 || cls > 2 ? 0 : (int)rt(cur_dev())->streams[cls].size(); }

// ---------------------------------------------------------------------------------------------- events
TB_EXPORT cudaEvent_t tb_rt_event_acquire(int timing) {
  if (ensure_device()) return nullptr;
  DeviceRuntime* r = rt(cur_dev());
  std::lock_guard<std::mutex> g(r->mu);
  auto& v = r->free_events[timing ? 1 : 0];
  if (!v.empty()) {
    cudaEvent_t e = v.back();
    v.pop_back();
    ++r->events_reused;
    return e;
  }
  cudaEvent_t e = nullptr;
  if (cudaEventCreateWithFlags(&e, timing ? cudaEventDefault : cudaEventDisableTiming) != cudaSuccess) return nullptr;
  ++r->events_created;
  return e;
}
TB_EXPORT void tb_rt_event_release(cudaEvent_t e, int timing) {
  DeviceRuntime* r = rt(cur_dev());
  std::lock_guard<std::mutex> g(r->mu);
  r->free_events[timing ? 1 : 0].push_back(e);
}
TB_EXPORT int tb_rt_event_record(cudaEvent_t e, cudaStream_t s) {
  TB_ENSURE_DEVICE();
  TB_CUDA_CHECK(cudaEventRecord(e, s));
  return 0;
}
TB_EXPORT int tb_rt_stream_wait_event(cudaStream_t s, cudaEvent_t e) {
  TB_ENSURE_DEVICE();
  TB_CUDA_CHECK(cudaStreamWaitEvent(s, e, 0));
  return 0;
}
TB_EXPORT int tb_rt_event_sync(cudaEvent_t e) {
  TB_ENSURE_DEVICE();
  TB_CUDA_CHECK(cudaEventSynchronize(e));
  return 0;
}
TB_EXPORT int tb_rt_event_query(cudaEvent_t e) {
  TB_ENSURE_DEVICE();
  cudaError_t r = cudaEventQuery(e);
  if (r == cudaSuccess) return 1;
  if (r == cudaErrorNotReady) return 0;
  TB_FAIL(TB_E_CUDA, "cudaEventQuery: %s", cudaGetErrorString(r));
}
TB_EXPORT float tb_rt_event_elapsed_ms(cudaEvent_t a, cudaEvent_t b) {
  float ms = -1.f;
  if (ensure_device() || cudaEventElapsedTime(&ms, a, b) != cudaSuccess) return -1.f;
  return ms;
}
TB_EXPORT void tb_rt_event_stats(uint64_t* out2) {
  DeviceRuntime* r = rt(cur_dev());
  out2[0] = r->events_created;
  out2[1] = r->events_reused;
}

// ---------------------------------------------------------------------------------------------- CUDA graphs
TB_EXPORT int tb_rt_graph_begin(cudaStream_t s) {
  TB_ENSURE_DEVICE();
  TB_CUDA_CHECK(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
  return 0;
}
// Ends the capture on `s`, instantiates the graph and stores it under `key` (replacing an older entry; the least
// recently launched entry is evicted beyond the capacity).
TB_EXPORT int tb_rt_graph_end(cudaStream_t s, uint64_t key) {
  TB_ENSURE_DEVICE();
  cudaGraph_t g = nullptr;
  TB_CUDA_CHECK(cudaStreamEndCapture(s, &g));
  cudaGraphExec_t ex = nullptr;
  cudaError_t e = cudaGraphInstantiate(&ex, g, 0);
  if (e != cudaSuccess) {
    cudaGraphDestroy(g);
    TB_FAIL(TB_E_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
  }
  DeviceRuntime* r = rt(cur_dev());
  std::lock_guard<std::mutex> lk(r->mu);
  auto it = r->graphs.find(key);
  if (it != r->graphs.end()) {
    cudaGraphExecDestroy(it->second.first.exec);
    cudaGraphDestroy(it->second.first.graph);
    r->lru.erase(it->second.second);
    r->graphs.erase(it);
  }
  while (r->graphs.size() >= r->graph_capacity && !r->lru.empty()) {
    uint64_t old = r->lru.back();
    r->lru.pop_back();
    auto o = r->graphs.find(old);
    cudaGraphExecDestroy(o->second.first.exec);
    cudaGraphDestroy(o->second.first.graph);
    r->graphs.erase(o);
    ++r->graph_evictions;
  }
  r->lru.push_front(key);
  r->graphs.emplace(key, std::make_pair(GraphEntry{ex, g, 0}, r->lru.begin()));
  return 0;
}
TB_EXPORT int tb_rt_graph_has(uint64_t key) {
  DeviceRuntime* r = rt(cur_dev());
  std::lock_guard<std::mutex> lk(r->mu);
  bool has = r->graphs.count(key) != 0;
  has ? ++r->graph_hits : ++r->graph_misses;
  return has;
}
TB_EXPORT int tb_rt_graph_launch(uint64_t key, cudaStream_t s) {
  TB_ENSURE_DEVICE();
  DeviceRuntime* r = rt(cur_dev());
  cudaGraphExec_t ex = nullptr;
  {
    std::lock_guard<std::mutex> lk(r->mu);
    auto it = r->graphs.find(key);
    if (it == r->graphs.end()) TB_FAIL(TB_E_ARG, "no graph cached under key %llu", (unsigned long long)key);
    r->lru.erase(it->second.second);
    r->lru.push_front(key);
    it->second.second = r->lru.begin();
    it->second.first.launches++;
    ex = it->second.first.exec;
  }
  TB_CUDA_CHECK(cudaGraphLaunch(ex, s));
  return 0;
}
TB_EXPORT int tb_rt_graph_node_count(uint64_t key) {
  DeviceRuntime* r = rt(cur_dev());
  std::lock_guard<std::mutex> lk(r->mu);
  auto it = r->graphs.find(key);
  if (it == r->graphs.end()) return -1;
  size_t n = 0;
  return cudaGraphGetNodes(it->second.first.graph, nullptr, &n) == cudaSuccess ? (int)n : -1;
}
TB_EXPORT void tb_rt_graph_set_capacity(uint64_t n) { rt(cur_dev())->graph_capacity = n ? n : 1; }
TB_EXPORT void tb_rt_graph_clear() {
  DeviceRuntime* r = rt(cur_dev());
  std::lock_guard<std::mutex> lk(r->mu);
  for (auto& kv : r->graphs) {
    cudaGraphExecDestroy(kv.second.first.exec);
    cudaGraphDestroy(kv.second.first.graph);
  }
  r->graphs.clear();
  r->lru.clear();
}
TB_EXPORT void tb_rt_graph_stats(uint64_t* out4) {
  DeviceRuntime* r = rt(cur_dev());
  std::lock_guard<std::mutex> lk(r->mu);
  out4[0] = r->graphs.size(); out4[1] = r->graph_hits; out4[2] = r->graph_misses; out4[3] = r->graph_evictions;
}

// Theoretical occupancy inputs for a launch configuration: resident CTAs per SM limited by threads, registers and
// shared memory (the role of crates/torsh-backend/src/cuda/occupancy.rs, with sm_100a limits read from the device).
TB_EXPORT int tb_rt_occupancy(int threads, int regs_per_thread, uint64_t smem_bytes, int* ctas_per_sm, int* limiter) {
  TB_ENSURE_DEVICE();
  cudaDeviceProp p;
  TB_CUDA_CHECK(cudaGetDeviceProperties(&p, cur_dev()));
  if (threads <= 0 || threads > p.maxThreadsPerBlock) TB_FAIL(TB_E_ARG, "threads per block %d out of range", threads);
  int by_thr = p.maxThreadsPerMultiProcessor / threads;
  int warps = (threads + 31) / 32;
  int regs_cta = ((regs_per_thread * 32 + 255) / 256 * 256) * warps;
  int by_reg = regs_cta ? p.regsPerMultiprocessor / regs_cta : 1 << 30;
  uint64_t smem_cta = smem_bytes + 1024;  // per-CTA reservation
  int by_smem = (int)(p.sharedMemPerMultiprocessor / smem_cta);
  int by_cta = p.maxBlocksPerMultiProcessor;
  int best = by_thr, lim = 0;
  if (by_reg < best) { best = by_reg; lim = 1; }
  if (by_smem < best) { best = by_smem; lim = 2; }
  if (by_cta < best) { best = by_cta; lim = 3; }
  *ctas_per_sm = best;
  *limiter = lim;  // 0 threads, 1 registers, 2 shared memory, 3 CTA slots
  return 0;
}

// ---------------------------------------------------------------------------------------------- profiler
// Scoped ranges: tb_prof_push(name, stream) opens an NVTX range (visible to Nsight tools) and records a CUDA event;
// tb_prof_pop records the closing event. tb_prof_collect synchronises the events and returns
// (name, depth, host start in microseconds since the first push, device duration in microseconds) per closed range.
// Role of the reference's ScopeGuard / CudaProfiler / NvtxRange, which only record host timestamps
// (crates/torsh-profiler/src/core/scope.rs, src/cuda.rs:21-437).
#include <nvtx3/nvToolsExt.h>

#include <chrono>
#include <string>

namespace tb {
namespace {
struct ProfRange {
  std::string name;
  int depth;
  double host_us;
  cudaEvent_t e0, e1;
  bool closed;
};
struct ProfState {
  std::mutex mu;
  std::vector<ProfRange> ranges;
  std::vector<size_t> open;
  std::chrono::steady_clock::time_point t0;
  bool started = false, enabled = true;
};
ProfState& prof() {
  static ProfState* s = new ProfState();
  return *s;
}
}  // namespace
}  // namespace tb

TB_EXPORT void tb_prof_enable(int on) { prof().enabled = on != 0; }
TB_EXPORT int tb_prof_push(const char* name, cudaStream_t st) {
  ProfState& s = prof();
  if (!s.enabled) return 0;
  TB_ENSURE_DEVICE();
  nvtxRangePushA(name);
  std::lock_guard<std::mutex> g(s.mu);
  if (!s.started) {
    s.t0 = std::chrono::steady_clock::now();
    s.started = true;
  }
  ProfRange r;
  r.name = name;
  r.depth = (int)s.open.size();
  r.host_us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - s.t0).count();
  r.closed = false;
  TB_CUDA_CHECK(cudaEventCreate(&r.e0));
  TB_CUDA_CHECK(cudaEventCreate(&r.e1));
  TB_CUDA_CHECK(cudaEventRecord(r.e0, st));
  s.open.push_back(s.ranges.size());
  s.ranges.push_back(r);
  return 0;
}
TB_EXPORT int tb_prof_pop(cudaStream_t st) {
  ProfState& s = prof();
  if (!s.enabled) return 0;
  TB_ENSURE_DEVICE();
  nvtxRangePop();
  std::lock_guard<std::mutex> g(s.mu);
  if (s.open.empty()) TB_FAIL(TB_E_ARG, "prof_pop without a matching push");
  ProfRange& r = s.ranges[s.open.back()];
  s.open.pop_back();
  TB_CUDA_CHECK(cudaEventRecord(r.e1, st));
  r.closed = true;
  return 0;
}
// Fills up to `cap` records; names are copied into name_buf (64 bytes each). Returns the number of records and
// clears them.
TB_EXPORT int tb_prof_collect(char* name_buf, int* depth, double* host_us, float* device_us, int cap) {
  ProfState& s = prof();
  if (ensure_device()) return 0;
  std::lock_guard<std::mutex> g(s.mu);
  int n = 0;
  std::vector<ProfRange> keep;
  for (ProfRange& r : s.ranges) {
    if (!r.closed) {
      keep.push_back(r);
      continue;
    }
    if (n < cap) {
      float ms = 0.f;
      cudaEventSynchronize(r.e1);
      cudaEventElapsedTime(&ms, r.e0, r.e1);
      snprintf(name_buf + 64 * n, 64, "%s", r.name.c_str());
      depth[n] = r.depth;
      host_us[n] = r.host_us;
      device_us[n] = ms * 1000.f;
      ++n;
    }
    cudaEventDestroy(r.e0);
    cudaEventDestroy(r.e1);
  }
  // indices of still-open ranges shift: rebuild
  s.open.clear();
  for (size_t i = 0; i < keep.size(); ++i) s.open.push_back(i);
  s.ranges.swap(keep);
  return n;
}
