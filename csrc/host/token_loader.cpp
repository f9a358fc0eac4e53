// Native token-batch loader: the data-loader worker pool of the reference (crates/torsh-data: DataLoader with workers,
// prefetch and pinned batches) specialised for language-model training. A token file (raw little-endian uint16 or
// int32 ids) is memory-mapped; worker threads cut [batch, seq + 1] windows at pseudo-random offsets and write them as
// int64 into a ring of caller-supplied buffers (pinned host memory when the caller allocated it so), so that the Python
// training loop only ever takes a finished batch and never touches the file or converts a token itself.
//
// Batches are deterministic: batch number b of (seed, rank, world) always holds the same windows, whichever worker fills
// it, and ranks draw disjoint streams (the generator is seeded with (seed, rank, b)).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <condition_variable>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>

#include "host_api.h"

namespace {
struct SplitMix {
  uint64_t s;
  uint64_t next() {
    uint64_t z = (s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  }
};

struct Loader {
  int fd = -1;
  const uint8_t* map = nullptr;
  size_t map_bytes = 0;
  long long n_tokens = 0;
  int token_bytes = 2;
  int batch = 0, seq = 0, slots = 0, rank = 0, world = 1;
  uint64_t seed = 0;
  std::vector<long long*> bufs;          // slots buffers of batch * (seq + 1) int64
  std::vector<long long> slot_batch;     // which batch number a slot holds (-1: free)
  std::vector<int> slot_state;           // 0 free, 1 being filled, 2 ready, 3 held by the consumer
  long long next_fill = 0, next_take = 0;
  std::mutex mu;
  std::condition_variable cv_fill, cv_take;
  std::vector<std::thread> workers;
  bool stop = false;
  std::atomic<long long> filled{0};

  long long token(long long i) const {
    if (token_bytes == 2) {
      uint16_t v;
      std::memcpy(&v, map + 2 * i, 2);
      return v;
    }
    int32_t v;
    std::memcpy(&v, map + 4 * i, 4);
    return v;
  }

  void fill(long long b, long long* dst) const {
    SplitMix g{seed * 0x100000001B3ull + (uint64_t)rank * 0x9E3779B1ull + (uint64_t)b * 0x85EBCA6Bull + 1};
    const long long span = (long long)seq + 1;
    const long long range = n_tokens - span + 1;
    for (int r = 0; r < batch; ++r) {
      const long long off = (long long)(g.next() % (uint64_t)range);
      for (long long j = 0; j < span; ++j) dst[(long long)r * span + j] = token(off + j);
    }
  }

  void run() {
    for (;;) {
      long long b;
      int slot;
      {
        std::unique_lock<std::mutex> lk(mu);
        // batch b lives in slot b % slots; it may be filled once the consumer has released batch b - slots
        cv_fill.wait(lk, [&] { return stop || slot_state[next_fill % slots] == 0; });
        if (stop) return;
        b = next_fill++;
        slot = (int)(b % slots);
        slot_state[slot] = 1;
        slot_batch[slot] = b;
      }
      fill(b, bufs[slot]);
      {
        std::lock_guard<std::mutex> lk(mu);
        slot_state[slot] = 2;
        filled.fetch_add(1);
      }
      cv_take.notify_all();
    }
  }
};
}  // namespace

// token_bytes: 2 (uint16) or 4 (int32). buffers: `slots` pointers to batch * (seq + 1) int64 each.
TSH_EXPORT void* tsh_tokens_open(const char* path, int token_bytes, int batch, int seq, int slots, long long** buffers,
                                 int workers, unsigned long long seed, int rank, int world) {
  if ((token_bytes != 2 && token_bytes != 4) || batch < 1 || seq < 1 || slots < 1 || workers < 1 || !buffers) {
    g_err = "token loader: bad arguments";
    return nullptr;
  }
  auto* L = new Loader();
  L->fd = ::open(path, O_RDONLY);
  struct stat st;
  if (L->fd < 0 || fstat(L->fd, &st) != 0) {
    g_err = std::string("token loader: cannot open ") + path;
    if (L->fd >= 0) ::close(L->fd);
    delete L;
    return nullptr;
  }
  L->map_bytes = (size_t)st.st_size;
  L->n_tokens = (long long)(L->map_bytes / token_bytes);
  if (L->n_tokens < (long long)seq + 1) {
    g_err = "token loader: file shorter than one sequence";
    ::close(L->fd);
    delete L;
    return nullptr;
  }
  void* m = mmap(nullptr, L->map_bytes, PROT_READ, MAP_PRIVATE, L->fd, 0);
  if (m == MAP_FAILED) {
    g_err = "token loader: mmap failed";
    ::close(L->fd);
    delete L;
    return nullptr;
  }
  madvise(m, L->map_bytes, MADV_RANDOM);
  L->map = (const uint8_t*)m;
  L->token_bytes = token_bytes;
  L->batch = batch; L->seq = seq; L->slots = slots; L->seed = seed; L->rank = rank; L->world = world;
  L->bufs.assign(buffers, buffers + slots);
  L->slot_batch.assign(slots, -1);
  L->slot_state.assign(slots, 0);
  for (int i = 0; i < workers; ++i) L->workers.emplace_back([L] { L->run(); });
  return L;
}

// Blocks until the next batch in order is ready; returns its slot (the caller reads buffers[slot]) or -1 on timeout.
TSH_EXPORT int tsh_tokens_next(void* h, double timeout_s, long long* batch_number) {
  auto* L = (Loader*)h;
  std::unique_lock<std::mutex> lk(L->mu);
  const int slot = (int)(L->next_take % L->slots);
  const long long want = L->next_take;
  if (!L->cv_take.wait_for(lk, std::chrono::duration<double>(timeout_s),
                           [&] { return L->slot_state[slot] == 2 && L->slot_batch[slot] == want; }))
    return -1;
  L->slot_state[slot] = 3;
  if (batch_number) *batch_number = want;
  L->next_take++;
  return slot;
}

// Hands a slot back to the workers once the consumer has copied (or finished using) its batch.
TSH_EXPORT int tsh_tokens_release(void* h, int slot) {
  auto* L = (Loader*)h;
  {
    std::lock_guard<std::mutex> lk(L->mu);
    if (slot < 0 || slot >= L->slots || L->slot_state[slot] != 3) return -1;
    L->slot_state[slot] = 0;
  }
  L->cv_fill.notify_all();
  return 0;
}

TSH_EXPORT long long tsh_tokens_count(void* h) { return ((Loader*)h)->n_tokens; }
TSH_EXPORT long long tsh_tokens_filled(void* h) { return ((Loader*)h)->filled.load(); }

TSH_EXPORT void tsh_tokens_close(void* h) {
  auto* L = (Loader*)h;
  {
    std::lock_guard<std::mutex> lk(L->mu);
    L->stop = true;
  }
  L->cv_fill.notify_all();
  for (auto& t : L->workers) t.join();
  munmap((void*)L->map, L->map_bytes);
  ::close(L->fd);
  delete L;
}
