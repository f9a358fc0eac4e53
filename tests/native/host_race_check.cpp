// Race check of the C++ host runtime under ThreadSanitizer: several threads hammer the caching pool, a token loader
// runs its workers against a consumer, and the TCP-store-free pieces are created and destroyed concurrently. Built and
// run by tests/test_native_tsan_cpu.py with -fsanitize=thread; any data race makes the program exit non-zero.
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <thread>
#include <vector>

extern "C" {
void* tsh_pool_create(uint64_t raw_budget_bytes, uint64_t limit_bytes);
void tsh_pool_destroy(void* h);
void* tsh_pool_alloc(void* h, uint64_t bytes, uint64_t stream);
int tsh_pool_free(void* h, void* p);
uint64_t tsh_pool_release_cached(void* h);
void* tsh_tokens_open(const char* path, int token_bytes, int batch, int seq, int slots, long long** buffers, int workers,
                      unsigned long long seed, int rank, int world);
int tsh_tokens_next(void* h, double timeout_s, long long* batch_number);
int tsh_tokens_release(void* h, int slot);
void tsh_tokens_close(void* h);
void* tsh_store_server_start(const char* host, int port, int* bound_port);
void tsh_store_server_stop(void* h);
void* tsh_store_client_connect(const char* host, int port, int timeout_ms);
void tsh_store_client_close(void* h);
int tsh_store_set(void* h, const char* key, const uint8_t* val, uint64_t n, int64_t ttl_secs);
int tsh_store_add(void* h, const char* key, int64_t delta, int64_t* result);
int tsh_store_wait(void* h, const char** keys, int nkeys, int timeout_ms);
void* tsh_watchdog_start(int rank, int world, double interval_s, double timeout_s, void (*publish)(int, long long, void*),
                         long long (*read)(int, void*), void* ctx);
int tsh_watchdog_failed(void* h, int* out);
long long tsh_watchdog_beats(void* h);
void tsh_watchdog_stop(void* h);
}

static std::atomic<long long> g_beats[2];
static void publish_beat(int rank, long long c, void*) { g_beats[rank].store(c); }
static long long read_beat(int rank, void*) { return g_beats[rank].load() ? g_beats[rank].load() : -1; }

int main(int argc, char** argv) {
  if (argc < 2) return 2;
  // ---- pool: 4 threads allocate, write, free
  void* pool = tsh_pool_create(0, 0);
  std::atomic<int> bad{0};
  std::vector<std::thread> ts;
  for (int t = 0; t < 4; ++t)
    ts.emplace_back([&, t] {
      std::vector<void*> mine;
      for (int i = 0; i < 400; ++i) {
        const uint64_t n = 64 + (uint64_t)((i * 37 + t * 101) % 5000);
        void* p = tsh_pool_alloc(pool, n, (uint64_t)t);
        if (!p) { bad++; continue; }
        std::memset(p, t + 1, n);
        mine.push_back(p);
        if (mine.size() > 8) {
          unsigned char* q = (unsigned char*)mine.front();
          if (q[0] != (unsigned char)(t + 1)) bad++;          // nobody else may have written into a live block
          tsh_pool_free(pool, mine.front());
          mine.erase(mine.begin());
        }
      }
      for (void* p : mine) tsh_pool_free(pool, p);
    });
  for (auto& t : ts) t.join();
  tsh_pool_release_cached(pool);
  tsh_pool_destroy(pool);
  // ---- token loader: 3 workers, one consumer, 3 slots
  const int batch = 2, seq = 8, slots = 3;
  std::vector<std::vector<long long>> store(slots, std::vector<long long>(batch * (seq + 1)));
  long long* bufs[slots];
  for (int i = 0; i < slots; ++i) bufs[i] = store[i].data();
  void* ld = tsh_tokens_open(argv[1], 2, batch, seq, slots, bufs, 3, 5, 0, 1);
  if (!ld) return 3;
  int held = -1;
  for (int i = 0; i < 200; ++i) {
    long long n = -1;
    int slot = tsh_tokens_next(ld, 10.0, &n);
    if (slot < 0 || n != i) { bad++; break; }
    for (int r = 0; r < batch; ++r)
      for (int j = 1; j <= seq; ++j)
        if (bufs[slot][r * (seq + 1) + j] != bufs[slot][r * (seq + 1)] + j) bad++;   // the file holds 0, 1, 2, ...
    if (held >= 0) tsh_tokens_release(ld, held);
    held = slot;
  }
  tsh_tokens_close(ld);
  // ---- TCP store: one server, 4 clients adding to one counter and waiting for each other's keys
  int port = 0;
  void* srv = tsh_store_server_start("127.0.0.1", 0, &port);
  if (!srv) return 4;
  std::vector<std::thread> cs;
  for (int t = 0; t < 4; ++t)
    cs.emplace_back([&, t] {
      void* c = tsh_store_client_connect("127.0.0.1", port, 5000);
      if (!c) { bad++; return; }
      int64_t v = 0;
      for (int i = 0; i < 50; ++i)
        if (tsh_store_add(c, "counter", 1, &v) != 0) bad++;
      char key[16];
      std::snprintf(key, sizeof key, "done%d", t);
      const uint8_t one = 1;
      tsh_store_set(c, key, &one, 1, -1);               // ttl < 0: no expiry
      const char* all[4] = {"done0", "done1", "done2", "done3"};
      if (tsh_store_wait(c, all, 4, 10000) != 0) bad++;
      if (tsh_store_add(c, "counter", 0, &v) != 0 || v != 200) bad++;
      tsh_store_client_close(c);
    });
  for (auto& t : cs) t.join();
  tsh_store_server_stop(srv);
  // ---- watchdog: two ranks beat through shared counters; rank 1 stops and rank 0 must report it as failed
  void* w0 = tsh_watchdog_start(0, 2, 0.01, 0.15, publish_beat, read_beat, nullptr);
  void* w1 = tsh_watchdog_start(1, 2, 0.01, 0.15, publish_beat, read_beat, nullptr);
  std::this_thread::sleep_for(std::chrono::milliseconds(100));
  int failed[2] = {0, 0};
  if (tsh_watchdog_failed(w0, failed) != 0) bad++;                  // nobody has failed yet
  tsh_watchdog_stop(w1);
  std::this_thread::sleep_for(std::chrono::milliseconds(400));
  if (tsh_watchdog_failed(w0, failed) != 1 || failed[1] != 1) bad++;
  if (tsh_watchdog_beats(w0) < 10) bad++;
  tsh_watchdog_stop(w0);
  std::printf("host race check: %d inconsistencies\n", bad.load());
  return bad.load() ? 1 : 0;
}
