// Heartbeat watchdog (roles of HealthChecker / ElasticTrainingManager heartbeats in
// crates/torsh-distributed/src/error_recovery.rs:377-497 and fault_tolerance.rs:451-855): a native thread beats for
// this rank at a fixed interval and keeps the time of the last beat seen from every peer; ranks whose beat is older
// than the timeout are reported as failed. Beats travel through caller-supplied callbacks (the Python side wires them to
// the TCP store), so the thread keeps running while the interpreter is busy inside a long kernel launch or collective.
#include <atomic>
#include <chrono>
#include <mutex>
#include <thread>
#include <vector>

#include "host_api.h"

namespace {
using Clock = std::chrono::steady_clock;
typedef void (*PublishFn)(int rank, long long counter, void* ctx);
typedef long long (*ReadFn)(int rank, void* ctx);  // latest counter of `rank`, or -1 when none was published

struct Watchdog {
  int rank, world;
  double interval_s, timeout_s;
  PublishFn publish;
  ReadFn read;
  void* ctx;
  std::thread th;
  std::atomic<bool> stop{false};
  std::mutex mu;
  std::vector<long long> last_counter;
  std::vector<Clock::time_point> last_change;
  std::atomic<long long> beats{0};

  void run() {
    while (!stop.load()) {
      long long c = beats.fetch_add(1) + 1;
      if (publish) publish(rank, c, ctx);
      auto now = Clock::now();
      if (read) {
        std::lock_guard<std::mutex> g(mu);
        for (int r = 0; r < world; ++r) {
          long long v = r == rank ? c : read(r, ctx);
          if (v != last_counter[r]) {
            last_counter[r] = v;
            last_change[r] = now;
          }
        }
      }
      std::this_thread::sleep_for(std::chrono::duration<double>(interval_s));
    }
  }
};
}  // namespace

TSH_EXPORT void* tsh_watchdog_start(int rank, int world, double interval_s, double timeout_s, PublishFn publish, ReadFn read,
                                    void* ctx) {
  if (rank < 0 || world < 1 || rank >= world || interval_s <= 0) return nullptr;
  auto* w = new Watchdog();
  w->rank = rank; w->world = world; w->interval_s = interval_s; w->timeout_s = timeout_s;
  w->publish = publish; w->read = read; w->ctx = ctx;
  w->last_counter.assign(world, -1);
  w->last_change.assign(world, Clock::now());
  w->th = std::thread([w] { w->run(); });
  return w;
}
// Writes 1 into failed[r] for every rank whose beat has not changed for longer than the timeout; returns their count.
TSH_EXPORT int tsh_watchdog_failed(void* h, int* failed) {
  auto* w = (Watchdog*)h;
  std::lock_guard<std::mutex> g(w->mu);
  auto now = Clock::now();
  int n = 0;
  for (int r = 0; r < w->world; ++r) {
    double age = std::chrono::duration<double>(now - w->last_change[r]).count();
    failed[r] = (r != w->rank && age > w->timeout_s) ? 1 : 0;
    n += failed[r];
  }
  return n;
}
TSH_EXPORT long long tsh_watchdog_beats(void* h) { return ((Watchdog*)h)->beats.load(); }
TSH_EXPORT void tsh_watchdog_stop(void* h) {
  auto* w = (Watchdog*)h;
  w->stop.store(true);
  if (w->th.joinable()) w->th.join();
  delete w;
}
