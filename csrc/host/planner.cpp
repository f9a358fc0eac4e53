// Host-side planning arithmetic of the parallel engines, native so the schedulers can call it from
// their launch paths without the interpreter:
//   * DDP gradient buckets   - parameters sorted largest first, greedy fill up to the cap
//                              (crates/torsh-distributed/src/ddp.rs:268-327; cap 25 MB, floor 1 MB)
//   * FSDP shard ranges      - base + (rank < rem) split (crates/torsh-distributed/src/fsdp.rs:239-303)
//   * 3-D rank mapping       - rank = dp*(tp*pp) + tp*pp_size + pp with pp fastest (the reference rule,
//                              crates/torsh-distributed/src/three_d_parallelism/config.rs:195-225), or the
//                              NVSwitch-friendly variant with tp fastest
//   * pipeline schedules     - GPipe and 1F1B action lists (warm-up = min(stages - stage - 1, M) forwards,
//                              steady one-forward-one-backward, cool-down backwards); the reference's
//                              1F1B skeleton is crates/torsh-distributed/src/pipeline.rs:254-340
#include <algorithm>
#include <cstdint>
#include <numeric>
#include <vector>

#include "host_api.h"

// bucket_of[i] receives the bucket index of parameter i. Returns the number of buckets.
TSH_EXPORT int tsh_ddp_assign_buckets(const int64_t* param_bytes, int n, int64_t cap_bytes, int32_t* bucket_of) {
  if (n <= 0) return 0;
  std::vector<int> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return param_bytes[a] > param_bytes[b]; });
  int bucket = 0;
  int64_t used = 0;
  bool open = false;
  for (int idx : order) {
    int64_t sz = param_bytes[idx];
    if (open && used + sz > cap_bytes) {
      ++bucket;
      used = 0;
      open = false;
    }
    bucket_of[idx] = bucket;
    used += sz;
    open = true;
  }
  return bucket + 1;
}

TSH_EXPORT void tsh_fsdp_shard_range(int64_t numel, int world, int rank, int64_t* start, int64_t* end) {
  int64_t base = numel / world, rem = numel % world;
  *start = rank * base + std::min<int64_t>(rank, rem);
  *end = *start + base + (rank < rem ? 1 : 0);
}

// order 0: pp fastest (reference); order 1: tp fastest (TP peers are adjacent ranks).
TSH_EXPORT int tsh_rank_of(int dp, int tp, int pp, int dp_size, int tp_size, int pp_size, int order) {
  if (dp < 0 || dp >= dp_size || tp < 0 || tp >= tp_size || pp < 0 || pp >= pp_size) return -1;
  if (order == 0) return dp * (tp_size * pp_size) + tp * pp_size + pp;
  return dp * (tp_size * pp_size) + pp * tp_size + tp;
}
TSH_EXPORT int tsh_coords_of(int rank, int dp_size, int tp_size, int pp_size, int order, int* dp, int* tp, int* pp) {
  if (rank < 0 || rank >= dp_size * tp_size * pp_size) return -1;
  *dp = rank / (tp_size * pp_size);
  int r = rank % (tp_size * pp_size);
  if (order == 0) { *tp = r / pp_size; *pp = r % pp_size; }
  else { *pp = r / tp_size; *tp = r % tp_size; }
  return 0;
}

// Action encoding: kind (0 = forward, 1 = backward) in bit 31..30... kept simple: actions[2*i] = kind,
// actions[2*i+1] = micro-batch. Returns the number of actions (2 * M) or -1.
// schedule 0 = GPipe (all forwards, then all backwards in reverse), 1 = 1F1B.
TSH_EXPORT int tsh_pipeline_schedule(int schedule, int stage, int num_stages, int num_micro, int32_t* actions, int cap) {
  if (stage < 0 || stage >= num_stages || num_micro <= 0 || cap < 2 * num_micro) return -1;
  int n = 0;
  auto push = [&](int kind, int mb) { actions[2 * n] = kind; actions[2 * n + 1] = mb; ++n; };
  if (schedule == 0) {
    for (int m = 0; m < num_micro; ++m) push(0, m);
    for (int m = num_micro - 1; m >= 0; --m) push(1, m);
    return n;
  }
  int warm = std::min(num_stages - stage - 1, num_micro);
  int f = 0, b = 0;
  for (int i = 0; i < warm; ++i) push(0, f++);
  int steady = num_micro - warm;
  for (int i = 0; i < steady; ++i) { push(0, f++); push(1, b++); }
  while (b < num_micro) push(1, b++);
  return n;
}

// Interleaved 1F1B over virtual stages: every rank holds `num_chunks` model chunks (chunk c of rank r is virtual stage
// c * num_stages + r), so a micro-batch crosses every rank num_chunks times and the pipeline bubble shrinks by that
// factor. Needs num_micro % num_stages == 0. actions[3*i] = kind (0 forward, 1 backward), [3*i+1] = micro-batch,
// [3*i+2] = chunk. Forward step k of a rank works on chunk (k / P) % V of micro-batch (k / (P*V)) * P + k % P;
// backward steps visit the chunks in reverse. Warm-up is (P - r - 1) * 2 + (V - 1) * P forwards, then one forward
// and one backward alternate, then the remaining backwards. Returns the number of actions (2 * M * V) or -1.
// The reference names this schedule and runs plain 1F1B for it (crates/torsh-distributed/src/pipeline.rs:343-347).
TSH_EXPORT int tsh_pipeline_schedule_interleaved(int stage, int num_stages, int num_micro, int num_chunks,
                                                 int32_t* actions, int cap) {
  const int P = num_stages, V = num_chunks, M = num_micro;
  if (stage < 0 || stage >= P || M <= 0 || V < 1 || M % P != 0 || cap < 2 * M * V) return -1;
  const int total = M * V;
  int n = 0;
  auto push = [&](int kind, int k) {
    const int group = k / (P * V), in_group = k % (P * V);
    int chunk = in_group / P;
    if (kind == 1) chunk = V - 1 - chunk;
    actions[3 * n] = kind;
    actions[3 * n + 1] = group * P + in_group % P;
    actions[3 * n + 2] = chunk;
    ++n;
  };
  int warm = std::min((P - stage - 1) * 2 + (V - 1) * P, total);
  int f = 0, b = 0;
  for (int i = 0; i < warm; ++i) push(0, f++);
  while (f < total) { push(0, f++); push(1, b++); }
  while (b < total) push(1, b++);
  return n;
}

// Peak number of activations a stage holds under the schedule (for the memory planner).
TSH_EXPORT int tsh_pipeline_peak_inflight(int schedule, int stage, int num_stages, int num_micro) {
  std::vector<int32_t> a(4 * (size_t)std::max(num_micro, 1));
  int n = tsh_pipeline_schedule(schedule, stage, num_stages, num_micro, a.data(), (int)a.size());
  int cur = 0, peak = 0;
  for (int i = 0; i < n; ++i) {
    cur += a[2 * i] == 0 ? 1 : -1;
    peak = std::max(peak, cur);
  }
  return peak;
}
