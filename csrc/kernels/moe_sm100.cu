// Mixture-of-experts token dispatch / combine over NVSwitch peer memory for sm_100a.
//
// Every rank owns E_local experts and a symmetric receive buffer laid out [E_local][world][C][H]: C capacity slots
// per (expert, source rank). The router has already given every (token, choice) pair its slot inside its expert
// (arrival order among the source rank's tokens) and a keep flag (false when the expert is over capacity), so both
// directions are pure data movement with fixed addresses and need no counting pass or size exchange:
//   scatter  (dispatch forward, combine backward): a warp copies scale * src[t, :] straight into the owner's buffer
//            row with 16-byte peer stores;
//   gather   (combine forward, dispatch backward): a warp sums w[t,k] * row over the token's K choices with 16-byte
//            peer loads, optionally also returning dot[t,k] = <dy[t,:], row> (the gate gradient).
// A one-CTA flag barrier (monotonic epochs, bounded waits) separates the phases. The reference's dispatch and combine
// move whole tensors through its mock all-to-all (crates/torsh-distributed/src/expert_parallelism/manager.rs:101-323).
#include "comm.cuh"
#include "common.cuh"
#include "host_util.h"

namespace tb {

struct MoeArgs {
  PeerTable bufs;        // symmetric [E_local][world][C][H] bf16 buffer on every rank
  const long* expert;    // [T, K] global expert id
  const long* slot;      // [T, K] slot inside (expert, this source rank)
  const uint8_t* keep;   // [T, K]
  const float* w;        // [T, K] weights (null = 1)
  int T, K, H, C, e_local, rank, world;
};

__device__ __forceinline__ bf16* moe_row(const MoeArgs& a, long e, long slot) {
  const int owner = (int)(e / a.e_local), le = (int)(e % a.e_local);
  return reinterpret_cast<bf16*>(a.bufs.ptr[owner]) + ((((long)le * a.world + a.rank) * a.C + slot) * a.H);
}

// one warp per (token, choice)
__global__ void moe_scatter_kernel(const MoeArgs a, const bf16* __restrict__ src, const int* __restrict__ counts,
                                   int* const* __restrict__ count_bufs) {
  const int lane = threadIdx.x & 31;
  const long wid = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long nwarps = ((long)gridDim.x * blockDim.x) >> 5;
  // the source also tells every owner how many of its slots are filled: counts_owner[le][src_rank]
  if (counts && blockIdx.x == 0) {
    for (int e = threadIdx.x; e < a.e_local * a.world; e += blockDim.x) {
      const int owner = e / a.e_local, le = e % a.e_local;
      count_bufs[owner][le * a.world + a.rank] = min(counts[e], a.C);
    }
  }
  const int nvec = a.H >> 3;
  for (long p = wid; p < (long)a.T * a.K; p += nwarps) {
    if (!a.keep[p]) continue;
    const long e = a.expert[p], s = a.slot[p];
    if (e < 0 || e >= (long)a.e_local * a.world || s < 0 || s >= a.C) {
      if (lane == 0) report_bad_index();
      continue;
    }
    const long t = p / a.K;
    const float sc = a.w ? a.w[p] : 1.f;
    const bf16* sp = src + t * a.H;
    bf16* dp = moe_row(a, e, s);
    for (int v = lane; v < nvec; v += 32) {
      Vec16<bf16> x;
      x.load_nc(sp + v * 8);
      if (a.w) {
        float f[8];
        x.get(f);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] *= sc;
        x.set(f);
      }
      x.store(dp + v * 8);
    }
  }
}

// one warp per token; y may be null when only the dot products are wanted
__global__ void moe_gather_kernel(const MoeArgs a, bf16* __restrict__ y, const bf16* __restrict__ dy,
                                  float* __restrict__ dot) {
  const int lane = threadIdx.x & 31;
  const long wid = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long nwarps = ((long)gridDim.x * blockDim.x) >> 5;
  const int nvec = a.H >> 3;
  constexpr int MAXK = 8;
  for (long t = wid; t < a.T; t += nwarps) {
    const bf16* rows[MAXK];
    float wk[MAXK], dk[MAXK];
#pragma unroll
    for (int k = 0; k < MAXK; ++k) {
      rows[k] = nullptr;
      wk[k] = dk[k] = 0.f;
      if (k < a.K) {
        const long p = t * a.K + k;
        const long e = a.expert[p], s = a.slot[p];
        if (a.keep[p] && e >= 0 && e < (long)a.e_local * a.world && s >= 0 && s < a.C) {
          rows[k] = moe_row(a, e, s);
          wk[k] = a.w ? a.w[p] : 1.f;
        }
      }
    }
    for (int v = lane; v < nvec; v += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, g[8];
      if (dot) {
        Vec16<bf16> gv;
        gv.load_nc(dy + t * a.H + v * 8);
        gv.get(g);
      }
#pragma unroll
      for (int k = 0; k < MAXK; ++k) {
        if (!rows[k]) continue;
        Vec16<bf16> x;
        x.load(rows[k] + v * 8);  // peer memory written during this step: plain (coherent) loads
        float f[8];
        x.get(f);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          acc[j] = fmaf(wk[k], f[j], acc[j]);
          if (dot) dk[k] = fmaf(g[j], f[j], dk[k]);
        }
      }
      if (y) {
        Vec16<bf16> o;
        o.set(acc);
        o.store(y + t * a.H + v * 8);
      }
    }
    if (dot) {
#pragma unroll
      for (int k = 0; k < MAXK; ++k)
        if (k < a.K) {
          const float s = warp_sum(dk[k]);
          if (lane == 0) dot[t * a.K + k] = s;
        }
    }
  }
}

// One CTA: every rank has reached this point of its stream (and its earlier peer stores are visible).
__global__ void comm_barrier_kernel(PeerTable flags, int rank, int world, uint32_t* epoch_ptr, int* status) {
  const uint32_t epoch = *epoch_ptr;
  cta_barrier_all_ranks(flags, 0, rank, world, 2 * epoch, status);
  if (threadIdx.x == 0) *epoch_ptr = epoch + 1;
}

static int fill_moe(MoeArgs& a, const void* const* bufs, const long* expert, const long* slot, const void* keep,
                    const float* w, int T, int K, int H, int C, int e_local, int rank, int world) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) TB_FAIL(TB_E_ARG, "moe: bad rank/world %d/%d", rank, world);
  if (K < 1 || K > 8) TB_FAIL(TB_E_ARG, "moe: top-k must be in [1, 8]");
  if (H % 8) TB_FAIL(TB_E_ARG, "moe: hidden size must be a multiple of 8");
  for (int i = 0; i < MAX_RANKS; ++i) a.bufs.ptr[i] = i < world ? const_cast<void*>(bufs[i]) : nullptr;
  a.expert = expert; a.slot = slot; a.keep = (const uint8_t*)keep; a.w = w;
  a.T = T; a.K = K; a.H = H; a.C = C; a.e_local = e_local; a.rank = rank; a.world = world;
  return 0;
}

}  // namespace tb
using namespace tb;

// src: [T, H] bf16. bufs: the symmetric destination buffers of all ranks. counts (optional): [E] int32 kept tokens per
// global expert on this rank, forwarded to count_bufs (device array of `world` pointers to each rank's [E_local][world]).
TB_EXPORT int tb_moe_scatter(const void* src, const void* const* bufs, const long* expert, const long* slot,
                             const void* keep, const float* scale, const int* counts, int* const* count_bufs, int T,
                             int K, int H, int C, int e_local, int rank, int world, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (T <= 0) return 0;
  MoeArgs a;
  if (int r = fill_moe(a, bufs, expert, slot, keep, scale, T, K, H, C, e_local, rank, world)) return r;
  if (((uintptr_t)src & 15)) TB_FAIL(TB_E_ARG, "moe_scatter: source must be 16-byte aligned");
  long warps = (long)T * K;
  int blocks = (int)((warps + 7) / 8);
  if (blocks > sm_count() * 8) blocks = sm_count() * 8;
  moe_scatter_kernel<<<blocks, 256, 0, st>>>(a, (const bf16*)src, counts, count_bufs);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// y: [T, H] bf16 (or null); dot: [T, K] fp32 with dy [T, H] bf16 (or both null).
TB_EXPORT int tb_moe_gather(const void* const* bufs, const long* expert, const long* slot, const void* keep,
                            const float* w, void* y, const void* dy, float* dot, int T, int K, int H, int C, int e_local,
                            int rank, int world, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (T <= 0) return 0;
  MoeArgs a;
  if (int r = fill_moe(a, bufs, expert, slot, keep, w, T, K, H, C, e_local, rank, world)) return r;
  if ((dot != nullptr) != (dy != nullptr)) TB_FAIL(TB_E_ARG, "moe_gather: dot and dy go together");
  int blocks = (int)(((long)T + 7) / 8);
  if (blocks > sm_count() * 8) blocks = sm_count() * 8;
  moe_gather_kernel<<<blocks, 256, 0, st>>>(a, (bf16*)y, (const bf16*)dy, dot);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

TB_EXPORT int tb_comm_barrier(const void* const* flags, int rank, int world, unsigned* epoch_ptr, int* status,
                              cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (world < 1 || world > MAX_RANKS) TB_FAIL(TB_E_ARG, "comm_barrier: bad world size %d", world);
  PeerTable f;
  for (int i = 0; i < MAX_RANKS; ++i) f.ptr[i] = i < world ? const_cast<void*>(flags[i]) : nullptr;
  comm_barrier_kernel<<<1, 32, 0, st>>>(f, rank, world, epoch_ptr, status);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int tb_set_check_word_moe(int* word) {
  TB_CUDA_CHECK(tb::set_check_word_this_tu(word));
  return 0;
}
