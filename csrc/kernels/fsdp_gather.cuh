// Un-shard ("all-gather") of one FSDP unit by copy CTAs, usable on its own or inside the GEMM that first
// consumes the unit's weights.
//
// Layout. A unit is a contiguous bf16 range cut into equal CHUNKS (a power of two >= 16 KB); rank q keeps chunks
// [q * cpr, (q + 1) * cpr) of it in its persistent shard (symmetric memory, so every rank can read every shard).
// The gather PULLS: each rank copies all chunks - its own included - into its private full-size unit buffer with
// bulk async copies (peer memory -> shared memory -> local memory), one elected thread per copy CTA driving a ring of
// 16 KB pieces (half of the ring loading, half storing). Chunks are fetched in the order first, first + 1, ... (wrapping), so the matrix that the consuming GEMM
// needs first arrives first; a chunk's ready word is published (release, gpu scope) once all its parts have landed,
// and the GEMM's TMA producer waits (bounded) on the words that cover the tile it is about to load.
//
// Synchronisation across ranks: ONE entry barrier among the copy CTAs (every rank has reached this gather in stream
// order, hence its shard of the unit holds the values of its last optimizer step). No exit barrier: a shard is
// rewritten only by the reduce-scatter + AdamW kernel of the same unit, whose own entry barrier every rank reaches
// after this gather in stream order.
//
// The reference gathers per parameter with `all_gather` and keeps the first tensor
// (crates/torsh-distributed/src/fsdp.rs:307-369).
#pragma once
#include "comm.cuh"
#include "sm100.cuh"

namespace tb {

struct GatherArgs {
  const void* src[MAX_RANKS];  // every rank's shard of this unit (cpr chunks each)
  void* dst;                   // local unit buffer: world * cpr chunks
  void* flag_tbl[MAX_RANKS];   // symmetric flag buffer (entry barrier, one slot per copy CTA)
  const uint32_t* epoch_ptr;   // device epoch counter of the launching stream's communication context
  uint32_t* ready;             // local: [nchunks] ready words (ready when >= epoch), then [nchunks] arrival counters
  int chunk_bytes, cpr, first; // bytes per chunk, chunks per rank, first chunk to fetch
  int ctas;                    // copy CTAs of this launch
  int rank, world;
  int* status;
};

constexpr int GATHER_PIECE = 16384;

// Bounded wait on a word in this GPU's own memory, written by a copy CTA of the same launch.
__device__ __forceinline__ bool wait_ready_gpu(const uint32_t* flag, uint32_t target, int* status) {
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if ((int32_t)(v - target) >= 0) return true;
    if ((++spins & 31u) == 0u) {
      if (status && *((volatile int*)status) != 0) return false;  // the copy side (or anyone) already gave up
      if (globaltimer_ns() - t0 > TB_PEER_WAIT_LIMIT_NS) {
        if (status) atomicCAS(status, 0, TB_ERR_WAIT_PEER);
        return false;
      }
    }
  }
}

// Cross-rank barrier for ONE WARP (all 32 lanes call it) on flag slot `slot`; same contract as
// cta_barrier_all_ranks, used where the rest of the CTA is busy with something else.
__device__ __forceinline__ bool warp_barrier_all_ranks(const PeerTable& flags, int slot, int rank, int world, uint32_t epoch,
                                                       int* status) {
  const int lane = threadIdx.x & 31;
  __syncwarp();
  int ok = 1;
  if (lane < world) {
    fence_sys();
    uint32_t* remote = reinterpret_cast<uint32_t*>(flags.ptr[lane]) + (size_t)slot * MAX_RANKS + rank;
    st_release_sys(remote, epoch);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(flags.ptr[rank]) + (size_t)slot * MAX_RANKS + lane;
    ok = wait_flag_ge(mine, epoch, status) ? 1 : 0;
    if (status && *((volatile int*)status) != 0) ok = 0;
    fence_sys();
  }
  return __all_sync(0xffffffffu, ok) != 0;
}

// The copy loop of one elected thread: units cta, cta + ctas, ... of the unit's (chunk, 64 KB part) list, in the fetch
// order that starts at chunk g.first, through a ring of NBUF pieces at `smem` with one mbarrier per buffer.
template <int NBUF, int PIECE>
__device__ __forceinline__ void unit_gather_thread(const GatherArgs& g, int cta, int ctas, uint32_t epoch, uint8_t* smem,
                                                   uint64_t* bars, volatile int* abort_flag) {
  static_assert(NBUF >= 2, "the gather ring needs at least two buffers");
  constexpr int STORES = NBUF / 2;  // stores allowed to be reading their buffers at once; the other buffers are being loaded
  const int nchunks = g.world * g.cpr;
  // parts of at most 64 KB: the first chunks are spread over several copy threads and land early
  const int part_bytes = g.chunk_bytes < 65536 ? g.chunk_bytes : (PIECE > 65536 ? PIECE : 65536);
  const int split = g.chunk_bytes / part_bytes;
  const int ppu = part_bytes / PIECE;  // pieces per unit
  const int units = nchunks * split;
  const int my_units = cta < units ? (units - cta + ctas - 1) / ctas : 0;
  const long total = (long)my_units * ppu;
  auto locate = [&](long i, const char*& src, char*& dst, int& chunk, int& piece) {
    const int ui = (int)(i / ppu);
    piece = (int)(i - (long)ui * ppu);
    const int u = cta + ui * ctas;
    const int part = u % split;
    int c = g.first + u / split;
    if (c >= nchunks) c -= nchunks;
    chunk = c;
    const int q = c / g.cpr;
    const long in_chunk = (long)part * part_bytes + (long)piece * PIECE;
    src = reinterpret_cast<const char*>(g.src[q]) + (long)(c - q * g.cpr) * g.chunk_bytes + in_chunk;
    dst = reinterpret_cast<char*>(g.dst) + (long)c * g.chunk_bytes + in_chunk;
  };
  auto issue_load = [&](long i) {
    const char* src; char* dst; int chunk, piece;
    locate(i, src, dst, chunk, piece);
    const int b = (int)(i % NBUF);
    mbar_expect_tx(&bars[b], PIECE);
    bulk_load(smem + b * PIECE, src, PIECE, &bars[b]);
  };
  // A part is published once the stores of all its pieces have completed. Stores complete in order, so instead of
  // draining the store queue at every part boundary, publication runs LAG pieces behind the store just issued:
  // `cp.async.bulk.wait_group LAG` leaves at most LAG store groups pending, hence every piece up to i - LAG has landed.
  constexpr int LAG = 16;
  long pub = 0;  // every part that ends before piece `pub` has been published
  auto publish_upto = [&](long done) {  // stores of pieces [0, done) are complete
    bool fenced = false;
    while (pub + ppu <= done) {
      const char* src; char* dst; int chunk, piece;
      locate(pub + ppu - 1, src, dst, chunk, piece);
      if (!fenced) {
        __threadfence();
        fenced = true;
      }
      uint32_t* cnt = g.ready + nchunks + chunk;
      uint32_t arrived;
      asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(arrived) : "l"(cnt) : "memory");
      if (arrived == (uint32_t)split - 1) {  // last part: reset the counter for the next launch, publish the chunk
        *cnt = 0;
        asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(g.ready + chunk), "r"(epoch) : "memory");
      }
      pub += ppu;
    }
  };
  long next_load = 0;
  for (; next_load < total && next_load < NBUF; ++next_load) issue_load(next_load);
  for (long i = 0; i < total; ++i) {
    const char* src; char* dst; int chunk, piece;
    locate(i, src, dst, chunk, piece);
    const int b = (int)(i % NBUF);
    mbar_wait(&bars[b], (uint32_t)((i / NBUF) & 1), abort_flag, g.status, TB_ERR_WAIT_FULL);
    bulk_store(dst, smem + b * PIECE, PIECE);
    bulk_commit();
    if (next_load < total) {
      // at most STORES stores still read their buffers, so the stores of pieces <= i - STORES have released theirs:
      // refill those buffers (piece j + NBUF goes into the buffer of piece j)
      asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(STORES) : "memory");
      while (next_load < total && next_load <= i - STORES + NBUF) issue_load(next_load++);
    }
    if (i >= LAG) {
      asm volatile("cp.async.bulk.wait_group %0;" ::"n"(LAG) : "memory");
      publish_upto(i - LAG + 1);
    }
  }
  bulk_wait_all();
  publish_upto(total);
  if (*abort_flag) {
    // a piece never landed: give copies still in flight time to settle before the CTA's shared memory is released
    uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) {
    }
  }
}

// Copy role of a whole CTA (stand-alone gather kernel, or the dedicated copy CTAs of a GEMM launch). `cta` is this
// CTA's index among the g.ctas copy CTAs; `smem` points at SMEM_BYTES of ring space (16-byte aligned), `bars` at 12
// mbarriers, `abort_flag` at a CTA-local word. Every thread of the CTA calls it.
template <int SMEM_BYTES, int PIECE = GATHER_PIECE>
__device__ __forceinline__ void unit_gather_role(const GatherArgs& g, int cta, uint8_t* smem, uint64_t* bars,
                                                 volatile int* abort_flag) {
  constexpr int NBUF = SMEM_BYTES / PIECE < 12 ? SMEM_BYTES / PIECE : 12;
  const uint32_t epoch = *g.epoch_ptr;
  PeerTable flags;
#pragma unroll
  for (int i = 0; i < MAX_RANKS; ++i) flags.ptr[i] = g.flag_tbl[i];
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int b = 0; b < NBUF; ++b) mbar_init(&bars[b], 1);
    fence_barrier_init();
  }
  const bool entry_ok = cta_barrier_all_ranks(flags, cta, g.rank, g.world, 2 * epoch, g.status);
  if (entry_ok && threadIdx.x == 0) unit_gather_thread<NBUF, PIECE>(g, cta, g.ctas, epoch, smem, bars, abort_flag);
  __syncthreads();
}

// Copy role of ONE WARP inside a CTA whose other warps compute (the GEMM that consumes the unit): every CTA of the
// launch contributes its bulk-copy engine, so the gather is spread over all SMs and costs no SM of its own. All 32
// lanes call it; `smem` is NBUF * PIECE bytes, `bars` NBUF mbarriers, `abort_flag` a word of this warp's own.
template <int NBUF, int PIECE = GATHER_PIECE>
__device__ __forceinline__ void unit_gather_warp(const GatherArgs& g, int cta, int ctas, uint8_t* smem, uint64_t* bars,
                                                 volatile int* abort_flag) {
  const uint32_t epoch = *g.epoch_ptr;
  PeerTable flags;
#pragma unroll
  for (int i = 0; i < MAX_RANKS; ++i) flags.ptr[i] = g.flag_tbl[i];
  if ((threadIdx.x & 31) == 0) {
    *abort_flag = 0;
    for (int b = 0; b < NBUF; ++b) mbar_init(&bars[b], 1);
    fence_barrier_init();
  }
  const bool entry_ok = warp_barrier_all_ranks(flags, cta, g.rank, g.world, 2 * epoch, g.status);
  if (entry_ok && (threadIdx.x & 31) == 0) unit_gather_thread<NBUF, PIECE>(g, cta, ctas, epoch, smem, bars, abort_flag);
  __syncwarp();
}

}  // namespace tb
