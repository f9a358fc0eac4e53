// bf16 GEMM for sm_100a: D[M,N] = A[M,K] * B[N,K]^T with fp32 accumulation in TMEM.
//
// Design (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: cp.async.bulk.tensor tiles into a STAGES-deep smem ring
//   warp 1      MMA issuer: one thread issues tcgen05.mma (128 x BN x 16) from smem
//               descriptors; accumulators live in TMEM, double-buffered (2 x BN columns)
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator, apply the fused epilogue
//               (bias, GELU, GELU-backward multiply, residual, cast) and store, while
//               the MMA warp already works on the next tile in the other TMEM buffer.
// Both operands may be K-major (contraction contiguous) or MN-major (the output index
// contiguous), so forward (x W^T), dgrad (dy W) and wgrad (dy^T x) all run without a
// transpose pass. Split-K with fp32 atomic accumulation keeps all SMs busy on wgrad.
//
// Replaces the reference's tiled SGEMM source string
// (crates/torsh-backend/src/kernel_generation/types/cuda_compiler.rs:104-167) and its
// unwired cuBLAS call (crates/torsh-backend/src/cuda/backend.rs:695-726).
#include "comm.cuh"
#include "fsdp_gather.cuh"
#include "host_util.h"
#include <stdlib.h>
#include <string.h>

#include "sm100.cuh"

namespace tb {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int A_TILE_BYTES = BM * BK * 2;
constexpr int GEMM_THREADS = 192;
constexpr int SCHED_DEPTH = 4;   // work indices the producer may publish ahead of the slowest consumer role

enum : int {
  EPI_BIAS = 1,          // += bias[n] (bf16)
  EPI_GELU = 2,          // tanh-GELU after bias
  EPI_RESIDUAL = 4,      // += residual[m,n] (bf16) after activation
  EPI_OUT_F32 = 8,       // D is fp32 (default bf16)
  EPI_ATOMIC = 16,       // fp32 atomic accumulate into D (split-K / grad accumulation)
  EPI_STORE_PREACT = 32, // also store the pre-activation (after bias) as bf16
  EPI_MUL_DGELU = 64,    // *= gelu'(aux[m,n]) (aux = forward pre-activation, bf16)
  EPI_ACCUM = 128,       // D = D + result (non-atomic read-modify-write)
  EPI_RASTER_M = 256,    // walk tiles with m fastest (B panel shared by concurrent CTAs)
};

struct GemmParams {
  int M, N, K;
  int ldd, ldr;
  void* D;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  __nv_bfloat16* preact;
  const __nv_bfloat16* aux;
  int flags;
  int split_k;
  int tiles_m, tiles_n;
  int kb_total, kb_per_split;
  int stream_k;  // 1: workers own equal contiguous ranges of (tile, K-block) units instead of whole K-splits
  // Dynamic tile scheduler: sched[0] is the launch's work counter, sched[1] counts CTAs that have drawn their last item
  // (the last one resets both). Null: work items are dealt round-robin. A CTA starts with item `worker` and draws every
  // further item from the counter, so a CTA that starts late or shares its SM with another kernel simply takes fewer
  // tiles instead of holding the launch back.
  unsigned* sched;
  int* status;
  // ---- tensor-parallel fusions (all zero / null for a plain GEMM) --------------------------------
  // GEMM -> reduce-scatter: output row r belongs to rank r / rs_rows; the epilogue stores the tile
  // straight into this rank's slot of that rank's buffer rs_dst[owner] ([world][rs_rows][ldd], bf16
  // or fp32) over NVLink, so the transfer of a tile overlaps the math of the next one.
  int rs_rows;
  void* rs_dst[MAX_RANKS];
  // all-gather -> GEMM: the first ag_ctas CTAs copy the peers' A shards (ag_rows rows of K elements
  // each, contiguous) into the local full A that map_a describes, 128-row tile by tile, and publish
  // a ready flag per tile; the GEMM CTAs start on the local shard and consume tiles as they land.
  int ag_ctas, ag_rows;
  const void* ag_src[MAX_RANKS];
  void* ag_dst;
  uint32_t* ag_ready;        // local: [tiles_m] ready words (ready when >= the launch's epoch), then [tiles_m]
                             // arrival counters of the copy CTAs that share a tile
  int ag_split;              // copy CTAs per 128-row tile (each moves 1/ag_split of the tile's bytes)
  void* flag_tbl[MAX_RANKS]; // symmetric flag buffer (cross-rank barriers of the copy CTAs)
  const uint32_t* epoch_ptr;
  int rank, world;
  int m_rot;                 // m-tiles are visited starting at this tile (own shard first / last)
  int tma_store;             // bf16 output leaves through shared memory + TMA tensor stores (out_maps)
  // Implicit-GEMM 3x3 / stride 1 / pad 1 convolution over a channels-last activation [N, H, W, C] (map_a is then a
  // 4-D map with box {64, W, TH, TN}): an M tile is TN images x TH full image rows (TN * TH * W <= 128 rows, which
  // are consecutive rows of the [N*H*W, Cout] output), K runs over 9 taps x C/64 channel chunks, and tap (kh, kw)
  // simply shifts the box by (kh - 1, kw - 1); the zero fill of out-of-range coordinates is the padding.
  int conv;                  // 0 off, 1 forward (B K-major [Cout, 9*C]), 2 input gradient (taps flipped, B MN-major),
                             // 3 weight gradient: D[Cout, 9*Cin] += dy^T x_shifted, K runs over pixel blocks of
                             // TN images x TH image rows (<= 64 pixels; unused K rows of a stage stay zero), both
                             // operands are 4-D boxes read MN-major, every 64-column chunk of B carries its own tap
  int cv_H, cv_W, cv_TH, cv_TN, cv_tiles_h, cv_cchunks, cv_a_bytes, cv_N;
  // FSDP un-shard fused into the unit's first GEMM: the first ag_ctas CTAs pull every rank's shard of the unit into
  // the local unit buffer (fsdp_gather.cuh) while the GEMM CTAs work; B lies inside that buffer at byte offset
  // wg_b_off with rows of wg_ldb_bytes, and the TMA producer waits for the chunks that cover each B tile (K-major B:
  // BN whole rows per tile; MN-major B: 64 whole rows per K block) before loading it.
  int wg_on;
  long wg_b_off, wg_ldb_bytes;
  GatherArgs wg;
};

template <int BN, int STAGES, int GBUFS = 0>
struct SmemLayout {
  static constexpr int B_TILE_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], tmem ptr, abort flag, then the dynamic scheduler's
  // sched_full[SCHED_DEPTH], sched_empty[SCHED_DEPTH] and its ring of work indices
  static constexpr int SCHED_OFFSET = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16;
  static constexpr int TOTAL = SCHED_OFFSET + 2 * SCHED_DEPTH * 8 + SCHED_DEPTH * 4;
  // Epilogue staging, 1024-byte aligned. bf16 outputs: 4 warps x 2 buffers x (32 rows x 128 B, 128B-swizzled),
  // each buffer leaves as one TMA tensor store. The fp32 reduce-scatter epilogue uses the same bytes as
  // 4 warps x 32 private rows of 144 B (128 B + pad).
  static constexpr int RS_ROW_PITCH = 144;
  static constexpr int RS_OFF = (TOTAL + 1023) / 1024 * 1024;
  static constexpr int EPI_OFF = RS_OFF;
  static constexpr int EPI_WARP_BYTES = 2 * 32 * 128;
  static constexpr int RS_BYTES = 4 * EPI_WARP_BYTES;
  // Ring of the FSDP gather warp (GBUFS pieces of 16 KB, their mbarriers and the warp's own abort word); 0 without it
  static constexpr int GATHER_OFF = RS_OFF + RS_BYTES;
  static constexpr int GATHER_BYTES = GBUFS ? GBUFS * GATHER_PIECE + 128 : 0;
  // No slack for a manual round-up: the dynamic shared-memory window is declared 1024-byte aligned (the kernel checks
  // it and refuses to run otherwise). The kilobyte this saves is what lets a small CTA of another kernel (the FSDP
  // reduce-scatter, 128 bytes of shared memory + the 1 KB the system reserves per CTA) share an SM with a GEMM CTA.
  static constexpr int ALLOC = RS_OFF + RS_BYTES + GATHER_BYTES;
  static_assert(4 * 32 * RS_ROW_PITCH <= RS_BYTES, "fp32 reduce-scatter rows must fit the staging region");
  static_assert(ALLOC <= 232448, "shared memory budget of one CTA exceeded");
};

// Output tensor maps of the TMA-store epilogue: [0] for a plain GEMM, one per destination rank for the
// GEMM -> reduce-scatter kernel (box 64 columns x 32 rows, 128-byte swizzle).
struct OutMaps {
  CUtensorMap m[MAX_RANKS];
};

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(x),
               "r"(y), "r"(smem_u32(smem_src))
               : "memory");
}
__device__ __forceinline__ void bulk_wait_read_le1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }

__device__ __forceinline__ void decode_tile(const GemmParams& p, int tile, int& m_t, int& n_t) {
  if (p.flags & EPI_RASTER_M) {
    n_t = tile / p.tiles_m;
    m_t = tile - n_t * p.tiles_m;
  } else {
    m_t = tile / p.tiles_n;
    n_t = tile - m_t * p.tiles_n;
  }
  if (p.m_rot) {
    m_t += p.m_rot;
    if (m_t >= p.tiles_m) m_t -= p.tiles_m;
  }
}

__device__ __forceinline__ void decode_work(const GemmParams& p, int work, int& m_t, int& n_t,
                                            int& kb0, int& kb1) {
  int tile = work / p.split_k;
  int ks = work - tile * p.split_k;
  if (p.flags & EPI_RASTER_M) {
    n_t = tile / p.tiles_m;
    m_t = tile - n_t * p.tiles_m;
  } else {
    m_t = tile / p.tiles_n;
    n_t = tile - m_t * p.tiles_n;
  }
  if (p.m_rot) {
    m_t += p.m_rot;
    if (m_t >= p.tiles_m) m_t -= p.tiles_m;
  }
  kb0 = ks * p.kb_per_split;
  kb1 = min(p.kb_total, kb0 + p.kb_per_split);
}

// The sequence of (tile, K-block range) pieces of one worker CTA; the TMA, MMA and epilogue roles each walk their own
// copy and see the same sequence. Split-K mode: work units worker, worker + nworkers, ... Stream-K mode (atomic fp32
// output only): the tiles x K-blocks units are cut into nworkers equal contiguous ranges, so every CTA does the same
// number of K-blocks whatever the tile count; a range that crosses a tile boundary becomes two pieces, and each
// piece adds its partial product into the output.
struct WorkIter {
  int pos, end, stride;
  __device__ __forceinline__ WorkIter(const GemmParams& p, int worker, int nworkers) {
    if (p.stream_k) {
      const long units = (long)p.tiles_m * p.tiles_n * p.kb_total;
      pos = (int)(units * worker / nworkers);
      end = (int)(units * (worker + 1) / nworkers);
      stride = 0;
    } else {
      pos = worker;
      end = p.tiles_m * p.tiles_n * p.split_k;
      stride = nworkers;
    }
  }
  __device__ __forceinline__ bool next(const GemmParams& p, int& m_t, int& n_t, int& kb0, int& kb1) {
    if (pos >= end) return false;
    if (p.stream_k) {
      const int tile = pos / p.kb_total;
      kb0 = pos - tile * p.kb_total;
      kb1 = min(p.kb_total, kb0 + (end - pos));
      decode_tile(p, tile, m_t, n_t);
      pos += kb1 - kb0;
    } else {
      decode_work(p, pos, m_t, n_t, kb0, kb1);
      pos += stride;
    }
    return true;
  }
};

// Work source of one role under either scheduler. Static: the WorkIter sequence. Dynamic: the TMA producer thread
// draws work indices (its first one is its worker number, later ones come from the global counter, fetched one item
// ahead so the atomic's latency hides behind the current tile's loads) and publishes them through a shared-memory
// ring; the MMA thread and the four epilogue warps read the ring. -1 ends the sequence.
struct TileSource {
  WorkIter st;
  bool dyn;
  int k;            // items taken so far
  int total;
  int cur, nxt;     // producer only
  volatile int* ring;
  uint64_t *sfull, *sempty;
  __device__ __forceinline__ TileSource(const GemmParams& p, int worker, int nworkers, uint8_t* sched_smem)
      : st(p, worker, nworkers), dyn(p.sched != nullptr), k(0), total(p.tiles_m * p.tiles_n * p.split_k), cur(worker), nxt(-1),
        raw(0), drew(false) {
    sfull = (uint64_t*)sched_smem;
    sempty = sfull + SCHED_DEPTH;
    ring = (volatile int*)(sempty + SCHED_DEPTH);
  }
  // producer: returns the next work index or -1 and publishes it to the other roles. The draw for the item AFTER the
  // returned one is issued here and only looked at in the next call, i.e. after this tile's loads have been issued, so
  // the atomic's round trip never sits in front of a load.
  unsigned raw;
  bool drew;
  __device__ __forceinline__ int produce(const GemmParams& p, int nworkers, volatile int* abort_flag) {
    int w;
    if (k == 0) {
      w = cur < total ? cur : -1;
      drew = false;
    } else if (drew) {
      const long d = (long)nworkers + raw;
      w = d < total ? (int)d : -1;
      if (w < 0 && atomicAdd(p.sched + 1, 1u) == gridDim.x - p.ag_ctas - 1u) {  // every CTA has drawn its last item
        p.sched[0] = 0;
        p.sched[1] = 0;
      }
    } else {
      w = -1;
    }
    drew = false;
    if (w >= 0 && !*abort_flag) {
      raw = atomicAdd(p.sched, 1u);
      drew = true;
    }
    const int slot = k % SCHED_DEPTH;
    if (k >= SCHED_DEPTH) mbar_wait(&sempty[slot], ((k / SCHED_DEPTH) & 1) ^ 1, abort_flag, p.status, TB_ERR_WAIT_MISC);
    ring[slot] = *abort_flag ? -1 : w;
    mbar_arrive(&sfull[slot]);
    ++k;
    return *abort_flag ? -1 : w;
  }
  // consumer (one thread per role instance reads; warps broadcast themselves)
  __device__ __forceinline__ int consume(const GemmParams& p, volatile int* abort_flag) {
    const int slot = k % SCHED_DEPTH;
    if (!mbar_wait(&sfull[slot], (k / SCHED_DEPTH) & 1, abort_flag, p.status, TB_ERR_WAIT_MISC)) return -1;
    const int w = ring[slot];
    ++k;
    return w;
  }
  __device__ __forceinline__ void release(int items_done) {  // consumer: item (items_done - 1) has been read
    mbar_arrive(&sempty[(items_done - 1) % SCHED_DEPTH]);
  }
};

// Convolution mode: first output row and number of valid rows of M tile m_t.
__device__ __forceinline__ void conv_tile(const GemmParams& p, int m_t, int& n0, int& h0, long& base_row, int& valid) {
  const int it = m_t / p.cv_tiles_h, ht = m_t - it * p.cv_tiles_h;
  n0 = it * p.cv_TN;
  h0 = ht * p.cv_TH;
  base_row = ((long)n0 * p.cv_H + h0) * p.cv_W;
  valid = min(p.cv_TN, p.cv_N - n0) * min(p.cv_TH, p.cv_H - h0) * p.cv_W;
}

// Bounded wait on a flag in this GPU's own memory (written by a copy CTA of the same launch).
__device__ __forceinline__ bool wait_flag_ge_gpu(const uint32_t* flag, uint32_t target, int* status) {
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if ((int32_t)(v - target) >= 0) return true;
    if ((++spins & 31u) == 0u && globaltimer_ns() - t0 > TB_PEER_WAIT_LIMIT_NS) {
      if (status) atomicCAS(status, 0, TB_ERR_WAIT_PEER);
      return false;
    }
  }
}

// Copy role of the all-gather -> GEMM kernel. One thread per CTA streams the peers' A shards through
// a shared-memory ring with bulk async copies (peer memory -> smem -> local memory), nearest peer
// first, and publishes one ready flag per 128-row tile. SMEM_BYTES of the CTA's dynamic shared
// memory serve as the ring; `bars` are mbarriers placed after it.
template <int SMEM_BYTES>
__device__ __forceinline__ void ag_copy_role(const GemmParams& p, uint8_t* smem, uint64_t* bars,
                                             volatile int* abort_flag) {
  constexpr int PIECE = 16384;
  constexpr int NBUF = SMEM_BYTES / PIECE < 12 ? SMEM_BYTES / PIECE : 12;
  constexpr int STORES = NBUF / 2;  // stores allowed to be reading their buffers at once; the other buffers are being loaded
  const uint32_t epoch = *p.epoch_ptr;
  PeerTable flags;
#pragma unroll
  for (int i = 0; i < MAX_RANKS; ++i) flags.ptr[i] = p.flag_tbl[i];
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int b = 0; b < NBUF; ++b) mbar_init(&bars[b], 1);
    fence_barrier_init();
  }
  // every rank's shard is complete once its kernel has started (stream order on that rank); without that
  // guarantee (a peer late beyond the wait limit) nothing is copied and the GEMM side gives up on its first flag
  const bool entry_ok = cta_barrier_all_ranks(flags, blockIdx.x, p.rank, p.world, 2 * epoch, p.status);
  if (entry_ok && threadIdx.x == 0) {
    // Work units: (peer, 128-row tile, part), peers nearest first, ag_split parts per tile so that a short shard
    // still keeps every copy CTA busy; this CTA takes the units blockIdx.x, blockIdx.x + ag_ctas, ... Their 16 KB
    // pieces form one stream that is pipelined through the ring: up to NBUF - 1 peer loads are in flight while the
    // piece that has landed is written to local memory; a buffer is refilled as soon as the store that read it has
    // released it (stores retire in order).
    const long tile_bytes = (long)BM * p.K * 2;
    const int tiles_per_rank = p.ag_rows / BM;
    const int split = p.ag_split;
    const int ppu = (int)(tile_bytes / PIECE) / split;  // pieces per unit; launcher guarantees divisibility
    const int units = (p.world - 1) * tiles_per_rank * split;
    const int my_units = (int)blockIdx.x < units ? (units - (int)blockIdx.x + p.ag_ctas - 1) / p.ag_ctas : 0;
    const long total = (long)my_units * ppu;
    const int pieces = ppu;  // a unit is complete after its last piece
    auto locate = [&](long g, const char*& src, char*& dst, int& q, int& t, int& piece) {
      const int ui = (int)(g / ppu);
      piece = (int)(g - (long)ui * ppu);
      const int u = (int)blockIdx.x + ui * p.ag_ctas;
      const int part = u % split;
      t = (u / split) % tiles_per_rank;
      const int step = 1 + u / (split * tiles_per_rank);
      q = (p.rank + step) % p.world;
      const long off = (long)t * tile_bytes + ((long)part * ppu + piece) * PIECE;
      src = reinterpret_cast<const char*>(p.ag_src[q]) + off;
      dst = reinterpret_cast<char*>(p.ag_dst) + (long)q * tiles_per_rank * tile_bytes + off;
    };
    auto issue_load = [&](long g) {
      const char* src; char* dst; int q, t, piece;
      locate(g, src, dst, q, t, piece);
      const int b = (int)(g % NBUF);
      mbar_expect_tx(&bars[b], PIECE);
      bulk_load(smem + b * PIECE, src, PIECE, &bars[b]);
    };
    // A part of a tile is published once the stores of all its pieces have completed. Stores complete in order, so
    // instead of draining the store queue at every part boundary (a full write round trip every few pieces),
    // publication runs LAG pieces behind the store just issued.
    constexpr int LAG = 16;  // a global write takes a few microseconds to complete: keep many stores in flight
    long pub = 0;  // every part that ends before piece `pub` has been published
    auto publish_upto = [&](long done) {  // stores of pieces [0, done) are complete
      bool fenced = false;
      while (pub + pieces <= done) {
        const char* src; char* dst; int q, t, piece;
        locate(pub + pieces - 1, src, dst, q, t, piece);
        if (!fenced) {
          __threadfence();
          fenced = true;
        }
        const int tile = q * tiles_per_rank + t;
        uint32_t* cnt = p.ag_ready + p.tiles_m + tile;
        uint32_t arrived;
        asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(arrived) : "l"(cnt) : "memory");
        if (arrived == (uint32_t)split - 1) {  // last part: reset the counter for the next launch, publish the tile
          *cnt = 0;
          asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.ag_ready + tile), "r"(epoch) : "memory");
        }
        pub += pieces;
      }
    };
    long next_load = 0;
    for (; next_load < total && next_load < NBUF; ++next_load) issue_load(next_load);
    for (long i = 0; i < total; ++i) {
      const char* src; char* dst; int q, t, piece;
      locate(i, src, dst, q, t, piece);
      const int b = (int)(i % NBUF);
      mbar_wait(&bars[b], (uint32_t)((i / NBUF) & 1), abort_flag, p.status, TB_ERR_WAIT_FULL);
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
      uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 2000000ull) {
      }
    }
  }
  // peers may overwrite their shards only after everybody has copied them
  cta_barrier_all_ranks(flags, blockIdx.x, p.rank, p.world, 2 * epoch + 1, p.status);
}

// Elementwise part of the epilogue on one thread's 32 consecutive output columns (a full, 16-byte aligned chunk):
// + bias, store of the pre-activation, tanh-GELU, multiply by GELU'(aux), + residual.
__device__ __forceinline__ void epi_math(const GemmParams& p, int flags, bool add_bias, int row, int n0, size_t off,
                                         float (&f)[32]) {
    if (add_bias) {
      const uint4* bp = reinterpret_cast<const uint4*>(p.bias + n0);
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 b = __ldg(bp + g);
        uint32_t w[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          f[g * 8 + e * 2] += bf16_lo(w[e]);
          f[g * 8 + e * 2 + 1] += bf16_hi(w[e]);
        }
      }
    }
    if (flags & EPI_STORE_PREACT) {
      uint4* pp = reinterpret_cast<uint4*>(p.preact + off);
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 o;
        o.x = pack_bf16x2(f[g * 8 + 0], f[g * 8 + 1]);
        o.y = pack_bf16x2(f[g * 8 + 2], f[g * 8 + 3]);
        o.z = pack_bf16x2(f[g * 8 + 4], f[g * 8 + 5]);
        o.w = pack_bf16x2(f[g * 8 + 6], f[g * 8 + 7]);
        pp[g] = o;
      }
    }
    if (flags & EPI_GELU) {
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = gelu_tanh(f[j]);
    }
    if (flags & EPI_MUL_DGELU) {
      const uint4* ap = reinterpret_cast<const uint4*>(p.aux + off);
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 a = ap[g];
        uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          f[g * 8 + e * 2] *= gelu_tanh_grad(bf16_lo(w[e]));
          f[g * 8 + e * 2 + 1] *= gelu_tanh_grad(bf16_hi(w[e]));
        }
      }
    }
    if (flags & EPI_RESIDUAL) {
      const uint4* rp =
          reinterpret_cast<const uint4*>(p.residual + (size_t)row * p.ldr + n0);
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 a = rp[g];
        uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          f[g * 8 + e * 2] += bf16_lo(w[e]);
          f[g * 8 + e * 2 + 1] += bf16_hi(w[e]);
        }
      }
    }
}

// GBUFS > 0: a seventh warp (threads 192..223) of EVERY CTA gathers its share of an FSDP unit through a ring of GBUFS 16 KB
// pieces while the CTA computes (the pipeline then has fewer stages to make room): the un-shard uses the bulk-copy engine
// of all SMs and costs the GEMM no SM.
template <int BN, int A_MAJOR, int B_MAJOR, int STAGES, int GBUFS = 0>
__global__ void __launch_bounds__(GBUFS ? GEMM_THREADS + 32 : GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ OutMaps out_maps, const GemmParams p) {
  using L = SmemLayout<BN, STAGES, GBUFS>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {  // the 128-byte swizzle of the TMA tiles needs this alignment; never seen, but never assumed
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, TB_ERR_BAD_ARG);
    return;
  }
  uint64_t* full = (uint64_t*)(smem + L::BAR_OFFSET);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_ptr = (uint32_t*)(tmem_empty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128 : (2 * BN <= 256) ? 256 : 512;

  if (p.ag_ctas > 0 && (int)blockIdx.x < p.ag_ctas) {
    ag_copy_role<L::BAR_OFFSET>(p, smem, full, abort_flag);
    return;
  }
  // GEMM CTAs are numbered from 0 after the copy CTAs
  const int worker = (int)blockIdx.x - p.ag_ctas;
  const int nworkers = (int)gridDim.x - p.ag_ctas;
  const uint32_t ag_epoch = (p.ag_ctas > 0 || p.wg_on) ? *p.epoch_ptr : 0u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);
    }
    {
      uint64_t* sb = (uint64_t*)(smem + L::SCHED_OFFSET);
      for (int d = 0; d < SCHED_DEPTH; ++d) {
        mbar_init(&sb[d], 1);                // published by the producer thread
        mbar_init(&sb[SCHED_DEPTH + d], 5);  // read by the MMA thread and the four epilogue warps
      }
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (p.conv == 3) {
    // K rows of a stage that the (shorter than 64-pixel) boxes never write must read as zero
    uint4* z = reinterpret_cast<uint4*>(smem);
    for (int i = threadIdx.x; i < L::BAR_OFFSET / 16; i += blockDim.x) z[i] = make_uint4(0, 0, 0, 0);
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&map_a);
      tma_prefetch_desc(&map_b);
      int s = 0;
      uint32_t phase = 0;
      TileSource it(p, worker, nworkers, smem + L::SCHED_OFFSET);
      auto next_work = [&](int& m_t, int& n_t, int& kb0, int& kb1) -> bool {
        if (!it.dyn) return it.st.next(p, m_t, n_t, kb0, kb1);
        const int w = it.produce(p, nworkers, abort_flag);
        if (w < 0) return false;
        decode_work(p, w, m_t, n_t, kb0, kb1);
        return true;
      };
      int m_t, n_t, kb0, kb1;
      // FSDP weight gather: chunks of the unit buffer this thread has already seen ready (indices below 64)
      uint64_t wg_seen = 0;
      auto wg_wait = [&](long byte0, long byte1) {
        const int c0 = (int)(byte0 / p.wg.chunk_bytes), c1 = (int)((byte1 - 1) / p.wg.chunk_bytes);
        bool waited = false;
        for (int c = c0; c <= c1; ++c) {
          if (c < 64 && ((wg_seen >> c) & 1ull)) continue;
          if (!*abort_flag && !wait_ready_gpu(p.wg.ready + c, ag_epoch, p.status)) *abort_flag = 1;
          if (c < 64) wg_seen |= 1ull << c;
          waited = true;
        }
        if (waited) fence_proxy_async_all();  // the chunk was written through the async proxy of another CTA
      };
      // Once any wait of this thread has given up (abort flag), nothing more is loaded: loads issued without a free
      // stage would pile transaction counts on one barrier beyond its range. The MMA and epilogue roles see the flag
      // too, stop waiting and drain their finite loops on whatever the stages hold.
      while (!*abort_flag && next_work(m_t, n_t, kb0, kb1)) {
        if (p.wg_on && B_MAJOR == 0)
          wg_wait(p.wg_b_off + (long)n_t * BN * p.wg_ldb_bytes, p.wg_b_off + (long)min(p.N, (n_t + 1) * BN) * p.wg_ldb_bytes);
        if (!p.wg_on && p.ag_ctas > 0 && (m_t * BM) / p.ag_rows != p.rank) {
          // rows of a peer: wait (bounded) until the copy CTAs have landed this 128-row tile locally
          if (!*abort_flag && !wait_flag_ge_gpu(p.ag_ready + m_t, ag_epoch, p.status)) *abort_flag = 1;
          fence_proxy_async_all();
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (p.wg_on && B_MAJOR == 1)
            wg_wait(p.wg_b_off + (long)kb * BK * p.wg_ldb_bytes, p.wg_b_off + (long)min(p.K, (kb + 1) * BK) * p.wg_ldb_bytes);
          if (*abort_flag || !mbar_wait(&empty[s], phase ^ 1, abort_flag, p.status, TB_ERR_WAIT_EMPTY)) break;
          uint8_t* sa = smem + s * L::STAGE_BYTES;
          uint8_t* sb = sa + A_TILE_BYTES;
          mbar_expect_tx(&full[s], p.conv == 3 ? (uint32_t)(p.cv_a_bytes * (BM / 64 + BN / 64))
                                  : p.conv ? (uint32_t)(p.cv_a_bytes + L::B_TILE_BYTES) : (uint32_t)L::STAGE_BYTES);
          if (A_MAJOR == 0 && p.conv) {
            const int tap = kb / p.cv_cchunks, cc = kb - tap * p.cv_cchunks;
            const int kh = tap / 3, kw = tap - kh * 3;
            int n0, h0, valid;
            long base_row;
            conv_tile(p, m_t, n0, h0, base_row, valid);
            tma_load_4d(sa, &map_a, &full[s], cc * 64, kw - 1, h0 + kh - 1, n0);
          } else if (A_MAJOR == 0) {
            tma_load_2d(sa, &map_a, &full[s], kb * BK, m_t * BM);
          } else if (p.conv == 3) {
            const int it = kb / p.cv_tiles_h, ht = kb - it * p.cv_tiles_h;
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_4d(sa + c * (64 * BK * 2), &map_a, &full[s], m_t * BM + c * 64, 0, ht * p.cv_TH, it * p.cv_TN);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d(sa + c * (64 * BK * 2), &map_a, &full[s], m_t * BM + c * 64, kb * BK);
          }
          if (B_MAJOR == 0) {
            tma_load_2d(sb, &map_b, &full[s], kb * BK, n_t * BN);
          } else if (p.conv == 3) {
            const int it = kb / p.cv_tiles_h, ht = kb - it * p.cv_tiles_h;
            const int cin = p.N / 9;
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) {
              const int col = n_t * BN + c * 64;
              const int tap = min(col / cin, 8);          // chunks past the last tap load something harmless
              const int ci0 = col - (col / cin) * cin;
              const int kh = tap / 3, kw = tap - kh * 3;
              tma_load_4d(sb + c * (64 * BK * 2), &map_b, &full[s], ci0, kw - 1, ht * p.cv_TH + kh - 1, it * p.cv_TN);
            }
          } else if (p.conv == 2) {
            // input gradient: weights [Cout, 9 * Cin] read MN-major; tap t of the gradient pairs with tap 8 - t of the
            // forward filter, whose Cin columns start at (8 - t) * Cin; the K rows are the Cout chunk
            const int tap = kb / p.cv_cchunks, cc = kb - tap * p.cv_cchunks;
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb + c * (64 * BK * 2), &map_b, &full[s], (8 - tap) * p.N + n_t * BN + c * 64, cc * BK);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb + c * (64 * BK * 2), &map_b, &full[s], n_t * BN + c * 64, kb * BK);
          }
          if (++s == STAGES) {
            s = 0;
            phase ^= 1;
          }
        }
      }
      if (*abort_flag) {
        if (it.dyn) {   // the other roles must not wait for a work index that will never come
          int a, b, c, d;
          next_work(a, b, c, d);
        }
        // give copies still in flight time to land before the CTA's smem is released
        uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MAJOR, B_MAJOR);
      int s = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      TileSource it(p, worker, nworkers, smem + L::SCHED_OFFSET);
      auto next_work = [&](int& m_t, int& n_t, int& kb0, int& kb1) -> bool {
        if (!it.dyn) return it.st.next(p, m_t, n_t, kb0, kb1);
        const int w = it.consume(p, abort_flag);
        it.release(it.k);
        if (w < 0) return false;
        decode_work(p, w, m_t, n_t, kb0, kb1);
        return true;
      };
      int m_t, n_t, kb0, kb1;
      while (next_work(m_t, n_t, kb0, kb1)) {
        mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.status, TB_ERR_WAIT_TMEM_EMPTY);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          mbar_wait(&full[s], phase, abort_flag, p.status, TB_ERR_WAIT_FULL);
          tc_fence_after();
          const uint32_t a_base = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t b_base = a_base + A_TILE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = (A_MAJOR == 0)
                                       ? make_smem_desc_sw128(a_base + k * 32, 16, 1024)
                                       : make_smem_desc_sw128(a_base + k * 2048, 64 * BK * 2, 1024);
            const uint64_t bdesc = (B_MAJOR == 0)
                                       ? make_smem_desc_sw128(b_base + k * 32, 16, 1024)
                                       : make_smem_desc_sw128(b_base + k * 2048, 64 * BK * 2, 1024);
            umma_ss(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty[s]);
          if (++s == STAGES) {
            s = 0;
            phase ^= 1;
          }
        }
        umma_commit(&tmem_full[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else if (GBUFS > 0 && warp == 6) {
    // ------------------------------------------------------------ FSDP gather warp
    uint8_t* gsm = smem + L::GATHER_OFF;
    uint64_t* gbars = (uint64_t*)(gsm + GBUFS * GATHER_PIECE);
    unit_gather_warp<(GBUFS > 0 ? GBUFS : 2)>(p.wg, (int)blockIdx.x, (int)gridDim.x, gsm, gbars, (volatile int*)(gbars + GBUFS));
  } else {
    // ------------------------------------------------------------ epilogue (4 warps)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t epi_cnt = 0;  // 64-column groups this warp has staged so far (selects the staging buffer)
    const int flags = p.flags;
    TileSource it(p, worker, nworkers, smem + L::SCHED_OFFSET);
    auto next_work = [&](int& m_t, int& n_t, int& kb0, int& kb1) -> bool {
      if (!it.dyn) return it.st.next(p, m_t, n_t, kb0, kb1);
      int w = 0;
      if (lane == 0) {
        w = it.consume(p, abort_flag);
        it.release(it.k);
      } else {
        ++it.k;
      }
      w = __shfl_sync(0xffffffffu, w, 0);
      if (w < 0) return false;
      decode_work(p, w, m_t, n_t, kb0, kb1);
      return true;
    };
    int m_t, n_t, kb0, kb1;
    while (next_work(m_t, n_t, kb0, kb1)) {
      mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.status, TB_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
      int row = m_t * BM + q * 32 + lane;
      bool row_ok = row < p.M;
      if (p.conv == 1 || p.conv == 2) {
        int n0, h0, valid;
        long base_row;
        conv_tile(p, m_t, n0, h0, base_row, valid);
        row = (int)base_row + q * 32 + lane;
        row_ok = (q * 32 + lane) < valid;
      }
      const bool add_bias = (flags & EPI_BIAS) && (kb0 == 0);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        const int n0 = n_t * BN + c0;
        if (n0 >= p.N) break;  // uniform across the warp
        uint32_t v[32];
        tmem_ld32(tmem_base + acc * BN + c0 + ((uint32_t)(q * 32) << 16), v);
        tmem_wait_ld();
        if (p.tma_store) {
          // bf16 output through shared memory: every lane packs its row's 32 columns into a 128B-swizzled
          // 32 x 64 staging tile; after the second half lane 0 sends the tile with one TMA tensor store
          // (rows >= M are clipped by the tensor map). N % 64 == 0 here, so every chunk is full.
          const int half = (c0 >> 5) & 1;
          uint8_t* sbuf = smem + L::EPI_OFF + q * L::EPI_WARP_BYTES + (epi_cnt & 1) * 4096;
          if (half == 0) {
            if (lane == 0) bulk_wait_read_le1();  // the store that last read this buffer has finished
            __syncwarp();
          }
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
          if (row_ok && p.rs_rows == 0) epi_math(p, flags, add_bias, row, n0, (size_t)row * p.ldd + n0, f);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int chunk = half * 4 + g;
            *reinterpret_cast<uint4*>(sbuf + lane * 128 + ((chunk ^ (lane & 7)) << 4)) =
                make_uint4(pack_bf16x2(f[g * 8 + 0], f[g * 8 + 1]), pack_bf16x2(f[g * 8 + 2], f[g * 8 + 3]),
                           pack_bf16x2(f[g * 8 + 4], f[g * 8 + 5]), pack_bf16x2(f[g * 8 + 6], f[g * 8 + 7]));
          }
          if (half == 1) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              const int row0 = m_t * BM + q * 32;
              if (p.rs_rows > 0) {
                const int owner = row0 / p.rs_rows;
                tma_store_2d(&out_maps.m[owner], sbuf, n0 - 32, p.rank * p.rs_rows + (row0 - owner * p.rs_rows));
              } else {
                tma_store_2d(&out_maps.m[0], sbuf, n0 - 32, row0);
              }
              bulk_commit();
            }
            ++epi_cnt;
          }
          continue;
        }
        if (!row_ok) continue;
        float f[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
        const bool full_chunk = (n0 + 32 <= p.N);
        const size_t off = (size_t)row * p.ldd + n0;
        if (p.rs_rows > 0) {
          // GEMM -> reduce-scatter: this thread's row segment goes into this rank's slot of the owner's
          // buffer ([world][rs_rows][ldd]). It is first packed into a private shared-memory row and then
          // leaves as ONE 128-byte bulk async store, so NVLink sees full-size write bursts instead of
          // thirty-two scattered 16-byte stores per instruction; the copy engine works while the thread
          // already unpacks the next chunk.
          const int owner = row / p.rs_rows;
          const size_t rbase = ((size_t)p.rank * p.rs_rows + (row - owner * p.rs_rows)) * p.ldd;
          uint8_t* srow = smem + L::RS_OFF + (q * 32 + lane) * L::RS_ROW_PITCH;
          if (flags & EPI_OUT_F32) {
            bulk_wait_read_all();  // my previous store has finished reading this row
            float4* s4 = reinterpret_cast<float4*>(srow);
#pragma unroll
            for (int g = 0; g < 8; ++g) s4[g] = make_float4(f[g * 4], f[g * 4 + 1], f[g * 4 + 2], f[g * 4 + 3]);
            fence_proxy_async_smem();
            bulk_store(reinterpret_cast<float*>(p.rs_dst[owner]) + rbase + n0, srow, 128);
            bulk_commit();
          } else {
            const int half = (c0 >> 5) & 1;
            if (half == 0) bulk_wait_read_all();
            uint4* s4 = reinterpret_cast<uint4*>(srow + half * 64);
#pragma unroll
            for (int g = 0; g < 4; ++g)
              s4[g] = make_uint4(pack_bf16x2(f[g * 8 + 0], f[g * 8 + 1]), pack_bf16x2(f[g * 8 + 2], f[g * 8 + 3]),
                                 pack_bf16x2(f[g * 8 + 4], f[g * 8 + 5]), pack_bf16x2(f[g * 8 + 6], f[g * 8 + 7]));
            if (half == 1 || n0 + 32 >= p.N || c0 + 32 >= BN) {
              fence_proxy_async_smem();
              bulk_store(reinterpret_cast<__nv_bfloat16*>(p.rs_dst[owner]) + rbase + (n0 - half * 32), srow,
                         (half + 1) * 64);
              bulk_commit();
            }
          }
          continue;
        }
        if (full_chunk && (p.ldd & 7) == 0) {
          epi_math(p, flags, add_bias, row, n0, off, f);
          if (flags & EPI_OUT_F32) {
            float* dp = reinterpret_cast<float*>(p.D) + off;
            if (flags & EPI_ATOMIC) {
#pragma unroll
              for (int g = 0; g < 8; ++g)
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dp + g * 4),
                             "f"(f[g * 4]), "f"(f[g * 4 + 1]), "f"(f[g * 4 + 2]),
                             "f"(f[g * 4 + 3])
                             : "memory");
            } else {
              float4* d4 = reinterpret_cast<float4*>(dp);
#pragma unroll
              for (int g = 0; g < 8; ++g) {
                float4 o = make_float4(f[g * 4], f[g * 4 + 1], f[g * 4 + 2], f[g * 4 + 3]);
                if (flags & EPI_ACCUM) {
                  float4 old = d4[g];
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                d4[g] = o;
              }
            }
          } else {
            uint4* d4 = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.D) + off);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              if (flags & EPI_ACCUM) {
                uint4 a = d4[g];
                uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  f[g * 8 + e * 2] += bf16_lo(w[e]);
                  f[g * 8 + e * 2 + 1] += bf16_hi(w[e]);
                }
              }
              uint4 o;
              o.x = pack_bf16x2(f[g * 8 + 0], f[g * 8 + 1]);
              o.y = pack_bf16x2(f[g * 8 + 2], f[g * 8 + 3]);
              o.z = pack_bf16x2(f[g * 8 + 4], f[g * 8 + 5]);
              o.w = pack_bf16x2(f[g * 8 + 6], f[g * 8 + 7]);
              d4[g] = o;
            }
          }
        } else {
          // ragged edge / unaligned leading dimension: scalar path
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int n = n0 + j;
            if (n >= p.N) continue;
            float x = f[j];
            if (add_bias) x += __bfloat162float(p.bias[n]);
            if (flags & EPI_STORE_PREACT) p.preact[off + j] = __float2bfloat16(x);
            if (flags & EPI_GELU) x = gelu_tanh(x);
            if (flags & EPI_MUL_DGELU) x *= gelu_tanh_grad(__bfloat162float(p.aux[off + j]));
            if (flags & EPI_RESIDUAL)
              x += __bfloat162float(p.residual[(size_t)row * p.ldr + n]);
            if (flags & EPI_OUT_F32) {
              float* dp = reinterpret_cast<float*>(p.D) + off + j;
              if (flags & EPI_ATOMIC)
                atomicAdd(dp, x);
              else
                *dp = (flags & EPI_ACCUM) ? (*dp + x) : x;
            } else {
              __nv_bfloat16* dp = reinterpret_cast<__nv_bfloat16*>(p.D) + off + j;
              if (flags & EPI_ACCUM) x += __bfloat162float(*dp);
              *dp = __float2bfloat16(x);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if (p.rs_rows > 0 || p.tma_store) bulk_wait_all();  // everything this thread sent has left shared memory and landed
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Counters of the dynamic tile scheduler: SCHED_SLOTS pairs (work counter, finished-CTA counter), all zero between
// launches (the last CTA of a launch resets its pair). Consecutive launches take consecutive pairs, so launches that run
// concurrently on different streams never share one; a pair is reused SCHED_SLOTS launches later.
constexpr int SCHED_SLOTS = 1024;
static __device__ unsigned g_sched_counters[2 * SCHED_SLOTS];

static bool g_dynamic_tiles = [] { const char* e = getenv("TB_GEMM_DYNAMIC"); return e && e[0] == '1'; }();

static int sched_pair(unsigned** out) {
  static unsigned* base[64] = {nullptr};
  static std::atomic<unsigned> seq{0};
  int dev = 0;
  TB_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) TB_FAIL(TB_E_ARG, "gemm: device index %d out of range", dev);
  if (!base[dev]) {
    unsigned* p = nullptr;
    TB_CUDA_CHECK(cudaGetSymbolAddress((void**)&p, g_sched_counters));
    base[dev] = p;
  }
  *out = base[dev] + 2 * (seq.fetch_add(1, std::memory_order_relaxed) % SCHED_SLOTS);
  return 0;
}

template <int BN, int A_MAJOR, int B_MAJOR, int STAGES, int GBUFS = 0>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const OutMaps& om, const GemmParams& p,
                       cudaStream_t stream) {
  using L = SmemLayout<BN, STAGES, GBUFS>;
  auto kern = gemm_bf16_kernel<BN, A_MAJOR, B_MAJOR, STAGES, GBUFS>;
  static bool configured = false;
  if (!configured) {
    TB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::ALLOC));
    configured = true;
  }
  long total = (long)p.tiles_m * p.tiles_n * (p.stream_k ? p.kb_total : p.split_k);
  int workers = sm_count() - p.ag_ctas;  // copy CTAs and GEMM CTAs must all be resident at once
  if (workers < 1) TB_FAIL(TB_E_ARG, "gemm: too many copy CTAs");
  int grid = (int)(total < workers ? total : workers) + p.ag_ctas;
  GemmParams q = p;
  // Dynamic dealing of the work items (more than one wave, no order that a fused collective relies on) is opt-in:
  // TB_GEMM_DYNAMIC=1 or tb_gemm_set_dynamic(1). It lets a CTA that was placed late (its SM held by a kernel of another
  // stream) take fewer tiles; with the GPU to itself the static deal measured 0.8 % faster on the GPT-2-medium step.
  q.sched = nullptr;
  if (g_dynamic_tiles && !p.stream_k && p.ag_ctas == 0 && total > workers) {
    if (int r = sched_pair(&q.sched)) return r;
  }
  kern<<<grid, GBUFS ? GEMM_THREADS + 32 : GEMM_THREADS, L::ALLOC, stream>>>(ma, mb, om, q);
  TB_CUDA_CHECK(cudaGetLastError());
  return TB_LAUNCH_OK;
}

}  // namespace tb

using namespace tb;

// D[M,N] = op(A) * op(B)^T with the fused epilogue selected by `flags`.
//   a_major = 0: A is stored [M, K] (row stride lda);  1: A is stored [K, M] (row stride lda)
//   b_major = 0: B is stored [N, K] (row stride ldb);  1: B is stored [K, N] (row stride ldb)
// lda / ldb must be multiples of 8 elements and the base pointers 16-byte aligned (TMA).
// `bn` selects the tile width (128 or 256); 0 lets the launcher choose.
struct TpFusion {
  int kind = 0;  // 0 none, 1 GEMM -> reduce-scatter, 2 all-gather -> GEMM
  int rank = 0, world = 1;
  const void* const* peers = nullptr;   // kind 1: per-rank accumulation buffers; kind 2: per-rank A shards
  const void* const* flags = nullptr;   // kind 2: symmetric flag buffers
  const unsigned* epoch_ptr = nullptr;  // kind 2
  unsigned* ready = nullptr;            // kind 2: local per-tile flags
  int copy_ctas = 0;                    // kind 2
  // implicit-GEMM convolution (kind 3): A is the channels-last activation [cv_n, cv_h, cv_w, K / 9]
  int cv_n = 0, cv_h = 0, cv_w = 0, cv_mode = 0;
  // FSDP unit gather fused into this GEMM (kind 5): B lies at byte offset wg_b_off of the unit buffer wg.dst
  GatherArgs wg{};
  long wg_b_off = 0;
};

static int gemm_dispatch(const void* A, const void* B, void* D, int M, int N, int K, int a_major,
                         int b_major, int lda, int ldb, int ldd, const void* bias,
                         const void* residual, int ldr, void* preact, const void* aux, int flags,
                         int split_k, int bn, int* status, cudaStream_t stream, const TpFusion& tp);

TB_EXPORT int tb_gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K, int a_major,
                           int b_major, int lda, int ldb, int ldd, const void* bias,
                           const void* residual, int ldr, void* preact, const void* aux, int flags,
                           int split_k, int bn, int* status, cudaStream_t stream) {
  TB_ENSURE_DEVICE();
  return gemm_dispatch(A, B, D, M, N, K, a_major, b_major, lda, ldb, ldd, bias, residual, ldr, preact, aux, flags,
                       split_k, bn, status, stream, TpFusion{});
}

// 3x3 / stride 1 / pad 1 convolution as an implicit GEMM (no im2col buffer). x: channels-last bf16 [n, h, w, c] with
// c % 64 == 0 and w <= 128. mode 1 (forward): wmat = [cout, 9*c] (taps row-major, channels innermost), y = [n*h*w, cout].
// mode 2 (input gradient): x is the output gradient [n, h, w, cout_fwd] (so c = cout_fwd), wmat is the SAME forward
// matrix [cout_fwd, 9*cin] and y = [n*h*w, cin]; `cout` is then the number of output columns cin.
TB_EXPORT int tb_conv3x3_gemm(const void* x, const void* wmat, void* y, int n, int h, int w, int c, int cout, int mode,
                              int ldw, int ldy, int bn, int* status, cudaStream_t stream) {
  TB_ENSURE_DEVICE();
  if (mode != 1 && mode != 2) TB_FAIL(TB_E_ARG, "conv3x3_gemm: mode must be 1 (forward) or 2 (input gradient)");
  TpFusion tp;
  tp.kind = 3;
  tp.cv_n = n; tp.cv_h = h; tp.cv_w = w; tp.cv_mode = mode;
  return gemm_dispatch(x, wmat, y, n * h * w, cout, 9 * c, 0, mode == 1 ? 0 : 1, c, ldw, ldy, nullptr, nullptr, 0, nullptr,
                       nullptr, 0, 1, bn, status, stream, tp);
}

// Weight gradient of the 3x3 / stride 1 / pad 1 convolution without a column matrix: dw[cout, 9*cin] (fp32,
// ACCUMULATED with atomics, taps row-major, channels innermost) += dy^T [cout, pixels] * shifted x [pixels, 9*cin].
// dy: [n, h, w, cout], x: [n, h, w, cin] channels-last bf16, cin % 64 == 0, w <= 64.
TB_EXPORT int tb_conv3x3_wgrad(const void* dy, const void* x, float* dw, int n, int h, int w, int cin, int cout, int lddw,
                               int split_k, int bn, int* status, cudaStream_t stream) {
  TB_ENSURE_DEVICE();
  TpFusion tp;
  tp.kind = 4;
  tp.cv_n = n; tp.cv_h = h; tp.cv_w = w;
  return gemm_dispatch(dy, x, dw, cout, 9 * cin, n * h * w, 1, 1, cout, cin, lddw, nullptr, nullptr, 0, nullptr, nullptr,
                       EPI_OUT_F32 | EPI_ATOMIC, split_k < 1 ? 1 : split_k, bn, status, stream, tp);
}

// Row-parallel linear with sequence parallelism: partial = A[M, K_local] * B[N, K_local]^T is
// reduce-scattered along M inside the epilogue. dst[r] is rank r's slot buffer
// [world][M / world][ldd] (bf16 or fp32 per `out_f32`): rank s writes slot s of the owner of each
// row. A cross-rank barrier must follow before the owner sums its slots (tb_rs_finalize), and the
// slots may be rewritten only after every owner has finished reading.
TB_EXPORT int tb_gemm_rs(const void* A, const void* B, const void* const* dst, int M, int N, int K, int b_major,
                         int lda, int ldb, int ldd, int out_f32, int rank, int world, int bn, int* status,
                         cudaStream_t stream) {
  TB_ENSURE_DEVICE();
  if (world < 1 || world > MAX_RANKS || M % (128 * world)) TB_FAIL(TB_E_ARG, "gemm_rs: M=%d must be a multiple of 128*world", M);
  if (N % 32 || ldd % 8) TB_FAIL(TB_E_ARG, "gemm_rs: N must be a multiple of 32 and ldd of 8");
  TpFusion tp;
  tp.kind = 1; tp.rank = rank; tp.world = world; tp.peers = dst;
  return gemm_dispatch(A, B, const_cast<void*>(dst[rank]), M, N, K, 0, b_major, lda, ldb, ldd, nullptr, nullptr, 0,
                       nullptr, nullptr, out_f32 ? EPI_OUT_F32 : 0, 1, bn, status, stream, tp);
}

// Column-parallel linear with sequence parallelism: D[M, N] = gather(A)[M, K] * B[N, K]^T where rank r
// owns rows [r*M/world, (r+1)*M/world) of A. a_full is the local [M, K] staging matrix (contiguous,
// lda = K) whose own-rank rows already hold this rank's shard; shards[r] is rank r's shard
// [M/world, K] (contiguous; may point into that rank's a_full). ready: local uint32 [M/128].
TB_EXPORT int tb_ag_gemm(void* a_full, const void* const* shards, const void* const* flag_bufs,
                         const unsigned* epoch_ptr, unsigned* ready, const void* B, void* D, int M, int N, int K,
                         int b_major, int ldb, int ldd, const void* bias, int flags, int rank, int world,
                         int copy_ctas, int bn, int* status, cudaStream_t stream);

static int gemm_dispatch(const void* A, const void* B, void* D, int M, int N, int K, int a_major,
                         int b_major, int lda, int ldb, int ldd, const void* bias,
                         const void* residual, int ldr, void* preact, const void* aux, int flags,
                         int split_k, int bn, int* status, cudaStream_t stream, const TpFusion& tp) {
  if (!A || !B || !D || M <= 0 || N <= 0 || K <= 0) TB_FAIL(TB_E_ARG, "tb_gemm_bf16: null pointer or empty shape");
  if ((lda & 7) || (ldb & 7)) TB_FAIL(TB_E_ARG, "tb_gemm_bf16: lda/ldb must be multiples of 8 (got %d, %d)", lda, ldb);
  if ((flags & EPI_BIAS) && !bias) TB_FAIL(TB_E_ARG, "tb_gemm_bf16: EPI_BIAS without bias");
  if ((flags & EPI_RESIDUAL) && !residual) TB_FAIL(TB_E_ARG, "tb_gemm_bf16: EPI_RESIDUAL without residual");
  if ((flags & EPI_STORE_PREACT) && !preact) TB_FAIL(TB_E_ARG, "tb_gemm_bf16: EPI_STORE_PREACT without buffer");
  if ((flags & EPI_MUL_DGELU) && !aux) TB_FAIL(TB_E_ARG, "tb_gemm_bf16: EPI_MUL_DGELU without aux");
  if ((flags & EPI_ATOMIC) && !(flags & EPI_OUT_F32)) TB_FAIL(TB_E_ARG, "tb_gemm_bf16: EPI_ATOMIC needs fp32 output");
  // split_k == -1: stream-K (every CTA gets the same number of K-blocks; partial tiles meet through fp32 atomics)
  const bool stream_k = split_k == -1;
  if (stream_k && (!(flags & EPI_ATOMIC) || tp.kind != 0)) TB_FAIL(TB_E_ARG, "tb_gemm_bf16: stream-K needs EPI_ATOMIC and no fused collective");
  if (split_k < 1) split_k = 1;
  if (split_k > 1 && !(flags & EPI_ATOMIC)) TB_FAIL(TB_E_ARG, "tb_gemm_bf16: split_k > 1 needs EPI_ATOMIC");
  if (bn == 0 && stream_k) bn = N > 128 ? 256 : 128;
  if (bn == 0) {
    // 256-wide tiles halve the smem traffic per FLOP; fall back to 128 when that
    // leaves SMs idle.
    long t256 = (long)((M + BM - 1) / BM) * ((N + 255) / 256) * split_k;
    bn = (N > 128 && t256 >= sm_count()) ? 256 : 128;
  }
  if (bn != 128 && bn != 256) TB_FAIL(TB_E_ARG, "tb_gemm_bf16: bn must be 128 or 256");

  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.ldd = ldd; p.ldr = ldr;
  p.D = D;
  p.bias = (const __nv_bfloat16*)bias;
  p.residual = (const __nv_bfloat16*)residual;
  p.preact = (__nv_bfloat16*)preact;
  p.aux = (const __nv_bfloat16*)aux;
  p.flags = flags;
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (N + bn - 1) / bn;
  p.kb_total = (K + BK - 1) / BK;
  if (split_k > p.kb_total) split_k = p.kb_total;
  p.kb_per_split = (p.kb_total + split_k - 1) / split_k;
  split_k = (p.kb_total + p.kb_per_split - 1) / p.kb_per_split;  // no empty split
  p.split_k = split_k;
  p.stream_k = stream_k ? 1 : 0;
  p.status = status;
  p.rank = tp.rank;
  p.world = tp.world;
  if (tp.kind == 3) {
    const int C = K / 9, H = tp.cv_h, W = tp.cv_w, Nimg = tp.cv_n;
    if (a_major != 0 || K != 9 * C || (C & 63) || W > 128 || H < 1 || W < 1 || M != Nimg * H * W)
      TB_FAIL(TB_E_ARG, "conv gemm: needs K-major A, channels %% 64 == 0, W <= 128 and M = N*H*W");
    if (split_k != 1 || (flags & (EPI_ATOMIC | EPI_ACCUM))) TB_FAIL(TB_E_ARG, "conv gemm: no split-K / accumulate");
    p.conv = tp.cv_mode;
    p.cv_H = H; p.cv_W = W; p.cv_N = Nimg;
    if (H * W <= 128) { p.cv_TH = H; p.cv_TN = 128 / (H * W); }
    else              { p.cv_TH = 128 / W; p.cv_TN = 1; }
    if (p.cv_TN > Nimg) p.cv_TN = Nimg;
    p.cv_tiles_h = (H + p.cv_TH - 1) / p.cv_TH;
    p.cv_cchunks = C / 64;
    p.cv_a_bytes = 128 * W * p.cv_TH * p.cv_TN;
    p.tiles_m = ((Nimg + p.cv_TN - 1) / p.cv_TN) * p.cv_tiles_h;
  }
  if (tp.kind == 4) {
    // weight gradient: M = Cout, N = 9 * Cin, the K loop runs over pixel blocks
    const int H = tp.cv_h, W = tp.cv_w, Nimg = tp.cv_n, cin = N / 9;
    if (a_major != 1 || b_major != 1 || N != 9 * cin || (cin & 63) || (M & 7) || W > 64 || H < 1)
      TB_FAIL(TB_E_ARG, "conv wgrad: needs Cin %% 64 == 0, W <= 64");
    if (!(flags & EPI_ATOMIC)) TB_FAIL(TB_E_ARG, "conv wgrad: fp32 atomic accumulation only");
    p.conv = 3;
    p.cv_H = H; p.cv_W = W; p.cv_N = Nimg;
    if (H * W <= 64) { p.cv_TH = H; p.cv_TN = 64 / (H * W); }
    else             { p.cv_TH = 64 / W; p.cv_TN = 1; }
    if (p.cv_TN > Nimg) p.cv_TN = Nimg;
    p.cv_tiles_h = (H + p.cv_TH - 1) / p.cv_TH;
    p.cv_a_bytes = 128 * W * p.cv_TH * p.cv_TN;   // bytes of one 64-column chunk box
    p.kb_total = ((Nimg + p.cv_TN - 1) / p.cv_TN) * p.cv_tiles_h;
    if (split_k > p.kb_total) split_k = p.kb_total;
    p.kb_per_split = (p.kb_total + split_k - 1) / split_k;
    split_k = (p.kb_total + p.kb_per_split - 1) / p.kb_per_split;
    p.split_k = split_k;
  }
  if (tp.kind == 1) {
    p.rs_rows = M / tp.world;
    for (int i = 0; i < tp.world; ++i) p.rs_dst[i] = const_cast<void*>(tp.peers[i]);
    // start with the tiles of the next rank and finish with the own rows: spreads the NVLink
    // traffic of the ranks over different destinations at any moment
    p.m_rot = ((tp.rank + 1) % tp.world) * (p.rs_rows / BM);
  } else if (tp.kind == 2) {
    p.ag_ctas = tp.copy_ctas;
    p.ag_rows = M / tp.world;
    for (int i = 0; i < tp.world; ++i) {
      p.ag_src[i] = tp.peers[i];
      p.flag_tbl[i] = const_cast<void*>(tp.flags[i]);
    }
    p.ag_dst = const_cast<void*>(A);
    p.ag_ready = tp.ready;
    {
      // parts per tile: enough that every copy CTA has work, a power of two that divides the K/64 pieces of a tile
      const int tiles_remote = (tp.world - 1) * (p.ag_rows / BM);
      int split = 1;
      while (split < 8 && tiles_remote * split < 2 * tp.copy_ctas && ((K / 64) % (split * 2)) == 0) split *= 2;
      p.ag_split = split;
    }
    p.epoch_ptr = tp.epoch_ptr;
    p.m_rot = tp.rank * (p.ag_rows / BM);  // own shard first
  } else if (tp.kind == 5) {
    if (split_k != 1 || stream_k) TB_FAIL(TB_E_ARG, "fsdp_ag_gemm: no split-K");
    const long b_bytes = (long)(b_major == 0 ? N : K) * ldb * 2;
    const long unit_bytes = (long)tp.wg.world * tp.wg.cpr * tp.wg.chunk_bytes;
    if (tp.wg_b_off < 0 || tp.wg_b_off + b_bytes > unit_bytes || (const char*)B != (const char*)tp.wg.dst + tp.wg_b_off)
      TB_FAIL(TB_E_ARG, "fsdp_ag_gemm: B must lie inside the unit buffer at the given offset");
    p.wg_on = 1;      // gathered by the seventh warp of every CTA (no dedicated copy CTAs)
    p.wg = tp.wg;
    p.wg.status = status;
    p.wg_b_off = tp.wg_b_off;
    p.wg_ldb_bytes = (long)ldb * 2;
    p.epoch_ptr = tp.wg.epoch_ptr;
  }

  CUtensorMap ma, mb;
  {
    uint64_t dims[2], str[1];
    uint32_t box[2];
    int r;
    if (tp.kind == 4) {
      uint32_t b4[4] = {64, (uint32_t)tp.cv_w, (uint32_t)p.cv_TH, (uint32_t)p.cv_TN};
      uint64_t da[4] = {(uint64_t)M, (uint64_t)tp.cv_w, (uint64_t)tp.cv_h, (uint64_t)tp.cv_n};
      uint64_t sa4[3] = {(uint64_t)lda * 2, (uint64_t)tp.cv_w * lda * 2, (uint64_t)tp.cv_h * tp.cv_w * lda * 2};
      r = make_tmap(&ma, A, 2, 4, da, sa4, b4);
      if (r) return r;
      const uint64_t cin = (uint64_t)N / 9;
      uint64_t db[4] = {cin, (uint64_t)tp.cv_w, (uint64_t)tp.cv_h, (uint64_t)tp.cv_n};
      uint64_t sb4[3] = {(uint64_t)ldb * 2, (uint64_t)tp.cv_w * ldb * 2, (uint64_t)tp.cv_h * tp.cv_w * ldb * 2};
      r = make_tmap(&mb, B, 2, 4, db, sb4, b4);
      if (r) return r;
    } else
    if (tp.kind == 3) {
      const uint64_t C = (uint64_t)K / 9;
      uint64_t d4[4] = {C, (uint64_t)tp.cv_w, (uint64_t)tp.cv_h, (uint64_t)tp.cv_n};
      uint64_t s4[3] = {C * 2, (uint64_t)tp.cv_w * C * 2, (uint64_t)tp.cv_h * tp.cv_w * C * 2};
      uint32_t b4[4] = {64, (uint32_t)tp.cv_w, (uint32_t)p.cv_TH, (uint32_t)p.cv_TN};
      r = make_tmap(&ma, A, 2, 4, d4, s4, b4);
    } else {
      if (a_major == 0) { dims[0] = K; dims[1] = M; box[0] = BK; box[1] = BM; }
      else              { dims[0] = M; dims[1] = K; box[0] = 64; box[1] = BK; }
      str[0] = (uint64_t)lda * 2;
      r = make_tmap(&ma, A, 2, 2, dims, str, box);
    }
    if (r) return r;
    if (tp.kind == 4) { /* both maps were built above */ }
    else {
    if (b_major == 0) { dims[0] = K; dims[1] = N; box[0] = BK; box[1] = bn; }
    else if (tp.kind == 3) { dims[0] = (uint64_t)9 * N; dims[1] = (uint64_t)K / 9; box[0] = 64; box[1] = BK; }
    else              { dims[0] = N; dims[1] = K; box[0] = 64; box[1] = BK; }
    str[0] = (uint64_t)ldb * 2;
    r = make_tmap(&mb, B, 2, 2, dims, str, box);
    if (r) return r;
    }
  }

  // TMA-store epilogue: bf16 output, whole 64-column groups, 16-byte aligned rows and operands
  OutMaps om;
  memset(&om, 0, sizeof(om));
  {
    static const bool enabled = [] {
      const char* e = getenv("TB_GEMM_TMA_STORE");
      return !(e && e[0] == '0');
    }();
    auto al16 = [](const void* q) { return ((uintptr_t)q & 15) == 0; };
    bool ok = enabled && tp.kind != 3 && !(flags & (EPI_OUT_F32 | EPI_ACCUM | EPI_ATOMIC)) && (N % 64) == 0 && (ldd & 7) == 0 &&
              split_k == 1 && (!bias || al16(bias)) && (!residual || (al16(residual) && (ldr & 7) == 0)) &&
              (!preact || al16(preact)) && (!aux || al16(aux));
    uint64_t dims[2], str[1] = {(uint64_t)ldd * 2};
    uint32_t box[2] = {64, 32};
    if (ok && tp.kind == 1) {
      dims[0] = (uint64_t)N;
      dims[1] = (uint64_t)tp.world * (uint64_t)(M / tp.world);
      for (int i = 0; i < tp.world && ok; ++i) ok = al16(tp.peers[i]) && make_tmap(&om.m[i], tp.peers[i], 2, 2, dims, str, box) == 0;
    } else if (ok) {
      dims[0] = (uint64_t)N;
      dims[1] = (uint64_t)M;
      ok = al16(D) && make_tmap(&om.m[0], D, 2, 2, dims, str, box) == 0;
    }
    p.tma_store = ok ? 1 : 0;
  }

#define TB_DISPATCH(BN_, ST_)                                                          \
  do {                                                                                 \
    if (a_major == 0 && b_major == 0) return launch_gemm<BN_, 0, 0, ST_>(ma, mb, om, p, stream); \
    if (a_major == 0 && b_major == 1) return launch_gemm<BN_, 0, 1, ST_>(ma, mb, om, p, stream); \
    if (a_major == 1 && b_major == 1) return launch_gemm<BN_, 1, 1, ST_>(ma, mb, om, p, stream); \
    if (a_major == 1 && b_major == 0) return launch_gemm<BN_, 1, 0, ST_>(ma, mb, om, p, stream); \
  } while (0)
  if (tp.kind == 5) {
    // one pipeline stage less than the plain GEMM: its 48 / 64 KB hold the gather warp's three-piece ring
    if (bn == 256) {
      if (b_major == 0) return launch_gemm<256, 0, 0, 3, 3>(ma, mb, om, p, stream);
      return launch_gemm<256, 0, 1, 3, 3>(ma, mb, om, p, stream);
    }
    if (b_major == 0) return launch_gemm<128, 0, 0, 4, 3>(ma, mb, om, p, stream);
    return launch_gemm<128, 0, 1, 4, 3>(ma, mb, om, p, stream);
  }
  if (bn == 256) TB_DISPATCH(256, 4);
  else TB_DISPATCH(128, 6);
#undef TB_DISPATCH
  TB_FAIL(TB_E_ARG, "tb_gemm_bf16: unsupported major combination");
}

__global__ void gemm_bump_epoch_kernel(uint32_t* e) { *e += 1; }

// Checks and fills the description of one unit gather (shared by the fused and the stand-alone launcher).
int tb_fill_gather(tb::GatherArgs& g, const void* const* shards, void* unit_buf, const void* const* flag_bufs,
                   const unsigned* epoch_ptr, unsigned* ready, int chunk_bytes, int cpr, int first_chunk, int rank,
                   int world, int ctas, int* status) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) TB_FAIL(TB_E_ARG, "fsdp gather: bad rank/world %d/%d", rank, world);
  if (chunk_bytes < GATHER_PIECE || (chunk_bytes & (chunk_bytes - 1))) TB_FAIL(TB_E_ARG, "fsdp gather: chunk bytes (%d) must be a power of two >= 16384", chunk_bytes);
  if (cpr < 1 || first_chunk < 0 || first_chunk >= world * cpr) TB_FAIL(TB_E_ARG, "fsdp gather: bad chunk counts");
  if (!unit_buf || !ready || !epoch_ptr || ((uintptr_t)unit_buf & 15)) TB_FAIL(TB_E_ARG, "fsdp gather: null or unaligned buffer");
  if (ctas < 1 || ctas > 128) TB_FAIL(TB_E_ARG, "fsdp gather: copy CTAs must be in [1, 128]");
  for (int i = 0; i < MAX_RANKS; ++i) {
    g.src[i] = i < world ? shards[i] : nullptr;
    g.flag_tbl[i] = i < world ? const_cast<void*>(flag_bufs[i]) : nullptr;
    if (i < world && (!shards[i] || ((uintptr_t)shards[i] & 15))) TB_FAIL(TB_E_ARG, "fsdp gather: null or unaligned shard");
  }
  g.dst = unit_buf; g.epoch_ptr = epoch_ptr; g.ready = ready; g.chunk_bytes = chunk_bytes; g.cpr = cpr;
  g.first = first_chunk; g.ctas = ctas; g.rank = rank; g.world = world; g.status = status;
  return 0;
}

// The GEMM that first consumes an FSDP unit, fused with the unit's un-shard: D = epilogue(A * op(B)^T) as tb_gemm_bf16,
// where B lives at byte offset b_off of the local unit buffer `unit_buf` that `copy_ctas` extra CTAs fill from every
// rank's shard (shards[r]: rank r's cpr chunks of chunk_bytes each, in symmetric memory) while the GEMM CTAs compute;
// the chunk that holds the start of B is fetched first. ready: local uint32 [2 * world * cpr], zero before first use.
// When the kernel has finished, the whole unit is in unit_buf. One communication context (flag_bufs, epoch_ptr) per
// stream; the launch bumps its epoch.
TB_EXPORT int tb_fsdp_ag_gemm(const void* A, const void* B, void* D, int M, int N, int K, int a_major, int b_major,
                              int lda, int ldb, int ldd, const void* bias, const void* residual, int ldr, void* preact,
                              const void* aux, int flags, int bn, const void* const* shards, void* unit_buf,
                              const void* const* flag_bufs, const unsigned* epoch_ptr, unsigned* ready, int chunk_bytes,
                              int cpr, long b_off, int rank, int world, int copy_ctas, int* status,
                              cudaStream_t stream) {
  TB_ENSURE_DEVICE();
  if (flags & (EPI_ATOMIC | EPI_ACCUM)) TB_FAIL(TB_E_ARG, "fsdp_ag_gemm: plain outputs only");
  if (ldb != (b_major == 0 ? K : N)) TB_FAIL(TB_E_ARG, "fsdp_ag_gemm: B must be contiguous (ldb %d)", ldb);
  TpFusion tp;
  tp.kind = 5;
  if (a_major != 0) TB_FAIL(TB_E_ARG, "fsdp_ag_gemm: A must be K-major");
  copy_ctas = 1;  // unused: every CTA of the launch carries a gather warp
  int r = tb_fill_gather(tp.wg, shards, unit_buf, flag_bufs, epoch_ptr, ready, chunk_bytes, cpr,
                         (int)(b_off / chunk_bytes) % (world * cpr > 0 ? world * cpr : 1), rank, world, copy_ctas, status);
  if (r) return r;
  tp.wg_b_off = b_off;
  tp.rank = rank; tp.world = world;
  r = gemm_dispatch(A, B, D, M, N, K, a_major, b_major, lda, ldb, ldd, bias, residual, ldr, preact, aux, flags, 1, bn,
                    status, stream, tp);
  if (r) return r;
  gemm_bump_epoch_kernel<<<1, 1, 0, stream>>>(const_cast<unsigned*>(epoch_ptr));
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

TB_EXPORT int tb_ag_gemm(void* a_full, const void* const* shards, const void* const* flag_bufs,
                         const unsigned* epoch_ptr, unsigned* ready, const void* B, void* D, int M, int N, int K,
                         int b_major, int ldb, int ldd, const void* bias, int flags, int rank, int world,
                         int copy_ctas, int bn, int* status, cudaStream_t stream) {
  TB_ENSURE_DEVICE();
  if (world < 1 || world > MAX_RANKS || M % (128 * world)) TB_FAIL(TB_E_ARG, "ag_gemm: M=%d must be a multiple of 128*world", M);
  if (((long)128 * K * 2) % 16384) TB_FAIL(TB_E_ARG, "ag_gemm: K=%d must be a multiple of 64", K);
  if (copy_ctas < 1) copy_ctas = 16;
  if (copy_ctas > 64) copy_ctas = 64;
  if (world == 1) copy_ctas = 0;
  TpFusion tp;
  tp.kind = world > 1 ? 2 : 0;
  tp.rank = rank; tp.world = world; tp.peers = shards; tp.flags = flag_bufs; tp.epoch_ptr = epoch_ptr; tp.ready = ready;
  tp.copy_ctas = copy_ctas;
  int r = gemm_dispatch(a_full, B, D, M, N, K, 0, b_major, K, ldb, ldd, bias, nullptr, 0, nullptr, nullptr, flags, 1,
                        bn, status, stream, tp);
  if (r) return r;
  if (world > 1) gemm_bump_epoch_kernel<<<1, 1, 0, stream>>>(const_cast<unsigned*>(epoch_ptr));
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// After a kernel gave up on a wait (status word set) its scheduler counters may not have been reset: clear them all.
// Turns the dynamic tile scheduler of the persistent GEMM on (1) or off (0); returns the previous setting.
TB_EXPORT int tb_gemm_set_dynamic(int on) {
  const int was = g_dynamic_tiles ? 1 : 0;
  g_dynamic_tiles = on != 0;
  return was;
}

TB_EXPORT int tb_gemm_reset_scheduler(cudaStream_t stream) {
  TB_ENSURE_DEVICE();
  unsigned* p = nullptr;
  TB_CUDA_CHECK(cudaGetSymbolAddress((void**)&p, tb::g_sched_counters));
  TB_CUDA_CHECK(cudaMemsetAsync(p, 0, sizeof(unsigned) * 2 * tb::SCHED_SLOTS, stream));
  return 0;
}

// Records the device that subsequent launches (from any thread) must run on.
TB_EXPORT void tb_set_device(int device) { tb::g_device().store(device); }

TB_EXPORT const char* tb_last_error() { return tb::last_error_buf(); }
