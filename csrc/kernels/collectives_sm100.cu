// Stand-alone collectives over NVSwitch peer memory for sm_100a: all-reduce (one-shot peer
// loads, two-shot NVLS multimem, two-shot plain peer loads/stores), all-gather and
// reduce-scatter, each with a fused scale (and the bf16 <-> fp32-accumulate cast).
//
// All buffers are "symmetric": the same allocation exists on every rank, and the kernel gets a
// table of the per-rank base pointers plus (when NVLS is available) one multicast address that the
// switch fans out to / reduces over all copies. The uniform NVSwitch topology needs no rings:
//   one-shot  : every rank reads all copies of the whole message and sums them (latency-optimal)
//   two-shot  : rank r reduces slice r (multimem.ld_reduce: the switch does the adds) and
//               broadcasts it (multimem.st) - bandwidth-optimal, 2 x N/world bytes per rank
// Entry and exit barriers use per-CTA flag slots with bounded waits (comm.cuh).
//
// The reference's collectives are no-ops / local clones (crates/torsh-distributed/src/collectives.rs:
// 232-288,797-845) and its only real all-reduce is a host-staged ring
// (crates/torsh-backend/src/cuda/multi_gpu.rs:130-217).
#include "comm.cuh"
#include "common.cuh"
#include "host_util.h"

namespace tb {

constexpr int COMM_THREADS = 512;
constexpr int COMM_MAX_BLOCKS = 320;  // flag slots per symmetric flag buffer (one per CTA: two CTAs per SM and some)

struct CommArgs {
  PeerTable bufs;    // symmetric data buffer
  PeerTable flags;   // symmetric flag buffer: uint32 [COMM_MAX_BLOCKS][MAX_RANKS]
  char* mc;          // multicast address of the data buffer (null: no NVLS)
  int rank, world;
  const uint32_t* epoch_ptr;  // device counter; this launch uses barrier values 2*e and 2*e+1, then bumps it
  long byte_off;     // offset of the message inside the symmetric buffer
  long n;            // elements
  float scale;
  int* status;
};

template <typename T> struct Acc;
template <> struct Acc<float> {
  static constexpr int N = 4;
  __device__ static void load(const void* p, float (&f)[4]) {
    float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  __device__ static void mc_reduce(const void* p, float (&f)[4]) {
    float4 v = multimem_ld_reduce_f32x4(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  __device__ static uint4 pack(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
};
template <> struct Acc<bf16> {
  static constexpr int N = 8;
  __device__ static void unpack(uint4 v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = bf16_lo(w[i]); f[2 * i + 1] = bf16_hi(w[i]); }
  }
  __device__ static void load(const void* p, float (&f)[8]) { unpack(*reinterpret_cast<const uint4*>(p), f); }
  __device__ static void mc_reduce(const void* p, float (&f)[8]) { unpack(multimem_ld_reduce_bf16x8(p), f); }
  __device__ static uint4 pack(const float (&f)[8]) {
    return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
  }
};

// Slice of rank r when n elements are split into `world` vector-aligned chunks.
__device__ __forceinline__ void slice_of(long n, int world, int r, int vec, long& begin, long& end) {
  long nv = (n + vec - 1) / vec;
  long per = (nv + world - 1) / world;
  begin = min(n, (long)r * per * vec);
  end = min(n, (long)(r + 1) * per * vec);
}

// MODE 0: one-shot (peer loads, result written to every rank's own copy by that rank)
// MODE 1: two-shot NVLS (multimem.ld_reduce own slice, multimem.st broadcast)
// MODE 2: two-shot plain peer memory (peer loads of own slice, peer stores to every copy)
template <typename T, int MODE>
__global__ void __launch_bounds__(COMM_THREADS)
allreduce_kernel(const CommArgs a) {
  constexpr int N = Acc<T>::N;
  const uint32_t epoch = *a.epoch_ptr;
  // a failed entry barrier means some peer's data is not known to be complete: touch nothing
  if (!cta_barrier_all_ranks(a.flags, blockIdx.x, a.rank, a.world, 2 * epoch, a.status)) return;
  const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const long nthreads = (long)gridDim.x * blockDim.x;
  if (MODE == 0) {
    char* mine = reinterpret_cast<char*>(a.bufs.ptr[a.rank]) + a.byte_off;
    // Every thread sums up to 4 vectors over all copies into registers; after a second barrier
    // (all ranks have finished reading) each rank overwrites its own copy with the result.
    const long nvec = a.n / N;  // launcher guarantees n % N == 0
    float acc[4][N];
    int cnt = 0;
    for (long v = tid; v < nvec && cnt < 4; v += nthreads, ++cnt) {
#pragma unroll
      for (int j = 0; j < N; ++j) acc[cnt][j] = 0.f;
      // copies are added in rank order 0, 1, ... on EVERY rank: a rank-rotated order would give each rank a differently
      // rounded sum beyond two ranks, and replicated parameters stepped with those sums would drift apart
      for (int q = 0; q < a.world; ++q) {
        float f[N];
        Acc<T>::load(reinterpret_cast<const char*>(a.bufs.ptr[q]) + a.byte_off + v * N * sizeof(T), f);
#pragma unroll
        for (int j = 0; j < N; ++j) acc[cnt][j] += f[j];
      }
    }
    // without the second barrier a peer may still be reading this rank's copy: leave it as it is
    if (!cta_barrier_all_ranks(a.flags, blockIdx.x, a.rank, a.world, 2 * epoch + 1, a.status)) return;
    cnt = 0;
    for (long v = tid; v < nvec && cnt < 4; v += nthreads, ++cnt) {
#pragma unroll
      for (int j = 0; j < N; ++j) acc[cnt][j] *= a.scale;
      *reinterpret_cast<uint4*>(mine + v * N * sizeof(T)) = Acc<T>::pack(acc[cnt]);
    }
    return;
  }
  long b0, b1;
  slice_of(a.n, a.world, a.rank, N, b0, b1);
  const long nvec = (b1 - b0) / N;
  constexpr int U = 4;  // vectors in flight per thread
  for (long v0 = tid; v0 < nvec; v0 += nthreads * U) {
    float f[U][N];
    long eoff[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long v = v0 + (long)u * nthreads;
      eoff[u] = a.byte_off + (b0 + v * N) * (long)sizeof(T);
      if (v < nvec) {
        if (MODE == 1) {
          Acc<T>::mc_reduce(a.mc + eoff[u], f[u]);
        } else {
#pragma unroll
          for (int j = 0; j < N; ++j) f[u][j] = 0.f;
          for (int p = 0; p < a.world; ++p) {
            const int q = (a.rank + p) % a.world;
            float g[N];
            Acc<T>::load(reinterpret_cast<const char*>(a.bufs.ptr[q]) + eoff[u], g);
#pragma unroll
            for (int j = 0; j < N; ++j) f[u][j] += g[j];
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long v = v0 + (long)u * nthreads;
      if (v < nvec) {
#pragma unroll
        for (int j = 0; j < N; ++j) f[u][j] *= a.scale;
        const uint4 o = Acc<T>::pack(f[u]);
        if (MODE == 1) {
          multimem_st_16(a.mc + eoff[u], o);
        } else {
          for (int p = 0; p < a.world; ++p) {
            const int q = (a.rank + p) % a.world;
            *reinterpret_cast<uint4*>(reinterpret_cast<char*>(a.bufs.ptr[q]) + eoff[u]) = o;
          }
        }
      }
    }
  }
  cta_barrier_all_ranks(a.flags, blockIdx.x, a.rank, a.world, 2 * epoch + 1, a.status);
}

// All-gather in place: the symmetric buffer holds world chunks of `n` elements; rank r's chunk is
// valid at chunk index r on entry and every chunk is valid on every rank on exit.
template <bool NVLS>
__global__ void __launch_bounds__(COMM_THREADS)
allgather_kernel(const CommArgs a, int elem_bytes) {
  const uint32_t epoch = *a.epoch_ptr;
  if (!cta_barrier_all_ranks(a.flags, blockIdx.x, a.rank, a.world, 2 * epoch, a.status)) return;
  const long bytes = a.n * elem_bytes;  // launcher guarantees a multiple of 16
  const long nvec = bytes / 16;
  const long base = a.byte_off + (long)a.rank * bytes;
  const char* src = reinterpret_cast<const char*>(a.bufs.ptr[a.rank]) + base;
  constexpr int U = 4;  // vectors in flight per thread
  const long nthreads = (long)gridDim.x * blockDim.x;
  for (long v0 = (long)blockIdx.x * blockDim.x + threadIdx.x; v0 < nvec; v0 += nthreads * U) {
    uint4 x[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long v = v0 + (long)u * nthreads;
      if (v < nvec) x[u] = *reinterpret_cast<const uint4*>(src + v * 16);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long v = v0 + (long)u * nthreads;
      if (v >= nvec) continue;
      if (NVLS) {
        multimem_st_16(a.mc + base + v * 16, x[u]);
      } else {
        for (int p = 1; p < a.world; ++p) {
          const int q = (a.rank + p) % a.world;
          *reinterpret_cast<uint4*>(reinterpret_cast<char*>(a.bufs.ptr[q]) + base + v * 16) = x[u];
        }
      }
    }
  }
  cta_barrier_all_ranks(a.flags, blockIdx.x, a.rank, a.world, 2 * epoch + 1, a.status);
}

// Reduce-scatter: the symmetric buffer holds world chunks of n elements on every rank;
// out[i] = scale * sum_p buf_p[rank * n + i], written to local (non-symmetric) memory.
template <typename T, bool NVLS>
__global__ void __launch_bounds__(COMM_THREADS)
reducescatter_kernel(const CommArgs a, T* __restrict__ out) {
  constexpr int N = Acc<T>::N;
  const uint32_t epoch = *a.epoch_ptr;
  if (!cta_barrier_all_ranks(a.flags, blockIdx.x, a.rank, a.world, 2 * epoch, a.status)) return;
  const long nvec = a.n / N;
  const long base = a.byte_off + (long)a.rank * a.n * (long)sizeof(T);
  constexpr int U = 4;  // vectors in flight per thread
  const long nthreads = (long)gridDim.x * blockDim.x;
  for (long v0 = (long)blockIdx.x * blockDim.x + threadIdx.x; v0 < nvec; v0 += nthreads * U) {
    float f[U][N];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long v = v0 + (long)u * nthreads;
      if (v >= nvec) continue;
      if (NVLS) {
        Acc<T>::mc_reduce(a.mc + base + v * 16, f[u]);
      } else {
#pragma unroll
        for (int j = 0; j < N; ++j) f[u][j] = 0.f;
        for (int p = 0; p < a.world; ++p) {
          const int q = (a.rank + p) % a.world;
          float g[N];
          Acc<T>::load(reinterpret_cast<const char*>(a.bufs.ptr[q]) + base + v * 16, g);
#pragma unroll
          for (int j = 0; j < N; ++j) f[u][j] += g[j];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long v = v0 + (long)u * nthreads;
      if (v >= nvec) continue;
#pragma unroll
      for (int j = 0; j < N; ++j) f[u][j] *= a.scale;
      *reinterpret_cast<uint4*>(reinterpret_cast<char*>(out) + v * 16) = Acc<T>::pack(f[u]);
    }
  }
  // peers may overwrite their chunks only after everyone has read them
  cta_barrier_all_ranks(a.flags, blockIdx.x, a.rank, a.world, 2 * epoch + 1, a.status);
}

// Second half of GEMM -> reduce-scatter: once every rank has stored its partial tiles into this rank's
// slot buffer ([world][rows][N]; entry barrier), sum the slots in fp32, add bias / residual, write the
// bf16 output, and hold everybody until all slot buffers have been read (exit barrier), after which
// they may be rewritten.
//
// The sum is a local HBM-bound pass, so it runs on a grid that fills the GPU (all CTAs resident), while the two
// cross-rank barriers involve one CTA only: CTA 0 performs the entry barrier and then publishes the epoch in
// local_sync[0]; the other CTAs wait (bounded) for that word. The CTA that finishes last (counter in
// local_sync[1], reset by that CTA) performs the exit barrier.
template <typename TA>
__global__ void __launch_bounds__(COMM_THREADS)
rs_finalize_kernel(const CommArgs a, const TA* __restrict__ acc, const bf16* __restrict__ bias,
                   const bf16* __restrict__ residual, bf16* __restrict__ out, long rows, int N,
                   uint32_t* __restrict__ local_sync) {
  const uint32_t epoch = *a.epoch_ptr;
  __shared__ int s_last;
  if (blockIdx.x == 0) {
    cta_barrier_all_ranks(a.flags, 0, a.rank, a.world, 2 * epoch, a.status);
    if (threadIdx.x == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(local_sync), "r"(epoch) : "memory");
  } else {
    if (threadIdx.x == 0) {
      const uint64_t t0 = globaltimer_ns();
      uint32_t spins = 0;
      while (true) {
        uint32_t v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(local_sync) : "memory");
        if ((int32_t)(v - epoch) >= 0) break;
        if ((++spins & 31u) == 0u) {
          if (a.status && *((volatile int*)a.status) != 0) break;
          if (globaltimer_ns() - t0 > TB_PEER_WAIT_LIMIT_NS) {
            if (a.status) atomicCAS(a.status, 0, TB_ERR_WAIT_PEER);
            break;
          }
        }
      }
    }
    __syncthreads();
  }
  // the slots are complete only if the entry barrier went through; otherwise leave the output alone
  if (a.status && *((volatile int*)a.status) != 0) return;
  const uint32_t nvec = (uint32_t)(rows * N / 8);
  const uint32_t vec_per_row = (uint32_t)N / 8;
  const long slot = rows * N;
  for (uint32_t v = blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += gridDim.x * blockDim.x) {
    const long e = (long)v * 8;
    const int c = (int)(v % vec_per_row) * 8;
    float f[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = 0.f;
#pragma unroll 4
    for (int s = 0; s < a.world; ++s) {
      float g[8];
      if (sizeof(TA) == 4) {
        const float4* src = reinterpret_cast<const float4*>(acc + s * slot + e);
        float4 x = src[0], y = src[1];
        g[0] = x.x; g[1] = x.y; g[2] = x.z; g[3] = x.w; g[4] = y.x; g[5] = y.y; g[6] = y.z; g[7] = y.w;
      } else {
        Acc<bf16>::load(acc + s * slot + e, g);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += g[j];
    }
    if (bias) {
      float b[8];
      Acc<bf16>::load(bias + c, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += b[j];
    }
    if (residual) {
      float r[8];
      Acc<bf16>::load(residual + e, r);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += r[j];
    }
    *reinterpret_cast<uint4*>(out + e) = Acc<bf16>::pack(f);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t done = atomicAdd(local_sync + 1, 1u);
    s_last = (done == gridDim.x - 1);
    if (s_last) local_sync[1] = 0;
  }
  __syncthreads();
  if (s_last) cta_barrier_all_ranks(a.flags, 0, a.rank, a.world, 2 * epoch + 1, a.status);
}

// Runs after a collective on the same stream: the next launch sees a fresh pair of barrier values.
__global__ void bump_epoch_kernel(uint32_t* e) { *e += 1; }

static int fill_args(CommArgs& a, const void* const* bufs, const void* const* flags, void* mc, int rank, int world,
                     const unsigned* epoch_ptr, long byte_off, long n, float scale, int* status) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) TB_FAIL(TB_E_ARG, "collective: bad rank/world %d/%d", rank, world);
  if (byte_off & 15) TB_FAIL(TB_E_ARG, "collective: byte offset must be a multiple of 16");
  for (int i = 0; i < MAX_RANKS; ++i) {
    a.bufs.ptr[i] = i < world ? const_cast<void*>(bufs[i]) : nullptr;
    a.flags.ptr[i] = i < world ? const_cast<void*>(flags[i]) : nullptr;
  }
  a.mc = static_cast<char*>(mc);
  a.rank = rank; a.world = world; a.epoch_ptr = epoch_ptr; a.byte_off = byte_off; a.n = n; a.scale = scale; a.status = status;
  return 0;
}

}  // namespace tb
using namespace tb;

TB_EXPORT int tb_comm_max_blocks() { return COMM_MAX_BLOCKS; }

// In-place all-reduce of n elements at byte_off of the symmetric buffer.
// dtype 0 = bf16 (fp32 accumulate), 1 = fp32. mode 0 one-shot, 1 two-shot NVLS, 2 two-shot peer memory.
TB_EXPORT int tb_allreduce(const void* const* bufs, const void* const* flags, void* mc, int rank, int world,
                           const unsigned* epoch_ptr, long byte_off, long n, int dtype, float scale, int mode, int nblocks,
                           int* status, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  CommArgs a;
  if (int r = fill_args(a, bufs, flags, mc, rank, world, epoch_ptr, byte_off, n, scale, status)) return r;
  const int vec = dtype == 0 ? 8 : 4;
  if (n % vec) TB_FAIL(TB_E_ARG, "all-reduce: n=%ld must be a multiple of %d", n, vec);
  if (mode == 1 && !mc) TB_FAIL(TB_E_ARG, "all-reduce: NVLS mode without a multicast address");
  if (nblocks < 1) nblocks = 1;
  if (nblocks > COMM_MAX_BLOCKS) nblocks = COMM_MAX_BLOCKS;
  if (mode == 0) {
    long need = (n / vec + (long)COMM_THREADS * 4 - 1) / ((long)COMM_THREADS * 4);
    if (need > COMM_MAX_BLOCKS) TB_FAIL(TB_E_TOO_LARGE, "one-shot all-reduce holds at most %d elements", COMM_MAX_BLOCKS * COMM_THREADS * 4 * vec);
    if (nblocks < need) nblocks = (int)need;
  }
#define TB_AR(T_)                                                                         \
  do {                                                                                    \
    if (mode == 0) allreduce_kernel<T_, 0><<<nblocks, COMM_THREADS, 0, st>>>(a);          \
    else if (mode == 1) allreduce_kernel<T_, 1><<<nblocks, COMM_THREADS, 0, st>>>(a);     \
    else allreduce_kernel<T_, 2><<<nblocks, COMM_THREADS, 0, st>>>(a);                    \
  } while (0)
  if (dtype == 0) TB_AR(bf16); else TB_AR(float);
#undef TB_AR
  bump_epoch_kernel<<<1, 1, 0, st>>>(const_cast<uint32_t*>(epoch_ptr));
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// In-place all-gather: chunk r (n elements of elem_bytes each) of the symmetric buffer is pushed to every rank.
TB_EXPORT int tb_allgather(const void* const* bufs, const void* const* flags, void* mc, int rank, int world,
                           const unsigned* epoch_ptr, long byte_off, long n, int elem_bytes, int use_nvls, int nblocks,
                           int* status, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  CommArgs a;
  if (int r = fill_args(a, bufs, flags, mc, rank, world, epoch_ptr, byte_off, n, 1.f, status)) return r;
  if ((n * elem_bytes) % 16) TB_FAIL(TB_E_ARG, "all-gather: chunk bytes must be a multiple of 16");
  if (use_nvls && !mc) TB_FAIL(TB_E_ARG, "all-gather: NVLS mode without a multicast address");
  if (nblocks < 1) nblocks = 1;
  if (nblocks > COMM_MAX_BLOCKS) nblocks = COMM_MAX_BLOCKS;
  if (use_nvls) allgather_kernel<true><<<nblocks, COMM_THREADS, 0, st>>>(a, elem_bytes);
  else allgather_kernel<false><<<nblocks, COMM_THREADS, 0, st>>>(a, elem_bytes);
  bump_epoch_kernel<<<1, 1, 0, st>>>(const_cast<uint32_t*>(epoch_ptr));
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// Reduce-scatter: out (local, n elements) = scale * sum over ranks of chunk `rank` of the symmetric buffer.
TB_EXPORT int tb_reducescatter(const void* const* bufs, const void* const* flags, void* mc, int rank, int world,
                               const unsigned* epoch_ptr, long byte_off, long n, int dtype, float scale, int use_nvls,
                               void* out, int nblocks, int* status, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  CommArgs a;
  if (int r = fill_args(a, bufs, flags, mc, rank, world, epoch_ptr, byte_off, n, scale, status)) return r;
  const int vec = dtype == 0 ? 8 : 4;
  if (n % vec) TB_FAIL(TB_E_ARG, "reduce-scatter: n=%ld must be a multiple of %d", n, vec);
  if (use_nvls && !mc) TB_FAIL(TB_E_ARG, "reduce-scatter: NVLS mode without a multicast address");
  if (nblocks < 1) nblocks = 1;
  if (nblocks > COMM_MAX_BLOCKS) nblocks = COMM_MAX_BLOCKS;
  if (dtype == 0) {
    if (use_nvls) reducescatter_kernel<bf16, true><<<nblocks, COMM_THREADS, 0, st>>>(a, (bf16*)out);
    else reducescatter_kernel<bf16, false><<<nblocks, COMM_THREADS, 0, st>>>(a, (bf16*)out);
  } else {
    if (use_nvls) reducescatter_kernel<float, true><<<nblocks, COMM_THREADS, 0, st>>>(a, (float*)out);
    else reducescatter_kernel<float, false><<<nblocks, COMM_THREADS, 0, st>>>(a, (float*)out);
  }
  bump_epoch_kernel<<<1, 1, 0, st>>>(const_cast<uint32_t*>(epoch_ptr));
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// One thread waits until *flag >= target or `limit_ns` nanoseconds have passed; on expiry it records
// TB_ERR_WAIT_PEER in the status word and returns, like every cross-GPU wait in this library. It lets a test (or a
// health check) see the time-out path with a flag that nothing sets, without a peer and without stalling the GPU for
// longer than the stated limit (at most one second is accepted).
__global__ void wait_probe_kernel(const uint32_t* flag, uint32_t target, unsigned long long limit_ns, int* status,
                                  unsigned long long* waited_ns) {
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if ((int32_t)(ld_acquire_sys(flag) - target) >= 0) break;
    if ((++spins & 31u) == 0u && globaltimer_ns() - t0 > limit_ns) {
      if (status) atomicCAS(status, 0, TB_ERR_WAIT_PEER);
      break;
    }
  }
  if (waited_ns) *waited_ns = globaltimer_ns() - t0;
}
TB_EXPORT int tb_wait_probe(const unsigned* flag, unsigned target, unsigned long long limit_ns, int* status,
                            unsigned long long* waited_ns, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (!flag) TB_FAIL(TB_E_ARG, "wait_probe: null flag");
  if (limit_ns > 1000000000ull) TB_FAIL(TB_E_TOO_LARGE, "wait_probe: the limit may not exceed one second");
  wait_probe_kernel<<<1, 1, 0, st>>>(flag, target, limit_ns, status, waited_ns);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// acc: this rank's slot buffer [world][rows][N] (contiguous; fp32 when acc_f32 else bf16).
// out: bf16 [rows, N]; bias [N] and residual [rows, N] are optional.
TB_EXPORT int tb_rs_finalize(const void* const* flags, int rank, int world, const unsigned* epoch_ptr, void* acc,
                             int acc_f32, const void* bias, const void* residual, void* out, long rows, int N,
                             unsigned* local_sync, int* status, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (N % 8) TB_FAIL(TB_E_ARG, "rs_finalize: N must be a multiple of 8");
  if (!local_sync) TB_FAIL(TB_E_ARG, "rs_finalize: local_sync (2 zero-initialised words) is required");
  if (rows * N / 8 >= (1L << 31)) TB_FAIL(TB_E_TOO_LARGE, "rs_finalize: more than 2^31 vectors");
  CommArgs a;
  const void* none[MAX_RANKS] = {nullptr};
  if (int r = fill_args(a, none, flags, nullptr, rank, world, epoch_ptr, 0, 0, 1.f, status)) return r;
  // every CTA must be resident at once (CTAs wait on CTA 0): at most two 512-thread CTAs per SM
  long want = (rows * N / 8 + COMM_THREADS - 1) / COMM_THREADS;
  int nblocks = (int)(want < 1 ? 1 : (want > 2L * sm_count() ? 2L * sm_count() : want));
  if (acc_f32) rs_finalize_kernel<float><<<nblocks, COMM_THREADS, 0, st>>>(a, (const float*)acc, (const bf16*)bias, (const bf16*)residual, (bf16*)out, rows, N, local_sync);
  else rs_finalize_kernel<bf16><<<nblocks, COMM_THREADS, 0, st>>>(a, (const bf16*)acc, (const bf16*)bias, (const bf16*)residual, (bf16*)out, rows, N, local_sync);
  bump_epoch_kernel<<<1, 1, 0, st>>>(const_cast<uint32_t*>(epoch_ptr));
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
