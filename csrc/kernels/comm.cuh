// Device primitives for kernels that talk to other GPUs over NVLink / NVSwitch:
// system-scope flag signalling with bounded waits, peer-pointer tables, and NVLS `multimem`
// loads / stores / reductions through a multicast address.
//
// Signalling scheme: every rank owns a flag array in symmetric memory, laid out
// [slot][world] of uint32. Rank r signals peer p by storing a monotonically increasing
// epoch into p's flags[slot][r] with release semantics at system scope; p waits until its
// own flags[slot][q] >= epoch for every q, with acquire loads. Each slot belongs to one CTA (or
// one logical barrier), each word has a single writer, values only grow, so no reset is needed.
// Every wait is bounded (about one second): on expiry the kernel records TB_ERR_WAIT_PEER in the
// launch's status word and the barrier reports failure, so a dead or late peer can never hang the GPU
// and the caller can skip the work that depended on the peers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sm100.cuh"

namespace tb {

constexpr int MAX_RANKS = 8;

#ifndef TB_PEER_WAIT_LIMIT_NS
#define TB_PEER_WAIT_LIMIT_NS 1000000000ull
#endif

struct PeerTable {
  void* ptr[MAX_RANKS];  // base address of the same symmetric buffer on every rank (own rank included)
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

// Bounded wait until *flag >= target. Returns false (and records the error) on expiry.
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* flag, uint32_t target, int* status) {
  if ((int32_t)(ld_acquire_sys(flag) - target) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if ((int32_t)(ld_acquire_sys(flag) - target) >= 0) return true;
    if ((++spins & 31u) == 0u) {
      if (status && *((volatile int*)status) != 0) return false;  // someone already gave up
      if (globaltimer_ns() - t0 > TB_PEER_WAIT_LIMIT_NS) {
        if (status) atomicCAS(status, 0, TB_ERR_WAIT_PEER);
        return false;
      }
    }
  }
}

// Cross-rank barrier for the calling CTA on flag slot `slot`. All threads of the CTA must call it.
// `flags` is the peer table of the flag arrays, `epoch` the value of this barrier instance.
// Orders all prior global writes of this CTA (to any GPU) before the peers' subsequent reads.
// Returns true when every peer arrived; false (the same value in every thread of the CTA) when a wait
// ran out or the launch's status word was already set. A caller whose ENTRY barrier failed must not
// touch peer data: the peers' buffers may be half written, and nothing orders this rank against them.
__device__ __forceinline__ bool cta_barrier_all_ranks(const PeerTable& flags, int slot, int rank, int world,
                                                      uint32_t epoch, int* status) {
  __syncthreads();
  int ok = 1;
  if (threadIdx.x < world) {
    fence_sys();
    uint32_t* remote = reinterpret_cast<uint32_t*>(flags.ptr[threadIdx.x]) + (size_t)slot * MAX_RANKS + rank;
    st_release_sys(remote, epoch);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(flags.ptr[rank]) + (size_t)slot * MAX_RANKS + threadIdx.x;
    ok = wait_flag_ge(mine, epoch, status) ? 1 : 0;
    if (status && *((volatile int*)status) != 0) ok = 0;  // an earlier wait of this launch (any CTA) gave up
    fence_sys();
  }
  return __syncthreads_and(ok) != 0;
}

// ---------------------------------------------------------------- multimem (NVLS)
// 16 bytes = 8 bf16: in-switch sum over all ranks' copies, accumulated in fp32.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
// 16 bytes = 4 fp32: in-switch sum over all ranks' copies.
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const void* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
// 16-byte store replicated by the switch into every rank's copy.
__device__ __forceinline__ void multimem_st_16(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void multimem_st_f32x4(void* mc_addr, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}

}  // namespace tb
