// FSDP step kernel for sm_100a: gradient reduce-scatter FUSED with the sharded AdamW update and
// with the all-gather of the updated bf16 parameters, in one launch over NVSwitch peer memory.
//
// Layout. One "unit" (a transformer block, or the whole model) is a contiguous range of the flat
// parameter space. Every rank holds, in symmetric memory, the full fp32 gradient range of the unit
// (what its own backward produced) and the full bf16 parameter range; it owns 1/world of the range
// (its shard) for which it keeps fp32 master weights and the two Adam moments locally.
//
// Per 8 elements of its shard a thread does:
//   g      = multimem.ld_reduce(grad)            the switch sums all ranks' copies (reduce-scatter)
//   p,m,v  = AdamW(master, m, v, g / world)      fp32 state stays local and sharded
//   multimem.st(param_bf16, bf16(p))             the switch writes every rank's copy (all-gather)
// and, after the exit barrier, every rank clears its own copy of the unit's gradient range.
// Without NVLS the same dataflow uses plain peer loads and peer stores.
// NVLink traffic per rank and step: 4 B x shard in (reduced), 2 B x shard out (replicated by the
// switch) - the minimum for a reduce-scatter plus all-gather - and no separate NCCL kernels,
// no bucket copies, no second pass over the optimizer state.
//
// Two parameter placements share the kernel:
//   SHARD_GRAD_OP (AG = true)   every rank keeps a full bf16 copy; the kernel refreshes all copies as described above.
//   FULL_SHARD    (AG = false)  only the rank's own bf16 shard is resident (param_shard, local memory, indexed like the
//                               optimizer state); the kernel writes just that, and the next forward / backward
//                               un-shards the unit again (fsdp_gather.cuh, tb_fsdp_ag_gemm, tb_fsdp_unit_gather).
// A failed entry barrier (a peer late by more than the wait limit, or an error already recorded for this launch)
// makes the CTA return before it reads a gradient or touches any state; a failed exit barrier skips the gradient
// clear, because a peer may still be reading. The host finds the code in the status word after the step.
//
// AdamW arithmetic follows crates/torsh-optim/src/adam.rs:809-950 (decoupled decay first, both
// moments bias-corrected). The reference's FSDP "reduce-scatter" is all_reduce + slice followed by
// shard -= grad (crates/torsh-distributed/src/fsdp.rs:373-419).
#include <stdlib.h>

#include "comm.cuh"
#include "common.cuh"
#include "fsdp_gather.cuh"
#include "host_util.h"

namespace tb {

constexpr int FSDP_THREADS = 512;
constexpr int FSDP_MAX_BLOCKS = 320;  // one cross-rank barrier slot per CTA (the flag buffer has 320 slots)

struct FsdpArgs {
  PeerTable grads;   // symmetric fp32 gradient buffer (full flat range)
  PeerTable params;  // symmetric bf16 parameter buffer (full flat range)
  PeerTable flags;   // symmetric flag buffer
  char* grad_mc;     // multicast addresses (null: plain peer memory)
  char* param_mc;
  float* master;     // local shard state, indexed from 0
  float* exp_avg;
  float* exp_avg_sq;
  long unit_off;     // element offset of the unit inside the flat range
  long unit_len;     // elements in the unit (multiple of 8 * world)
  long state_off;    // element offset of this unit's shard inside the local shard arrays
  int rank, world;
  const uint32_t* epoch_ptr;
  float lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale;
  const float* dyn;  // optional device scalars (lr, bc1, bc2) for CUDA-graph replay
  __nv_bfloat16* param_shard;  // FULL_SHARD: local bf16 shard array, indexed like master (null: write every rank's full copy)
  int* status;
};

template <bool NVLS, bool AG>
// two CTAs per SM (at most 64 registers per thread): the whole-GPU launches of 2 x SM-count CTAs are resident at once
__global__ void __launch_bounds__(FSDP_THREADS, 2)
fsdp_rs_adamw_ag_kernel(FsdpArgs a) {
  const uint32_t epoch = *a.epoch_ptr;
  float lr = a.lr, bc1 = a.bc1, bc2 = a.bc2;
  if (a.dyn) {
    lr = a.dyn[0];
    bc1 = a.dyn[1];
    bc2 = a.dyn[2];
  }
  // peer base pointers in shared memory: indexing the kernel-parameter arrays with a run-time rank would move
  // them to local memory and put a local load in front of every peer access
  __shared__ const float* s_grads[MAX_RANKS];
  __shared__ __nv_bfloat16* s_params[MAX_RANKS];
#pragma unroll
  for (int i = 0; i < MAX_RANKS; ++i)
    if (threadIdx.x == i) {
      s_grads[i] = reinterpret_cast<const float*>(a.grads.ptr[i]);
      s_params[i] = reinterpret_cast<__nv_bfloat16*>(a.params.ptr[i]);
    }
  __syncthreads();
  // every rank's backward has finished writing this unit's gradients
  if (!cta_barrier_all_ranks(a.flags, blockIdx.x, a.rank, a.world, 2 * epoch, a.status)) return;
  const long shard = a.unit_len / a.world;
  const long g0 = a.unit_off + (long)a.rank * shard;  // my shard inside the flat range
  const long nvec = shard / 8;
  const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const long nthreads = (long)gridDim.x * blockDim.x;
  for (long v = tid; v < nvec; v += nthreads) {
    const long ge = g0 + v * 8;          // flat element index
    const long se = a.state_off + v * 8; // local state index
    float g[8];
    if (NVLS) {
      float4 x = multimem_ld_reduce_f32x4(a.grad_mc + ge * 4);
      float4 y = multimem_ld_reduce_f32x4(a.grad_mc + ge * 4 + 16);
      g[0] = x.x; g[1] = x.y; g[2] = x.z; g[3] = x.w; g[4] = y.x; g[5] = y.y; g[6] = y.z; g[7] = y.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] = 0.f;
      for (int p = 0; p < a.world; ++p) {
        const int q = (a.rank + p) % a.world;
        const float4* src = reinterpret_cast<const float4*>(s_grads[q] + ge);
        float4 x = src[0], y = src[1];
        g[0] += x.x; g[1] += x.y; g[2] += x.z; g[3] += x.w; g[4] += y.x; g[5] += y.y; g[6] += y.z; g[7] += y.w;
      }
    }
    float w[8], m[8], s[8];
    *reinterpret_cast<float4*>(w) = *reinterpret_cast<const float4*>(a.master + se);
    *reinterpret_cast<float4*>(w + 4) = *reinterpret_cast<const float4*>(a.master + se + 4);
    *reinterpret_cast<float4*>(m) = *reinterpret_cast<const float4*>(a.exp_avg + se);
    *reinterpret_cast<float4*>(m + 4) = *reinterpret_cast<const float4*>(a.exp_avg + se + 4);
    *reinterpret_cast<float4*>(s) = *reinterpret_cast<const float4*>(a.exp_avg_sq + se);
    *reinterpret_cast<float4*>(s + 4) = *reinterpret_cast<const float4*>(a.exp_avg_sq + se + 4);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gi = g[j] * a.grad_scale;
      float p = w[j];
      p -= lr * a.wd * p;
      m[j] = a.beta1 * m[j] + (1.f - a.beta1) * gi;
      s[j] = a.beta2 * s[j] + (1.f - a.beta2) * gi * gi;
      p -= lr * (m[j] / bc1) / (sqrtf(s[j] / bc2) + a.eps);
      w[j] = p;
    }
    *reinterpret_cast<float4*>(a.master + se) = *reinterpret_cast<float4*>(w);
    *reinterpret_cast<float4*>(a.master + se + 4) = *reinterpret_cast<float4*>(w + 4);
    *reinterpret_cast<float4*>(a.exp_avg + se) = *reinterpret_cast<float4*>(m);
    *reinterpret_cast<float4*>(a.exp_avg + se + 4) = *reinterpret_cast<float4*>(m + 4);
    *reinterpret_cast<float4*>(a.exp_avg_sq + se) = *reinterpret_cast<float4*>(s);
    *reinterpret_cast<float4*>(a.exp_avg_sq + se + 4) = *reinterpret_cast<float4*>(s + 4);
    const uint4 o = make_uint4(pack_bf16x2(w[0], w[1]), pack_bf16x2(w[2], w[3]), pack_bf16x2(w[4], w[5]),
                               pack_bf16x2(w[6], w[7]));
    if (!AG) {
      *reinterpret_cast<uint4*>(a.param_shard + se) = o;
    } else if (NVLS) {
      multimem_st_16(a.param_mc + ge * 2, o);
    } else {
      for (int p = 0; p < a.world; ++p) {
        const int q = (a.rank + p) % a.world;
        *reinterpret_cast<uint4*>(s_params[q] + ge) = o;
      }
    }
  }
  // all shards of the unit have been reduced everywhere and every parameter copy is complete
  if (!cta_barrier_all_ranks(a.flags, blockIdx.x, a.rank, a.world, 2 * epoch + 1, a.status)) return;
  // Clear my own copy of the gradient for the next accumulation. This CTA's exit barrier only proves
  // that the CTAs with the same index on the other ranks are done reading, so it clears exactly the
  // vectors those CTAs read: the same vector indices, in every rank's shard.
  float* gmine = const_cast<float*>(s_grads[a.rank]) + a.unit_off;
  for (int q = 0; q < a.world; ++q) {
    float4* gz = reinterpret_cast<float4*>(gmine + (long)q * shard);
    for (long v = tid; v < nvec; v += nthreads) {
      gz[2 * v] = make_float4(0.f, 0.f, 0.f, 0.f);
      gz[2 * v + 1] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
}

__global__ void fsdp_bump_epoch_kernel(uint32_t* e) { *e += 1; }

}  // namespace tb
using namespace tb;

// grads / params / flags: per-rank base pointers of the three symmetric buffers.
// unit_off, unit_len in elements; unit_len must be a multiple of 8 * world and unit_off of 8.
// master / exp_avg / exp_avg_sq: local fp32 shard arrays; this unit's shard starts at state_off.
// param_shard (may be null): local bf16 shard array indexed like master. When given, the refreshed parameters are
// written there only (FULL_SHARD) and `params` / `param_mc` are not used; `unit_off` then addresses the gradient
// buffer alone.
static int fsdp_step_launch(const void* const* grads, const void* const* params, const void* const* flags,
                            void* grad_mc, void* param_mc, float* master, float* exp_avg, float* exp_avg_sq,
                            void* param_shard, long unit_off, long unit_len, long state_off, int rank, int world,
                            const unsigned* epoch_ptr, float lr, float beta1, float beta2, float eps, float wd,
                            float bc1, float bc2, float grad_scale, const float* dyn, int nblocks, int* status,
                            cudaStream_t st, int threads = FSDP_THREADS) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) TB_FAIL(TB_E_ARG, "fsdp step: bad rank/world");
  if (threads < 64 || threads > FSDP_THREADS || threads % 32) TB_FAIL(TB_E_ARG, "fsdp step: threads per CTA must be a multiple of 32 in [64, 512]");
  if (unit_len % (8L * world) || unit_off % 8 || state_off % 8)
    TB_FAIL(TB_E_ARG, "fsdp step: unit_len (%ld) must be a multiple of 8*world, offsets of 8", unit_len);
  const bool full_shard = param_shard != nullptr;
  if (!full_shard && (grad_mc == nullptr) != (param_mc == nullptr))
    TB_FAIL(TB_E_ARG, "fsdp step: give both multicast addresses or none");
  FsdpArgs a;
  for (int i = 0; i < MAX_RANKS; ++i) {
    a.grads.ptr[i] = i < world ? const_cast<void*>(grads[i]) : nullptr;
    a.params.ptr[i] = (i < world && params) ? const_cast<void*>(params[i]) : nullptr;
    a.flags.ptr[i] = i < world ? const_cast<void*>(flags[i]) : nullptr;
  }
  a.grad_mc = static_cast<char*>(grad_mc);
  a.param_mc = static_cast<char*>(param_mc);
  a.master = master; a.exp_avg = exp_avg; a.exp_avg_sq = exp_avg_sq;
  a.unit_off = unit_off; a.unit_len = unit_len; a.state_off = state_off;
  a.rank = rank; a.world = world; a.epoch_ptr = epoch_ptr;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.wd = wd; a.bc1 = bc1; a.bc2 = bc2;
  a.grad_scale = grad_scale; a.dyn = dyn; a.status = status;
  a.param_shard = static_cast<__nv_bfloat16*>(param_shard);
  if (nblocks < 1) nblocks = 1;
  if (nblocks > FSDP_MAX_BLOCKS) nblocks = FSDP_MAX_BLOCKS;
  if (full_shard) {
    if (grad_mc) fsdp_rs_adamw_ag_kernel<true, false><<<nblocks, threads, 0, st>>>(a);
    else fsdp_rs_adamw_ag_kernel<false, false><<<nblocks, threads, 0, st>>>(a);
  } else {
    if (grad_mc) fsdp_rs_adamw_ag_kernel<true, true><<<nblocks, FSDP_THREADS, 0, st>>>(a);
    else fsdp_rs_adamw_ag_kernel<false, true><<<nblocks, FSDP_THREADS, 0, st>>>(a);
  }
  fsdp_bump_epoch_kernel<<<1, 1, 0, st>>>(const_cast<uint32_t*>(epoch_ptr));
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

TB_EXPORT int tb_fsdp_rs_adamw_ag(const void* const* grads, const void* const* params, const void* const* flags,
                                  void* grad_mc, void* param_mc, float* master, float* exp_avg, float* exp_avg_sq,
                                  long unit_off, long unit_len, long state_off, int rank, int world,
                                  const unsigned* epoch_ptr, float lr, float beta1, float beta2, float eps, float wd,
                                  float bc1, float bc2, float grad_scale, const float* dyn, int nblocks, int* status,
                                  cudaStream_t st) {
  TB_ENSURE_DEVICE();
  return fsdp_step_launch(grads, params, flags, grad_mc, param_mc, master, exp_avg, exp_avg_sq, nullptr, unit_off,
                          unit_len, state_off, rank, world, epoch_ptr, lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale,
                          dyn, nblocks, status, st);
}

// FULL_SHARD step of one unit: reduce-scatter of the unit's gradient (in the switch with grad_mc, else by peer loads)
// fused with AdamW on the rank's shard; the refreshed bf16 shard goes to param_shard[state_off ...] in local memory.
// grads: per-rank base pointers of the symmetric gradient workspace; the unit's gradient starts at element grad_off.
TB_EXPORT int tb_fsdp_rs_adamw(const void* const* grads, const void* const* flags, void* grad_mc, float* master,
                               float* exp_avg, float* exp_avg_sq, void* param_shard, long grad_off, long unit_len,
                               long state_off, int rank, int world, const unsigned* epoch_ptr, float lr, float beta1,
                               float beta2, float eps, float wd, float grad_scale, const float* dyn, int nblocks,
                               int threads, int* status, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (!param_shard) TB_FAIL(TB_E_ARG, "fsdp step: null parameter shard");
  // `threads` per CTA: small CTAs (128 threads = 8 K registers) fit next to the CTAs of the backward kernels they overlap
  return fsdp_step_launch(grads, nullptr, flags, grad_mc, nullptr, master, exp_avg, exp_avg_sq, param_shard, grad_off,
                          unit_len, state_off, rank, world, epoch_ptr, lr, beta1, beta2, eps, wd, 1.f, 1.f, grad_scale,
                          dyn, nblocks, status, st, threads > 0 ? threads : FSDP_THREADS);
}

namespace tb {
constexpr int GATHER_SMEM = 12 * GATHER_PIECE;
template <int PIECE>
__global__ void __launch_bounds__(32, 1) fsdp_unit_gather_kernel(const GatherArgs g) {
  extern __shared__ uint8_t gsm_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)gsm_raw + 127) & ~(uintptr_t)127);
  uint64_t* bars = (uint64_t*)(smem + GATHER_SMEM);
  volatile int* abort_flag = (volatile int*)(bars + 12);
  unit_gather_role<GATHER_SMEM, PIECE>(g, (int)blockIdx.x, smem, bars, abort_flag);
}
}  // namespace tb

int tb_fill_gather(tb::GatherArgs& g, const void* const* shards, void* unit_buf, const void* const* flag_bufs,
                   const unsigned* epoch_ptr, unsigned* ready, int chunk_bytes, int cpr, int first_chunk, int rank,
                   int world, int ctas, int* status);

// Stand-alone un-shard of one unit (no consuming GEMM in the same launch): `ctas` copy CTAs (one per SM at most)
// pull every rank's shard into unit_buf; arguments as in tb_fsdp_ag_gemm.
TB_EXPORT int tb_fsdp_unit_gather(const void* const* shards, void* unit_buf, const void* const* flag_bufs,
                                  const unsigned* epoch_ptr, unsigned* ready, int chunk_bytes, int cpr, int rank,
                                  int world, int ctas, int* status, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  GatherArgs g;
  if (ctas < 1) ctas = 64;
  if (ctas > 128) ctas = 128;
  if (int r = tb_fill_gather(g, shards, unit_buf, flag_bufs, epoch_ptr, ready, chunk_bytes, cpr, 0, rank, world, ctas, status))
    return r;
  static bool configured = false;
  constexpr int SMEM = GATHER_SMEM + 12 * 8 + 16 + 128;
  if (!configured) {
    TB_CUDA_CHECK(cudaFuncSetAttribute(fsdp_unit_gather_kernel<16384>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    TB_CUDA_CHECK(cudaFuncSetAttribute(fsdp_unit_gather_kernel<32768>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    TB_CUDA_CHECK(cudaFuncSetAttribute(fsdp_unit_gather_kernel<65536>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    configured = true;
  }
  // piece size of the copy ring (experiment knob: TB_GATHER_PIECE_KB = 16, 32 or 64)
  static const int piece_kb = [] { const char* e = getenv("TB_GATHER_PIECE_KB"); return e ? atoi(e) : 16; }();
  if (piece_kb == 64 && chunk_bytes % 65536 == 0) fsdp_unit_gather_kernel<65536><<<ctas, 32, SMEM, st>>>(g);
  else if (piece_kb == 32 && chunk_bytes % 32768 == 0) fsdp_unit_gather_kernel<32768><<<ctas, 32, SMEM, st>>>(g);
  else fsdp_unit_gather_kernel<16384><<<ctas, 32, SMEM, st>>>(g);
  fsdp_bump_epoch_kernel<<<1, 1, 0, st>>>(const_cast<uint32_t*>(epoch_ptr));
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
