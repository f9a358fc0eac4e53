// Shared device helpers for the memory-bound kernels: 16-byte vector access for
// bf16 / fp32, warp and block reductions, type conversion.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

namespace tb {

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16(v); }

// A 16-byte vector of T (8 bf16 or 4 fp32) with float views.
template <typename T> struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
  uint4 raw;
  __device__ __forceinline__ void load(const T* p) { raw = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void load_nc(const T* p) { raw = __ldg(reinterpret_cast<const uint4*>(p)); }
  __device__ __forceinline__ void store(T* p) const { *reinterpret_cast<uint4*>(p) = raw; }
  __device__ __forceinline__ void get(float (&f)[N]) const {
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < N; ++i) f[i] = to_f<T>(e[i]);
  }
  __device__ __forceinline__ void set(const float (&f)[N]) {
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < N; ++i) e[i] = from_f<T>(f[i]);
  }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide reductions; `scratch` holds >= 32 floats of shared memory. All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nw) ? scratch[lane] : 0.f;
  return warp_sum(r);
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nw) ? scratch[lane] : -FLT_MAX;
  return warp_max(r);
}

__host__ __device__ inline int ceil_div(long a, long b) { return (int)((a + b - 1) / b); }

}  // namespace tb

// ---------------------------------------------------------------- device-side index checks
// Kernels that index memory with values they read from tensors (token ids, class targets, expert slots, graph
// edges) never follow a bad index: they skip or clamp it. With checks enabled (TORSH_KERNEL_CHECKS=1 ->
// tb_set_kernel_checks) they also record TB_ERR_BAD_INDEX in the device status word, which the host turns into an
// exception at its next status read; there is no trap and no assert, the context stays usable. Every translation unit
// that includes this header has its own copy of the pointer; tb_set_kernel_checks sets them all.
#define TB_KERNEL_CHECK_WORD 1
namespace tb {
constexpr int TB_ERR_BAD_INDEX = 108;
static __device__ int* d_check_word = nullptr;
__device__ __forceinline__ void report_bad_index() {
  int* w = d_check_word;
  if (w) atomicCAS(w, 0, TB_ERR_BAD_INDEX);
}
// Host: point this translation unit's check word at `word` (null switches the reports off).
static inline cudaError_t set_check_word_this_tu(int* word) {
  return cudaMemcpyToSymbol(d_check_word, &word, sizeof(word));
}
}  // namespace tb
