// Gradient compression kernels (roles of crates/torsh-distributed/src/gradient_compression.rs: Quantization, SignSGD,
// Threshold sparsification), one pass over the gradient each:
//   int8 quantisation with one fp32 scale per chunk of 1024 values (symmetric, absmax / 127);
//   sign packing: 32 signs per word plus the mean absolute value as the single scale;
//   threshold sparsification: (index, value) pairs of |x| > thr compacted through one atomic counter per warp ballot.
#include "common.cuh"
#include "host_util.h"

namespace tb {

constexpr int QCHUNK = 1024;

template <typename T>
__global__ void quant_int8_kernel(const T* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ scales, long n) {
  __shared__ float red[32];
  const long c0 = (long)blockIdx.x * QCHUNK;
  float v[4], amax = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long idx = c0 + threadIdx.x + i * 256;
    v[i] = idx < n ? to_f<T>(x[idx]) : 0.f;
    amax = fmaxf(amax, fabsf(v[i]));
  }
  amax = block_max(amax, red);
  const float scale = amax > 0.f ? amax / 127.f : 1.f;
  if (threadIdx.x == 0) scales[blockIdx.x] = scale;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long idx = c0 + threadIdx.x + i * 256;
    if (idx < n) q[idx] = (int8_t)max(-127, min(127, __float2int_rn(v[i] / scale)));
  }
}
template <typename T>
__global__ void dequant_int8_kernel(const int8_t* __restrict__ q, const float* __restrict__ scales, T* __restrict__ y, long n) {
  const long stride = (long)gridDim.x * blockDim.x;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) y[i] = from_f<T>((float)q[i] * scales[i / QCHUNK]);
}

template <typename T>
__global__ void sign_pack_kernel(const T* __restrict__ x, uint32_t* __restrict__ bits, float* __restrict__ abs_sum, long n) {
  __shared__ float red[32];
  const long stride = (long)gridDim.x * blockDim.x;
  float s = 0.f;
  const long nround = (n + 31) / 32 * 32;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nround; i += stride) {
    const float v = i < n ? to_f<T>(x[i]) : 0.f;
    s += fabsf(v);
    const uint32_t b = __ballot_sync(0xffffffffu, i < n && v >= 0.f);
    if ((threadIdx.x & 31) == 0) bits[i >> 5] = b;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) atomicAdd(abs_sum, s);
}
template <typename T>
__global__ void sign_unpack_kernel(const uint32_t* __restrict__ bits, const float* __restrict__ abs_sum, T* __restrict__ y,
                                   long n) {
  const float scale = *abs_sum / (float)n;
  const long stride = (long)gridDim.x * blockDim.x;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = from_f<T>(((bits[i >> 5] >> (i & 31)) & 1u) ? scale : -scale);
}

template <typename T>
__global__ void threshold_kernel(const T* __restrict__ x, float thr, int* __restrict__ idx, float* __restrict__ vals,
                                 int* __restrict__ count, int capacity, long n) {
  const long stride = (long)gridDim.x * blockDim.x;
  const long nround = (n + 31) / 32 * 32;
  const int lane = threadIdx.x & 31;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nround; i += stride) {
    const float v = i < n ? to_f<T>(x[i]) : 0.f;
    const bool keep = i < n && fabsf(v) > thr;
    const uint32_t m = __ballot_sync(0xffffffffu, keep);
    int base = 0;
    if (lane == 0 && m) base = atomicAdd(count, __popc(m));
    base = __shfl_sync(0xffffffffu, base, 0);
    if (keep) {
      const int pos = base + __popc(m & ((1u << lane) - 1u));
      if (pos < capacity) {
        idx[pos] = (int)i;
        vals[pos] = v;
      }
    }
  }
}

static inline int cgrid(long n) {
  long b = (n + 255) / 256;
  long cap = (long)sm_count() * 8;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace tb
using namespace tb;

// dtype 0 bf16, 1 fp32. scales: fp32 [ceil(n / 1024)].
TB_EXPORT int tb_quantize_int8(const void* x, void* q, float* scales, long n, int dtype, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (n <= 0) return 0;
  const int blocks = (int)((n + QCHUNK - 1) / QCHUNK);
  if (dtype == 0) quant_int8_kernel<bf16><<<blocks, 256, 0, st>>>((const bf16*)x, (int8_t*)q, scales, n);
  else quant_int8_kernel<float><<<blocks, 256, 0, st>>>((const float*)x, (int8_t*)q, scales, n);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
TB_EXPORT int tb_dequantize_int8(const void* q, const float* scales, void* y, long n, int dtype, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (n <= 0) return 0;
  if (dtype == 0) dequant_int8_kernel<bf16><<<cgrid(n), 256, 0, st>>>((const int8_t*)q, scales, (bf16*)y, n);
  else dequant_int8_kernel<float><<<cgrid(n), 256, 0, st>>>((const int8_t*)q, scales, (float*)y, n);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
// bits: uint32 [ceil(n / 32)]; abs_sum: fp32 [1], zeroed here, holds sum |x| afterwards.
TB_EXPORT int tb_sign_pack(const void* x, void* bits, float* abs_sum, long n, int dtype, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (n <= 0) return 0;
  TB_CUDA_CHECK(cudaMemsetAsync(abs_sum, 0, sizeof(float), st));
  if (dtype == 0) sign_pack_kernel<bf16><<<cgrid(n), 256, 0, st>>>((const bf16*)x, (uint32_t*)bits, abs_sum, n);
  else sign_pack_kernel<float><<<cgrid(n), 256, 0, st>>>((const float*)x, (uint32_t*)bits, abs_sum, n);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
TB_EXPORT int tb_sign_unpack(const void* bits, const float* abs_sum, void* y, long n, int dtype, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (n <= 0) return 0;
  if (dtype == 0) sign_unpack_kernel<bf16><<<cgrid(n), 256, 0, st>>>((const uint32_t*)bits, abs_sum, (bf16*)y, n);
  else sign_unpack_kernel<float><<<cgrid(n), 256, 0, st>>>((const uint32_t*)bits, abs_sum, (float*)y, n);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
// idx / vals hold up to `capacity` entries; count (int32 [1], zeroed here) receives the number of values above the
// threshold, which may exceed the capacity (the surplus is dropped).
TB_EXPORT int tb_threshold_sparsify(const void* x, float thr, int* idx, float* vals, int* count, int capacity, long n,
                                    int dtype, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (n <= 0) return 0;
  if (n >= (1L << 31)) TB_FAIL(TB_E_TOO_LARGE, "threshold_sparsify: at most 2^31 - 1 elements");
  TB_CUDA_CHECK(cudaMemsetAsync(count, 0, sizeof(int), st));
  if (dtype == 0) threshold_kernel<bf16><<<cgrid(n), 256, 0, st>>>((const bf16*)x, thr, idx, vals, count, capacity, n);
  else threshold_kernel<float><<<cgrid(n), 256, 0, st>>>((const float*)x, thr, idx, vals, count, capacity, n);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
