// Device-resident elementwise kernels for sm_100a: unary / binary / scalar ops, fill, cast,
// GELU / SiLU / SwiGLU forward and backward, bias-column-sum, 2-D transpose.
//
// 16-byte vector accesses, grid sized to the SM count, no host round trips. They stand in for the
// reference's run-time generated f32 PTX (crates/torsh-tensor/src/cuda_backend/ptx_ops.rs:61-95,
// 203-282: unary relu/sigmoid/tanh/exp/log/sqrt/abs/neg, binary add/sub/mul/div/max/min), which
// pays two PCIe copies and a module load per call (crates/torsh-tensor/src/gpu_dispatch.rs:85-100),
// and for the empty launch stubs in crates/torsh-backend/src/cuda/kernels/mod.rs:20-330.
#include "common.cuh"
#include "host_util.h"
#include "sm100.cuh"

namespace tb {

enum UnaryOp { U_RELU = 0, U_SIGMOID, U_TANH, U_EXP, U_LOG, U_SQRT, U_ABS, U_NEG, U_GELU_TANH, U_SILU, U_GELU_ERF, U_RSQRT, U_SQUARE, U_COPY };
enum BinaryOp { B_ADD = 0, B_SUB, B_MUL, B_DIV, B_MAX, B_MIN, B_RELU_BWD, B_GELU_BWD, B_SILU_BWD, B_SIGMOID_BWD, B_TANH_BWD };

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float silu_grad(float x) {
  float s = 1.f / (1.f + __expf(-x));
  return s * (1.f + x * (1.f - s));
}

__device__ __forceinline__ float unary_apply(int op, float x, float alpha) {
  switch (op) {
    case U_RELU: return fmaxf(x, 0.f);
    case U_SIGMOID: return 1.f / (1.f + __expf(-x));
    case U_TANH: return tanhf(x);
    case U_EXP: return __expf(x);
    case U_LOG: return __logf(x);
    case U_SQRT: return sqrtf(x);
    case U_ABS: return fabsf(x);
    case U_NEG: return -x;
    case U_GELU_TANH: return gelu_tanh(x);
    case U_SILU: return silu(x);
    case U_GELU_ERF: return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
    case U_RSQRT: return rsqrtf(x);
    case U_SQUARE: return x * x;
    default: return x * alpha;  // U_COPY doubles as scalar multiply
  }
}
// For the *_BWD ops: a = upstream gradient, b = forward input (or output for sigmoid/tanh).
__device__ __forceinline__ float binary_apply(int op, float a, float b) {
  switch (op) {
    case B_ADD: return a + b;
    case B_SUB: return a - b;
    case B_MUL: return a * b;
    case B_DIV: return a / b;
    case B_MAX: return fmaxf(a, b);
    case B_MIN: return fminf(a, b);
    case B_RELU_BWD: return b > 0.f ? a : 0.f;
    case B_GELU_BWD: return a * gelu_tanh_grad(b);
    case B_SILU_BWD: return a * silu_grad(b);
    case B_SIGMOID_BWD: return a * b * (1.f - b);
    default: return a * (1.f - b * b);  // B_TANH_BWD
  }
}

template <typename T>
__global__ void unary_kernel(const T* __restrict__ x, T* __restrict__ y, long n, int op, float alpha) {
  constexpr int N = Vec16<T>::N;
  const long nvec = n / N;
  const long stride = (long)gridDim.x * blockDim.x;
  for (long v = (long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += stride) {
    Vec16<T> t;
    t.load(x + v * N);
    float f[N];
    t.get(f);
#pragma unroll
    for (int j = 0; j < N; ++j) f[j] = unary_apply(op, f[j], alpha);
    t.set(f);
    t.store(y + v * N);
  }
  for (long i = nvec * N + (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = from_f<T>(unary_apply(op, to_f<T>(x[i]), alpha));
}

// y = op(a, b); b_scalar != 0 broadcasts the single value *b... here passed by value in `sb`.
template <typename T>
__global__ void binary_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ y,
                              long n, int op, int use_scalar, float sb) {
  constexpr int N = Vec16<T>::N;
  const long nvec = n / N;
  const long stride = (long)gridDim.x * blockDim.x;
  for (long v = (long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += stride) {
    Vec16<T> ta, tb2;
    ta.load(a + v * N);
    float fa[N], fb[N];
    ta.get(fa);
    if (use_scalar) {
#pragma unroll
      for (int j = 0; j < N; ++j) fb[j] = sb;
    } else {
      tb2.load(b + v * N);
      tb2.get(fb);
    }
#pragma unroll
    for (int j = 0; j < N; ++j) fa[j] = binary_apply(op, fa[j], fb[j]);
    ta.set(fa);
    ta.store(y + v * N);
  }
  for (long i = nvec * N + (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = from_f<T>(binary_apply(op, to_f<T>(a[i]), use_scalar ? sb : to_f<T>(b[i])));
}

template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ x, TO* __restrict__ y, long n) {
  const long stride = (long)gridDim.x * blockDim.x;
  const long n4 = n / 4;
  for (long v = (long)blockIdx.x * blockDim.x + threadIdx.x; v < n4; v += stride) {
    float f[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) f[j] = to_f<TI>(x[v * 4 + j]);
#pragma unroll
    for (int j = 0; j < 4; ++j) y[v * 4 + j] = from_f<TO>(f[j]);
  }
  for (long i = n4 * 4 + (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = from_f<TO>(to_f<TI>(x[i]));
}

template <typename T>
__global__ void fill_kernel(T* __restrict__ y, long n, float value) {
  const long stride = (long)gridDim.x * blockDim.x;
  const T v = from_f<T>(value);
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) y[i] = v;
}

// SwiGLU over the last dim: x = [a | b] (each `half` wide); y = a * silu(b) — the gate is the
// SECOND half, as in crates/torsh-nn/src/layers/activation/gated.rs:536-608.
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, long rows, int half) {
  constexpr int N = Vec16<T>::N;
  const int hv = half / N;
  const long total = rows * hv;
  const long stride = (long)gridDim.x * blockDim.x;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    long r = idx / hv;
    int c = (int)(idx - r * hv) * N;
    Vec16<T> ta, tg;
    ta.load(x + r * 2 * half + c);
    tg.load(x + r * 2 * half + half + c);
    float fa[N], fg[N];
    ta.get(fa);
    tg.get(fg);
#pragma unroll
    for (int j = 0; j < N; ++j) fa[j] = fa[j] * silu(fg[j]);
    ta.set(fa);
    ta.store(y + r * half + c);
  }
}
template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                  T* __restrict__ dx, long rows, int half) {
  constexpr int N = Vec16<T>::N;
  const int hv = half / N;
  const long total = rows * hv;
  const long stride = (long)gridDim.x * blockDim.x;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    long r = idx / hv;
    int c = (int)(idx - r * hv) * N;
    Vec16<T> ta, tg, td;
    ta.load(x + r * 2 * half + c);
    tg.load(x + r * 2 * half + half + c);
    td.load(dy + r * half + c);
    float fa[N], fg[N], fd[N], da[N], dg[N];
    ta.get(fa);
    tg.get(fg);
    td.get(fd);
#pragma unroll
    for (int j = 0; j < N; ++j) {
      da[j] = fd[j] * silu(fg[j]);
      dg[j] = fd[j] * fa[j] * silu_grad(fg[j]);
    }
    ta.set(da);
    tg.set(dg);
    ta.store(dx + r * 2 * half + c);
    tg.store(dx + r * 2 * half + half + c);
  }
}

// out[c] += sum_r x[r, c] (fp32 accumulate, atomics across row blocks): bias gradients.
// Block = 32 x 8 threads: x-threads own one 16-byte vector of columns each, y-threads split the
// rows of the block; partial sums meet in shared memory, one atomic per column per block.
template <typename T>
__global__ void colsum_kernel(const T* __restrict__ x, float* __restrict__ out, long rows, int cols,
                              long ld, int rows_per_block) {
  constexpr int N = Vec16<T>::N;
  __shared__ float part[8][32 * N + 1];
  const int c0 = (blockIdx.x * 32 + threadIdx.x) * N;
  const long r0 = (long)blockIdx.y * rows_per_block;
  const long r1 = min(rows, r0 + rows_per_block);
  float acc[N];
#pragma unroll
  for (int j = 0; j < N; ++j) acc[j] = 0.f;
  const bool vec_ok = (c0 + N <= cols) && ((ld % N) == 0) && (((uintptr_t)x & 15) == 0);
  if (c0 < cols) {
    long r = r0 + threadIdx.y;
    if (vec_ok) {
      // eight, then four rows in flight per thread
      for (; r + 56 < r1; r += 64) {
        Vec16<T> t[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) t[u].load_nc(x + (r + 8 * u) * ld + c0);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          float f[N];
          t[u].get(f);
#pragma unroll
          for (int j = 0; j < N; ++j) acc[j] += f[j];
        }
      }
      for (; r + 24 < r1; r += 32) {
        Vec16<T> t[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) t[u].load_nc(x + (r + 8 * u) * ld + c0);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          float f[N];
          t[u].get(f);
#pragma unroll
          for (int j = 0; j < N; ++j) acc[j] += f[j];
        }
      }
    }
    for (; r < r1; r += 8) {
      if (vec_ok) {
        Vec16<T> t;
        t.load(x + r * ld + c0);
        float f[N];
        t.get(f);
#pragma unroll
        for (int j = 0; j < N; ++j) acc[j] += f[j];
      } else {
#pragma unroll
        for (int j = 0; j < N; ++j)
          if (c0 + j < cols) acc[j] += to_f<T>(x[r * ld + c0 + j]);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < N; ++j) part[threadIdx.y][threadIdx.x * N + j] = acc[j];
  __syncthreads();
  const int tid = threadIdx.y * 32 + threadIdx.x;
  for (int c = tid; c < 32 * N; c += 256) {
    const int col = blockIdx.x * 32 * N + c;
    if (col < cols) {
      float s = 0.f;
#pragma unroll
      for (int y = 0; y < 8; ++y) s += part[y][c];
      atomicAdd(out + col, s);
    }
  }
}

template <typename T>
__global__ void transpose_kernel(const T* __restrict__ x, T* __restrict__ y, int rows, int cols) {
  __shared__ T tile[32][33];
  int bx = blockIdx.x * 32, by = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int r = by + j, c = bx + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = x[(size_t)r * cols + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int r = bx + j, c = by + threadIdx.x;
    if (r < cols && c < rows) y[(size_t)r * rows + c] = tile[threadIdx.x][j];
  }
}

static inline int ew_grid(long work_items) {
  long b = (work_items + 255) / 256;
  long cap = (long)sm_count() * 16;
  return (int)(b < 1 ? 1 : (b < cap ? b : cap));
}

}  // namespace tb
using namespace tb;

// dtype: 0 = bf16, 1 = fp32
TB_EXPORT int tb_unary(const void* x, void* y, long n, int op, float alpha, int dtype, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (n <= 0) return 0;
  if (dtype == 0) unary_kernel<bf16><<<ew_grid(n / 8 + 1), 256, 0, st>>>((const bf16*)x, (bf16*)y, n, op, alpha);
  else unary_kernel<float><<<ew_grid(n / 4 + 1), 256, 0, st>>>((const float*)x, (float*)y, n, op, alpha);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
TB_EXPORT int tb_binary(const void* a, const void* b, void* y, long n, int op, int use_scalar,
                        float scalar, int dtype, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (n <= 0) return 0;
  if (dtype == 0) binary_kernel<bf16><<<ew_grid(n / 8 + 1), 256, 0, st>>>((const bf16*)a, (const bf16*)b, (bf16*)y, n, op, use_scalar, scalar);
  else binary_kernel<float><<<ew_grid(n / 4 + 1), 256, 0, st>>>((const float*)a, (const float*)b, (float*)y, n, op, use_scalar, scalar);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
// kind: 0 = f32 -> bf16, 1 = bf16 -> f32
TB_EXPORT int tb_cast(const void* x, void* y, long n, int kind, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (n <= 0) return 0;
  if (kind == 0) cast_kernel<float, bf16><<<ew_grid(n / 4 + 1), 256, 0, st>>>((const float*)x, (bf16*)y, n);
  else cast_kernel<bf16, float><<<ew_grid(n / 4 + 1), 256, 0, st>>>((const bf16*)x, (float*)y, n);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
TB_EXPORT int tb_fill(void* y, long n, float value, int dtype, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (n <= 0) return 0;
  if (dtype == 0) fill_kernel<bf16><<<ew_grid(n), 256, 0, st>>>((bf16*)y, n, value);
  else fill_kernel<float><<<ew_grid(n), 256, 0, st>>>((float*)y, n, value);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
TB_EXPORT int tb_swiglu_fwd(const void* x, void* y, long rows, int half, int dtype, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (rows <= 0) return 0;
  int N = dtype == 0 ? 8 : 4;
  if (half % N) TB_FAIL(TB_E_ARG, "swiglu: half width %d must be a multiple of %d", half, N);
  long total = rows * (half / N);
  if (dtype == 0) swiglu_fwd_kernel<bf16><<<ew_grid(total), 256, 0, st>>>((const bf16*)x, (bf16*)y, rows, half);
  else swiglu_fwd_kernel<float><<<ew_grid(total), 256, 0, st>>>((const float*)x, (float*)y, rows, half);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
TB_EXPORT int tb_swiglu_bwd(const void* dy, const void* x, void* dx, long rows, int half, int dtype, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (rows <= 0) return 0;
  int N = dtype == 0 ? 8 : 4;
  if (half % N) TB_FAIL(TB_E_ARG, "swiglu: half width %d must be a multiple of %d", half, N);
  long total = rows * (half / N);
  if (dtype == 0) swiglu_bwd_kernel<bf16><<<ew_grid(total), 256, 0, st>>>((const bf16*)dy, (const bf16*)x, (bf16*)dx, rows, half);
  else swiglu_bwd_kernel<float><<<ew_grid(total), 256, 0, st>>>((const float*)dy, (const float*)x, (float*)dx, rows, half);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
// out (fp32 [cols]) is ACCUMULATED into.
TB_EXPORT int tb_colsum(const void* x, float* out, long rows, int cols, long ld, int dtype, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (rows <= 0 || cols <= 0) return 0;
  const int N = dtype == 0 ? 8 : 4;
  const int cols_per_block = 32 * N;
  const int col_blocks = (cols + cols_per_block - 1) / cols_per_block;
  // enough row blocks for about six CTAs per SM (the loads of one thread cover 64 rows at a time), at least 64 rows each
  long want = (6L * sm_count() + col_blocks - 1) / col_blocks;
  long rpb = (rows + want - 1) / want;
  if (rpb < 64) rpb = 64;
  dim3 grid(col_blocks, (unsigned)((rows + rpb - 1) / rpb)), block(32, 8);
  if (dtype == 0) colsum_kernel<bf16><<<grid, block, 0, st>>>((const bf16*)x, out, rows, cols, ld, (int)rpb);
  else colsum_kernel<float><<<grid, block, 0, st>>>((const float*)x, out, rows, cols, ld, (int)rpb);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
TB_EXPORT int tb_transpose(const void* x, void* y, int rows, int cols, int dtype, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (rows <= 0 || cols <= 0) return 0;
  dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
  if (dtype == 0) transpose_kernel<bf16><<<grid, block, 0, st>>>((const bf16*)x, (bf16*)y, rows, cols);
  else transpose_kernel<float><<<grid, block, 0, st>>>((const float*)x, (float*)y, rows, cols);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
