// Row softmax / log-softmax (forward, backward) and fused cross-entropy for sm_100a.
//
// One CTA per row. The row is staged once into shared memory (up to ~200 KB, e.g. a
// 50 304-wide bf16 vocabulary row is 100 KB) so HBM sees one read and one write per element;
// wider rows fall back to re-reading global memory. All statistics are fp32.
//
// The cross-entropy kernel produces the per-row loss and, in the same pass, the gradient
// (softmax - onehot) * scale, optionally in place over the logits. The reference computes
// cross_entropy as log_softmax + one-hot NLL with seven temporaries
// (crates/torsh-nn/src/functional/loss.rs:15-60, crates/torsh-tensor/src/advanced_ops.rs:1045-1090).
#include "common.cuh"
#include "host_util.h"

namespace tb {

constexpr int SM_THREADS = 512;
constexpr int SM_MAX_CACHE_BYTES = 200 * 1024;

template <typename T, bool CACHE>
__device__ __forceinline__ float row_get(const T* g, const T* s, int i) {
  return to_f<T>(CACHE ? s[i] : g[i]);
}

// Loads row into smem (if CACHE) and returns the row maximum over [0, C).
template <typename T, bool CACHE>
__device__ __forceinline__ float load_row_max(const T* __restrict__ xr, T* srow, int C,
                                              float* scratch) {
  constexpr int N = Vec16<T>::N;
  float m = -FLT_MAX;
  const bool vec_ok = ((uintptr_t)xr & 15) == 0;
  const int nvec = vec_ok ? C / N : 0;
  // four 16-byte loads in flight per thread: with one, a 512-thread CTA keeps 8 KB outstanding and two such CTAs per SM
  // cannot cover the memory latency (the kernel then ran at 0.40 of the copy bandwidth)
  int v = threadIdx.x;
  const int bd = blockDim.x;
  for (; v + 3 * bd < nvec; v += 4 * bd) {
    Vec16<T> t[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) t[u].load(xr + (size_t)(v + u * bd) * N);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (CACHE) t[u].store(srow + (v + u * bd) * N);
      float f[N];
      t[u].get(f);
#pragma unroll
      for (int j = 0; j < N; ++j) m = fmaxf(m, f[j]);
    }
  }
  for (; v < nvec; v += bd) {
    Vec16<T> t;
    t.load(xr + (size_t)v * N);
    if (CACHE) t.store(srow + v * N);
    float f[N];
    t.get(f);
#pragma unroll
    for (int j = 0; j < N; ++j) m = fmaxf(m, f[j]);
  }
  for (int i = nvec * N + threadIdx.x; i < C; i += blockDim.x) {
    T e = xr[i];
    if (CACHE) srow[i] = e;
    m = fmaxf(m, to_f<T>(e));
  }
  m = block_max(m, scratch);  // includes the __syncthreads that publishes srow
  return m;
}

template <typename T, bool CACHE, bool LOG>
__global__ void __launch_bounds__(SM_THREADS)
softmax_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int rows, int C, long ldx, long ldy) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __shared__ float scratch[32];
  T* srow = reinterpret_cast<T*>(smem_raw);
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + (size_t)row * ldx;
    T* yr = y + (size_t)row * ldy;
    float m = load_row_max<T, CACHE>(xr, srow, C, scratch);
    float s = 0.f;
    for (int i = threadIdx.x; i < C; i += blockDim.x) s += __expf(row_get<T, CACHE>(xr, srow, i) - m);
    s = block_sum(s, scratch);
    const float lse = m + __logf(s);
    const float inv = 1.f / s;
    for (int i = threadIdx.x; i < C; i += blockDim.x) {
      float v = row_get<T, CACHE>(xr, srow, i);
      yr[i] = from_f<T>(LOG ? (v - lse) : __expf(v - m) * inv);
    }
    __syncthreads();
  }
}

// softmax:      dx = y * (dy - sum(dy * y));  log_softmax: dx = dy - exp(y) * sum(dy)
template <typename T, bool LOG>
__global__ void __launch_bounds__(SM_THREADS)
softmax_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ y, T* __restrict__ dx, int rows,
                   int C) {
  __shared__ float scratch[32];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* dyr = dy + (size_t)row * C;
    const T* yr = y + (size_t)row * C;
    float s = 0.f;
    for (int i = threadIdx.x; i < C; i += blockDim.x)
      s += LOG ? to_f<T>(dyr[i]) : to_f<T>(dyr[i]) * to_f<T>(yr[i]);
    s = block_sum(s, scratch);
    for (int i = threadIdx.x; i < C; i += blockDim.x) {
      float d = to_f<T>(dyr[i]), yy = to_f<T>(yr[i]);
      dx[(size_t)row * C + i] = from_f<T>(LOG ? (d - __expf(yy) * s) : yy * (d - s));
    }
  }
}

// Fused cross-entropy. logits [rows, ld] with C valid classes (columns C..ld-1 are padding and get
// zero gradient). loss_rows[row] = lse - logit[target] (0 for ignored rows). When dlogits != null
// it receives (softmax - onehot) * scale, `scale` typically 1 / number_of_counted_rows.
template <typename T, bool CACHE>
__global__ void __launch_bounds__(SM_THREADS)
xent_kernel(const T* __restrict__ logits, const long* __restrict__ targets,
            float* __restrict__ loss_rows, float* __restrict__ lse_rows, T* __restrict__ dlogits,
            int rows, int C, long ld, float scale, long ignore_index) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __shared__ float scratch[32];
  T* srow = reinterpret_cast<T*>(smem_raw);
  constexpr int N = Vec16<T>::N;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = logits + (size_t)row * ld;
    const long tgt = targets[row];
    const bool ignored = (tgt == ignore_index) || tgt < 0 || tgt >= C;
    if (ignored && tgt != ignore_index && threadIdx.x == 0) report_bad_index();   // a target outside [0, C) that is not the ignore value
    float m = load_row_max<T, CACHE>(xr, srow, C, scratch);
    float s = 0.f;
    {
      // the staged row is read back 16 bytes at a time (the row start is 16-byte aligned in shared memory)
      const int nv = CACHE ? C / N : 0;
      for (int v = threadIdx.x; v < nv; v += blockDim.x) {
        Vec16<T> t;
        t.load(srow + v * N);
        float f[N];
        t.get(f);
#pragma unroll
        for (int j = 0; j < N; ++j) s += __expf(f[j] - m);
      }
      for (int i = nv * N + threadIdx.x; i < C; i += blockDim.x) s += __expf(row_get<T, CACHE>(xr, srow, i) - m);
    }
    s = block_sum(s, scratch);
    const float lse = m + __logf(s);
    if (threadIdx.x == 0) {
      float xt = ignored ? lse : row_get<T, CACHE>(xr, srow, (int)tgt);
      loss_rows[row] = lse - xt;
      if (lse_rows) lse_rows[row] = lse;
    }
    if (!CACHE) __syncthreads();  // the target logit is read before an in-place gradient overwrites it
    if (dlogits) {
      T* dr = dlogits + (size_t)row * ld;
      const float sc = ignored ? 0.f : scale;
      const bool vec_ok = (((uintptr_t)dr & 15) == 0) && CACHE;
      const int nvec = vec_ok ? (int)(ld / N) : 0;
      for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
        float o[N];
#pragma unroll
        for (int j = 0; j < N; ++j) {
          int i = v * N + j;
          float p = (i < C) ? __expf(to_f<T>(srow[i]) - lse) : 0.f;
          if (i == tgt) p -= 1.f;
          o[j] = p * sc;
        }
        Vec16<T> t;
        t.set(o);
        t.store(dr + v * N);
      }
      for (int i = nvec * N + threadIdx.x; i < ld; i += blockDim.x) {
        float p = (i < C) ? __expf(row_get<T, CACHE>(xr, srow, i) - lse) : 0.f;
        if (i == tgt) p -= 1.f;
        dr[i] = from_f<T>(p * sc);
      }
    }
    __syncthreads();
  }
}

template <typename K>
static int set_smem(K kern, size_t bytes) {
  if (bytes > 48 * 1024) TB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return 0;
}

template <typename T>
static int softmax_fwd_launch(const void* x, void* y, int rows, int C, long ldx, long ldy, int log,
                              cudaStream_t st) {
  size_t bytes = (size_t)C * sizeof(T);
  bool cache = bytes <= SM_MAX_CACHE_BYTES;
  int grid = rows < sm_count() * 4 ? rows : sm_count() * 4;
  int threads = C >= 4096 ? SM_THREADS : (C >= 1024 ? 256 : 128);
  size_t smem = cache ? ((bytes + 15) / 16 * 16) : 0;
#define TB_SF(CACHE_, LOG_)                                                                        \
  {                                                                                                \
    auto k = softmax_fwd_kernel<T, CACHE_, LOG_>;                                                  \
    if (int r = set_smem(k, smem)) return r;                                                       \
    k<<<grid, threads, smem, st>>>((const T*)x, (T*)y, rows, C, ldx, ldy);                         \
  }
  if (cache) { if (log) TB_SF(true, true) else TB_SF(true, false) }
  else { if (log) TB_SF(false, true) else TB_SF(false, false) }
#undef TB_SF
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

template <typename T>
static int xent_launch(const void* logits, const long* targets, float* loss_rows, float* lse_rows,
                       void* dlogits, int rows, int C, long ld, float scale, long ignore_index,
                       cudaStream_t st) {
  size_t bytes = (size_t)C * sizeof(T);
  bool cache = bytes <= SM_MAX_CACHE_BYTES;
  int grid = rows < sm_count() * 4 ? rows : sm_count() * 4;
  int threads = C >= 4096 ? SM_THREADS : (C >= 1024 ? 256 : 128);
  size_t smem = cache ? ((bytes + 15) / 16 * 16) : 0;
  if (cache) {
    auto k = xent_kernel<T, true>;
    if (int r = set_smem(k, smem)) return r;
    k<<<grid, threads, smem, st>>>((const T*)logits, targets, loss_rows, lse_rows, (T*)dlogits, rows, C, ld, scale, ignore_index);
  } else {
    auto k = xent_kernel<T, false>;
    k<<<grid, threads, 0, st>>>((const T*)logits, targets, loss_rows, lse_rows, (T*)dlogits, rows, C, ld, scale, ignore_index);
  }
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

}  // namespace tb
using namespace tb;

// dtype: 0 = bf16, 1 = fp32. ldx / ldy are row strides in elements.
TB_EXPORT int tb_softmax_fwd(const void* x, void* y, int rows, int C, long ldx, long ldy, int log,
                             int dtype, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (rows <= 0 || C <= 0) return 0;
  return dtype == 0 ? softmax_fwd_launch<bf16>(x, y, rows, C, ldx, ldy, log, st)
                    : softmax_fwd_launch<float>(x, y, rows, C, ldx, ldy, log, st);
}

TB_EXPORT int tb_softmax_bwd(const void* dy, const void* y, void* dx, int rows, int C, int log,
                             int dtype, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (rows <= 0 || C <= 0) return 0;
  int grid = rows < sm_count() * 8 ? rows : sm_count() * 8;
  int threads = C >= 4096 ? SM_THREADS : (C >= 1024 ? 256 : 128);
  if (dtype == 0) {
    if (log) softmax_bwd_kernel<bf16, true><<<grid, threads, 0, st>>>((const bf16*)dy, (const bf16*)y, (bf16*)dx, rows, C);
    else softmax_bwd_kernel<bf16, false><<<grid, threads, 0, st>>>((const bf16*)dy, (const bf16*)y, (bf16*)dx, rows, C);
  } else {
    if (log) softmax_bwd_kernel<float, true><<<grid, threads, 0, st>>>((const float*)dy, (const float*)y, (float*)dx, rows, C);
    else softmax_bwd_kernel<float, false><<<grid, threads, 0, st>>>((const float*)dy, (const float*)y, (float*)dx, rows, C);
  }
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// Fused cross-entropy forward (+ backward when dlogits != null; dlogits may alias logits).
TB_EXPORT int tb_cross_entropy(const void* logits, const long* targets, float* loss_rows,
                               float* lse_rows, void* dlogits, int rows, int C, long ld, float scale,
                               long ignore_index, int dtype, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (rows <= 0 || C <= 0) return 0;
  if (ld < C) TB_FAIL(TB_E_ARG, "tb_cross_entropy: ld (%ld) < C (%d)", ld, C);
  return dtype == 0 ? xent_launch<bf16>(logits, targets, loss_rows, lse_rows, dlogits, rows, C, ld, scale, ignore_index, st)
                    : xent_launch<float>(logits, targets, loss_rows, lse_rows, dlogits, rows, C, ld, scale, ignore_index, st);
}

int tb_set_check_word_xent(int* word) {
  TB_CUDA_CHECK(tb::set_check_word_this_tu(word));
  return 0;
}
