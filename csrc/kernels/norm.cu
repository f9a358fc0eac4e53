// LayerNorm and RMSNorm forward / backward for sm_100a.
//
// One CTA walks rows (grid-stride); each thread owns up to VPT 16-byte vectors of the row and
// keeps them in registers, so every element is read from HBM exactly once per pass. Row
// statistics use two block reductions (mean, then centred variance) for accuracy. The backward
// keeps per-thread fp32 partial sums of d(gamma) / d(beta) for its own columns across all rows of
// the CTA and flushes them once with atomics into fp32 gradient buffers.
//
// Semantics follow the reference layers: LayerNorm eps 1e-5 (biased variance) and
// RMSNorm y = x / sqrt(mean(x^2) + eps) * w with eps 1e-6
// (crates/torsh-nn/src/layers/normalization/layer_group/mod.rs:491-514,539-623).
#include "common.cuh"
#include "host_util.h"

namespace tb {

template <typename T, int VPT, bool RMS>
__global__ void norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gamma,
                                const T* __restrict__ beta, T* __restrict__ y,
                                float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows,
                                int H, float eps) {
  constexpr int N = Vec16<T>::N;
  __shared__ float scratch[32];
  const int nvec = H / N;
  Vec16<T> g[VPT], b[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      g[i].load_nc(gamma + v * N);
      if (!RMS && beta) b[i].load_nc(beta + v * N);
    }
  }
  // the next row's vectors are requested before this row's reductions, so their latency hides behind the block sums
  Vec16<T> nxt[VPT];
  if ((int)blockIdx.x < rows) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) nxt[i].load(x + (size_t)blockIdx.x * H + v * N);
    }
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    float f[VPT][N];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        nxt[i].get(f[i]);
#pragma unroll
        for (int j = 0; j < N; ++j) s += RMS ? f[i][j] * f[i][j] : f[i][j];
      }
    }
    if (row + (int)gridDim.x < rows) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) nxt[i].load(x + (size_t)(row + gridDim.x) * H + v * N);
      }
    }
    float mean = 0.f, rstd;
    if (RMS) {
      float ms = block_sum(s, scratch) / H;
      rstd = rsqrtf(ms + eps);
    } else {
      mean = block_sum(s, scratch) / H;
      float sq = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) {
#pragma unroll
          for (int j = 0; j < N; ++j) {
            float d = f[i][j] - mean;
            sq += d * d;
          }
        }
      }
      float var = block_sum(sq, scratch) / H;
      rstd = rsqrtf(var + eps);
    }
    if (threadIdx.x == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
    T* yr = y + (size_t)row * H;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        float gf[N], bf[N], o[N];
        g[i].get(gf);
        if (!RMS && beta) b[i].get(bf);
#pragma unroll
        for (int j = 0; j < N; ++j) {
          float xh = (f[i][j] - mean) * rstd;
          o[j] = xh * gf[j] + ((!RMS && beta) ? bf[j] : 0.f);
        }
        Vec16<T> t;
        t.set(o);
        t.store(yr + v * N);
      }
    }
  }
}

// dx = rstd * (dy*g - mean(dy*g) - xhat * mean(dy*g*xhat))      (LayerNorm)
// dx = rstd * (dy*g - xhat * mean(dy*g*xhat))                   (RMSNorm, xhat = x*rstd)
// Optionally dx += dres (gradient arriving through the residual branch).
template <typename T, int VPT, bool RMS>
__global__ void norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                const T* __restrict__ gamma, const float* __restrict__ mean_in,
                                const float* __restrict__ rstd_in, const T* __restrict__ dres,
                                T* __restrict__ dx, float* __restrict__ dgamma,
                                float* __restrict__ dbeta, float* __restrict__ partial, int rows, int H) {
  constexpr int N = Vec16<T>::N;
  __shared__ float scratch[32];
  const int nvec = H / N;
  float gf[VPT][N], dg[VPT][N], db[VPT][N];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    int v = threadIdx.x + i * blockDim.x;
#pragma unroll
    for (int j = 0; j < N; ++j) dg[i][j] = db[i][j] = gf[i][j] = 0.f;
    if (v < nvec) {
      Vec16<T> t;
      t.load_nc(gamma + v * N);
      t.get(gf[i]);
    }
  }
  // the next row's vectors are requested before this row's reductions, so their latency hides behind the block sums
  Vec16<T> nx[VPT], nd[VPT], nr[VPT];
  auto request = [&](int row) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        nx[i].load(x + (size_t)row * H + v * N);
        nd[i].load(dy + (size_t)row * H + v * N);
        if (dres) nr[i].load(dres + (size_t)row * H + v * N);
      }
    }
  };
  if ((int)blockIdx.x < rows) request(blockIdx.x);
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float mean = RMS ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    float xh[VPT][N], dyg[VPT][N], res[VPT][N];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        float xf[N], df[N];
        nx[i].get(xf);
        nd[i].get(df);
        if (dres) nr[i].get(res[i]);
#pragma unroll
        for (int j = 0; j < N; ++j) {
          xh[i][j] = (xf[j] - mean) * rstd;
          dyg[i][j] = df[j] * gf[i][j];
          dg[i][j] += df[j] * xh[i][j];
          db[i][j] += df[j];
          s1 += dyg[i][j];
          s2 += dyg[i][j] * xh[i][j];
        }
      }
    }
    if (row + (int)gridDim.x < rows) request(row + gridDim.x);
    if (!RMS) s1 = block_sum(s1, scratch) / H; else s1 = 0.f;
    s2 = block_sum(s2, scratch) / H;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        float o[N];
#pragma unroll
        for (int j = 0; j < N; ++j) o[j] = dres ? res[i][j] : 0.f;
#pragma unroll
        for (int j = 0; j < N; ++j) o[j] += rstd * (dyg[i][j] - s1 - xh[i][j] * s2);
        Vec16<T> t;
        t.set(o);
        t.store(dx + (size_t)row * H + v * N);
      }
    }
  }
  // Per-CTA partial sums: written to the workspace (reduced by norm_bwd_reduce_kernel, no atomic
  // contention) or, without a workspace, added straight into the gradient with atomics.
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      if (partial) {
        float* pg = partial + (size_t)blockIdx.x * 2 * H + v * N;
#pragma unroll
        for (int j = 0; j < N; j += 4) {
          *reinterpret_cast<float4*>(pg + j) = make_float4(dg[i][j], dg[i][j + 1], dg[i][j + 2], dg[i][j + 3]);
          if (!RMS) *reinterpret_cast<float4*>(pg + H + j) = make_float4(db[i][j], db[i][j + 1], db[i][j + 2], db[i][j + 3]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < N; ++j) {
          if (dgamma) atomicAdd(dgamma + v * N + j, dg[i][j]);
          if (!RMS && dbeta) atomicAdd(dbeta + v * N + j, db[i][j]);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Warp-per-row forms for rows of at most 32 * VPL 16-byte vectors (H <= 2048 bf16, 1024 fp32). A warp owns a row: its
// statistics are two shuffle reductions with no block barrier, eight rows are in flight per CTA and the next row of
// every warp is requested before the current one is reduced. With one CTA per row a 2 KB row left too few bytes in
// flight per SM and two block barriers per row on the critical path (0.43 of the copy bandwidth at 32768 x 1024).
constexpr int NORM_WARPS = 8;

template <typename T, int VPL, bool RMS>
__global__ void __launch_bounds__(NORM_WARPS * 32, VPL <= 4 ? 2 : 1) norm_fwd_warp_kernel(
    const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta, T* __restrict__ y,
    float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int H, float eps) {
  constexpr int N = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int nvec = H / N;
  const int nwarps = gridDim.x * NORM_WARPS;
  Vec16<T> g[VPL], b[VPL], nxt[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int v = lane + 32 * i;
    if (v < nvec) {
      g[i].load_nc(gamma + v * N);
      if (!RMS && beta) b[i].load_nc(beta + v * N);
    }
  }
  int row = blockIdx.x * NORM_WARPS + (threadIdx.x >> 5);
  if (row < rows) {
#pragma unroll
    for (int i = 0; i < VPL; ++i)
      if (lane + 32 * i < nvec) nxt[i].load(x + (size_t)row * H + (lane + 32 * i) * N);
  }
  const float inv_h = 1.f / (float)H;
  for (; row < rows; row += nwarps) {
    float f[VPL][N];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      if (lane + 32 * i < nvec) {
        nxt[i].get(f[i]);
#pragma unroll
        for (int j = 0; j < N; ++j) s += RMS ? f[i][j] * f[i][j] : f[i][j];
      }
    }
    if (row + nwarps < rows) {
#pragma unroll
      for (int i = 0; i < VPL; ++i)
        if (lane + 32 * i < nvec) nxt[i].load(x + (size_t)(row + nwarps) * H + (lane + 32 * i) * N);
    }
    float mean = 0.f, rstd;
    if (RMS) {
      rstd = rsqrtf(warp_sum(s) * inv_h + eps);
    } else {
      mean = warp_sum(s) * inv_h;
      float sq = 0.f;
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        if (lane + 32 * i < nvec) {
#pragma unroll
          for (int j = 0; j < N; ++j) {
            const float d = f[i][j] - mean;
            sq += d * d;
          }
        }
      }
      rstd = rsqrtf(warp_sum(sq) * inv_h + eps);
    }
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
    T* yr = y + (size_t)row * H;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        float gf[N], bf[N], o[N];
        g[i].get(gf);
        if (!RMS && beta) b[i].get(bf);
#pragma unroll
        for (int j = 0; j < N; ++j) {
          o[j] = (f[i][j] - mean) * rstd * gf[j];
          if (!RMS && beta) o[j] += bf[j];
        }
        Vec16<T> t;
        t.set(o);
        t.store(yr + v * N);
      }
    }
  }
}

// Same arithmetic as norm_bwd_kernel. Every lane keeps fp32 partial sums of d(gamma) / d(beta) for its own columns
// over all rows of its warp; the CTA's eight warps then add theirs in shared memory (2 * H floats) and the CTA writes
// one partial row of the workspace (or adds into the gradients with atomics when there is none).
template <typename T, int VPL, bool RMS>
__global__ void __launch_bounds__(NORM_WARPS * 32) norm_bwd_warp_kernel(
    const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma, const float* __restrict__ mean_in,
    const float* __restrict__ rstd_in, const T* __restrict__ dres, T* __restrict__ dx, float* __restrict__ dgamma,
    float* __restrict__ dbeta, float* __restrict__ partial, int rows, int H) {
  constexpr int N = Vec16<T>::N;
  extern __shared__ float nb_sums[];  // [2][H]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = H / N;
  const int nwarps = gridDim.x * NORM_WARPS;
  float gf[VPL][N], dg[VPL][N], db[VPL][N];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
#pragma unroll
    for (int j = 0; j < N; ++j) dg[i][j] = db[i][j] = gf[i][j] = 0.f;
    if (lane + 32 * i < nvec) {
      Vec16<T> t;
      t.load_nc(gamma + (lane + 32 * i) * N);
      t.get(gf[i]);
    }
  }
  Vec16<T> nx[VPL], nd[VPL], nr[VPL];
  auto request = [&](int r) {
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        nx[i].load(x + (size_t)r * H + v * N);
        nd[i].load(dy + (size_t)r * H + v * N);
        if (dres) nr[i].load(dres + (size_t)r * H + v * N);
      }
    }
  };
  int row = blockIdx.x * NORM_WARPS + warp;
  if (row < rows) request(row);
  const float inv_h = 1.f / (float)H;
  for (; row < rows; row += nwarps) {
    const float mean = RMS ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    float xh[VPL][N], dyg[VPL][N], res[VPL][N];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      if (lane + 32 * i < nvec) {
        float xf[N], df[N];
        nx[i].get(xf);
        nd[i].get(df);
        if (dres) nr[i].get(res[i]);
#pragma unroll
        for (int j = 0; j < N; ++j) {
          xh[i][j] = (xf[j] - mean) * rstd;
          dyg[i][j] = df[j] * gf[i][j];
          dg[i][j] += df[j] * xh[i][j];
          db[i][j] += df[j];
          s1 += dyg[i][j];
          s2 += dyg[i][j] * xh[i][j];
        }
      }
    }
    if (row + nwarps < rows) request(row + nwarps);
    s1 = RMS ? 0.f : warp_sum(s1) * inv_h;
    s2 = warp_sum(s2) * inv_h;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        float o[N];
#pragma unroll
        for (int j = 0; j < N; ++j) o[j] = (dres ? res[i][j] : 0.f) + rstd * (dyg[i][j] - s1 - xh[i][j] * s2);
        Vec16<T> t;
        t.set(o);
        t.store(dx + (size_t)row * H + v * N);
      }
    }
  }
  // the eight warps take turns adding their column sums into shared memory
  for (int w = 0; w < NORM_WARPS; ++w) {
    if (warp == w) {
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int v = lane + 32 * i;
        if (v < nvec) {
#pragma unroll
          for (int j = 0; j < N; ++j) {
            float* pg = nb_sums + v * N + j;
            if (w == 0) {
              pg[0] = dg[i][j];
              pg[H] = db[i][j];
            } else {
              pg[0] += dg[i][j];
              pg[H] += db[i][j];
            }
          }
        }
      }
    }
    __syncthreads();
  }
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    if (partial) {
      partial[(size_t)blockIdx.x * 2 * H + c] = nb_sums[c];
      if (!RMS) partial[(size_t)blockIdx.x * 2 * H + H + c] = nb_sums[H + c];
    } else {
      if (dgamma) atomicAdd(dgamma + c, nb_sums[c]);
      if (!RMS && dbeta) atomicAdd(dbeta + c, nb_sums[H + c]);
    }
  }
}

// dgamma[c] += sum_b partial[b][0][c]; dbeta[c] += sum_b partial[b][1][c].
// A CTA owns 32 columns; its 32 x 32 threads split the nblk partial rows 32 ways (coalesced 128-byte reads), then
// the 32 row-groups meet in shared memory. With hundreds of partial rows a one-thread-per-column loop is a chain of
// dependent cache misses (47 us measured for H = 1024); this form takes a few microseconds.
__global__ void __launch_bounds__(1024) norm_bwd_reduce_kernel(const float* __restrict__ partial,
                                                               float* __restrict__ dgamma, float* __restrict__ dbeta,
                                                               int nblk, int H) {
  __shared__ float red[32][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  const int which = blockIdx.y;  // 0 = gamma, 1 = beta
  float* out = which == 0 ? dgamma : dbeta;
  if (!out) return;
  float s = 0.f;
  if (c < H) {
    const float* p = partial + (size_t)which * H + c;
    for (int b = threadIdx.y; b < nblk; b += 32) s += p[(size_t)b * 2 * H];
  }
  red[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < H) {
    float t = 0.f;
#pragma unroll
    for (int y = 0; y < 32; ++y) t += red[y][threadIdx.x];
    out[c] += t;
  }
}

static inline int norm_bwd_grid(int rows) { return rows < sm_count() * 4 ? rows : sm_count() * 4; }

template <typename T, bool RMS>
static int norm_fwd_launch(const void* x, const void* gamma, const void* beta, void* y, float* mean,
                           float* rstd, int rows, int H, float eps, cudaStream_t st) {
  constexpr int N = Vec16<T>::N;
  if (H % N) TB_FAIL(TB_E_ARG, "norm: H=%d must be a multiple of %d", H, N);
  int nvec = H / N;
  if (nvec <= 32 * 8) {
    // resident CTAs only (two per SM up to four vectors per lane, one above): every warp then streams several rows
    // with the next one already requested
    const int want = (rows + NORM_WARPS - 1) / NORM_WARPS;
    const int cap = sm_count() * (nvec <= 128 ? 2 : 1);
    const int wgrid = want < cap ? want : cap;
#define TB_NFW(VPL_)                                                                                                  \
  norm_fwd_warp_kernel<T, VPL_, RMS><<<wgrid, NORM_WARPS * 32, 0, st>>>((const T*)x, (const T*)gamma, (const T*)beta, \
                                                                        (T*)y, mean, rstd, rows, H, eps);
    if (nvec <= 32) TB_NFW(1) else if (nvec <= 64) TB_NFW(2) else if (nvec <= 128) TB_NFW(4) else TB_NFW(8)
#undef TB_NFW
    TB_CUDA_CHECK(cudaGetLastError());
    return 0;
  }
  int grid = rows < sm_count() * 8 ? rows : sm_count() * 8;
#define TB_NF(VPT_)                                                                                 \
  {                                                                                                 \
    int threads = ((nvec + VPT_ - 1) / VPT_ + 31) / 32 * 32;                                        \
    norm_fwd_kernel<T, VPT_, RMS><<<grid, threads, 0, st>>>((const T*)x, (const T*)gamma,           \
                                                             (const T*)beta, (T*)y, mean, rstd,     \
                                                             rows, H, eps);                         \
  }
  if (nvec <= 256) TB_NF(1) else if (nvec <= 1024) TB_NF(2) else if (nvec <= 4096) TB_NF(4) else
    TB_FAIL(TB_E_ARG, "norm: H=%d too large", H);
#undef TB_NF
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

template <typename T, bool RMS>
static int norm_bwd_launch(const void* dy, const void* x, const void* gamma, const float* mean,
                           const float* rstd, const void* dres, void* dx, float* dgamma,
                           float* dbeta, float* partial, int rows, int H, cudaStream_t st) {
  constexpr int N = Vec16<T>::N;
  if (H % N) TB_FAIL(TB_E_ARG, "norm: H=%d must be a multiple of %d", H, N);
  int nvec = H / N;
  int grid = norm_bwd_grid(rows);
  if (nvec <= 32 * 4) {  // eight vectors per lane would spill: wider rows keep the CTA-per-row kernel
    // never more CTAs than the cap above: the workspace (also the fixed one of tb_norm_bwd_static) is sized for it
    const int want = (rows + NORM_WARPS - 1) / NORM_WARPS;
    const int cap = sm_count() * (nvec <= 32 ? 3 : 1);  // resident CTAs: 80 / 158 / 255 registers per thread
    const int wgrid = want < (cap < grid ? cap : grid) ? want : (cap < grid ? cap : grid);
    const size_t smem = (size_t)2 * H * sizeof(float);
#define TB_NBW(VPL_)                                                                                           \
  norm_bwd_warp_kernel<T, VPL_, RMS><<<wgrid, NORM_WARPS * 32, smem, st>>>(                                    \
      (const T*)dy, (const T*)x, (const T*)gamma, mean, rstd, (const T*)dres, (T*)dx, dgamma, dbeta, partial, rows, H);
    if (nvec <= 32) TB_NBW(1) else if (nvec <= 64) TB_NBW(2) else TB_NBW(4)
#undef TB_NBW
    if (partial) {
      dim3 rgrid((H + 31) / 32, RMS ? 1 : 2);
      norm_bwd_reduce_kernel<<<rgrid, dim3(32, 32), 0, st>>>(partial, dgamma, dbeta, wgrid, H);
    }
    TB_CUDA_CHECK(cudaGetLastError());
    return 0;
  }
#define TB_NB(VPT_)                                                                               \
  {                                                                                               \
    int threads = ((nvec + VPT_ - 1) / VPT_ + 31) / 32 * 32;                                      \
    norm_bwd_kernel<T, VPT_, RMS><<<grid, threads, 0, st>>>((const T*)dy, (const T*)x,            \
                                                             (const T*)gamma, mean, rstd,         \
                                                             (const T*)dres, (T*)dx, dgamma,      \
                                                             dbeta, partial, rows, H);            \
  }
  if (nvec <= 256) TB_NB(1) else if (nvec <= 1024) TB_NB(2) else if (nvec <= 4096) TB_NB(4) else
    TB_FAIL(TB_E_ARG, "norm: H=%d too large", H);
#undef TB_NB
  if (partial) {
    dim3 rgrid((H + 31) / 32, RMS ? 1 : 2);
    norm_bwd_reduce_kernel<<<rgrid, dim3(32, 32), 0, st>>>(partial, dgamma, dbeta, grid, H);
  }
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

}  // namespace tb
using namespace tb;

// dtype: 0 = bf16, 1 = fp32. rms: 0 = LayerNorm, 1 = RMSNorm. beta / mean may be null.
TB_EXPORT int tb_norm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean,
                          float* rstd, int rows, int H, float eps, int rms, int dtype,
                          cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (rows <= 0) return 0;
  if (dtype == 0)
    return rms ? norm_fwd_launch<bf16, true>(x, gamma, beta, y, mean, rstd, rows, H, eps, st)
               : norm_fwd_launch<bf16, false>(x, gamma, beta, y, mean, rstd, rows, H, eps, st);
  return rms ? norm_fwd_launch<float, true>(x, gamma, beta, y, mean, rstd, rows, H, eps, st)
             : norm_fwd_launch<float, false>(x, gamma, beta, y, mean, rstd, rows, H, eps, st);
}

// Number of fp32 elements of scratch memory tb_norm_bwd wants for (rows, H).
TB_EXPORT long tb_norm_bwd_workspace(int rows, int H) {
  if (rows <= 0) return 0;
  if (tb::ensure_device()) return 0;
  return (long)norm_bwd_grid(rows) * 2 * H;
}

// dgamma / dbeta are fp32 buffers that the kernel ACCUMULATES into (zero them for a fresh
// gradient). dres (optional) is added to dx. `partial` is scratch memory of
// tb_norm_bwd_workspace(rows, H) floats holding per-CTA partial sums that a second kernel
// reduces; with partial == null the partial sums are added with atomics instead (slower).
TB_EXPORT int tb_norm_bwd(const void* dy, const void* x, const void* gamma, const float* mean,
                          const float* rstd, const void* dres, void* dx, float* dgamma,
                          float* dbeta, float* partial, int rows, int H, int rms, int dtype,
                          cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (rows <= 0) return 0;
  if (dtype == 0)
    return rms ? norm_bwd_launch<bf16, true>(dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, partial, rows, H, st)
               : norm_bwd_launch<bf16, false>(dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, partial, rows, H, st);
  return rms ? norm_bwd_launch<float, true>(dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, partial, rows, H, st)
             : norm_bwd_launch<float, false>(dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, partial, rows, H, st);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of tb_norm_bwd (declared in csrc/include/torsh_b200_noalloc.h).
//
// tb_norm_bwd needs scratch memory for its per-CTA partial sums and expects the caller to provide
// it. Some callers cannot: code running inside a CUDA-graph capture or a real-time serving loop must
// not touch an allocator, and a plain C / FFI host has no caching allocator to ask. For them the
// scratch lives in the library image itself, in a file-scope device array of fixed size. Every GPU
// that loads the library holds these 8 MiB until the process exits.
//
// Rules that follow from sharing one array:
//  * the request is refused (TB_E_TOO_LARGE) when it needs more than the array holds;
//  * the array keeps whatever the previous call left in it. Nothing has to start at zero here: every
//    partial-sum row that the reduce kernel reads is fully overwritten by the CTA that owns it;
//  * two calls whose kernels overlap on the GPU (different streams, or graphs replayed concurrently)
//    race on the array. Issue them on one stream, or serialise them with events.
// The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
// device current) and caches it; make that first call before any stream capture begins.
namespace tb {
constexpr long NOALLOC_SCRATCH_FLOATS = 2L * 1024 * 1024;  // 8 MiB
static __device__ __align__(256) float g_norm_bwd_scratch[NOALLOC_SCRATCH_FLOATS];
// In host code the name above is only a handle for the symbol, never a device address.
static float* g_norm_bwd_scratch_dev[64] = {nullptr};

static int noalloc_scratch_ptr(float** out) {
  int dev = 0;
  TB_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) TB_FAIL(TB_E_ARG, "tb_norm_bwd_static: device index %d out of range", dev);
  if (!g_norm_bwd_scratch_dev[dev]) {
    float* p = nullptr;
    TB_CUDA_CHECK(cudaGetSymbolAddress((void**)&p, g_norm_bwd_scratch));
    if (!p) TB_FAIL(TB_E_CUDA, "tb_norm_bwd_static: cudaGetSymbolAddress returned a null address");
    g_norm_bwd_scratch_dev[dev] = p;
  }
  *out = g_norm_bwd_scratch_dev[dev];
  return 0;
}
}  // namespace tb

TB_EXPORT long tb_norm_bwd_static_capacity() { return tb::NOALLOC_SCRATCH_FLOATS; }

TB_EXPORT int tb_norm_bwd_static(const void* dy, const void* x, const void* gamma, const float* mean,
                                 const float* rstd, const void* dres, void* dx, float* dgamma, float* dbeta,
                                 int rows, int H, int rms, int dtype, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (rows <= 0) return 0;
  const long need = (long)tb::norm_bwd_grid(rows) * 2 * H;
  if (need > tb::NOALLOC_SCRATCH_FLOATS)
    TB_FAIL(tb::TB_E_TOO_LARGE,
            "tb_norm_bwd_static: rows=%d, H=%d needs %ld floats of scratch, the built-in array holds %ld; "
            "use tb_norm_bwd with caller-provided scratch",
            rows, H, need, tb::NOALLOC_SCRATCH_FLOATS);
  float* scratch = nullptr;
  if (int r = tb::noalloc_scratch_ptr(&scratch)) return r;
  return tb_norm_bwd(dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, scratch, rows, H, rms, dtype, st);
}
