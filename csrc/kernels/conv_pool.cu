// Channels-last (NHWC, bf16) convolution support, BatchNorm2d and pooling for sm_100a.
//
// A convolution is a GEMM on the tcgen05 kernel of gemm_sm100.cu: 1x1 stride-1 convolutions pass the activation
// matrix [N*H*W, C] straight through; every other shape goes through im2col_nhwc (forward, weight gradient) and
// col2im_nhwc (input gradient, written as a gather so no atomics are needed). BatchNorm2d keeps per-channel
// statistics in fp32 and fuses the affine transform, the residual add and ReLU into one pass forward and one
// reduce + one apply pass backward. The reference runs these layers through host loops or cuDNN calls
// (crates/torsh-backend/src/cuda/cudnn/operations.rs:99-1319; crates/torsh-nn/src/layers/normalization.rs) and its
// own conv2d / batchnorm2d / maxpool2d launchers are empty (crates/torsh-backend/src/cuda/kernels/mod.rs:20-330).
#include <type_traits>

#include "common.cuh"
#include "host_util.h"

namespace tb {

struct ConvGeom {
  int N, H, W, C, KH, KW, stride, pad, Ho, Wo;
  long ld;  // row pitch of the column matrix in elements (>= KH*KW*C, multiple of 8)
};

// cols[m, (kh*KW + kw)*C + c] = x[n, ho*stride - pad + kh, wo*stride - pad + kw, c], zero outside the image.
// One thread moves V channels: 16 bytes when C % 8 == 0, 8 bytes when C % 4 == 0 (the stem with its 3 input
// channels padded to 4). Columns between KH*KW*C and the row pitch are zero-filled by the last tap's threads.
template <int V>
__global__ void im2col_vec_kernel(const bf16* __restrict__ x, bf16* __restrict__ cols, ConvGeom g) {
  typedef typename std::conditional<V == 8, uint4, uint2>::type vec_t;
  const int cv = g.C / V;
  const int K = g.KH * g.KW * g.C;
  const int tail = (int)(g.ld - K) / V;  // zero vectors after the last tap
  const long per_row = (long)g.KH * g.KW * cv + tail;
  const long total = (long)g.N * g.Ho * g.Wo * per_row;
  const long stride = (long)gridDim.x * blockDim.x;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const long m = idx / per_row;
    int r = (int)(idx - m * per_row);
    vec_t v;
    memset(&v, 0, sizeof(v));
    if (r >= g.KH * g.KW * cv) {
      *reinterpret_cast<vec_t*>(cols + m * g.ld + K + (long)(r - g.KH * g.KW * cv) * V) = v;
      continue;
    }
    const int tap = r / cv, c = (r - tap * cv) * V;
    const int kh = tap / g.KW, kw = tap - kh * g.KW;
    const int wo = (int)(m % g.Wo);
    const long t = m / g.Wo;
    const int ho = (int)(t % g.Ho), n = (int)(t / g.Ho);
    const int h = ho * g.stride - g.pad + kh, w = wo * g.stride - g.pad + kw;
    if (h >= 0 && h < g.H && w >= 0 && w < g.W)
      v = __ldg(reinterpret_cast<const vec_t*>(x + (((long)n * g.H + h) * g.W + w) * g.C + c));
    *reinterpret_cast<vec_t*>(cols + m * g.ld + (long)tap * g.C + c) = v;
  }
}
// Any C (the 3-channel stem): one thread per column-matrix element, pad columns written as zero.
__global__ void im2col_scalar_kernel(const bf16* __restrict__ x, bf16* __restrict__ cols, ConvGeom g) {
  const int K = g.KH * g.KW * g.C;
  const long total = (long)g.N * g.Ho * g.Wo * g.ld;
  const long stride = (long)gridDim.x * blockDim.x;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const long m = idx / g.ld;
    const int k = (int)(idx - m * g.ld);
    bf16 v = __float2bfloat16(0.f);
    if (k < K) {
      const int tap = k / g.C, c = k - tap * g.C;
      const int kh = tap / g.KW, kw = tap - kh * g.KW;
      const int wo = (int)(m % g.Wo);
      const long t = m / g.Wo;
      const int ho = (int)(t % g.Ho), n = (int)(t / g.Ho);
      const int h = ho * g.stride - g.pad + kh, w = wo * g.stride - g.pad + kw;
      if (h >= 0 && h < g.H && w >= 0 && w < g.W) v = x[(((long)n * g.H + h) * g.W + w) * g.C + c];
    }
    cols[idx] = v;
  }
}

// dx[n, h, w, c] = sum over the taps (kh, kw) whose output pixel exists of dcols[(n, ho, wo), (kh, kw, c)]:
// the transpose of im2col as a gather, fp32 accumulation, one thread per 8 channels of one input pixel.
__global__ void col2im_kernel(const bf16* __restrict__ dcols, bf16* __restrict__ dx, ConvGeom g) {
  const int c8 = g.C >> 3;
  const long total = (long)g.N * g.H * g.W * c8;
  const long stride = (long)gridDim.x * blockDim.x;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const long pix = idx / c8;
    const int c = (int)(idx - pix * c8) << 3;
    const int w = (int)(pix % g.W);
    const long t = pix / g.W;
    const int h = (int)(t % g.H), n = (int)(t / g.H);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int kh = 0; kh < g.KH; ++kh) {
      const int hn = h + g.pad - kh;
      if (hn < 0 || hn % g.stride) continue;
      const int ho = hn / g.stride;
      if (ho >= g.Ho) continue;
      for (int kw = 0; kw < g.KW; ++kw) {
        const int wn = w + g.pad - kw;
        if (wn < 0 || wn % g.stride) continue;
        const int wo = wn / g.stride;
        if (wo >= g.Wo) continue;
        Vec16<bf16> v;
        v.load_nc(dcols + (((long)n * g.Ho + ho) * g.Wo + wo) * g.ld + (long)(kh * g.KW + kw) * g.C + c);
        float f[8];
        v.get(f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += f[j];
      }
    }
    Vec16<bf16> o;
    o.set(acc);
    o.store(dx + pix * g.C + c);
  }
}

// ------------------------------------------------------------------------------------------------ BatchNorm2d
// Per-channel sum and sum of squares of x [rows, C] into sums[0..C) and sums[C..2C) (fp32, accumulated with one
// atomic per column per block). 32 x 8 threads; a thread owns 8 adjacent channels of every 8th row of its row block.
__global__ void bn_stats_kernel(const bf16* __restrict__ x, float* __restrict__ sums, long rows, int C,
                                int rows_per_block) {
  __shared__ float part[2][8][32 * 8 + 1];
  const int c0 = (blockIdx.x * 32 + threadIdx.x) * 8;
  const long r0 = (long)blockIdx.y * rows_per_block, r1 = min(rows, r0 + rows_per_block);
  float s[8], q[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) s[j] = q[j] = 0.f;
  if (c0 < C) {
    for (long r = r0 + threadIdx.y; r < r1; r += 8) {
      Vec16<bf16> v;
      v.load_nc(x + r * C + c0);
      float f[8];
      v.get(f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        s[j] += f[j];
        q[j] += f[j] * f[j];
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    part[0][threadIdx.y][threadIdx.x * 8 + j] = s[j];
    part[1][threadIdx.y][threadIdx.x * 8 + j] = q[j];
  }
  __syncthreads();
  const int tid = threadIdx.y * 32 + threadIdx.x;
  const int col = blockIdx.x * 256 + tid;
  if (col < C) {
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int y = 0; y < 8; ++y) {
      a += part[0][y][tid];
      b += part[1][y][tid];
    }
    atomicAdd(sums + col, a);
    atomicAdd(sums + C + col, b);
  }
}
// mean / rstd from the sums; running statistics updated with `momentum` and the unbiased variance, as
// torch.nn.BatchNorm2d and the reference's BatchNorm2d do.
__global__ void bn_finalize_kernel(const float* __restrict__ sums, float* __restrict__ mean, float* __restrict__ rstd,
                                   float* __restrict__ run_mean, float* __restrict__ run_var, long rows, int C,
                                   float eps, float momentum) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const float m = sums[c] / (float)rows;
  const float var = fmaxf(sums[C + c] / (float)rows - m * m, 0.f);
  mean[c] = m;
  rstd[c] = rsqrtf(var + eps);
  if (run_mean) {
    run_mean[c] = (1.f - momentum) * run_mean[c] + momentum * m;
    const float unb = rows > 1 ? var * (float)rows / (float)(rows - 1) : var;
    run_var[c] = (1.f - momentum) * run_var[c] + momentum * unb;
  }
}
// y = act((x - mean) * rstd * gamma + beta + residual)
__global__ void bn_apply_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res, bf16* __restrict__ y,
                                const float* __restrict__ mean, const float* __restrict__ rstd,
                                const float* __restrict__ gamma, const float* __restrict__ beta, long rows, int C,
                                int relu) {
  const int c8 = C >> 3;
  const long total = rows * c8;
  const long stride = (long)gridDim.x * blockDim.x;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const long r = idx / c8;
    const int c = (int)(idx - r * c8) << 3;
    Vec16<bf16> v;
    v.load_nc(x + r * C + c);
    float f[8], rr[8];
    v.get(f);
    if (res) {
      Vec16<bf16> rv;
      rv.load_nc(res + r * C + c);
      rv.get(rr);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sc = rstd[c + j] * gamma[c + j];
      float o = (f[j] - mean[c + j]) * sc + beta[c + j];
      if (res) o += rr[j];
      f[j] = relu ? fmaxf(o, 0.f) : o;
    }
    v.set(f);
    v.store(y + r * C + c);
  }
}
// Backward reduction: sums[0..C) += sum g, sums[C..2C) += sum g * xhat, with g = dy masked by (y > 0) when the
// forward applied ReLU.
__global__ void bn_bwd_reduce_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ y,
                                     const bf16* __restrict__ x, const float* __restrict__ mean,
                                     const float* __restrict__ rstd, float* __restrict__ sums, long rows, int C,
                                     int relu, int rows_per_block) {
  __shared__ float part[2][8][32 * 8 + 1];
  const int c0 = (blockIdx.x * 32 + threadIdx.x) * 8;
  const long r0 = (long)blockIdx.y * rows_per_block, r1 = min(rows, r0 + rows_per_block);
  float s[8], q[8], mu[8], rs[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) s[j] = q[j] = 0.f;
  if (c0 < C) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      mu[j] = mean[c0 + j];
      rs[j] = rstd[c0 + j];
    }
    for (long r = r0 + threadIdx.y; r < r1; r += 8) {
      Vec16<bf16> vg, vx;
      vg.load_nc(dy + r * C + c0);
      vx.load_nc(x + r * C + c0);
      float g[8], xf[8], yf[8];
      vg.get(g);
      vx.get(xf);
      if (relu) {
        Vec16<bf16> vy;
        vy.load_nc(y + r * C + c0);
        vy.get(yf);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gj = (relu && yf[j] <= 0.f) ? 0.f : g[j];
        s[j] += gj;
        q[j] += gj * (xf[j] - mu[j]) * rs[j];
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    part[0][threadIdx.y][threadIdx.x * 8 + j] = s[j];
    part[1][threadIdx.y][threadIdx.x * 8 + j] = q[j];
  }
  __syncthreads();
  const int tid = threadIdx.y * 32 + threadIdx.x;
  const int col = blockIdx.x * 256 + tid;
  if (col < C) {
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int yy = 0; yy < 8; ++yy) {
      a += part[0][yy][tid];
      b += part[1][yy][tid];
    }
    atomicAdd(sums + col, a);
    atomicAdd(sums + C + col, b);
  }
}
// dx = gamma * rstd * (g - (sum_g + xhat * sum_gx) / rows); dres = g (when the forward added a residual);
// dgamma += sum_gx, dbeta += sum_g (fp32, by the first row-block of threads that sees each channel).
__global__ void bn_bwd_apply_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ y,
                                    const bf16* __restrict__ x, const float* __restrict__ mean,
                                    const float* __restrict__ rstd, const float* __restrict__ gamma,
                                    const float* __restrict__ sums, bf16* __restrict__ dx, bf16* __restrict__ dres,
                                    long rows, int C, int relu) {
  const int c8 = C >> 3;
  const long total = rows * c8;
  const long stride = (long)gridDim.x * blockDim.x;
  const float inv = 1.f / (float)rows;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const long r = idx / c8;
    const int c = (int)(idx - r * c8) << 3;
    Vec16<bf16> vg, vx;
    vg.load_nc(dy + r * C + c);
    vx.load_nc(x + r * C + c);
    float g[8], xf[8], yf[8], o[8];
    vg.get(g);
    vx.get(xf);
    if (relu) {
      Vec16<bf16> vy;
      vy.load_nc(y + r * C + c);
      vy.get(yf);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (relu && yf[j] <= 0.f) g[j] = 0.f;
      const float xh = (xf[j] - mean[c + j]) * rstd[c + j];
      o[j] = gamma[c + j] * rstd[c + j] * (g[j] - (sums[c + j] + xh * sums[C + c + j]) * inv);
    }
    vx.set(o);
    vx.store(dx + r * C + c);
    if (dres) {
      vg.set(g);
      vg.store(dres + r * C + c);
    }
  }
}
__global__ void bn_param_grad_kernel(const float* __restrict__ sums, float* __restrict__ dgamma,
                                     float* __restrict__ dbeta, int C) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  dbeta[c] += sums[c];
  dgamma[c] += sums[C + c];
}

// ---- fast BatchNorm forms for C/8 a power of two <= 256 (every ResNet width): a thread keeps one group of 8
// channels for its whole life, so the per-channel constants sit in registers and a row costs one 16-byte load per
// operand; 256 / (C/8) rows are in flight per block iteration and there is no integer division in the loop.
constexpr int BN_U = 4;   // rows in flight per thread, forward kernels
constexpr int BN_UB = 2;  // rows in flight per thread, backward kernels (three operands per row)
struct BnMap {
  int cv, r_in, rpb;  // channel-vector index, row inside the block's row group, rows per block iteration
};
__device__ __forceinline__ BnMap bn_map(int c8) {
  BnMap m;
  m.cv = threadIdx.x & (c8 - 1);
  m.r_in = threadIdx.x / c8;
  m.rpb = blockDim.x / c8;
  return m;
}
// Sum the per-thread partials of threads that share a channel group and add them to sums[] with one atomic per
// channel per block. part: shared [2][256][9] floats.
__device__ __forceinline__ void bn_block_reduce(float (&s)[8], float (&q)[8], float* part, float* sums, int C, int c8,
                                                const BnMap& m) {
  float* p0 = part;
  float* p1 = part + 256 * 9;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    p0[threadIdx.x * 9 + j] = s[j];
    p1[threadIdx.x * 9 + j] = q[j];
  }
  __syncthreads();
  // thread t < 2*C handles (which = t / C, channel = t % C); loops when 2*C > blockDim
  for (int t = threadIdx.x; t < 2 * C; t += blockDim.x) {
    const int which = t / C, ch = t - which * C;
    const int cv = ch >> 3, j = ch & 7;
    const float* src = which ? p1 : p0;
    float a = 0.f;
    for (int r = 0; r < m.rpb; ++r) a += src[(r * c8 + cv) * 9 + j];
    atomicAdd(sums + which * C + ch, a);
  }
}
__global__ void __launch_bounds__(256) bn_stats_fast_kernel(const bf16* __restrict__ x, float* __restrict__ sums,
                                                            long rows, int C) {
  __shared__ float part[2 * 256 * 9];
  const int c8 = C >> 3;
  const BnMap m = bn_map(c8);
  float s[8], q[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) s[j] = q[j] = 0.f;
  const bf16* xp = x + (long)m.cv * 8;
  const long step = (long)gridDim.x * m.rpb;
  for (long r = (long)blockIdx.x * m.rpb + m.r_in; r < rows; r += step * BN_U) {
    Vec16<bf16> v[BN_U];
#pragma unroll
    for (int u = 0; u < BN_U; ++u)
      if (r + u * step < rows) v[u].load_nc(xp + (r + u * step) * C);
#pragma unroll
    for (int u = 0; u < BN_U; ++u) {
      if (r + u * step >= rows) break;
      float f[8];
      v[u].get(f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        s[j] += f[j];
        q[j] += f[j] * f[j];
      }
    }
  }
  bn_block_reduce(s, q, part, sums, C, c8, m);
}
__global__ void __launch_bounds__(256) bn_apply_fast_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res,
                                                            bf16* __restrict__ y, const float* __restrict__ mean,
                                                            const float* __restrict__ rstd,
                                                            const float* __restrict__ gamma,
                                                            const float* __restrict__ beta, long rows, int C,
                                                            int relu) {
  const int c8 = C >> 3;
  const BnMap m = bn_map(c8);
  float sc[8], sh[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int c = m.cv * 8 + j;
    sc[j] = rstd[c] * gamma[c];
    sh[j] = beta[c] - mean[c] * sc[j];
  }
  const long off = (long)m.cv * 8;
  const long step = (long)gridDim.x * m.rpb;
  for (long r = (long)blockIdx.x * m.rpb + m.r_in; r < rows; r += step * BN_U) {
    Vec16<bf16> v[BN_U], rv[BN_U];
#pragma unroll
    for (int u = 0; u < BN_U; ++u) {
      const long ru = r + u * step;
      if (ru < rows) {
        v[u].load_nc(x + ru * C + off);
        if (res) rv[u].load_nc(res + ru * C + off);
      }
    }
#pragma unroll
    for (int u = 0; u < BN_U; ++u) {
      const long ru = r + u * step;
      if (ru >= rows) break;
      float f[8];
      v[u].get(f);
      if (res) {
        float rr[8];
        rv[u].get(rr);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = fmaf(f[j], sc[j], sh[j]) + rr[j];
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = fmaf(f[j], sc[j], sh[j]);
      }
      if (relu) {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = fmaxf(f[j], 0.f);
      }
      v[u].set(f);
      v[u].store(y + ru * C + off);
    }
  }
}
template <int RELU>
__global__ void __launch_bounds__(256, RELU == 2 ? 3 : 4) bn_bwd_reduce_fast_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ y,
                                                                 const bf16* __restrict__ x,
                                                                 const float* __restrict__ mean,
                                                                 const float* __restrict__ rstd,
                                                                 const float* __restrict__ gamma,
                                                                 const float* __restrict__ beta,
                                                                 float* __restrict__ sums, long rows, int C) {
  constexpr int relu = RELU;
  // relu == 1: mask from the saved output y; relu == 2: no residual was added, so the mask is recomputed from x with
  // the forward's own fused multiply-add (one tensor less to read)
  __shared__ float part[2 * 256 * 9];
  const int c8 = C >> 3;
  const BnMap m = bn_map(c8);
  float s[8], q[8], mu[8], sc[8], sh[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    s[j] = q[j] = 0.f;
    mu[j] = mean[m.cv * 8 + j];
    sc[j] = sh[j] = 0.f;
    if (relu == 2) {
      sc[j] = rstd[m.cv * 8 + j] * gamma[m.cv * 8 + j];
      sh[j] = beta[m.cv * 8 + j] - mu[j] * sc[j];
    }
  }
  const long off = (long)m.cv * 8;
  const long step = (long)gridDim.x * m.rpb;
  for (long r = (long)blockIdx.x * m.rpb + m.r_in; r < rows; r += step * BN_UB) {
    Vec16<bf16> vg[BN_UB], vx[BN_UB], vy[BN_UB];
#pragma unroll
    for (int u = 0; u < BN_UB; ++u) {
      const long ru = r + u * step;
      if (ru < rows) {
        vg[u].load_nc(dy + ru * C + off);
        vx[u].load_nc(x + ru * C + off);
        if (relu == 1) vy[u].load_nc(y + ru * C + off);
      }
    }
#pragma unroll
    for (int u = 0; u < BN_UB; ++u) {
      if (r + u * step >= rows) break;
      float g[8], xf[8];
      vg[u].get(g);
      vx[u].get(xf);
      if (relu == 1) {
        float yf[8];
        vy[u].get(yf);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (yf[j] <= 0.f) g[j] = 0.f;
      } else if (relu == 2) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (fmaf(xf[j], sc[j], sh[j]) <= 0.f) g[j] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        s[j] += g[j];
        q[j] = fmaf(g[j], xf[j] - mu[j], q[j]);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) q[j] *= rstd[m.cv * 8 + j];
  bn_block_reduce(s, q, part, sums, C, c8, m);
}
template <int RELU>
__global__ void __launch_bounds__(256, 3) bn_bwd_apply_fast_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ y,
                                                                const bf16* __restrict__ x,
                                                                const float* __restrict__ mean,
                                                                const float* __restrict__ rstd,
                                                                const float* __restrict__ gamma,
                                                                const float* __restrict__ beta,
                                                                const float* __restrict__ sums, bf16* __restrict__ dx,
                                                                bf16* __restrict__ dres, long rows, int C) {
  constexpr int relu = RELU;
  const int c8 = C >> 3;
  const BnMap m = bn_map(c8);
  // dx = a * g + b * x + d with a = gamma*rstd, b = -a * rstd * sum_gx / rows, d = -a * sum_g / rows - b * mean
  float a[8], b[8], d[8], sh[8];
  const float inv = 1.f / (float)rows;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int c = m.cv * 8 + j;
    a[j] = gamma[c] * rstd[c];
    b[j] = -a[j] * rstd[c] * sums[C + c] * inv;
    d[j] = -a[j] * sums[c] * inv - b[j] * mean[c];
    sh[j] = relu == 2 ? beta[c] - mean[c] * a[j] : 0.f;   // forward: y = relu(fma(x, a, sh))
  }
  const long off = (long)m.cv * 8;
  const long step = (long)gridDim.x * m.rpb;
  for (long r = (long)blockIdx.x * m.rpb + m.r_in; r < rows; r += step * BN_UB) {
    Vec16<bf16> vg[BN_UB], vx[BN_UB], vy[BN_UB];
#pragma unroll
    for (int u = 0; u < BN_UB; ++u) {
      const long ru = r + u * step;
      if (ru < rows) {
        vg[u].load_nc(dy + ru * C + off);
        vx[u].load_nc(x + ru * C + off);
        if (relu == 1) vy[u].load_nc(y + ru * C + off);
      }
    }
#pragma unroll
    for (int u = 0; u < BN_UB; ++u) {
      const long ru = r + u * step;
      if (ru >= rows) break;
      float g[8], xf[8];
      vg[u].get(g);
      vx[u].get(xf);
      if (relu == 1) {
        float yf[8];
        vy[u].get(yf);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (yf[j] <= 0.f) g[j] = 0.f;
      } else if (relu == 2) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (fmaf(xf[j], a[j], sh[j]) <= 0.f) g[j] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) xf[j] = fmaf(a[j], g[j], fmaf(b[j], xf[j], d[j]));
      vx[u].set(xf);
      vx[u].store(dx + ru * C + off);
      if (dres) {
        vg[u].set(g);
        vg[u].store(dres + ru * C + off);
      }
    }
  }
}
static inline bool bn_fast_ok(int C) {
  const int c8 = C >> 3;
  return (C & 7) == 0 && c8 >= 1 && c8 <= 256 && (c8 & (c8 - 1)) == 0;
}
static inline int bn_fast_grid(long rows, int C) {
  const long rpb = 256 / (C >> 3);
  long blocks = (rows + rpb - 1) / rpb;
  const long cap = (long)sm_count() * 8;
  return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

// ------------------------------------------------------------------------------------------------ pooling
// Max pooling k x k / stride / pad over NHWC; idx records which tap won (first maximum in row-major tap order, the
// choice torch makes), so the backward pass is an exact gather.
__global__ void maxpool_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, uint8_t* __restrict__ idx,
                                   int N, int H, int W, int C, int k, int stride, int pad, int Ho, int Wo) {
  const int c8 = C >> 3;
  const long total = (long)N * Ho * Wo * c8;
  const long gs = (long)gridDim.x * blockDim.x;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gs) {
    const long pix = i / c8;
    const int c = (int)(i - pix * c8) << 3;
    const int wo = (int)(pix % Wo);
    const long t = pix / Wo;
    const int ho = (int)(t % Ho), n = (int)(t / Ho);
    float best[8];
    uint8_t bi[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      best[j] = -INFINITY;
      bi[j] = 0;
    }
    for (int kh = 0; kh < k; ++kh) {
      const int h = ho * stride - pad + kh;
      if (h < 0 || h >= H) continue;
      for (int kw = 0; kw < k; ++kw) {
        const int w = wo * stride - pad + kw;
        if (w < 0 || w >= W) continue;
        Vec16<bf16> v;
        v.load_nc(x + (((long)n * H + h) * W + w) * C + c);
        float f[8];
        v.get(f);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (f[j] > best[j]) {
            best[j] = f[j];
            bi[j] = (uint8_t)(kh * k + kw);
          }
      }
    }
    Vec16<bf16> o;
    o.set(best);
    o.store(y + pix * C + c);
    uint2 packed;
    packed.x = bi[0] | (bi[1] << 8) | (bi[2] << 16) | (bi[3] << 24);
    packed.y = bi[4] | (bi[5] << 8) | (bi[6] << 16) | (bi[7] << 24);
    *reinterpret_cast<uint2*>(idx + pix * C + c) = packed;
  }
}
__global__ void maxpool_bwd_kernel(const bf16* __restrict__ dy, const uint8_t* __restrict__ idx,
                                   bf16* __restrict__ dx, int N, int H, int W, int C, int k, int stride, int pad,
                                   int Ho, int Wo) {
  const int c8 = C >> 3;
  const long total = (long)N * H * W * c8;
  const long gs = (long)gridDim.x * blockDim.x;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gs) {
    const long pix = i / c8;
    const int c = (int)(i - pix * c8) << 3;
    const int w = (int)(pix % W);
    const long t = pix / W;
    const int h = (int)(t % H), n = (int)(t / H);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int kh = 0; kh < k; ++kh) {
      const int hn = h + pad - kh;
      if (hn < 0 || hn % stride) continue;
      const int ho = hn / stride;
      if (ho >= Ho) continue;
      for (int kw = 0; kw < k; ++kw) {
        const int wn = w + pad - kw;
        if (wn < 0 || wn % stride) continue;
        const int wo = wn / stride;
        if (wo >= Wo) continue;
        const long op = ((long)n * Ho + ho) * Wo + wo;
        const uint2 pk = __ldg(reinterpret_cast<const uint2*>(idx + op * C + c));
        Vec16<bf16> v;
        v.load_nc(dy + op * C + c);
        float f[8];
        v.get(f);
        const int tap = kh * k + kw;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int who = ((j < 4 ? pk.x : pk.y) >> ((j & 3) * 8)) & 0xFF;
          if (who == tap) acc[j] += f[j];
        }
      }
    }
    Vec16<bf16> o;
    o.set(acc);
    o.store(dx + pix * C + c);
  }
}
// Global average pooling: y[n, c] = mean over hw of x[n, hw, c]; backward broadcasts dy / hw.
__global__ void avgpool_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, int N, int HW, int C) {
  const int c8 = C >> 3;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N * c8) return;
  const int n = i / c8, c = (i - n * c8) << 3;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int p = 0; p < HW; ++p) {
    Vec16<bf16> v;
    v.load_nc(x + ((long)n * HW + p) * C + c);
    float f[8];
    v.get(f);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] += f[j];
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] /= (float)HW;
  Vec16<bf16> o;
  o.set(acc);
  o.store(y + (long)n * C + c);
}
__global__ void avgpool_bwd_kernel(const bf16* __restrict__ dy, bf16* __restrict__ dx, int N, int HW, int C) {
  const int c8 = C >> 3;
  const long total = (long)N * HW * c8;
  const long gs = (long)gridDim.x * blockDim.x;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gs) {
    const long pix = i / c8;
    const int c = (int)(i - pix * c8) << 3;
    const int n = (int)(pix / HW);
    Vec16<bf16> v;
    v.load_nc(dy + (long)n * C + c);
    float f[8];
    v.get(f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] /= (float)HW;
    v.set(f);
    v.store(dx + pix * C + c);
  }
}

static inline int grid_1d(long items, int threads = 256) {
  long b = (items + threads - 1) / threads;
  long cap = (long)sm_count() * 16;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}
static inline bool al16(const void* p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace tb
using namespace tb;

TB_EXPORT int tb_im2col_nhwc(const void* x, void* cols, int N, int H, int W, int C, int KH, int KW, int stride, int pad,
                             long ld, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (N <= 0 || stride <= 0 || KH <= 0 || KW <= 0) TB_FAIL(TB_E_ARG, "im2col: bad geometry");
  ConvGeom g{N, H, W, C, KH, KW, stride, pad, (H + 2 * pad - KH) / stride + 1, (W + 2 * pad - KW) / stride + 1, ld};
  if (g.Ho <= 0 || g.Wo <= 0) TB_FAIL(TB_E_ARG, "im2col: empty output");
  if (ld < (long)KH * KW * C || (ld & 7)) TB_FAIL(TB_E_ARG, "im2col: row pitch %ld too small or not a multiple of 8", ld);
  const long rows = (long)N * g.Ho * g.Wo;
  const long K = (long)KH * KW * C;
  if ((C & 7) == 0 && al16(x) && al16(cols) && ((ld - K) & 7) == 0) {
    im2col_vec_kernel<8><<<grid_1d(rows * (KH * KW * (C >> 3) + (ld - K) / 8)), 256, 0, st>>>((const bf16*)x, (bf16*)cols, g);
  } else if ((C & 3) == 0 && al16(x) && al16(cols) && ((ld - K) & 3) == 0) {
    im2col_vec_kernel<4><<<grid_1d(rows * (KH * KW * (C >> 2) + (ld - K) / 4)), 256, 0, st>>>((const bf16*)x, (bf16*)cols, g);
  } else {
    im2col_scalar_kernel<<<grid_1d(rows * ld), 256, 0, st>>>((const bf16*)x, (bf16*)cols, g);
  }
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
TB_EXPORT int tb_col2im_nhwc(const void* dcols, void* dx, int N, int H, int W, int C, int KH, int KW, int stride,
                             int pad, long ld, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (N <= 0 || stride <= 0) TB_FAIL(TB_E_ARG, "col2im: bad geometry");
  if ((C & 7) || (ld & 7) || !al16(dcols) || !al16(dx)) TB_FAIL(TB_E_ARG, "col2im: C and pitch must be multiples of 8, pointers 16-byte aligned");
  ConvGeom g{N, H, W, C, KH, KW, stride, pad, (H + 2 * pad - KH) / stride + 1, (W + 2 * pad - KW) / stride + 1, ld};
  col2im_kernel<<<grid_1d((long)N * H * W * (C >> 3)), 256, 0, st>>>((const bf16*)dcols, (bf16*)dx, g);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

static inline void bn_grid(long rows, int C, dim3* grid, int* rpb) {
  const int col_blocks = (C + 255) / 256;
  long want = (4L * sm_count() + col_blocks - 1) / col_blocks;
  long r = (rows + want - 1) / want;
  if (r < 64) r = 64;
  *rpb = (int)r;
  *grid = dim3(col_blocks, (unsigned)((rows + r - 1) / r));
}
// sums: fp32 [2*C] scratch (zeroed here). mean / rstd: fp32 [C] outputs. run_mean / run_var may be null.
TB_EXPORT int tb_bn_fwd(const void* x, const void* res, void* y, float* sums, float* mean, float* rstd,
                        const float* gamma, const float* beta, float* run_mean, float* run_var, long rows, int C,
                        float eps, float momentum, int relu, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (rows <= 0 || C <= 0) return 0;
  if ((C & 7) || !al16(x) || !al16(y) || (res && !al16(res))) TB_FAIL(TB_E_ARG, "bn_fwd: C %% 8 and 16-byte alignment required");
  TB_CUDA_CHECK(cudaMemsetAsync(sums, 0, sizeof(float) * 2 * C, st));
  if (bn_fast_ok(C)) {
    const int g = bn_fast_grid(rows, C);
    bn_stats_fast_kernel<<<g, 256, 0, st>>>((const bf16*)x, sums, rows, C);
    bn_finalize_kernel<<<(C + 255) / 256, 256, 0, st>>>(sums, mean, rstd, run_mean, run_var, rows, C, eps, momentum);
    bn_apply_fast_kernel<<<g, 256, 0, st>>>((const bf16*)x, (const bf16*)res, (bf16*)y, mean, rstd, gamma, beta, rows, C, relu);
  } else {
    dim3 grid;
    int rpb;
    bn_grid(rows, C, &grid, &rpb);
    bn_stats_kernel<<<grid, dim3(32, 8), 0, st>>>((const bf16*)x, sums, rows, C, rpb);
    bn_finalize_kernel<<<(C + 255) / 256, 256, 0, st>>>(sums, mean, rstd, run_mean, run_var, rows, C, eps, momentum);
    bn_apply_kernel<<<grid_1d(rows * (C >> 3)), 256, 0, st>>>((const bf16*)x, (const bf16*)res, (bf16*)y, mean, rstd, gamma, beta, rows, C, relu);
  }
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
// Inference form: mean / rstd given (from the running statistics).
TB_EXPORT int tb_bn_apply(const void* x, const void* res, void* y, const float* mean, const float* rstd,
                          const float* gamma, const float* beta, long rows, int C, int relu, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (rows <= 0) return 0;
  if ((C & 7) || !al16(x) || !al16(y) || (res && !al16(res))) TB_FAIL(TB_E_ARG, "bn_apply: C %% 8 and 16-byte alignment required");
  if (bn_fast_ok(C))
    bn_apply_fast_kernel<<<bn_fast_grid(rows, C), 256, 0, st>>>((const bf16*)x, (const bf16*)res, (bf16*)y, mean, rstd, gamma, beta, rows, C, relu);
  else
    bn_apply_kernel<<<grid_1d(rows * (C >> 3)), 256, 0, st>>>((const bf16*)x, (const bf16*)res, (bf16*)y, mean, rstd, gamma, beta, rows, C, relu);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
// dgamma / dbeta (fp32 [C]) are accumulated into; dres may be null; y is read only when relu != 0.
TB_EXPORT int tb_bn_bwd(const void* dy, const void* y, const void* x, const float* mean, const float* rstd,
                        const float* gamma, const float* beta, float* sums, void* dx, void* dres, float* dgamma,
                        float* dbeta, long rows, int C, int relu, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (rows <= 0 || C <= 0) return 0;
  // relu: 0 none, 1 mask from the saved output y. With y == null (allowed when the forward added no residual) the
  // register-resident kernels recompute the mask from x, gamma and beta instead.
  if (relu && !y) {
    if (dres || !beta || !bn_fast_ok(C)) TB_FAIL(TB_E_ARG, "bn_bwd: the ReLU mask can be recomputed only without a residual, with beta, and for power-of-two channel groups");
    relu = 2;
  }
  if ((C & 7) || !al16(dy) || !al16(x) || !al16(dx) || (relu == 1 && !al16(y)) || (dres && !al16(dres)))
    TB_FAIL(TB_E_ARG, "bn_bwd: C %% 8 and 16-byte alignment required");
  TB_CUDA_CHECK(cudaMemsetAsync(sums, 0, sizeof(float) * 2 * C, st));
  if (bn_fast_ok(C)) {
    const int g = bn_fast_grid(rows, C);
#define TB_BN_BWD_FAST(R)                                                                                              \
  bn_bwd_reduce_fast_kernel<R><<<g, 256, 0, st>>>((const bf16*)dy, (const bf16*)y, (const bf16*)x, mean, rstd, gamma,  \
                                                  beta, sums, rows, C);                                                \
  bn_bwd_apply_fast_kernel<R><<<g, 256, 0, st>>>((const bf16*)dy, (const bf16*)y, (const bf16*)x, mean, rstd, gamma,   \
                                                 beta, sums, (bf16*)dx, (bf16*)dres, rows, C)
    if (relu == 2) { TB_BN_BWD_FAST(2); }
    else if (relu == 1) { TB_BN_BWD_FAST(1); }
    else { TB_BN_BWD_FAST(0); }
#undef TB_BN_BWD_FAST
  } else {
    dim3 grid;
    int rpb;
    bn_grid(rows, C, &grid, &rpb);
    bn_bwd_reduce_kernel<<<grid, dim3(32, 8), 0, st>>>((const bf16*)dy, (const bf16*)y, (const bf16*)x, mean, rstd, sums, rows, C, relu, rpb);
    bn_bwd_apply_kernel<<<grid_1d(rows * (C >> 3)), 256, 0, st>>>((const bf16*)dy, (const bf16*)y, (const bf16*)x, mean, rstd, gamma, sums, (bf16*)dx, (bf16*)dres, rows, C, relu);
  }
  bn_param_grad_kernel<<<(C + 255) / 256, 256, 0, st>>>(sums, dgamma, dbeta, C);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

TB_EXPORT int tb_maxpool_fwd(const void* x, void* y, void* idx, int N, int H, int W, int C, int k, int stride, int pad,
                             cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if ((C & 7) || k * k > 255 || !al16(x) || !al16(y) || ((uintptr_t)idx & 7)) TB_FAIL(TB_E_ARG, "maxpool: C %% 8, k*k <= 255, aligned pointers required");
  const int Ho = (H + 2 * pad - k) / stride + 1, Wo = (W + 2 * pad - k) / stride + 1;
  maxpool_fwd_kernel<<<grid_1d((long)N * Ho * Wo * (C >> 3)), 256, 0, st>>>((const bf16*)x, (bf16*)y, (uint8_t*)idx, N, H, W, C, k, stride, pad, Ho, Wo);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
TB_EXPORT int tb_maxpool_bwd(const void* dy, const void* idx, void* dx, int N, int H, int W, int C, int k, int stride,
                             int pad, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if ((C & 7) || !al16(dy) || !al16(dx) || ((uintptr_t)idx & 7)) TB_FAIL(TB_E_ARG, "maxpool_bwd: C %% 8 and aligned pointers required");
  const int Ho = (H + 2 * pad - k) / stride + 1, Wo = (W + 2 * pad - k) / stride + 1;
  maxpool_bwd_kernel<<<grid_1d((long)N * H * W * (C >> 3)), 256, 0, st>>>((const bf16*)dy, (const uint8_t*)idx, (bf16*)dx, N, H, W, C, k, stride, pad, Ho, Wo);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
TB_EXPORT int tb_avgpool_fwd(const void* x, void* y, int N, int HW, int C, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if ((C & 7) || !al16(x) || !al16(y)) TB_FAIL(TB_E_ARG, "avgpool: C %% 8 and aligned pointers required");
  avgpool_fwd_kernel<<<(N * (C >> 3) + 127) / 128, 128, 0, st>>>((const bf16*)x, (bf16*)y, N, HW, C);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
TB_EXPORT int tb_avgpool_bwd(const void* dy, void* dx, int N, int HW, int C, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if ((C & 7) || !al16(dy) || !al16(dx)) TB_FAIL(TB_E_ARG, "avgpool_bwd: C %% 8 and aligned pointers required");
  avgpool_bwd_kernel<<<grid_1d((long)N * HW * (C >> 3)), 256, 0, st>>>((const bf16*)dy, (bf16*)dx, N, HW, C);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
