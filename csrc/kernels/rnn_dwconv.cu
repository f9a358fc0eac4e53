// Recurrent-cell and depthwise-convolution kernels for sm_100a: the parts of a cuDNN-style layer library that are
// not GEMMs.
//
// LSTM: the input projection of ALL time steps is one GEMM and each step's recurrent projection is one small GEMM
// (both on the tcgen05 kernel); what remains per step is the gate arithmetic, fused here into one pass that reads the
// two pre-activation tensors and the previous cell state once and writes h, c and the activated gates (kept for the
// backward). Gate order i, f, g, o as in PyTorch and in the reference's `lstm_forward`
// (crates/torsh-backend/src/cuda/cudnn/operations.rs:1198, which forwards to cudnnRNNForward).
//
// Depthwise convolution (groups == channels, the `group_count` case of operations.rs:364 that has no GEMM shape):
// channels-last bf16, one thread per output pixel and vector of 8 channels, weights [kh][kw][C] so a tap is one 16-byte
// load; the input gradient is the gather form of the same sum (any stride), the weight gradient a two-stage reduction.
#include "common.cuh"
#include "host_util.h"

namespace tb {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// gx, gh: [B, 4H] pre-activations (input and recurrent projection, biases already inside gx), c_prev [B, H].
// Writes h, c [B, H] and act [B, 4H] = (i, f, g, o) after their nonlinearities.
template <typename T>
__global__ void lstm_cell_fwd_kernel(const T* __restrict__ gx, const T* __restrict__ gh, const float* __restrict__ c_prev,
                                     T* __restrict__ h, float* __restrict__ c, T* __restrict__ act, int B, int H) {
  const long total = (long)B * H;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
    const int b = (int)(idx / H), j = (int)(idx - (long)b * H);
    const size_t base = (size_t)b * 4 * H + j;
    const float pi = to_f<T>(gx[base]) + to_f<T>(gh[base]);
    const float pf = to_f<T>(gx[base + H]) + to_f<T>(gh[base + H]);
    const float pg = to_f<T>(gx[base + 2 * H]) + to_f<T>(gh[base + 2 * H]);
    const float po = to_f<T>(gx[base + 3 * H]) + to_f<T>(gh[base + 3 * H]);
    const float i = sigmoidf_(pi), f = sigmoidf_(pf), g = tanhf(pg), o = sigmoidf_(po);
    const float cn = f * c_prev[idx] + i * g;
    c[idx] = cn;
    h[idx] = from_f<T>(o * tanhf(cn));
    act[base] = from_f<T>(i);
    act[base + H] = from_f<T>(f);
    act[base + 2 * H] = from_f<T>(g);
    act[base + 3 * H] = from_f<T>(o);
  }
}

// dh, dc_next: gradients w.r.t. this step's h and c (dc_next may be null = 0). Writes dgates [B, 4H] (w.r.t. the
// pre-activations, shared by the input and the recurrent projection) and dc_prev [B, H].
template <typename T>
__global__ void lstm_cell_bwd_kernel(const T* __restrict__ dh, const float* __restrict__ dc_next, const T* __restrict__ act,
                                     const float* __restrict__ c, const float* __restrict__ c_prev, T* __restrict__ dgates,
                                     float* __restrict__ dc_prev, int B, int H) {
  const long total = (long)B * H;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
    const int b = (int)(idx / H), j = (int)(idx - (long)b * H);
    const size_t base = (size_t)b * 4 * H + j;
    const float i = to_f<T>(act[base]), f = to_f<T>(act[base + H]), g = to_f<T>(act[base + 2 * H]), o = to_f<T>(act[base + 3 * H]);
    const float tc = tanhf(c[idx]);
    const float dhv = to_f<T>(dh[idx]);
    const float dcv = (dc_next ? dc_next[idx] : 0.f) + dhv * o * (1.f - tc * tc);
    dgates[base] = from_f<T>(dcv * g * i * (1.f - i));
    dgates[base + H] = from_f<T>(dcv * c_prev[idx] * f * (1.f - f));
    dgates[base + 2 * H] = from_f<T>(dcv * i * (1.f - g * g));
    dgates[base + 3 * H] = from_f<T>(dhv * tc * o * (1.f - o));
    dc_prev[idx] = dcv * f;
  }
}

// y[n, ho, wo, c] = sum_{kh, kw} x[n, ho * s - p + kh, wo * s - p + kw, c] * w[kh, kw, c]   (bf16 in / out, fp32 sums)
__global__ void __launch_bounds__(256) dwconv_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                     const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ y, int N,
                                                     int H, int W, int C, int Ho, int Wo, int K, int stride, int pad) {
  const int cv = C / 8;
  const long total = (long)N * Ho * Wo * cv;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
    const int c8 = (int)(idx % cv);
    long p = idx / cv;
    const int wo = (int)(p % Wo);
    p /= Wo;
    const int ho = (int)(p % Ho);
    const int n = (int)(p / Ho);
    float acc[8];
    if (bias) {
      Vec16<__nv_bfloat16> bv;
      bv.load_nc(bias + c8 * 8);
      bv.get(acc);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    }
    for (int kh = 0; kh < K; ++kh) {
      const int hi = ho * stride - pad + kh;
      if (hi < 0 || hi >= H) continue;
      for (int kw = 0; kw < K; ++kw) {
        const int wi = wo * stride - pad + kw;
        if (wi < 0 || wi >= W) continue;
        Vec16<__nv_bfloat16> xv, wv;
        xv.load(x + (((size_t)n * H + hi) * W + wi) * C + c8 * 8);
        const int tap = kh * K + kw;
        wv.load_nc(w + (size_t)tap * C + c8 * 8);
        float xf[8], wf[8];
        xv.get(xf);
        wv.get(wf);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += xf[j] * wf[j];
      }
    }
    Vec16<__nv_bfloat16> out;
    out.set(acc);
    out.store(y + (((size_t)n * Ho + ho) * Wo + wo) * C + c8 * 8);
  }
}

// dx[n, hi, wi, c] = sum over the taps (kh, kw) and outputs (ho, wo) with ho * s - p + kh == hi, wo * s - p + kw == wi of
// dy[n, ho, wo, c] * w[kh, kw, c]: the gather form of the input gradient, any stride.
__global__ void __launch_bounds__(256) dwconv_dgrad_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ w,
                                                           __nv_bfloat16* __restrict__ dx, int N, int H, int W, int C, int Ho, int Wo,
                                                           int K, int stride, int pad) {
  const int cv = C / 8;
  const long total = (long)N * H * W * cv;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
    const int c8 = (int)(idx % cv);
    long p = idx / cv;
    const int wi = (int)(p % W);
    p /= W;
    const int hi = (int)(p % H);
    const int n = (int)(p / H);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int kh = 0; kh < K; ++kh) {
      const int th = hi + pad - kh;
      if (th < 0 || th % stride) continue;
      const int ho = th / stride;
      if (ho >= Ho) continue;
      for (int kw = 0; kw < K; ++kw) {
        const int tw = wi + pad - kw;
        if (tw < 0 || tw % stride) continue;
        const int wo = tw / stride;
        if (wo >= Wo) continue;
        Vec16<__nv_bfloat16> dv, wv;
        dv.load(dy + (((size_t)n * Ho + ho) * Wo + wo) * C + c8 * 8);
        wv.load_nc(w + (size_t)(kh * K + kw) * C + c8 * 8);
        float df[8], wf[8];
        dv.get(df);
        wv.get(wf);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += df[j] * wf[j];
      }
    }
    Vec16<__nv_bfloat16> out;
    out.set(acc);
    out.store(dx + (((size_t)n * H + hi) * W + wi) * C + c8 * 8);
  }
}

// dw[kh, kw, c] += sum_{n, ho, wo} x[n, ho * s - p + kh, wo * s - p + kw, c] * dy[n, ho, wo, c]; db[c] += sum dy.
// Grid (C / 8 / 32 rounded up, K * K, row blocks): 32 channel vectors x 8 row lanes per CTA; each CTA reduces its share
// of the output pixels in registers, then across the 8 row lanes in shared memory, then one atomic per channel.
__global__ void __launch_bounds__(256) dwconv_wgrad_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                                           float* __restrict__ dw, float* __restrict__ db, int N, int H, int W, int C,
                                                           int Ho, int Wo, int K, int stride, int pad) {
  __shared__ float part[8][32 * 8 + 1];
  const int cv = C / 8;
  const int c8 = blockIdx.x * 32 + (threadIdx.x & 31);
  const int lane_r = threadIdx.x >> 5;
  const int kh = blockIdx.y / K, kw = blockIdx.y % K;
  const bool do_bias = db != nullptr && blockIdx.y == 0;
  float acc[8], bacc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = bacc[j] = 0.f;
  if (c8 < cv) {
    const long pixels = (long)N * Ho * Wo;
    for (long p = (long)blockIdx.z * 8 + lane_r; p < pixels; p += (long)gridDim.z * 8) {
      const int wo = (int)(p % Wo);
      const long q = p / Wo;
      const int ho = (int)(q % Ho), n = (int)(q / Ho);
      Vec16<__nv_bfloat16> dv;
      float df[8];
      const int hi = ho * stride - pad + kh, wi = wo * stride - pad + kw;
      const bool inside = hi >= 0 && hi < H && wi >= 0 && wi < W;
      if (!inside && !do_bias) continue;
      dv.load(dy + (size_t)p * C + c8 * 8);
      dv.get(df);
      if (do_bias) {
#pragma unroll
        for (int j = 0; j < 8; ++j) bacc[j] += df[j];
      }
      if (inside) {
        Vec16<__nv_bfloat16> xv;
        float xf[8];
        xv.load(x + (((size_t)n * H + hi) * W + wi) * C + c8 * 8);
        xv.get(xf);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += xf[j] * df[j];
      }
    }
  }
  for (int pass = 0; pass < (do_bias ? 2 : 1); ++pass) {
#pragma unroll
    for (int j = 0; j < 8; ++j) part[lane_r][(threadIdx.x & 31) * 8 + j] = pass == 0 ? acc[j] : bacc[j];
    __syncthreads();
    const int col = threadIdx.x;  // 256 threads = 32 vectors x 8 channels
    const int ch = blockIdx.x * 256 + col;
    if (ch < C) {
      float t = 0.f;
#pragma unroll
      for (int r = 0; r < 8; ++r) t += part[r][col];
      if (pass == 0) atomicAdd(dw + (size_t)blockIdx.y * C + ch, t);
      else atomicAdd(db + ch, t);
    }
    __syncthreads();
  }
}

}  // namespace tb
using namespace tb;

static inline int ew_grid(long total) {
  long g = (total + 255) / 256;
  long cap = (long)sm_count() * 16;
  return (int)(g < cap ? g : cap);
}

// dtype: 0 = bf16, 1 = fp32 for gx / gh / h / act; cell states are always fp32.
TB_EXPORT int tb_lstm_cell_fwd(const void* gx, const void* gh, const float* c_prev, void* h, float* c, void* act, int B, int H,
                               int dtype, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (B <= 0 || H <= 0) return 0;
  const int grid = ew_grid((long)B * H);
  if (dtype == 0) lstm_cell_fwd_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)gx, (const bf16*)gh, c_prev, (bf16*)h, c, (bf16*)act, B, H);
  else lstm_cell_fwd_kernel<float><<<grid, 256, 0, st>>>((const float*)gx, (const float*)gh, c_prev, (float*)h, c, (float*)act, B, H);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

TB_EXPORT int tb_lstm_cell_bwd(const void* dh, const float* dc_next, const void* act, const float* c, const float* c_prev, void* dgates,
                               float* dc_prev, int B, int H, int dtype, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (B <= 0 || H <= 0) return 0;
  const int grid = ew_grid((long)B * H);
  if (dtype == 0)
    lstm_cell_bwd_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)dh, dc_next, (const bf16*)act, c, c_prev, (bf16*)dgates, dc_prev, B, H);
  else
    lstm_cell_bwd_kernel<float><<<grid, 256, 0, st>>>((const float*)dh, dc_next, (const float*)act, c, c_prev, (float*)dgates, dc_prev, B, H);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// x [N, H, W, C] bf16, w [K, K, C] bf16, bias [C] or null, y [N, Ho, Wo, C]; C a multiple of 8.
TB_EXPORT int tb_dwconv_fwd(const void* x, const void* w, const void* bias, void* y, int N, int H, int W, int C, int Ho, int Wo, int K,
                            int stride, int pad, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (N <= 0 || C <= 0) return 0;
  if (C % 8) TB_FAIL(TB_E_ARG, "depthwise conv: channels (%d) must be a multiple of 8", C);
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y | (uintptr_t)bias) & 15) TB_FAIL(TB_E_ARG, "depthwise conv: pointers must be 16-byte aligned");
  const int grid = ew_grid((long)N * Ho * Wo * (C / 8));
  dwconv_kernel<<<grid, 256, 0, st>>>((const bf16*)x, (const bf16*)w, (const bf16*)bias, (bf16*)y, N, H, W, C, Ho, Wo, K, stride, pad);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// dy [N, Ho, Wo, C] -> dx [N, H, W, C] (every element written).
TB_EXPORT int tb_dwconv_dgrad(const void* dy, const void* w, void* dx, int N, int H, int W, int C, int Ho, int Wo, int K, int stride,
                              int pad, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (N <= 0 || C <= 0) return 0;
  if (C % 8) TB_FAIL(TB_E_ARG, "depthwise conv: channels (%d) must be a multiple of 8", C);
  if (((uintptr_t)dy | (uintptr_t)w | (uintptr_t)dx) & 15) TB_FAIL(TB_E_ARG, "depthwise conv: pointers must be 16-byte aligned");
  const int grid = ew_grid((long)N * H * W * (C / 8));
  dwconv_dgrad_kernel<<<grid, 256, 0, st>>>((const bf16*)dy, (const bf16*)w, (bf16*)dx, N, H, W, C, Ho, Wo, K, stride, pad);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// dw [K, K, C] and db [C] (may be null) are fp32 and ACCUMULATED into (zero them first).
TB_EXPORT int tb_dwconv_wgrad(const void* x, const void* dy, float* dw, float* db, int N, int H, int W, int C, int Ho, int Wo, int K,
                              int stride, int pad, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (N <= 0 || C <= 0) return 0;
  if (C % 8) TB_FAIL(TB_E_ARG, "depthwise conv: channels (%d) must be a multiple of 8", C);
  const long pixels = (long)N * Ho * Wo;
  const int cblocks = (C / 8 + 31) / 32;
  long want = (4L * sm_count()) / ((long)cblocks * K * K) + 1;   // about four CTAs per SM in total
  long maxz = (pixels + 63) / 64;                               // at least 64 pixels per CTA row lane group
  if (want > maxz) want = maxz;
  if (want < 1) want = 1;
  if (want > 65535) want = 65535;
  dim3 grid(cblocks, K * K, (unsigned)want);
  dwconv_wgrad_kernel<<<grid, 256, 0, st>>>((const bf16*)x, (const bf16*)dy, dw, db, N, H, W, C, Ho, Wo, K, stride, pad);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
