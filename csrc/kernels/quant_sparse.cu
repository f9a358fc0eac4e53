// Quantised and sparse device kernels for sm_100a.
//
// INT4 group-wise weights: a row of K values is cut into groups of `group` (32 / 64 / 128 / 256) consecutive elements;
// each group has one fp32 scale = max|w| / 7 and its codes q = rint(w / scale) in [-7, 7] are packed two per byte,
// element 2i in the low nibble and 2i+1 in the high nibble (two's complement nibbles). The weight-only linear kernel
// multiplies a few activation rows by such a matrix without ever materialising the bf16 weights: it is bound by the
// K/2 bytes per output that must come from HBM, which is the point of the format for decoding.
// INT8 per-row: scale = max|x| / 127 per row.
// CSR x dense: one warp per (row, 128-column tile), 4 columns per lane, fp32 accumulation.
//
// The reference lists these as modules of torsh-quantization (crates/torsh-quantization/src/lib.rs: INT4 / group-wise
// schemes, `quantize_per_channel`) and as `CudaSparseTensor` (crates/torsh-sparse/src/gpu.rs:13-250, which forwards to
// a cuSPARSE wrapper that is not implemented there).
#include "common.cuh"
#include "host_util.h"

namespace tb {

__device__ __forceinline__ int clamp_q(float v, int qmax) {
  int q = __float2int_rn(v);
  return q < -qmax ? -qmax : (q > qmax ? qmax : q);
}

// One warp per group. PAIRS = group / 64 pairs of elements per lane.
template <typename T, int PAIRS>
__global__ void __launch_bounds__(256) quant_int4_group_kernel(const T* __restrict__ w, uint8_t* __restrict__ packed,
                                                               float* __restrict__ scales, long ngroups, int group) {
  const int lane = threadIdx.x & 31;
  const long g = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (g >= ngroups) return;
  const T* src = w + g * group;
  float v[PAIRS][2];
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < PAIRS; ++i) {
    const int e = 2 * (lane + 32 * i);
    const bool in = e < group;  // group 32: only the first 16 lanes hold a pair
    v[i][0] = in ? to_f<T>(src[e]) : 0.f;
    v[i][1] = in ? to_f<T>(src[e + 1]) : 0.f;
    m = fmaxf(m, fmaxf(fabsf(v[i][0]), fabsf(v[i][1])));
  }
  m = warp_max(m);
  const float scale = fmaxf(m, 1e-12f) / 7.f;
  const float inv = 1.f / scale;
  if (lane == 0) scales[g] = scale;
#pragma unroll
  for (int i = 0; i < PAIRS; ++i) {
    const int e = 2 * (lane + 32 * i);
    if (e < group) {
      const int lo = clamp_q(v[i][0] * inv, 7), hi = clamp_q(v[i][1] * inv, 7);
      packed[(g * group + e) >> 1] = (uint8_t)((lo & 0xF) | ((hi & 0xF) << 4));
    }
  }
}

__device__ __forceinline__ void unpack8(uint32_t word, float (&out)[8]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int nib = (word >> (4 * j)) & 0xF;
    out[j] = (float)((nib ^ 8) - 8);  // sign-extend the nibble
  }
}

template <typename T>
__global__ void dequant_int4_group_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ scales,
                                          T* __restrict__ out, long nwords, int group) {
  // one thread per 4 packed bytes = 8 elements (group is a multiple of 8, so they share a scale)
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nwords; i += (long)gridDim.x * blockDim.x) {
    const uint32_t word = reinterpret_cast<const uint32_t*>(packed)[i];
    const float s = scales[(i * 8) / group];
    float f[8];
    unpack8(word, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) out[i * 8 + j] = from_f<T>(f[j] * s);
  }
}

// y[m, n] = sum_k x[m, k] * deq(W)[n, k] (+ bias[n]); one warp per output column n, all MROWS activation rows at once.
// A lane takes 8 consecutive k (one 32-bit word of codes) per step; the warp covers 256 k per step.
template <int MROWS>
__global__ void __launch_bounds__(256) int4_linear_kernel(const __nv_bfloat16* __restrict__ x, const uint8_t* __restrict__ packed,
                                                          const float* __restrict__ scales, const __nv_bfloat16* __restrict__ bias,
                                                          __nv_bfloat16* __restrict__ y, int M, int N, int K, int group) {
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (n >= N) return;
  const uint32_t* wrow = reinterpret_cast<const uint32_t*>(packed + (size_t)n * (K / 2));
  const float* srow = scales + (size_t)n * (K / group);
  float acc[MROWS];
#pragma unroll
  for (int m = 0; m < MROWS; ++m) acc[m] = 0.f;
  for (int k0 = lane * 8; k0 < K; k0 += 256) {
    const uint32_t word = __ldg(wrow + (k0 >> 3));
    const float s = __ldg(srow + k0 / group);
    float wv[8];
    unpack8(word, wv);
#pragma unroll
    for (int m = 0; m < MROWS; ++m) {
      if (m < M) {
        const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)m * K + k0);
        const __nv_bfloat16* xe = reinterpret_cast<const __nv_bfloat16*>(&raw);
        float part = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) part += __bfloat162float(xe[j]) * wv[j];
        acc[m] += part * s;
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MROWS; ++m) {
    const float t = warp_sum(acc[m]);
    if (lane == 0 && m < M) y[(size_t)m * N + n] = __float2bfloat16(t + (bias ? __bfloat162float(bias[n]) : 0.f));
  }
}

// One CTA row-loop: scale[row] = max|x[row]| / 127, q = rint(x / scale).
template <typename T>
__global__ void quant_int8_row_kernel(const T* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ scale, int rows, int cols) {
  __shared__ float scratch[32];
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + (size_t)r * cols;
    float m = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, fabsf(to_f<T>(xr[c])));
    m = block_max(m, scratch);
    const float s = fmaxf(m, 1e-12f) / 127.f, inv = 1.f / s;
    if (threadIdx.x == 0) scale[r] = s;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) q[(size_t)r * cols + c] = (int8_t)clamp_q(to_f<T>(xr[c]) * inv, 127);
    __syncthreads();
  }
}

template <typename T>
__global__ void dequant_int8_row_kernel(const int8_t* __restrict__ q, const float* __restrict__ scale, T* __restrict__ out, long total,
                                        int cols) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x)
    out[i] = from_f<T>((float)q[i] * scale[i / cols]);
}

// C[r, :] = sum_j vals[j] * B[col[j], :] over the non-zeros j of row r. Grid (ceil(M / 4), ceil(N / 128)), 4 warps per CTA.
template <typename T>
__global__ void __launch_bounds__(128) csr_spmm_kernel(const int* __restrict__ rowptr, const int* __restrict__ colidx,
                                                       const float* __restrict__ vals, const T* __restrict__ B, T* __restrict__ C,
                                                       int M, int K, int N) {
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (r >= M) return;
  const int n0 = blockIdx.y * 128 + lane * 4;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const int j0 = rowptr[r], j1 = rowptr[r + 1];
  for (int j = j0; j < j1; ++j) {
    const int c = __ldg(colidx + j);
    const float a = __ldg(vals + j);
    if (c < 0 || c >= K) {  // a column index outside B: recorded when kernel checks are on, skipped either way
      if (lane == 0) report_bad_index();
      continue;
    }
    const T* brow = B + (size_t)c * N;
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (n0 + u < N) acc[u] += a * to_f<T>(brow[n0 + u]);
  }
#pragma unroll
  for (int u = 0; u < 4; ++u)
    if (n0 + u < N) C[(size_t)r * N + n0 + u] = from_f<T>(acc[u]);
}

}  // namespace tb
using namespace tb;

static bool group_ok(int group) { return group == 32 || group == 64 || group == 128 || group == 256; }

// w: [rows, cols] bf16 (dtype 0) or fp32 (1), cols a multiple of `group`; packed: rows * cols / 2 bytes; scales: rows * cols / group.
TB_EXPORT int tb_quantize_int4_group(const void* w, int dtype, void* packed, float* scales, long rows, int cols, int group,
                                     cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (rows <= 0 || cols <= 0) return 0;
  if (!group_ok(group) || cols % group) TB_FAIL(TB_E_ARG, "int4: group must be 32 / 64 / 128 / 256 and divide cols (%d, %d)", group, cols);
  const long ngroups = rows * (cols / group);
  const int grid = (int)((ngroups + 7) / 8);
#define TB_Q4(T, PAIRS) quant_int4_group_kernel<T, PAIRS><<<grid, 256, 0, st>>>((const T*)w, (uint8_t*)packed, scales, ngroups, group)
  if (dtype == 0) {
    if (group <= 64) TB_Q4(bf16, 1); else if (group == 128) TB_Q4(bf16, 2); else TB_Q4(bf16, 4);
  } else {
    if (group <= 64) TB_Q4(float, 1); else if (group == 128) TB_Q4(float, 2); else TB_Q4(float, 4);
  }
#undef TB_Q4
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

TB_EXPORT int tb_dequantize_int4_group(const void* packed, const float* scales, void* out, int dtype, long rows, int cols, int group,
                                       cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (rows <= 0 || cols <= 0) return 0;
  if (!group_ok(group) || cols % group) TB_FAIL(TB_E_ARG, "int4: group must be 32 / 64 / 128 / 256 and divide cols (%d, %d)", group, cols);
  if (((uintptr_t)packed & 3) != 0) TB_FAIL(TB_E_ARG, "int4: packed codes must be 4-byte aligned");
  const long nwords = rows * cols / 8;
  const int grid = (int)((nwords + 255) / 256 < 148 * 16 ? (nwords + 255) / 256 : 148 * 16);
  if (dtype == 0) dequant_int4_group_kernel<bf16><<<grid, 256, 0, st>>>((const uint8_t*)packed, scales, (bf16*)out, nwords, group);
  else dequant_int4_group_kernel<float><<<grid, 256, 0, st>>>((const uint8_t*)packed, scales, (float*)out, nwords, group);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// Weight-only INT4 linear for up to 8 activation rows: x [M, K] bf16, packed [N, K / 2], scales [N, K / group], y [M, N] bf16.
TB_EXPORT int tb_int4_linear(const void* x, const void* packed, const float* scales, const void* bias, void* y, int M, int N, int K,
                             int group, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (M <= 0 || N <= 0) return 0;
  if (M > 8) TB_FAIL(TB_E_TOO_LARGE, "int4 linear: at most 8 activation rows per call (got %d); dequantise and use the GEMM beyond", M);
  if (!group_ok(group) || K % group || K % 8) TB_FAIL(TB_E_ARG, "int4 linear: K (%d) must be a multiple of the group (%d) and of 8", K, group);
  if (((uintptr_t)x & 15) || ((uintptr_t)packed & 3)) TB_FAIL(TB_E_ARG, "int4 linear: x must be 16-byte and the codes 4-byte aligned");
  const int grid = (N + 7) / 8;
#define TB_L4(MR) int4_linear_kernel<MR><<<grid, 256, 0, st>>>((const bf16*)x, (const uint8_t*)packed, scales, (const bf16*)bias, (bf16*)y, M, N, K, group)
  if (M == 1) TB_L4(1); else if (M == 2) TB_L4(2); else if (M <= 4) TB_L4(4); else TB_L4(8);
#undef TB_L4
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

TB_EXPORT int tb_quantize_int8_row(const void* x, int dtype, void* q, float* scale, int rows, int cols, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (rows <= 0 || cols <= 0) return 0;
  const int grid = rows < sm_count() * 8 ? rows : sm_count() * 8;
  if (dtype == 0) quant_int8_row_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)x, (int8_t*)q, scale, rows, cols);
  else quant_int8_row_kernel<float><<<grid, 256, 0, st>>>((const float*)x, (int8_t*)q, scale, rows, cols);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

TB_EXPORT int tb_dequantize_int8_row(const void* q, const float* scale, void* out, int dtype, int rows, int cols, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (rows <= 0 || cols <= 0) return 0;
  const long total = (long)rows * cols;
  const int grid = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  if (dtype == 0) dequant_int8_row_kernel<bf16><<<grid, 256, 0, st>>>((const int8_t*)q, scale, (bf16*)out, total, cols);
  else dequant_int8_row_kernel<float><<<grid, 256, 0, st>>>((const int8_t*)q, scale, (float*)out, total, cols);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// C [M, N] = A (CSR: rowptr [M + 1], colidx / vals [nnz], fp32 values) x B [K, N]; B and C bf16 (dtype 0) or fp32 (1).
TB_EXPORT int tb_csr_spmm(const int* rowptr, const int* colidx, const float* vals, const void* B, void* C, int M, int K, int N, int dtype,
                          cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (M <= 0 || N <= 0) return 0;
  dim3 grid((M + 3) / 4, (N + 127) / 128);
  if (dtype == 0) csr_spmm_kernel<bf16><<<grid, 128, 0, st>>>(rowptr, colidx, vals, (const bf16*)B, (bf16*)C, M, K, N);
  else csr_spmm_kernel<float><<<grid, 128, 0, st>>>(rowptr, colidx, vals, (const float*)B, (float*)C, M, K, N);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int tb_set_check_word_quant_sparse(int* word) {
  TB_CUDA_CHECK(tb::set_check_word_this_tu(word));
  return 0;
}
