// Axis reductions, embedding gather / scatter-add and rotary position embedding for sm_100a.
//
// Reductions view the tensor as [outer, axis, inner]. The reference assigns one thread per output
// element and loops serially over the axis with no shared memory or shuffles
// (crates/torsh-tensor/src/cuda_backend/ptx_ops.rs:106-184,285-356). Here inner == 1 uses one CTA
// per output row with warp-shuffle + shared-memory reduction, and inner > 1 maps threads across
// the contiguous inner index so loads stay coalesced while the axis is split over blockDim.y.
#include "common.cuh"
#include "host_util.h"

namespace tb {

enum ReduceOp { R_SUM = 0, R_MAX = 1, R_MIN = 2, R_MEAN = 3 };

__device__ __forceinline__ float red_init(int op) { return op == R_MAX ? -FLT_MAX : (op == R_MIN ? FLT_MAX : 0.f); }
__device__ __forceinline__ float red_comb(int op, float a, float b) {
  return op == R_MAX ? fmaxf(a, b) : (op == R_MIN ? fminf(a, b) : a + b);
}

template <typename T>
__global__ void reduce_rows_kernel(const T* __restrict__ x, T* __restrict__ y, long outer, long axis, int op) {
  __shared__ float scratch[32];
  for (long o = blockIdx.x; o < outer; o += gridDim.x) {
    const T* xr = x + o * axis;
    float acc = red_init(op);
    for (long i = threadIdx.x; i < axis; i += blockDim.x) acc = red_comb(op, acc, to_f<T>(xr[i]));
    // block reduce with the right combiner
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc = red_comb(op, acc, __shfl_xor_sync(0xffffffffu, acc, s));
    __syncthreads();
    if (lane == 0) scratch[warp] = acc;
    __syncthreads();
    if (warp == 0) {
      float r = lane < nw ? scratch[lane] : red_init(op);
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) r = red_comb(op, r, __shfl_xor_sync(0xffffffffu, r, s));
      if (lane == 0) y[o] = from_f<T>(op == R_MEAN ? r / (float)axis : r);
    }
  }
}

// inner > 1: block (32 x 8): x-threads walk the inner index, y-threads split the axis.
template <typename T>
__global__ void reduce_inner_kernel(const T* __restrict__ x, T* __restrict__ y, long outer, long axis,
                                    long inner, int op) {
  __shared__ float part[8][33];
  const long in = (long)blockIdx.x * 32 + threadIdx.x;
  const long o = blockIdx.y;
  float acc = red_init(op);
  if (in < inner)
    for (long a = threadIdx.y; a < axis; a += blockDim.y)
      acc = red_comb(op, acc, to_f<T>(x[(o * axis + a) * inner + in]));
  part[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && in < inner) {
    for (int j = 1; j < blockDim.y; ++j) acc = red_comb(op, acc, part[j][threadIdx.x]);
    y[o * inner + in] = from_f<T>(op == R_MEAN ? acc / (float)axis : acc);
  }
}

// Deterministic sum of n fp32 values, scaled: out[0] = scale * sum(x). Single CTA, fixed order.
__global__ void sum_f32_kernel(const float* __restrict__ x, float* __restrict__ out, long n, float scale) {
  __shared__ float scratch[32];
  float s = 0.f;
  for (long i = threadIdx.x; i < n; i += blockDim.x) s += x[i];
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) out[0] = s * scale;
}

// out[t, :] = wte[ids[t], :] (+ wpe[t % seq, :])
template <typename T>
__global__ void embedding_fwd_kernel(const long* __restrict__ ids, const T* __restrict__ wte,
                                     const T* __restrict__ wpe, T* __restrict__ out, long tokens,
                                     int H, int seq, long vocab) {
  constexpr int N = Vec16<T>::N;
  const int hv = H / N;
  const long total = tokens * hv;
  const long stride = (long)gridDim.x * blockDim.x;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    long t = idx / hv;
    int c = (int)(idx - t * hv) * N;
    long id = ids[t];
    if (id < 0 || id >= vocab) {
      if (c == 0) report_bad_index();
      id = 0;
    }
    Vec16<T> a;
    a.load(wte + id * H + c);
    if (wpe) {
      Vec16<T> p;
      p.load(wpe + (long)(t % seq) * H + c);
      float fa[N], fp[N];
      a.get(fa);
      p.get(fp);
#pragma unroll
      for (int j = 0; j < N; ++j) fa[j] += fp[j];
      a.set(fa);
    }
    a.store(out + t * H + c);
  }
}
// dwte[ids[t], :] += dout[t, :]; dwpe[t % seq, :] += dout[t, :]  (fp32 atomics)
template <typename T>
__global__ void embedding_bwd_kernel(const long* __restrict__ ids, const T* __restrict__ dout,
                                     float* __restrict__ dwte, float* __restrict__ dwpe, long tokens,
                                     int H, int seq, long vocab) {
  const long total = tokens * H;
  const long stride = (long)gridDim.x * blockDim.x;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    long t = idx / H;
    int c = (int)(idx - t * H);
    float g = to_f<T>(dout[idx]);
    long id = ids[t];
    if (dwte && id >= 0 && id < vocab) atomicAdd(dwte + id * H + c, g);
    else if (dwte && c == 0) report_bad_index();
    if (dwpe) atomicAdd(dwpe + (long)(t % seq) * H + c, g);
  }
}

// Message passing without the [E, F] message tensor: out[dst[e], :] += w[e] * x[src[e], :] for every edge e.
// One thread owns four consecutive features of one edge and issues one 16-byte vector reduction
// (red.global.add.v4.f32), so each edge row costs F/4 atomics. The CUDA string the reference emits for the
// same step adds into the output without atomics (crates/torsh-graph/src/jit.rs:405-450). src == nullptr reads
// row e of x (plain scatter-add); w == nullptr is weight 1. Indices outside [0, n_src) / [0, n_dst) are skipped.
template <typename T>
__global__ void gnn_scatter_kernel(const T* __restrict__ x, const long* __restrict__ src,
                                   const long* __restrict__ dst, const float* __restrict__ w,
                                   float* __restrict__ out, long E, int F, long n_src, long n_dst) {
  const int fq = F >> 2;
  const long total = E * fq;
  const long stride = (long)gridDim.x * blockDim.x;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const long e = idx / fq;
    const int c = (int)(idx - e * fq) << 2;
    const long s = src ? src[e] : e;
    const long d = dst[e];
    if (s < 0 || s >= n_src || d < 0 || d >= n_dst) {
      if (c == 0) report_bad_index();
      continue;
    }
    const float we = w ? w[e] : 1.f;
    const T* xp = x + s * F + c;
    float4 v = make_float4(to_f<T>(xp[0]) * we, to_f<T>(xp[1]) * we, to_f<T>(xp[2]) * we, to_f<T>(xp[3]) * we);
    float* op = out + d * F + c;
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(op), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
  }
}

// Rotary embedding on x [B, S, heads, D] (in place allowed). Adjacent pairs (2i, 2i+1) rotate by
// pos * base^(-2i/D): the pairing and frequency rule of RotaryPositionalEmbedding
// (crates/torsh-nn/src/layers/embedding.rs:372-430), whose rotate step is a no-op in the
// reference. sign = -1 applies the inverse rotation (the backward pass).
template <typename T>
__global__ void rope_kernel(const T* __restrict__ x, T* __restrict__ y, long B, int S, int heads,
                            int D, float base, int pos_offset, float sign) {
  const int half = D / 2;
  const long total = B * S * heads * half;
  const long stride = (long)gridDim.x * blockDim.x;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    int i = (int)(idx % half);
    long rest = idx / half;
    long bs = rest / heads;
    int s = (int)(bs % S);
    float freq = __powf(base, -2.f * (float)i / (float)D);
    float ang = (float)(s + pos_offset) * freq;
    float sn, cs;
    sincosf(ang, &sn, &cs);
    sn *= sign;
    long o = rest * D + 2 * i;
    float a = to_f<T>(x[o]), b = to_f<T>(x[o + 1]);
    y[o] = from_f<T>(a * cs - b * sn);
    y[o + 1] = from_f<T>(a * sn + b * cs);
  }
}

static inline int grid_for(long items) {
  long b = (items + 255) / 256;
  long cap = (long)sm_count() * 16;
  return (int)(b < 1 ? 1 : (b < cap ? b : cap));
}

}  // namespace tb
using namespace tb;

TB_EXPORT int tb_reduce_axis(const void* x, void* y, long outer, long axis, long inner, int op, int dtype, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (outer <= 0 || axis <= 0 || inner <= 0) return 0;
  if (inner == 1) {
    int threads = axis >= 2048 ? 512 : (axis >= 256 ? 128 : 32);
    int grid = (int)(outer < (long)sm_count() * 16 ? outer : (long)sm_count() * 16);
    if (dtype == 0) reduce_rows_kernel<bf16><<<grid, threads, 0, st>>>((const bf16*)x, (bf16*)y, outer, axis, op);
    else reduce_rows_kernel<float><<<grid, threads, 0, st>>>((const float*)x, (float*)y, outer, axis, op);
  } else {
    if (outer > 65535) TB_FAIL(TB_E_ARG, "reduce: outer=%ld exceeds grid.y limit", outer);
    dim3 grid((unsigned)((inner + 31) / 32), (unsigned)outer), block(32, 8);
    if (dtype == 0) reduce_inner_kernel<bf16><<<grid, block, 0, st>>>((const bf16*)x, (bf16*)y, outer, axis, inner, op);
    else reduce_inner_kernel<float><<<grid, block, 0, st>>>((const float*)x, (float*)y, outer, axis, inner, op);
  }
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
TB_EXPORT int tb_sum_f32(const float* x, float* out, long n, float scale, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  sum_f32_kernel<<<1, 1024, 0, st>>>(x, out, n, scale);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
// Device-side index checks (see common.cuh): `word` is the device status word, or null to switch the reports off.
int tb_set_check_word_xent(int* word);
int tb_set_check_word_moe(int* word);
int tb_set_check_word_quant_sparse(int* word);
TB_EXPORT int tb_set_kernel_checks(int* word) {
  TB_ENSURE_DEVICE();
  TB_CUDA_CHECK(set_check_word_this_tu(word));
  if (int r = tb_set_check_word_xent(word)) return r;
  if (int r = tb_set_check_word_moe(word)) return r;
  return tb_set_check_word_quant_sparse(word);
}

TB_EXPORT int tb_embedding_fwd(const long* ids, const void* wte, const void* wpe, void* out, long tokens,
                               int H, int seq, long vocab, int dtype, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (tokens <= 0) return 0;
  int N = dtype == 0 ? 8 : 4;
  if (H % N) TB_FAIL(TB_E_ARG, "embedding: H=%d must be a multiple of %d", H, N);
  long total = tokens * (H / N);
  if (dtype == 0) embedding_fwd_kernel<bf16><<<grid_for(total), 256, 0, st>>>(ids, (const bf16*)wte, (const bf16*)wpe, (bf16*)out, tokens, H, seq, vocab);
  else embedding_fwd_kernel<float><<<grid_for(total), 256, 0, st>>>(ids, (const float*)wte, (const float*)wpe, (float*)out, tokens, H, seq, vocab);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
TB_EXPORT int tb_embedding_bwd(const long* ids, const void* dout, float* dwte, float* dwpe, long tokens,
                               int H, int seq, long vocab, int dtype, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (tokens <= 0) return 0;
  long total = tokens * H;
  if (dtype == 0) embedding_bwd_kernel<bf16><<<grid_for(total), 256, 0, st>>>(ids, (const bf16*)dout, dwte, dwpe, tokens, H, seq, vocab);
  else embedding_bwd_kernel<float><<<grid_for(total), 256, 0, st>>>(ids, (const float*)dout, dwte, dwpe, tokens, H, seq, vocab);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
TB_EXPORT int tb_gnn_scatter(const void* x, const long* src, const long* dst, const float* w, float* out, long E,
                             int F, long n_src, long n_dst, int dtype, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (E <= 0) return 0;
  if (F % 4) TB_FAIL(TB_E_ARG, "gnn_scatter: feature count must be a multiple of 4");
  if (((uintptr_t)out & 15) != 0) TB_FAIL(TB_E_ARG, "gnn_scatter: output must be 16-byte aligned");
  long total = E * (F / 4);
  if (dtype == 0) gnn_scatter_kernel<bf16><<<grid_for(total), 256, 0, st>>>((const bf16*)x, src, dst, w, out, E, F, n_src, n_dst);
  else gnn_scatter_kernel<float><<<grid_for(total), 256, 0, st>>>((const float*)x, src, dst, w, out, E, F, n_src, n_dst);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
TB_EXPORT int tb_rope(const void* x, void* y, long B, int S, int heads, int D, float base, int pos_offset,
                      int inverse, int dtype, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (B <= 0) return 0;
  if (D % 2) TB_FAIL(TB_E_ARG, "rope: head dim must be even");
  long total = B * S * heads * (D / 2);
  float sign = inverse ? -1.f : 1.f;
  if (dtype == 0) rope_kernel<bf16><<<grid_for(total), 256, 0, st>>>((const bf16*)x, (bf16*)y, B, S, heads, D, base, pos_offset, sign);
  else rope_kernel<float><<<grid_for(total), 256, 0, st>>>((const float*)x, (float*)y, B, S, heads, D, base, pos_offset, sign);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
