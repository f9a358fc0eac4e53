// Fused multi-tensor optimizer kernels for sm_100a: AdamW / Adam, SGD-momentum, LAMB,
// gradient norm, clip / unscale with inf check, zero.
//
// tb_adam_multi's `dyn` (optional, 3 floats on the device: lr, 1-beta1^t, 1-beta2^t) overrides the
// by-value scalars, so that a step captured in a CUDA graph keeps advancing.
// All kernels take a device-resident table of tensors (pointers + length) and a block map
// (tensor index, chunk index per CTA), so one launch updates every parameter of a model; a flat
// FSDP shard is simply a table with one entry. State is fp32 (master weights, exp_avg,
// exp_avg_sq); a bf16 copy of each parameter is written in the same pass for the next forward.
//
// Arithmetic follows the reference optimizers exactly:
//   AdamW (crates/torsh-optim/src/adam.rs:809-950): p -= lr*wd*p; m,v update; BOTH moments are
//     bias-corrected (m/(1-b1^t), v/(1-b2^t)) before p -= lr * mhat / (sqrt(vhat) + eps).
//   SGD (crates/torsh-optim/src/sgd.rs:443-610): d = g + wd*p; buf = mu*buf + (1-damp)*d with
//     buf starting at zero; nesterov d += mu*buf else d = buf; p -= lr*d.
//   LAMB (crates/torsh-optim/src/lamb.rs:24-140): g' = g + wd*p before the moments;
//     u = mhat/(sqrt(vhat)+eps); trust = |p|/|u| if both > eps else 1, clamped to <= threshold.
#include "common.cuh"
#include "host_util.h"

namespace tb {

constexpr int MT_CHUNK = 16384;  // elements per CTA
constexpr int MT_THREADS = 256;

struct MtEntry {
  void* p[6];
  long n;
};

// grad dtype: 0 = bf16, 1 = fp32
__device__ __forceinline__ float load_grad(const void* g, long i, int gdtype) {
  return gdtype == 0 ? __bfloat162float(reinterpret_cast<const bf16*>(g)[i])
                     : reinterpret_cast<const float*>(g)[i];
}

struct AdamArgs {
  float lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale;
  int decoupled;   // 1 = AdamW, 0 = Adam (L2 added to the gradient)
  int amsgrad;
  int gdtype;
  int zero_grad;
};

// slots: 0 = low-precision param copy (bf16, may be null), 1 = master fp32, 2 = grad,
//        3 = exp_avg, 4 = exp_avg_sq, 5 = max_exp_avg_sq (amsgrad only)
__global__ void __launch_bounds__(MT_THREADS)
adam_kernel(const MtEntry* __restrict__ table, const int* __restrict__ blk_tensor,
            const int* __restrict__ blk_chunk, AdamArgs a, const float* __restrict__ found_inf,
            const float* __restrict__ dyn) {
  if (found_inf && *found_inf != 0.f) return;  // AMP: skip the step on overflow
  if (dyn) {  // step-dependent scalars read from device memory so a captured graph stays valid
    a.lr = dyn[0];
    a.bc1 = dyn[1];
    a.bc2 = dyn[2];
  }
  const MtEntry e = table[blk_tensor[blockIdx.x]];
  const long base = (long)blk_chunk[blockIdx.x] * MT_CHUNK;
  const long end = min(e.n, base + MT_CHUNK);
  bf16* lowp = reinterpret_cast<bf16*>(e.p[0]);
  float* w = reinterpret_cast<float*>(e.p[1]);
  void* g = e.p[2];
  float* m = reinterpret_cast<float*>(e.p[3]);
  float* v = reinterpret_cast<float*>(e.p[4]);
  float* vmax = reinterpret_cast<float*>(e.p[5]);
  auto step = [&](float& p, float gi, float& mi, float& vi, float& vm) {
    gi *= a.grad_scale;
    if (a.decoupled) p -= a.lr * a.wd * p; else gi += a.wd * p;
    mi = a.beta1 * mi + (1.f - a.beta1) * gi;
    vi = a.beta2 * vi + (1.f - a.beta2) * gi * gi;
    float vh = vi / a.bc2;
    if (a.amsgrad) {
      vm = fmaxf(vm, vh);
      vh = vm;
    }
    p -= a.lr * (mi / a.bc1) / (sqrtf(vh) + a.eps);
  };
  const bool vec_ok = !a.amsgrad && a.gdtype == 1 && ((base & 3) == 0) && ((end & 3) == 0) &&
                      ((((uintptr_t)w | (uintptr_t)g | (uintptr_t)m | (uintptr_t)v) & 15) == 0) &&
                      (((uintptr_t)lowp & 7) == 0);
  if (vec_ok) {
    // 16-byte path: 4 elements per thread per iteration
    for (long i = base + 4 * threadIdx.x; i < end; i += 4 * MT_THREADS) {
      float4 p4 = *reinterpret_cast<float4*>(w + i);
      float4 g4 = *reinterpret_cast<float4*>(reinterpret_cast<float*>(g) + i);
      float4 m4 = *reinterpret_cast<float4*>(m + i);
      float4 v4 = *reinterpret_cast<float4*>(v + i);
      float dummy = 0.f;
      step(p4.x, g4.x, m4.x, v4.x, dummy);
      step(p4.y, g4.y, m4.y, v4.y, dummy);
      step(p4.z, g4.z, m4.z, v4.z, dummy);
      step(p4.w, g4.w, m4.w, v4.w, dummy);
      *reinterpret_cast<float4*>(w + i) = p4;
      *reinterpret_cast<float4*>(m + i) = m4;
      *reinterpret_cast<float4*>(v + i) = v4;
      if (lowp) {
        uint2 o;
        __nv_bfloat162 lo = __floats2bfloat162_rn(p4.x, p4.y), hi = __floats2bfloat162_rn(p4.z, p4.w);
        o.x = *reinterpret_cast<uint32_t*>(&lo);
        o.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(lowp + i) = o;
      }
      if (a.zero_grad) *reinterpret_cast<float4*>(reinterpret_cast<float*>(g) + i) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    return;
  }
  for (long i = base + threadIdx.x; i < end; i += MT_THREADS) {
    float gi = load_grad(g, i, a.gdtype);
    float p = w[i], mi = m[i], vi = v[i];
    float vm = a.amsgrad ? vmax[i] : 0.f;
    step(p, gi, mi, vi, vm);
    m[i] = mi;
    v[i] = vi;
    if (a.amsgrad) vmax[i] = vm;
    w[i] = p;
    if (lowp) lowp[i] = __float2bfloat16(p);
    if (a.zero_grad) {
      if (a.gdtype == 0) reinterpret_cast<bf16*>(g)[i] = __float2bfloat16(0.f);
      else reinterpret_cast<float*>(g)[i] = 0.f;
    }
  }
}

struct SgdArgs {
  float lr, momentum, dampening, wd, grad_scale;
  int nesterov, gdtype, zero_grad;
};
// slots: 0 = bf16 copy (nullable), 1 = master fp32, 2 = grad, 3 = momentum buffer (nullable if mu == 0)
__global__ void __launch_bounds__(MT_THREADS)
sgd_kernel(const MtEntry* __restrict__ table, const int* __restrict__ blk_tensor,
           const int* __restrict__ blk_chunk, SgdArgs a, const float* __restrict__ found_inf) {
  if (found_inf && *found_inf != 0.f) return;
  const MtEntry e = table[blk_tensor[blockIdx.x]];
  const long base = (long)blk_chunk[blockIdx.x] * MT_CHUNK;
  const long end = min(e.n, base + MT_CHUNK);
  bf16* lowp = reinterpret_cast<bf16*>(e.p[0]);
  float* w = reinterpret_cast<float*>(e.p[1]);
  void* g = e.p[2];
  float* buf = reinterpret_cast<float*>(e.p[3]);
  for (long i = base + threadIdx.x; i < end; i += MT_THREADS) {
    float p = w[i];
    float d = load_grad(g, i, a.gdtype) * a.grad_scale + a.wd * p;
    if (a.momentum != 0.f) {
      float b = a.momentum * buf[i] + (1.f - a.dampening) * d;
      buf[i] = b;
      d = a.nesterov ? d + a.momentum * b : b;
    }
    p -= a.lr * d;
    w[i] = p;
    if (lowp) lowp[i] = __float2bfloat16(p);
    if (a.zero_grad) {
      if (a.gdtype == 0) reinterpret_cast<bf16*>(g)[i] = __float2bfloat16(0.f);
      else reinterpret_cast<float*>(g)[i] = 0.f;
    }
  }
}

struct LambArgs {
  float lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale, trust_clip;
  int gdtype;
};
// Phase 1: moments + update direction u (stored in slot 5), per-tensor |p|^2 and |u|^2 in norms[2*t].
// slots: 0 = bf16 copy, 1 = master, 2 = grad, 3 = exp_avg, 4 = exp_avg_sq, 5 = update scratch (fp32)
__global__ void __launch_bounds__(MT_THREADS)
lamb_phase1_kernel(const MtEntry* __restrict__ table, const int* __restrict__ blk_tensor,
                   const int* __restrict__ blk_chunk, LambArgs a, float* __restrict__ norms) {
  __shared__ float scratch[32];
  const int t = blk_tensor[blockIdx.x];
  const MtEntry e = table[t];
  const long base = (long)blk_chunk[blockIdx.x] * MT_CHUNK;
  const long end = min(e.n, base + MT_CHUNK);
  float* w = reinterpret_cast<float*>(e.p[1]);
  void* g = e.p[2];
  float* m = reinterpret_cast<float*>(e.p[3]);
  float* v = reinterpret_cast<float*>(e.p[4]);
  float* u = reinterpret_cast<float*>(e.p[5]);
  float pn = 0.f, un = 0.f;
  for (long i = base + threadIdx.x; i < end; i += MT_THREADS) {
    float p = w[i];
    float gi = load_grad(g, i, a.gdtype) * a.grad_scale + a.wd * p;
    float mi = a.beta1 * m[i] + (1.f - a.beta1) * gi;
    float vi = a.beta2 * v[i] + (1.f - a.beta2) * gi * gi;
    m[i] = mi;
    v[i] = vi;
    float ui = (mi / a.bc1) / (sqrtf(vi / a.bc2) + a.eps);
    u[i] = ui;
    pn += p * p;
    un += ui * ui;
  }
  pn = block_sum(pn, scratch);
  un = block_sum(un, scratch);
  if (threadIdx.x == 0) {
    atomicAdd(norms + 2 * t, pn);
    atomicAdd(norms + 2 * t + 1, un);
  }
}
__global__ void __launch_bounds__(MT_THREADS)
lamb_phase2_kernel(const MtEntry* __restrict__ table, const int* __restrict__ blk_tensor,
                   const int* __restrict__ blk_chunk, LambArgs a, const float* __restrict__ norms) {
  const int t = blk_tensor[blockIdx.x];
  const MtEntry e = table[t];
  const long base = (long)blk_chunk[blockIdx.x] * MT_CHUNK;
  const long end = min(e.n, base + MT_CHUNK);
  bf16* lowp = reinterpret_cast<bf16*>(e.p[0]);
  float* w = reinterpret_cast<float*>(e.p[1]);
  const float* u = reinterpret_cast<const float*>(e.p[5]);
  const float pn = sqrtf(norms[2 * t]), un = sqrtf(norms[2 * t + 1]);
  float trust = (pn > a.eps && un > a.eps) ? pn / un : 1.f;
  trust = fminf(trust, a.trust_clip);
  for (long i = base + threadIdx.x; i < end; i += MT_THREADS) {
    float p = w[i] - a.lr * trust * u[i];
    w[i] = p;
    if (lowp) lowp[i] = __float2bfloat16(p);
  }
}

// Sum of squares of slot `slot` over all tensors, accumulated into *out (fp32). With
// per_tensor != null also accumulates per-tensor sums.
__global__ void __launch_bounds__(MT_THREADS)
sqnorm_kernel(const MtEntry* __restrict__ table, const int* __restrict__ blk_tensor,
              const int* __restrict__ blk_chunk, int slot, int dtype, float* __restrict__ out,
              float* __restrict__ per_tensor) {
  __shared__ float scratch[32];
  const int t = blk_tensor[blockIdx.x];
  const MtEntry e = table[t];
  const long base = (long)blk_chunk[blockIdx.x] * MT_CHUNK;
  const long end = min(e.n, base + MT_CHUNK);
  float s = 0.f;
  for (long i = base + threadIdx.x; i < end; i += MT_THREADS) {
    float x = load_grad(e.p[slot], i, dtype);
    s += x * x;
  }
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) {
    atomicAdd(out, s);
    if (per_tensor) atomicAdd(per_tensor + t, s);
  }
}

// g *= scale where scale = *scale_ptr (if non-null) else scale_imm; records non-finite values in
// *found_inf (set to 1). mode 1: scale = min(1, max_norm / (sqrt(*sqnorm) + 1e-6)) (clip by norm).
__global__ void __launch_bounds__(MT_THREADS)
scale_kernel(const MtEntry* __restrict__ table, const int* __restrict__ blk_tensor,
             const int* __restrict__ blk_chunk, int slot, int dtype, float scale_imm,
             const float* __restrict__ sqnorm, float max_norm, int mode,
             float* __restrict__ found_inf) {
  const MtEntry e = table[blk_tensor[blockIdx.x]];
  const long base = (long)blk_chunk[blockIdx.x] * MT_CHUNK;
  const long end = min(e.n, base + MT_CHUNK);
  float scale = scale_imm;
  if (mode == 1) {
    float nrm = sqrtf(*sqnorm);
    scale = fminf(1.f, max_norm / (nrm + 1e-6f));
    if (scale == 1.f && !found_inf) return;
  }
  bool bad = false;
  for (long i = base + threadIdx.x; i < end; i += MT_THREADS) {
    float x = load_grad(e.p[slot], i, dtype);
    if (!isfinite(x)) bad = true;
    x *= scale;
    if (dtype == 0) reinterpret_cast<bf16*>(e.p[slot])[i] = __float2bfloat16(x);
    else reinterpret_cast<float*>(e.p[slot])[i] = x;
  }
  if (bad && found_inf) *found_inf = 1.f;
}

}  // namespace tb
using namespace tb;

TB_EXPORT int tb_mt_chunk() { return MT_CHUNK; }

TB_EXPORT int tb_adam_multi(const void* table, const int* blk_tensor, const int* blk_chunk,
                            int nblocks, float lr, float beta1, float beta2, float eps, float wd,
                            float bc1, float bc2, float grad_scale, int decoupled, int amsgrad,
                            int gdtype, int zero_grad, const float* found_inf, const float* dyn,
                            cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (nblocks <= 0) return 0;
  AdamArgs a{lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale, decoupled, amsgrad, gdtype, zero_grad};
  adam_kernel<<<nblocks, MT_THREADS, 0, st>>>((const MtEntry*)table, blk_tensor, blk_chunk, a, found_inf, dyn);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

TB_EXPORT int tb_sgd_multi(const void* table, const int* blk_tensor, const int* blk_chunk,
                           int nblocks, float lr, float momentum, float dampening, float wd,
                           float grad_scale, int nesterov, int gdtype, int zero_grad,
                           const float* found_inf, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (nblocks <= 0) return 0;
  SgdArgs a{lr, momentum, dampening, wd, grad_scale, nesterov, gdtype, zero_grad};
  sgd_kernel<<<nblocks, MT_THREADS, 0, st>>>((const MtEntry*)table, blk_tensor, blk_chunk, a, found_inf);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// norms: fp32 [2 * num_tensors], zeroed by this call.
TB_EXPORT int tb_lamb_multi(const void* table, const int* blk_tensor, const int* blk_chunk,
                            int nblocks, int ntensors, float lr, float beta1, float beta2, float eps,
                            float wd, float bc1, float bc2, float grad_scale, float trust_clip,
                            int gdtype, float* norms, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (nblocks <= 0) return 0;
  LambArgs a{lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale, trust_clip, gdtype};
  TB_CUDA_CHECK(cudaMemsetAsync(norms, 0, sizeof(float) * 2 * ntensors, st));
  lamb_phase1_kernel<<<nblocks, MT_THREADS, 0, st>>>((const MtEntry*)table, blk_tensor, blk_chunk, a, norms);
  lamb_phase2_kernel<<<nblocks, MT_THREADS, 0, st>>>((const MtEntry*)table, blk_tensor, blk_chunk, a, norms);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// out (1 float) is zeroed by this call, then receives the sum of squares of slot `slot`.
TB_EXPORT int tb_sqnorm_multi(const void* table, const int* blk_tensor, const int* blk_chunk,
                              int nblocks, int slot, int dtype, float* out, float* per_tensor,
                              cudaStream_t st) {
  TB_ENSURE_DEVICE();
  TB_CUDA_CHECK(cudaMemsetAsync(out, 0, sizeof(float), st));
  if (nblocks <= 0) return 0;
  sqnorm_kernel<<<nblocks, MT_THREADS, 0, st>>>((const MtEntry*)table, blk_tensor, blk_chunk, slot, dtype, out, per_tensor);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}

TB_EXPORT int tb_scale_multi(const void* table, const int* blk_tensor, const int* blk_chunk,
                             int nblocks, int slot, int dtype, float scale, const float* sqnorm,
                             float max_norm, int mode, float* found_inf, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (nblocks <= 0) return 0;
  scale_kernel<<<nblocks, MT_THREADS, 0, st>>>((const MtEntry*)table, blk_tensor, blk_chunk, slot, dtype, scale, sqnorm, max_norm, mode, found_inf);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
