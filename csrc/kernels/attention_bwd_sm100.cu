// Flash attention backward for sm_100a (tcgen05 / TMEM / TMA), causal or full, head dim 64 / 128.
//
// One CTA per (batch, head, 128-key block); it walks the query blocks that see those keys:
//   S  = Q_i K_j^T          dP = dO_i V_j^T                   (tensor core, into TMEM)
//   P  = exp(S*scale - L_i) dS = P * (dP - delta_i) * scale   (compute warps, fp32)
//   dV_j += P^T dO_i        dK_j += dS^T Q_i                  (accumulate in TMEM over i)
//   dQ_i += dS K_j                                            (TMEM -> fp32 atomics in global)
// P and dS are written by the compute warps into shared memory in the 128-byte-swizzled layout
// that tcgen05.mma descriptors read, once, and that one buffer serves both as the K-major A
// operand (dQ) and as the MN-major A operand (dK, dV) - no transposes anywhere. Q, dO, K, V tiles
// are the TMA-loaded tiles themselves, used K-major or MN-major as each product needs.
// TMEM: S | dP (128 cols each) | dV | dK (D each) | dQ partial (D; aliases S when D = 128).
// Warps 0-7 compute (two threads per query row = TMEM lane, each owning half of the columns), warp 8
// issues MMAs, warp 9 drives TMA.
//
// The reference has no attention backward at all (its autograd tape covers only
// add/sub/mul/matmul/pow/mean/sum: crates/torsh-tensor/src/core_ops/types.rs:1497-1658).
#include "host_util.h"
#include "sm100.cuh"

namespace tb {

constexpr int FB_THREADS = 320;  // 8 compute warps + MMA warp + TMA warp

struct FaBwdParams {
  const float* LSE;    // [B, H, S]
  const float* delta;  // [B, H, S]  rowsum(dO * O)
  float* dQ_acc;       // fp32 [B*S, H*D] accumulated with atomics
  __nv_bfloat16* dK;   // [B*S, dkv_stride], head h at column h*D
  __nv_bfloat16* dV;
  int B, S, H;
  long dkv_stride;
  float scale;
  int causal;
  int* status;
};

template <int D>
struct FaBwdSmem {
  static constexpr int TILE = 128 * D * 2;
  static constexpr int QST = (D == 64) ? 2 : 1;  // Q / dO ring depth
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = TILE;
  static constexpr int Q_OFF = 2 * TILE;
  static constexpr int DO_OFF = Q_OFF + QST * TILE;
  static constexpr int P_OFF = DO_OFF + QST * TILE;
  static constexpr int DS_OFF = P_OFF + 32768;
  static constexpr int BAR_OFF = DS_OFF + 32768;
  // kv_full, q_full[2], q_empty[2], do_full[2], do_empty[2], s_full, dp_full, ds_full,
  // pds_empty, dq_full, dq_empty, dkv_full, s_free, dp_free
  static constexpr int NBARS = 18;
  static constexpr int TOTAL = BAR_OFF + NBARS * 8 + 16;
  static constexpr int ALLOC = TOTAL + 1024;
};

// P = exp2(S * sl2 - L) and dS = P * (dP - delta) * scale for 32 scores of one row, both packed to bf16 pairs. The
// scale-and-shift steps run as packed two-wide fp32 instructions; MASK is a template parameter so that blocks away from
// the diagonal and the ragged edge carry no compare / select instructions.
template <bool MASK>
__device__ __forceinline__ void fa_bwd_p_ds(const uint32_t (&sv)[32], const uint32_t (&dv)[32], float sl2, float Lr,
                                            float scale, float dr, int kvbase, int col_limit, uint32_t (&pp)[16],
                                            uint32_t (&dd)[16]) {
  const float2 s2 = make_float2(sl2, sl2), l2 = make_float2(-Lr, -Lr);
  const float2 c2 = make_float2(scale, scale), d2 = make_float2(-dr * scale, -dr * scale);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float2 t = __ffma2_rn(make_float2(__uint_as_float(sv[2 * i]), __uint_as_float(sv[2 * i + 1])), s2, l2);
    float2 e = make_float2(exp2f(t.x), exp2f(t.y));
    if (MASK) {
      if (kvbase + 2 * i > col_limit) e.x = 0.f;
      if (kvbase + 2 * i + 1 > col_limit) e.y = 0.f;
    }
    const float2 g = __ffma2_rn(make_float2(__uint_as_float(dv[2 * i]), __uint_as_float(dv[2 * i + 1])), c2, d2);
    const float2 ds = __fmul2_rn(e, g);
    pp[i] = pack_bf16x2(e.x, e.y);
    dd[i] = pack_bf16x2(ds.x, ds.y);
  }
}

template <int D>
__global__ void __launch_bounds__(FB_THREADS, 1)
fa_bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
              const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
              const FaBwdParams p) {
  using L = FaBwdSmem<D>;
  constexpr int KCH = D / 64;
  constexpr int QST = L::QST;
  constexpr uint32_t TM_S = 0, TM_DP = 128, TM_DV = 256, TM_DK = 256 + D;
  constexpr uint32_t TM_DQ = (D == 64) ? 384 : 0;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + L::BAR_OFF);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;
  uint64_t* q_empty = bars + 3;
  uint64_t* do_full = bars + 5;
  uint64_t* do_empty = bars + 7;
  uint64_t* s_full = bars + 9;
  uint64_t* dp_full = bars + 10;
  uint64_t* ds_full = bars + 11;
  uint64_t* pds_empty = bars + 12;
  uint64_t* dq_full = bars + 13;
  uint64_t* dq_empty = bars + 14;
  uint64_t* dkv_full = bars + 15;
  uint64_t* s_free = bars + 16;    // compute warps have read S of the current block out of TMEM (head dim 64 only)
  uint64_t* dp_free = bars + 17;   // ... and dP
  // Head dim 64 runs software-pipelined: the score MMAs of query block t + 1 are issued as soon as the compute warps
  // have copied S[t] / dP[t] into registers, so the tensor core works on block t + 1 while they evaluate the
  // exponentials of block t, and the dQ partial of block t is drained (TMEM -> fp32 reductions) after the compute of
  // block t + 1, when its MMAs have long finished. With head dim 128 dQ shares TMEM columns with S, which forbids the
  // early issue, and the blocks run one after the other.
  constexpr bool PIPELINED = (D == 64);
  uint32_t* tmem_ptr = (uint32_t*)(bars + L::NBARS);
  volatile int* abort_flag = (volatile int*)(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_blk = (p.S + 127) / 128;
  const int jb = blockIdx.x % n_blk;  // key block; early key blocks (most work when causal) first
  const int bh = blockIdx.x / n_blk;
  const int h = bh % p.H, b = bh / p.H;
  const int kv0 = jb * 128;
  const int i0 = p.causal ? jb : 0;
  const int n_it = n_blk - i0;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
      mbar_init(&do_full[i], 1);
      mbar_init(&do_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(ds_full, 256);
    mbar_init(pds_empty, 1);
    mbar_init(dq_full, 1);
    mbar_init(dq_empty, 256);
    mbar_init(dkv_full, 1);
    mbar_init(s_free, 256);
    mbar_init(dp_free, 256);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 8) {
    tmem_alloc(tmem_ptr, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;

  if (warp == 9) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      tma_prefetch_desc(&map_do);
      mbar_expect_tx(kv_full, 2 * L::TILE);
#pragma unroll
      for (int c = 0; c < KCH; ++c) {
        tma_load_4d(smem + L::K_OFF + c * 16384, &map_k, kv_full, c * 64, h, kv0, b);
        tma_load_4d(smem + L::V_OFF + c * 16384, &map_v, kv_full, c * 64, h, kv0, b);
      }
      for (int t = 0; t < n_it; ++t) {
        const int s = t % QST;
        const uint32_t ph = (t / QST) & 1;
        const int qrow0 = (i0 + t) * 128;
        // once a wait has given up, nothing more is loaded: loads without a free slot would pile transaction counts
        // on one barrier beyond its range
        if (!mbar_wait(&q_empty[s], ph ^ 1, abort_flag, p.status, TB_ERR_WAIT_EMPTY)) break;
        mbar_expect_tx(&q_full[s], L::TILE);
#pragma unroll
        for (int c = 0; c < KCH; ++c)
          tma_load_4d(smem + L::Q_OFF + s * L::TILE + c * 16384, &map_q, &q_full[s], c * 64, h, qrow0, b);
        if (!mbar_wait(&do_empty[s], ph ^ 1, abort_flag, p.status, TB_ERR_WAIT_EMPTY)) break;
        mbar_expect_tx(&do_full[s], L::TILE);
#pragma unroll
        for (int c = 0; c < KCH; ++c)
          tma_load_4d(smem + L::DO_OFF + s * L::TILE + c * 16384, &map_do, &do_full[s], c * 64, h, qrow0, b);
      }
      if (*abort_flag) {
        uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) {
        }
      }
    }
  } else if (warp == 8) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_dkv = make_idesc_bf16(128, D, 1, 1);
      constexpr uint32_t idesc_dq = make_idesc_bf16(128, D, 0, 1);
      const uint32_t k_base = smem_u32(smem + L::K_OFF);
      const uint32_t v_base = smem_u32(smem + L::V_OFF);
      const uint32_t p_base = smem_u32(smem + L::P_OFF);
      const uint32_t ds_base = smem_u32(smem + L::DS_OFF);
      mbar_wait(kv_full, 0, abort_flag, p.status, TB_ERR_WAIT_FULL);
      // S = Q_t K^T and dP = dO_t V^T of query block t (each waits for its TMEM columns when pipelined)
      auto issue_scores = [&](int t) {
        const int s = t % QST;
        const uint32_t ph = (t / QST) & 1;
        const uint32_t q_base = smem_u32(smem + L::Q_OFF + s * L::TILE);
        const uint32_t do_base = smem_u32(smem + L::DO_OFF + s * L::TILE);
        if (PIPELINED && t > 0) mbar_wait(s_free, (t - 1) & 1, abort_flag, p.status, TB_ERR_WAIT_TMEM_EMPTY);
        mbar_wait(&q_full[s], ph, abort_flag, p.status, TB_ERR_WAIT_FULL);
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < KCH; ++c)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_ss(tmem_base + TM_S, make_smem_desc_sw128(q_base + c * 16384 + k * 32, 16, 1024),
                    make_smem_desc_sw128(k_base + c * 16384 + k * 32, 16, 1024), idesc_s, (c | k) ? 1u : 0u);
        umma_commit(s_full);
        if (PIPELINED && t > 0) mbar_wait(dp_free, (t - 1) & 1, abort_flag, p.status, TB_ERR_WAIT_TMEM_EMPTY);
        mbar_wait(&do_full[s], ph, abort_flag, p.status, TB_ERR_WAIT_FULL);
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < KCH; ++c)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_ss(tmem_base + TM_DP, make_smem_desc_sw128(do_base + c * 16384 + k * 32, 16, 1024),
                    make_smem_desc_sw128(v_base + c * 16384 + k * 32, 16, 1024), idesc_s, (c | k) ? 1u : 0u);
        umma_commit(dp_full);
      };
      if (PIPELINED && n_it > 0) issue_scores(0);
      for (int t = 0; t < n_it; ++t) {
        const int s = t % QST;
        const uint32_t q_base = smem_u32(smem + L::Q_OFF + s * L::TILE);
        const uint32_t do_base = smem_u32(smem + L::DO_OFF + s * L::TILE);
        if (PIPELINED) {
          if (t + 1 < n_it) issue_scores(t + 1);   // runs on the tensor core while the compute warps work on block t
        } else {
          // when dQ aliases S (D = 128) the previous dQ partial must be drained first
          if (t > 0) mbar_wait(dq_empty, (t - 1) & 1, abort_flag, p.status, TB_ERR_WAIT_TMEM_EMPTY);
          issue_scores(t);
        }
        // P and dS are in shared memory once the compute warps arrive here
        mbar_wait(ds_full, t & 1, abort_flag, p.status, TB_ERR_WAIT_MISC);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ss(tmem_base + TM_DV, make_smem_desc_sw128(p_base + kk * 2048, 16384, 1024),
                  make_smem_desc_sw128(do_base + kk * 2048, 16384, 1024), idesc_dkv, (t | kk) ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ss(tmem_base + TM_DK, make_smem_desc_sw128(ds_base + kk * 2048, 16384, 1024),
                  make_smem_desc_sw128(q_base + kk * 2048, 16384, 1024), idesc_dkv, (t | kk) ? 1u : 0u);
        if (D == 64 && t > 0) mbar_wait(dq_empty, (t - 1) & 1, abort_flag, p.status, TB_ERR_WAIT_TMEM_EMPTY);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ss(tmem_base + TM_DQ,
                  make_smem_desc_sw128(ds_base + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                  make_smem_desc_sw128(k_base + kk * 2048, 16384, 1024), idesc_dq, kk ? 1u : 0u);
        umma_commit(dq_full);
        umma_commit(pds_empty);
        umma_commit(&q_empty[s]);
        umma_commit(&do_empty[s]);
      }
      umma_commit(dkv_full);
    }
  } else {
    // ---------------------------------------------------------------- compute (8 warps)
    // Two warps per group of 32 rows: warps 0-3 take key columns 0-63 (and the first half of the
    // dQ / dK / dV columns), warps 4-7 the rest; no exchange is needed, L and delta are per row.
    const int half = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const float sl2 = p.scale * 1.4426950408889634f;
    uint8_t* p_smem = smem + L::P_OFF;
    uint8_t* ds_smem = smem + L::DS_OFF;
    const int sw = row & 7;
    // dQ partial of query block tt: TMEM -> fp32 reductions into the global accumulator
    auto drain_dq = [&](int tt) {
      const int qd = (i0 + tt) * 128 + row;
      const bool ok = qd < p.S;
      mbar_wait(dq_full, tt & 1, abort_flag, p.status, TB_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
      float* dq_row = p.dQ_acc + ((size_t)b * p.S + (ok ? qd : 0)) * ((size_t)p.H * D) + (size_t)h * D;
#pragma unroll 1
      for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_base + TM_DQ + c * 32 + lane_off, v);
        tmem_wait_ld();
        if (ok) {
#pragma unroll
          for (int g = 0; g < 8; ++g)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dq_row + c * 32 + g * 4),
                         "f"(__uint_as_float(v[g * 4])), "f"(__uint_as_float(v[g * 4 + 1])),
                         "f"(__uint_as_float(v[g * 4 + 2])), "f"(__uint_as_float(v[g * 4 + 3]))
                         : "memory");
        }
      }
      tc_fence_before();
      mbar_arrive(dq_empty);
    };
    for (int t = 0; t < n_it; ++t) {
      const int qi = (i0 + t) * 128 + row;
      const bool q_ok = qi < p.S;
      const size_t stat_idx = ((size_t)b * p.H + h) * p.S + (q_ok ? qi : 0);
      const float Lr = q_ok ? p.LSE[stat_idx] * 1.4426950408889634f : INFINITY;
      const float dr = q_ok ? p.delta[stat_idx] : 0.f;
      const bool need_mask = (p.causal && (i0 + t) == jb) || (kv0 + 128 > p.S);
      const int col_limit = p.causal ? min(qi, p.S - 1) : p.S - 1;
      mbar_wait(s_full, t & 1, abort_flag, p.status, TB_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
      // this thread's 64 score columns go to registers at once, so that the tensor core may overwrite S
      uint32_t sv0[32], sv1[32];
      tmem_ld32(tmem_base + TM_S + (half * 2) * 32 + lane_off, sv0);
      tmem_ld32(tmem_base + TM_S + (half * 2 + 1) * 32 + lane_off, sv1);
      tmem_wait_ld();
      if (PIPELINED) {
        tc_fence_before();
        mbar_arrive(s_free);
      }
      mbar_wait(dp_full, t & 1, abort_flag, p.status, TB_ERR_WAIT_TMEM_FULL);
      // the previous iteration's MMAs must be done reading P / dS from shared memory
      mbar_wait(pds_empty, (t & 1) ^ 1, abort_flag, p.status, TB_ERR_WAIT_EMPTY);
      tc_fence_after();
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = half * 2 + cc;
        uint32_t dv[32];
        tmem_ld32(tmem_base + TM_DP + c * 32 + lane_off, dv);
        tmem_wait_ld();
        if (PIPELINED && cc == 1) {
          tc_fence_before();
          mbar_arrive(dp_free);
        }
        uint32_t pp[16], dd[16];
        const uint32_t (&sv)[32] = cc == 0 ? sv0 : sv1;
        if (need_mask) fa_bwd_p_ds<true>(sv, dv, sl2, Lr, p.scale, dr, kv0 + c * 32, col_limit, pp, dd);
        else fa_bwd_p_ds<false>(sv, dv, sl2, Lr, p.scale, dr, kv0 + c * 32, col_limit, pp, dd);
        // columns c*32 .. c*32+31 = four 16-byte chunks of sub-tile c/2 (64 keys per sub-tile)
        const int sub = c >> 1;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int ch = (c & 1) * 4 + g;
          const int off = sub * 16384 + row * 128 + ((ch ^ sw) << 4);
          *reinterpret_cast<uint4*>(p_smem + off) = make_uint4(pp[g * 4], pp[g * 4 + 1], pp[g * 4 + 2], pp[g * 4 + 3]);
          *reinterpret_cast<uint4*>(ds_smem + off) = make_uint4(dd[g * 4], dd[g * 4 + 1], dd[g * 4 + 2], dd[g * 4 + 3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(ds_full);
      if (PIPELINED) {
        if (t > 0) drain_dq(t - 1);   // finished long ago: the MMAs of block t - 1 ran under this block's exponentials
      } else {
        drain_dq(t);
      }
    }
    if (PIPELINED && n_it > 0) drain_dq(n_it - 1);
    // dK, dV of this key block: thread = key row
    mbar_wait(dkv_full, 0, abort_flag, p.status, TB_ERR_WAIT_TMEM_FULL);
    tc_fence_after();
    const int kvi = kv0 + row;
    const bool kv_ok = kvi < p.S;
    __nv_bfloat16* dk_row = p.dK + ((size_t)b * p.S + (kv_ok ? kvi : 0)) * p.dkv_stride + (size_t)h * D;
    __nv_bfloat16* dv_row = p.dV + ((size_t)b * p.S + (kv_ok ? kvi : 0)) * p.dkv_stride + (size_t)h * D;
#pragma unroll 1
    for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
      uint32_t kvv[32], vvv[32];
      tmem_ld32(tmem_base + TM_DK + c * 32 + lane_off, kvv);
      tmem_ld32(tmem_base + TM_DV + c * 32 + lane_off, vvv);
      tmem_wait_ld();
      if (kv_ok) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 a, d2;
          a.x = pack_bf16x2(__uint_as_float(kvv[g * 8 + 0]), __uint_as_float(kvv[g * 8 + 1]));
          a.y = pack_bf16x2(__uint_as_float(kvv[g * 8 + 2]), __uint_as_float(kvv[g * 8 + 3]));
          a.z = pack_bf16x2(__uint_as_float(kvv[g * 8 + 4]), __uint_as_float(kvv[g * 8 + 5]));
          a.w = pack_bf16x2(__uint_as_float(kvv[g * 8 + 6]), __uint_as_float(kvv[g * 8 + 7]));
          d2.x = pack_bf16x2(__uint_as_float(vvv[g * 8 + 0]), __uint_as_float(vvv[g * 8 + 1]));
          d2.y = pack_bf16x2(__uint_as_float(vvv[g * 8 + 2]), __uint_as_float(vvv[g * 8 + 3]));
          d2.z = pack_bf16x2(__uint_as_float(vvv[g * 8 + 4]), __uint_as_float(vvv[g * 8 + 5]));
          d2.w = pack_bf16x2(__uint_as_float(vvv[g * 8 + 6]), __uint_as_float(vvv[g * 8 + 7]));
          reinterpret_cast<uint4*>(dk_row + c * 32)[g] = a;
          reinterpret_cast<uint4*>(dv_row + c * 32)[g] = d2;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b, h, s] = sum_d O[b, s, h, d] * dO[b, s, h, d]. Each thread reads one 16-byte vector of O
// and dO (8 elements); the D/8 lanes of a (token, head) pair combine with shuffles.
template <int D>
__global__ void fa_delta_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO,
                                float* __restrict__ delta, int B, int S, int H, long o_stride, long do_stride) {
  constexpr int LPG = D / 8;  // lanes per (token, head)
  const long gid = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const long pair = gid / LPG;
  const int sub = (int)(gid % LPG);
  const long total = (long)B * S * H;
  float s = 0.f;
  int hh = 0;
  long tok = 0;
  if (pair < total) {
    hh = (int)(pair % H);
    tok = pair / H;
    const uint4 a = *reinterpret_cast<const uint4*>(O + tok * o_stride + (long)hh * D + sub * 8);
    const uint4 c = *reinterpret_cast<const uint4*>(dO + tok * do_stride + (long)hh * D + sub * 8);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, cw[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) s += bf16_lo(aw[i]) * bf16_lo(cw[i]) + bf16_hi(aw[i]) * bf16_hi(cw[i]);
  }
#pragma unroll
  for (int off = LPG / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (pair < total && sub == 0) {
    const long bb = tok / S, ss = tok % S;
    delta[(bb * H + hh) * S + ss] = s;
  }
}

// dst[t, col0 + c] = bf16(src[t, c]) for c < cols (fp32 accumulator -> strided bf16 gradient)
__global__ void fa_cvt_dq_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long rows,
                                 int cols, long dst_stride) {
  const long total = rows * (cols / 4);
  const long stride = (long)gridDim.x * blockDim.x;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    long r = idx / (cols / 4);
    int c = (int)(idx - r * (cols / 4)) * 4;
    float4 v = *reinterpret_cast<const float4*>(src + r * cols + c);
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(dst + r * dst_stride + c) = o;
  }
}

inline int make_bshd_map_bwd(CUtensorMap* m, const void* base, int B, int S, int H, int D, long row_stride) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)S, (uint64_t)B};
  uint64_t str[3] = {(uint64_t)D * 2, (uint64_t)row_stride * 2, (uint64_t)S * row_stride * 2};
  uint32_t box[4] = {64, 1, 128, 1};
  return make_tmap(m, base, 2, 4, dims, str, box);
}

}  // namespace tb
using namespace tb;

// Workspace (caller-provided): delta fp32 [B*H*S], dq_acc fp32 [B*S*H*D] (zeroed here).
// dq, dk, dv: bf16 [B*S, dqkv_stride] with head h at column h*D (may be the three column bands of
// one fused dQKV buffer).
TB_EXPORT int tb_flash_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                                const float* lse, void* dq, void* dk, void* dv, float* delta, float* dq_acc,
                                int B, int S, int H, int D, long q_stride, long kv_stride, long o_stride,
                                long do_stride, long dqkv_stride, float scale, int causal, int* status,
                                cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (!q || !k || !v || !o || !dout || !lse || !dq || !dk || !dv || !delta || !dq_acc)
    TB_FAIL(TB_E_ARG, "flash_attn_bwd: null pointer");
  if (D != 64 && D != 128) TB_FAIL(TB_E_ARG, "flash_attn_bwd: head dim %d not supported (64 or 128)", D);
  if ((dqkv_stride & 7) || ((uintptr_t)dq & 15) || ((uintptr_t)dk & 15) || ((uintptr_t)dv & 15))
    TB_FAIL(TB_E_ARG, "flash_attn_bwd: gradients must be 16-byte aligned");
  CUtensorMap mq, mk, mv, mdo;
  int r;
  if ((r = make_bshd_map_bwd(&mq, q, B, S, H, D, q_stride))) return r;
  if ((r = make_bshd_map_bwd(&mk, k, B, S, H, D, kv_stride))) return r;
  if ((r = make_bshd_map_bwd(&mv, v, B, S, H, D, kv_stride))) return r;
  if ((r = make_bshd_map_bwd(&mdo, dout, B, S, H, D, do_stride))) return r;
  if ((o_stride & 7) || (do_stride & 7) || ((uintptr_t)o & 15) || ((uintptr_t)dout & 15))
    TB_FAIL(TB_E_ARG, "flash_attn_bwd: o / dout must be 16-byte aligned with strides that are multiples of 8");
  const long nthreads = (long)B * S * H * (D / 8);
  if (D == 64)
    fa_delta_kernel<64><<<(unsigned)((nthreads + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta, B, S, H, o_stride, do_stride);
  else
    fa_delta_kernel<128><<<(unsigned)((nthreads + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta, B, S, H, o_stride, do_stride);
  TB_CUDA_CHECK(cudaMemsetAsync(dq_acc, 0, sizeof(float) * (size_t)B * S * H * D, st));
  FaBwdParams p{lse, delta, dq_acc, (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, B, S, H, dqkv_stride, scale, causal, status};
  const int n_blk = (S + 127) / 128;
  const long grid = (long)n_blk * B * H;
  if (D == 64) {
    static bool cfg = false;
    if (!cfg) { TB_CUDA_CHECK(cudaFuncSetAttribute(fa_bwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, FaBwdSmem<64>::ALLOC)); cfg = true; }
    fa_bwd_kernel<64><<<(unsigned)grid, FB_THREADS, FaBwdSmem<64>::ALLOC, st>>>(mq, mk, mv, mdo, p);
  } else {
    static bool cfg = false;
    if (!cfg) { TB_CUDA_CHECK(cudaFuncSetAttribute(fa_bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, FaBwdSmem<128>::ALLOC)); cfg = true; }
    fa_bwd_kernel<128><<<(unsigned)grid, FB_THREADS, FaBwdSmem<128>::ALLOC, st>>>(mq, mk, mv, mdo, p);
  }
  const long rows = (long)B * S;
  long items = rows * (H * D / 4);
  int g = (int)((items + 255) / 256 < (long)sm_count() * 16 ? (items + 255) / 256 : (long)sm_count() * 16);
  fa_cvt_dq_kernel<<<g, 256, 0, st>>>(dq_acc, (__nv_bfloat16*)dq, rows, H * D, dqkv_stride);
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
