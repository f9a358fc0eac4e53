// Flash attention forward for sm_100a (tcgen05 / TMEM / TMA), causal or full, head dim 64 or 128.
//
// One CTA per (batch, head, 128-query block), 320 threads:
//   warps 0-7  softmax: two threads per query row (= TMEM lane), each owning half of the key
//              columns of a score block and half of the output columns. Read S = Q K^T from TMEM,
//              online softmax in fp32 (exp2, running max / sum), write P as packed bf16 back to
//              TMEM, accumulate O in registers from the per-block P V partials.
//   warp 8     MMA issuer (one thread): S[j+1] = Q K[j+1]^T is issued before waiting for P[j],
//              so the tensor core works on the next block while the softmax warps run.
//   warp 9     TMA producer (one thread): Q once, K / V tiles through 2-deep rings.
// TMEM (512 columns): S0 | S1 (128 each, fp32) | P0 | P1 (64 each, bf16 pairs) | O partial (D).
// Memory is O(S): nothing of size S x S is ever written. Q, K, V are addressed through 4-D tensor
// maps [B, S, H, D] with arbitrary token stride, so the fused QKV projection output is consumed
// in place; O is written token-major [B*S, H*D] ready for the output projection GEMM.
//
// The reference's "flash attention" tiles queries in blocks of 64 but still materialises a
// [block, S] score matrix against all keys and has no backward
// (crates/torsh-functional/src/attention.rs:493-629).
#include "host_util.h"
#include "sm100.cuh"

namespace tb {

constexpr int FA_BM = 128;
constexpr int FA_BN = 128;
constexpr int FA_THREADS = 320;  // 8 softmax warps + MMA warp + TMA warp

struct FaFwdParams {
  __nv_bfloat16* O;  // [B*S, o_stride] with head h at column h*D
  float* LSE;        // [B, H, S] natural-log-sum-exp of the scaled scores (may be null)
  int B, S, H;
  long o_stride;
  float scale;       // softmax scale (1/sqrt(D))
  int causal;
  int* status;
};

template <int D>
struct FaFwdSmem {
  static constexpr int TILE = 128 * D * 2;       // one Q / K / V tile
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = TILE;             // 2 stages
  static constexpr int V_OFF = 3 * TILE;         // 2 stages
  static constexpr int BAR_OFF = 5 * TILE;
  // q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full[2], o_full, o_empty
  static constexpr int NBARS = 15;
  static constexpr int XMAX_OFF = BAR_OFF + NBARS * 8 + 16;   // float [2][2][128]: row-max / row-sum exchange
  static constexpr int TOTAL = XMAX_OFF + 2 * 2 * 128 * 4;
  static constexpr int ALLOC = TOTAL + 1024;
};

template <int D>
__global__ void __launch_bounds__(FA_THREADS, 1)
fa_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
              const __grid_constant__ CUtensorMap map_v, const FaFwdParams p) {
  using L = FaFwdSmem<D>;
  constexpr int KCH = D / 64;
  constexpr uint32_t TM_S = 0, TM_P = 256, TM_O = 384;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + L::BAR_OFF);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = bars + 3;
  uint64_t* v_full = bars + 5;
  uint64_t* v_empty = bars + 7;
  uint64_t* s_full = bars + 9;
  uint64_t* p_full = bars + 11;
  uint64_t* o_full = bars + 13;
  uint64_t* o_empty = bars + 14;
  uint32_t* tmem_ptr = (uint32_t*)(bars + L::NBARS);
  volatile int* abort_flag = (volatile int*)(tmem_ptr + 1);
  volatile float* xmax = (volatile float*)(smem + L::XMAX_OFF);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qb = (p.S + FA_BM - 1) / FA_BM;
  // heavy (late) query blocks first so the causal triangle balances across SMs
  const int qb = n_qb - 1 - (int)(blockIdx.x % n_qb);
  const int bh = blockIdx.x / n_qb;
  const int h = bh % p.H, b = bh / p.H;
  const int q0 = qb * FA_BM;
  const int n_kv_all = (p.S + FA_BN - 1) / FA_BN;
  const int n_kv = p.causal ? min(n_kv_all, qb + 1) : n_kv_all;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 256);
    }
    mbar_init(o_full, 1);
    mbar_init(o_empty, 256);
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
      mbar_expect_tx(q_full, L::TILE);
#pragma unroll
      for (int c = 0; c < KCH; ++c) tma_load_4d(smem + L::Q_OFF + c * 16384, &map_q, q_full, c * 64, h, q0, b);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        mbar_wait(&k_empty[s], ph ^ 1, abort_flag, p.status, TB_ERR_WAIT_EMPTY);
        mbar_expect_tx(&k_full[s], L::TILE);
#pragma unroll
        for (int c = 0; c < KCH; ++c)
          tma_load_4d(smem + L::K_OFF + s * L::TILE + c * 16384, &map_k, &k_full[s], c * 64, h, j * FA_BN, b);
        mbar_wait(&v_empty[s], ph ^ 1, abort_flag, p.status, TB_ERR_WAIT_EMPTY);
        mbar_expect_tx(&v_full[s], L::TILE);
#pragma unroll
        for (int c = 0; c < KCH; ++c)
          tma_load_4d(smem + L::V_OFF + s * L::TILE + c * 16384, &map_v, &v_full[s], c * 64, h, j * FA_BN, b);
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
      constexpr uint32_t idesc_qk = make_idesc_bf16(128, FA_BN, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, D, 0, 1);
      const uint32_t q_base = smem_u32(smem + L::Q_OFF);
      auto issue_qk = [&](int j) {
        const int s = j & 1;
        mbar_wait(&k_full[s], (j >> 1) & 1, abort_flag, p.status, TB_ERR_WAIT_FULL);
        tc_fence_after();
        const uint32_t k_base = smem_u32(smem + L::K_OFF + s * L::TILE);
#pragma unroll
        for (int c = 0; c < KCH; ++c)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_ss(tmem_base + TM_S + s * 128,
                    make_smem_desc_sw128(q_base + c * 16384 + k * 32, 16, 1024),
                    make_smem_desc_sw128(k_base + c * 16384 + k * 32, 16, 1024), idesc_qk,
                    (c | k) ? 1u : 0u);
        umma_commit(&s_full[s]);
        umma_commit(&k_empty[s]);
      };
      mbar_wait(q_full, 0, abort_flag, p.status, TB_ERR_WAIT_FULL);
      issue_qk(0);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        if (j + 1 < n_kv) issue_qk(j + 1);
        mbar_wait(&p_full[s], (j >> 1) & 1, abort_flag, p.status, TB_ERR_WAIT_MISC);
        mbar_wait(&v_full[s], (j >> 1) & 1, abort_flag, p.status, TB_ERR_WAIT_FULL);
        mbar_wait(o_empty, (j & 1) ^ 1, abort_flag, p.status, TB_ERR_WAIT_TMEM_EMPTY);
        tc_fence_after();
        const uint32_t v_base = smem_u32(smem + L::V_OFF + s * L::TILE);
#pragma unroll
        for (int kk = 0; kk < FA_BN / 16; ++kk)
          umma_ts(tmem_base + TM_O, tmem_base + TM_P + s * 64 + kk * 8,
                  make_smem_desc_sw128(v_base + kk * 2048, 16384, 1024), idesc_pv, kk ? 1u : 0u);
        umma_commit(o_full);
        umma_commit(&v_empty[s]);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax (8 warps)
    // Two warps share each group of 32 query rows: warps 0-3 take key columns 0-63 of every score
    // block and the first half of the output columns, warps 4-7 the other halves. Two warps per
    // scheduler keep the exp2 / convert stream issuing while the partner waits on TMEM or the
    // special-function unit. The row maximum is the only value the two halves must agree on per
    // block (one shared-memory exchange + one named barrier); the row sums meet once at the end.
    const int half = warp >> 2;                 // 0: columns 0-63, 1: columns 64-127
    const int row = (warp & 3) * 32 + lane;     // row inside the query block = TMEM lane
    const int qi = q0 + row;                    // global query index
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const float sl2 = p.scale * 1.4426950408889634f;
    constexpr int DH = D / 2;                   // output columns owned by this thread
    float m = -INFINITY, l = 0.f, alpha_prev = 1.f;
    float o[DH];
#pragma unroll
    for (int i = 0; i < DH; ++i) o[i] = 0.f;

    auto accumulate_o = [&](int jdone) {
      mbar_wait(o_full, jdone & 1, abort_flag, p.status, TB_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < DH / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_base + TM_O + half * DH + c * 32 + lane_off, v);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = o[c * 32 + i] * alpha_prev + __uint_as_float(v[i]);
      }
      tc_fence_before();
      mbar_arrive(o_empty);
    };

    for (int j = 0; j < n_kv; ++j) {
      const int s = j & 1;
      const int kv0 = j * FA_BN + half * 64;   // first key column of this thread's half
      const bool need_mask = (p.causal && j * FA_BN + FA_BN - 1 > q0) || (j * FA_BN + FA_BN > p.S);
      const int col_limit = p.causal ? min(qi, p.S - 1) : p.S - 1;  // last visible key index
      mbar_wait(&s_full[s], (j >> 1) & 1, abort_flag, p.status, TB_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
      const uint32_t ts = tmem_base + TM_S + s * 128 + half * 64 + lane_off;
      uint32_t v0[32], v1[32];
      tmem_ld32(ts, v0);
      tmem_ld32(ts + 32, v1);
      tmem_wait_ld();
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float x0 = __uint_as_float(v0[i]), x1 = __uint_as_float(v1[i]);
        if (need_mask) {
          if (kv0 + i > col_limit) x0 = -INFINITY;
          if (kv0 + 32 + i > col_limit) x1 = -INFINITY;
        }
        mx = fmaxf(mx, fmaxf(x0, x1));
      }
      xmax[(j & 1) * 256 + half * 128 + row] = mx;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      mx = fmaxf(m, fmaxf(mx, xmax[(j & 1) * 256 + (half ^ 1) * 128 + row]));
      const float msafe = (mx == -INFINITY) ? 0.f : mx;
      const float alpha = exp2f((m - msafe) * sl2);
      const float moff = msafe * sl2;
      float rowsum = 0.f;
      const uint32_t tp = tmem_base + TM_P + s * 64 + half * 32 + lane_off;
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float p0 = exp2f(__uint_as_float(v0[2 * i]) * sl2 - moff), p1 = exp2f(__uint_as_float(v0[2 * i + 1]) * sl2 - moff);
        if (need_mask) {
          if (kv0 + 2 * i > col_limit) p0 = 0.f;
          if (kv0 + 2 * i + 1 > col_limit) p1 = 0.f;
        }
        rowsum += p0 + p1;
        pk[i] = pack_bf16x2(p0, p1);
      }
      tmem_st16(tp, pk);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float p0 = exp2f(__uint_as_float(v1[2 * i]) * sl2 - moff), p1 = exp2f(__uint_as_float(v1[2 * i + 1]) * sl2 - moff);
        if (need_mask) {
          if (kv0 + 32 + 2 * i > col_limit) p0 = 0.f;
          if (kv0 + 32 + 2 * i + 1 > col_limit) p1 = 0.f;
        }
        rowsum += p0 + p1;
        pk[i] = pack_bf16x2(p0, p1);
      }
      tmem_st16(tp + 16, pk);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&p_full[s]);
      l = l * alpha + rowsum;
      m = mx;
      if (j > 0) accumulate_o(j - 1);
      alpha_prev = alpha;
    }
    accumulate_o(n_kv - 1);
    // the two halves of a row add their partial sums, through the exchange buffer that the last block did
    // not use (its readers may still be behind this thread)
    xmax[(n_kv & 1) * 256 + half * 128 + row] = l;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    l += xmax[(n_kv & 1) * 256 + (half ^ 1) * 128 + row];
    if (qi < p.S) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = p.O + ((size_t)b * p.S + qi) * p.o_stride + (size_t)h * D + half * DH;
#pragma unroll
      for (int g = 0; g < DH / 8; ++g) {
        uint4 w;
        w.x = pack_bf16x2(o[g * 8 + 0] * inv, o[g * 8 + 1] * inv);
        w.y = pack_bf16x2(o[g * 8 + 2] * inv, o[g * 8 + 3] * inv);
        w.z = pack_bf16x2(o[g * 8 + 4] * inv, o[g * 8 + 5] * inv);
        w.w = pack_bf16x2(o[g * 8 + 6] * inv, o[g * 8 + 7] * inv);
        reinterpret_cast<uint4*>(orow)[g] = w;
      }
      if (p.LSE && half == 0) p.LSE[((size_t)b * p.H + h) * p.S + qi] = (l > 0.f) ? (m * p.scale + logf(l)) : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// 4-D map over a [B, S, H, D] bf16 view with token stride `row_stride` elements; box = 64 x 1 x 128 x 1.
inline int make_bshd_map(CUtensorMap* m, const void* base, int B, int S, int H, int D, long row_stride) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)S, (uint64_t)B};
  uint64_t str[3] = {(uint64_t)D * 2, (uint64_t)row_stride * 2, (uint64_t)S * row_stride * 2};
  uint32_t box[4] = {64, 1, 128, 1};
  return make_tmap(m, base, 2, 4, dims, str, box);
}

}  // namespace tb
using namespace tb;

// q, k, v: bf16 views [B, S, H, D] with token strides q_stride / kv_stride (elements); head h starts
// at element h*D of a token row; D in {64, 128}. o: [B*S, o_stride]. lse: fp32 [B, H, S] or null.
TB_EXPORT int tb_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B,
                                int S, int H, int D, long q_stride, long kv_stride, long o_stride,
                                float scale, int causal, int* status, cudaStream_t st) {
  TB_ENSURE_DEVICE();
  if (!q || !k || !v || !o || B <= 0 || S <= 0 || H <= 0) TB_FAIL(TB_E_ARG, "flash_attn_fwd: bad arguments");
  if (D != 64 && D != 128) TB_FAIL(TB_E_ARG, "flash_attn_fwd: head dim %d not supported (64 or 128)", D);
  if ((o_stride & 7) || ((uintptr_t)o & 15)) TB_FAIL(TB_E_ARG, "flash_attn_fwd: output must be 16-byte aligned");
  CUtensorMap mq, mk, mv;
  int r;
  if ((r = make_bshd_map(&mq, q, B, S, H, D, q_stride))) return r;
  if ((r = make_bshd_map(&mk, k, B, S, H, D, kv_stride))) return r;
  if ((r = make_bshd_map(&mv, v, B, S, H, D, kv_stride))) return r;
  FaFwdParams p{(__nv_bfloat16*)o, lse, B, S, H, o_stride, scale, causal, status};
  const int n_qb = (S + FA_BM - 1) / FA_BM;
  const long grid = (long)n_qb * B * H;
  if (D == 64) {
    static bool cfg = false;
    if (!cfg) { TB_CUDA_CHECK(cudaFuncSetAttribute(fa_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, FaFwdSmem<64>::ALLOC)); cfg = true; }
    fa_fwd_kernel<64><<<(unsigned)grid, FA_THREADS, FaFwdSmem<64>::ALLOC, st>>>(mq, mk, mv, p);
  } else {
    static bool cfg = false;
    if (!cfg) { TB_CUDA_CHECK(cudaFuncSetAttribute(fa_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, FaFwdSmem<128>::ALLOC)); cfg = true; }
    fa_fwd_kernel<128><<<(unsigned)grid, FA_THREADS, FaFwdSmem<128>::ALLOC, st>>>(mq, mk, mv, p);
  }
  TB_CUDA_CHECK(cudaGetLastError());
  return 0;
}
