// Flash attention forward for sm_100a (tcgen05 / TMEM / TMA), causal or full, head dim 64 or 128.
//
// Persistent CTAs (one per SM) walk the (batch, head, 128-query block) tiles, heaviest causal tiles first; the
// three roles keep running counters across tiles, so the TMA warp already loads the next tile's Q / K / V and the
// MMA warp already issues its first Q K^T while the softmax warps still normalise and store the previous tile.
// 320 threads:
//   warps 0-7  softmax: two threads per query row (= TMEM lane), each owning half of the key
//              columns of a score block and half of the output columns. Read S = Q K^T from TMEM,
//              online softmax in fp32 (exp2, running max / sum), write P as packed bf16 back to
//              TMEM, accumulate O in registers from the per-block P V partials.
//   warp 8     MMA issuer (one thread): S[j+1] = Q K[j+1]^T is issued before waiting for P[j],
//              so the tensor core works on the next block while the softmax warps run.
//   warp 9     TMA producer (one thread): Q through a 2-deep ring (one slot per tile), K / V tiles through 2-deep rings.
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
  static constexpr int Q_OFF = 0;                // 2 stages
  static constexpr int K_OFF = 2 * TILE;         // 2 stages
  static constexpr int V_OFF = 4 * TILE;         // 2 stages
  static constexpr int BAR_OFF = 6 * TILE;
  // q_full[2], q_empty[2], k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full[2], o_full, o_empty
  static constexpr int NBARS = 18;
  static constexpr int XMAX_OFF = BAR_OFF + NBARS * 8 + 16;   // float [3][2][128]: row-max (2 buffers) / row-sum exchange
  static constexpr int TOTAL = XMAX_OFF + 3 * 2 * 128 * 4;
  static constexpr int ALLOC = TOTAL + 1024;
};

// max of three fp32 values in one instruction (sm_100)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Row maximum over this thread's 64 scores (two 32-column TMEM loads). MASK is a template parameter so that the
// unmasked blocks (all but the diagonal and the ragged last one) carry no compare / select instructions at all.
template <bool MASK>
__device__ __forceinline__ float fa_row_max(const uint32_t (&v0)[32], const uint32_t (&v1)[32], int kv0, int col_limit) {
  float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    float a0 = __uint_as_float(v0[i]), a1 = __uint_as_float(v0[i + 1]);
    float b0 = __uint_as_float(v1[i]), b1 = __uint_as_float(v1[i + 1]);
    if (MASK) {
      if (kv0 + i > col_limit) a0 = -INFINITY;
      if (kv0 + i + 1 > col_limit) a1 = -INFINITY;
      if (kv0 + 32 + i > col_limit) b0 = -INFINITY;
      if (kv0 + 32 + i + 1 > col_limit) b1 = -INFINITY;
    }
    m0 = fmax3(m0, a0, a1);
    m1 = fmax3(m1, b0, b1);
  }
  return fmaxf(m0, m1);
}

// p = exp2(s * sl2 - moff) for 32 scores, packed to bf16 pairs; the scale-and-shift and the row sum run as packed
// two-wide fp32 instructions (fma.rn.f32x2 / add.f32x2), so each pair costs one FFMA2, two MUFU.EX2, one FADD2 and
// one pack.
template <bool MASK>
__device__ __forceinline__ void fa_exp_pack(const uint32_t (&v)[32], float sl2, float moff, int kvbase, int col_limit,
                                            uint32_t (&pk)[16], float2& rowsum) {
  const float2 s2 = make_float2(sl2, sl2), o2 = make_float2(-moff, -moff);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float2 t = __ffma2_rn(make_float2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1])), s2, o2);
    float2 e = make_float2(exp2f(t.x), exp2f(t.y));
    if (MASK) {
      if (kvbase + 2 * i > col_limit) e.x = 0.f;
      if (kvbase + 2 * i + 1 > col_limit) e.y = 0.f;
    }
    rowsum = __fadd2_rn(rowsum, e);
    pk[i] = pack_bf16x2(e.x, e.y);
  }
}

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
  uint64_t* q_empty = bars + 2;
  uint64_t* k_full = bars + 4;
  uint64_t* k_empty = bars + 6;
  uint64_t* v_full = bars + 8;
  uint64_t* v_empty = bars + 10;
  uint64_t* s_full = bars + 12;
  uint64_t* p_full = bars + 14;
  uint64_t* o_full = bars + 16;
  uint64_t* o_empty = bars + 17;
  uint32_t* tmem_ptr = (uint32_t*)(bars + L::NBARS);
  volatile int* abort_flag = (volatile int*)(tmem_ptr + 1);
  volatile float* xmax = (volatile float*)(smem + L::XMAX_OFF);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qb = (p.S + FA_BM - 1) / FA_BM;
  const int n_kv_all = (p.S + FA_BN - 1) / FA_BN;
  const int BH = p.B * p.H;
  const int n_tiles = n_qb * BH;
  // tile t -> (query block, batch*head): heavy (late) query blocks first, so the causal triangle balances over the SMs
  auto tile_qb = [&](int t) { return n_qb - 1 - t / BH; };
  auto tile_nkv = [&](int t) { return p.causal ? min(n_kv_all, tile_qb(t) + 1) : n_kv_all; };

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
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
      uint32_t it = 0, tcount = 0;  // K/V blocks and tiles handled so far by this CTA
      // once a wait has given up, nothing more is loaded: loads without a free slot would pile transaction counts on
      // one barrier beyond its range
      for (int t = blockIdx.x; t < n_tiles && !*abort_flag; t += gridDim.x, ++tcount) {
        const int bh = t % BH, h = bh % p.H, b = bh / p.H, q0 = tile_qb(t) * FA_BM, n_kv = tile_nkv(t);
        const int qs = tcount & 1;
        if (!mbar_wait(&q_empty[qs], ((tcount >> 1) & 1) ^ 1, abort_flag, p.status, TB_ERR_WAIT_EMPTY)) break;
        mbar_expect_tx(&q_full[qs], L::TILE);
#pragma unroll
        for (int c = 0; c < KCH; ++c)
          tma_load_4d(smem + L::Q_OFF + qs * L::TILE + c * 16384, &map_q, &q_full[qs], c * 64, h, q0, b);
        for (int j = 0; j < n_kv; ++j, ++it) {
          const int s = it & 1;
          const uint32_t ph = (it >> 1) & 1;
          if (!mbar_wait(&k_empty[s], ph ^ 1, abort_flag, p.status, TB_ERR_WAIT_EMPTY)) break;
          mbar_expect_tx(&k_full[s], L::TILE);
#pragma unroll
          for (int c = 0; c < KCH; ++c)
            tma_load_4d(smem + L::K_OFF + s * L::TILE + c * 16384, &map_k, &k_full[s], c * 64, h, j * FA_BN, b);
          if (!mbar_wait(&v_empty[s], ph ^ 1, abort_flag, p.status, TB_ERR_WAIT_EMPTY)) break;
          mbar_expect_tx(&v_full[s], L::TILE);
#pragma unroll
          for (int c = 0; c < KCH; ++c)
            tma_load_4d(smem + L::V_OFF + s * L::TILE + c * 16384, &map_v, &v_full[s], c * 64, h, j * FA_BN, b);
        }
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
      // Two cursors over the same flattened (tile, K/V block) sequence: `a` issues S = Q K^T, `b` issues O = P V one
      // block behind, so the score MMA of the next block (possibly of the next tile) runs while the softmax warps work.
      struct Cursor {
        int t, j, n_kv;
        uint32_t it, tcount;
      };
      auto advance = [&](Cursor& c) {
        ++c.it;
        if (++c.j == c.n_kv) {
          c.t += gridDim.x;
          ++c.tcount;
          c.j = 0;
          c.n_kv = c.t < n_tiles ? tile_nkv(c.t) : 0;
        }
      };
      auto issue_qk = [&](const Cursor& c) {
        const int s = c.it & 1, qs = c.tcount & 1;
        if (c.j == 0) mbar_wait(&q_full[qs], (c.tcount >> 1) & 1, abort_flag, p.status, TB_ERR_WAIT_FULL);
        mbar_wait(&k_full[s], (c.it >> 1) & 1, abort_flag, p.status, TB_ERR_WAIT_FULL);
        tc_fence_after();
        const uint32_t q_base = smem_u32(smem + L::Q_OFF + qs * L::TILE);
        const uint32_t k_base = smem_u32(smem + L::K_OFF + s * L::TILE);
#pragma unroll
        for (int ch = 0; ch < KCH; ++ch)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_ss(tmem_base + TM_S + s * 128,
                    make_smem_desc_sw128(q_base + ch * 16384 + k * 32, 16, 1024),
                    make_smem_desc_sw128(k_base + ch * 16384 + k * 32, 16, 1024), idesc_qk,
                    (ch | k) ? 1u : 0u);
        umma_commit(&s_full[s]);
        umma_commit(&k_empty[s]);
        if (c.j == c.n_kv - 1) umma_commit(&q_empty[qs]);  // last score MMA of the tile: its Q slot may be refilled
      };
      Cursor a{(int)blockIdx.x, 0, 0, 0u, 0u}, bcur{(int)blockIdx.x, 0, 0, 0u, 0u};
      a.n_kv = bcur.n_kv = a.t < n_tiles ? tile_nkv(a.t) : 0;
      if (a.t < n_tiles) {
        issue_qk(a);
        advance(a);
      }
      while (bcur.t < n_tiles) {
        if (a.t < n_tiles) {
          issue_qk(a);
          advance(a);
        }
        const int s = bcur.it & 1;
        mbar_wait(&p_full[s], (bcur.it >> 1) & 1, abort_flag, p.status, TB_ERR_WAIT_MISC);
        mbar_wait(&v_full[s], (bcur.it >> 1) & 1, abort_flag, p.status, TB_ERR_WAIT_FULL);
        mbar_wait(o_empty, (bcur.it & 1) ^ 1, abort_flag, p.status, TB_ERR_WAIT_TMEM_EMPTY);
        tc_fence_after();
        const uint32_t v_base = smem_u32(smem + L::V_OFF + s * L::TILE);
#pragma unroll
        for (int kk = 0; kk < FA_BN / 16; ++kk)
          umma_ts(tmem_base + TM_O, tmem_base + TM_P + s * 64 + kk * 8,
                  make_smem_desc_sw128(v_base + kk * 2048, 16384, 1024), idesc_pv, kk ? 1u : 0u);
        umma_commit(o_full);
        umma_commit(&v_empty[s]);
        advance(bcur);
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
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const float sl2 = p.scale * 1.4426950408889634f;
    constexpr int DH = D / 2;                   // output columns owned by this thread
    uint32_t it = 0;                            // K/V blocks handled so far by this CTA (all tiles)
    for (int t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    const int bh = t % BH, h = bh % p.H, b = bh / p.H, q0 = tile_qb(t) * FA_BM, n_kv = tile_nkv(t);
    const int qi = q0 + row;                    // global query index
    float m = -INFINITY, l = 0.f, alpha_prev = 1.f;
    float o[DH];
#pragma unroll
    for (int i = 0; i < DH; ++i) o[i] = 0.f;

    auto accumulate_o = [&](uint32_t it_done) {
      mbar_wait(o_full, it_done & 1, abort_flag, p.status, TB_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < DH / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_base + TM_O + half * DH + c * 32 + lane_off, v);
        tmem_wait_ld();
        const float2 a2 = make_float2(alpha_prev, alpha_prev);
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float2 r = __ffma2_rn(make_float2(o[c * 32 + i], o[c * 32 + i + 1]), a2,
                                      make_float2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])));
          o[c * 32 + i] = r.x;
          o[c * 32 + i + 1] = r.y;
        }
      }
      tc_fence_before();
      mbar_arrive(o_empty);
    };

    for (int j = 0; j < n_kv; ++j, ++it) {
      const int s = it & 1;
      const int kv0 = j * FA_BN + half * 64;   // first key column of this thread's half
      const bool need_mask = (p.causal && j * FA_BN + FA_BN - 1 > q0) || (j * FA_BN + FA_BN > p.S);
      const int col_limit = p.causal ? min(qi, p.S - 1) : p.S - 1;  // last visible key index
      mbar_wait(&s_full[s], (it >> 1) & 1, abort_flag, p.status, TB_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
      const uint32_t ts = tmem_base + TM_S + s * 128 + half * 64 + lane_off;
      uint32_t v0[32], v1[32];
      tmem_ld32(ts, v0);
      tmem_ld32(ts + 32, v1);
      tmem_wait_ld();
      float mx = need_mask ? fa_row_max<true>(v0, v1, kv0, col_limit) : fa_row_max<false>(v0, v1, kv0, col_limit);
      xmax[s * 256 + half * 128 + row] = mx;
      asm volatile("bar.sync %0, 64;" ::"r"(1 + (warp & 3)) : "memory");  // only the two warps that share these rows
      mx = fmax3(m, mx, xmax[s * 256 + (half ^ 1) * 128 + row]);
      const float msafe = (mx == -INFINITY) ? 0.f : mx;
      const float alpha = exp2f((m - msafe) * sl2);
      const float moff = msafe * sl2;
      float2 rs2 = make_float2(0.f, 0.f);
      const uint32_t tp = tmem_base + TM_P + s * 64 + half * 32 + lane_off;
      uint32_t pk[16];
      if (need_mask) fa_exp_pack<true>(v0, sl2, moff, kv0, col_limit, pk, rs2);
      else fa_exp_pack<false>(v0, sl2, moff, kv0, col_limit, pk, rs2);
      tmem_st16(tp, pk);
      if (need_mask) fa_exp_pack<true>(v1, sl2, moff, kv0 + 32, col_limit, pk, rs2);
      else fa_exp_pack<false>(v1, sl2, moff, kv0 + 32, col_limit, pk, rs2);
      tmem_st16(tp + 16, pk);
      const float rowsum = rs2.x + rs2.y;
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&p_full[s]);
      l = l * alpha + rowsum;
      m = mx;
      if (j > 0) accumulate_o(it - 1);
      alpha_prev = alpha;
    }
    accumulate_o(it - 1);
    // the two halves of a row add their partial sums through a third exchange buffer: the row-max buffers may
    // already be in use by a faster thread's next block or next tile
    xmax[512 + half * 128 + row] = l;
    asm volatile("bar.sync %0, 64;" ::"r"(1 + (warp & 3)) : "memory");
    l += xmax[512 + (half ^ 1) * 128 + row];
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
    }  // tile loop
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
  const long tiles = (long)n_qb * B * H;
  const long grid = tiles < sm_count() ? tiles : sm_count();  // persistent CTAs, one per SM
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
