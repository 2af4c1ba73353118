// Bucketed (windowed) multi-head self-attention forward on tcgen05 tensor cores, sm_100a.
//
// Implements buck_swin_fwd(Q, K, V, O, L, Scope_buckets, bucket_size), which the reference's Python layer calls
// (flash3dxfmr/layers/buck_swin.py:57) but whose kernel source and binding are absent from the reference snapshot
// (declaration src/f3d_frontend.cu:90-92, binding commented out :136).  Semantics follow the reference's tests
// (tests/test_attn_fwd.py:295-452, tests/test_lib.py:24-48) and scope helpers (flash3dxfmr/psh/bucket_scope.py:
// 143-181): for every batch row b, head h and scope s (a row of Scope_buckets listing k buckets), the tokens of
// those buckets attend to each other with softmax(Q K^T / sqrt(D)) V; LSE is the natural-log row normaliser.
// Buckets that no scope lists are left untouched.
//
// Kernel shape: one CTA = NQ tiles of 128 query rows of one (scope, head, batch row) that share one stream of K/V
// tiles (the library instantiates NQ = 1; the scope's query tiles must be a multiple of NQ); 32 + 128 * NQ threads:
//   warp 0        one elected thread is both the TMA producer and the MMA issuer.  It loads the Q tiles once and K/V
//                 tiles of 64 keys through a 4-stage ring (3-D tensor maps over [token, head, dim], swizzle width =
//                 min(128, 2*D) bytes), issues S_t = Q_t K^T (M=128, N=64) and O_t += P_t V (A operand P read from
//                 tensor memory, V as MN-major B operand) for every query tile t and commits mbarriers.  A ring stage
//                 is refilled without a barrier of its own: when the softmax warps of every tile have delivered P of
//                 key tile j, they had all seen O complete up to tile j-1, so the MMAs that read stage (j-1) % 4 are
//                 done and key tile j+3 may land there.
//   warps 1..4NQ  softmax, four warps per query tile, one thread per query row; S is read with tcgen05.ld, the
//                 running maximum and sum are kept in the base-2 domain, P is written as bf16 with tcgen05.st, O is
//                 rescaled in tensor memory only when the row maximum moved, and the epilogue normalises and stores O
//                 and LSE
// Per query tile, tensor memory holds S (64 columns), P (32) and O (D) side by side: because P does not overwrite S,
// the next key tile's Q K^T is issued as soon as the softmax threads have pulled S into registers, so the tensor pipe
// computes S(j+1) while the warps exponentiate tile j.  At D = 32 the kernel is bound by the special-function unit
// (one ex2 per score against 4*D = 128 tensor FLOPs) and by instruction issue of the softmax warps, not by the tensor
// pipe; three of every sixteen exponentials are therefore computed on the FMA pipe (poly_exp2_pair).
#include "f3d_common.cuh"
#include "tc_sm100.cuh"
#include "../../include/f3d_b200.h"

namespace f3d {

int *status_word(int device);

constexpr int kBQ = 128;      // query rows per tile
constexpr int kBKV = 64;      // keys per tile
constexpr int kKvStages = 4;

struct AttnFwdArgs {
  __nv_bfloat16 *O; float *lse; const uint32_t *scopes;
  int B, L, H, num_scopes, k, bucket, q_blocks_per_bucket;   // q_blocks_per_bucket = bucket / 128
  float scale_log2;          // log2(e) / sqrt(D)
  int *status;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float m;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(m) : "f"(a), "f"(b), "f"(c));
  return m;
}

// packed fp32 pairs (Blackwell executes fma / add on two fp32 values per instruction)
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// two fp32 values as a packed pair in the kernel's 16-bit element type (P in tensor memory, O in global memory)
template <bool F16> __device__ __forceinline__ uint32_t pack_p2(float a, float b) {
  if (F16) { __half2 h = __floats2half2_rn(a, b); return *reinterpret_cast<uint32_t *>(&h); }
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&h);
}

// 2^x for a pair of arguments (at most a few units above zero, any distance below) on the FMA pipe instead of the special-function unit: n = round(x) by the
// magic-number addition (the sum x + 1.5 * 2^23 carries n in its low mantissa bits), f = x - n in [-0.5, 0.5], a cubic
// for 2^f (largest relative error 7.5e-5, against the 3.9e-3 of the bf16 rounding P gets anyway), and n added to the
// exponent field with integer arithmetic.  The integer maximum keeps the result at 2^-126 or above (times the cubic),
// so arguments far below the range of an fp32 exponent come out as tiny numbers instead of wrapping around.
__device__ __forceinline__ void poly_exp2_pair(uint64_t x2, float &e0, float &e1) {
  const uint64_t magic2 = pack2(12582912.f, 12582912.f), nmagic2 = pack2(-12582912.f, -12582912.f);
  const uint64_t t2 = add2(x2, magic2);
  const uint64_t u2 = add2(t2, nmagic2);                              // n as a float, exact
  const uint64_t f2 = fma2(u2, pack2(-1.f, -1.f), x2);                // x - n
  uint64_t p2 = fma2(pack2(0.055171459913253784f, 0.055171459913253784f), f2, pack2(0.2426108568906784f, 0.2426108568906784f));
  p2 = fma2(p2, f2, pack2(0.6932609677314758f, 0.6932609677314758f));
  p2 = fma2(p2, f2, pack2(0.9999281167984009f, 0.9999281167984009f));
  float t0, t1, p0, p1;
  unpack2(t2, t0, t1);
  unpack2(p2, p0, p1);
  const int lowest = 0x4B400000 - 126;                                // bits of 1.5 * 2^23 - 126
  const int n0 = max(__float_as_int(t0), lowest), n1 = max(__float_as_int(t1), lowest);
  e0 = __int_as_float(__float_as_int(p0) + (n0 << 23));               // the bits of 1.5 * 2^23 vanish in the shift
  e1 = __int_as_float(__float_as_int(p1) + (n1 << 23));
}

template <int D, int BKV, int NQ> struct AttnCfg {
  static constexpr int DCH = D < 64 ? D : 64;       // columns per swizzled row
  static constexpr int NDCH = D / DCH;
  static constexpr int RB = DCH * 2;                // bytes per swizzled row
  static constexpr uint64_t SWZ = RB == 128 ? tc::kSwizzle128 : (RB == 64 ? tc::kSwizzle64 : tc::kSwizzle32);
  static constexpr int kQBytes = kBQ * D * 2;       // one Q tile
  static constexpr int kTileBytes = BKV * D * 2;    // one K or V tile
  static constexpr int kStageBytes = 2 * kTileBytes;
  static constexpr int kSmem = NQ * kQBytes + kKvStages * kStageBytes + 512 + 1024;
  static constexpr int kThreads = 32 + 128 * NQ;
  // Tensor memory columns of one query tile: S (fp32 scores, BKV), P (bf16 probabilities, two per column, BKV / 2),
  // O (fp32, D).  P has columns of its own so that the next tile's S = Q K^T can be issued as soon as the softmax
  // warps have read S, while they are still computing P.
  static constexpr uint32_t kPCol = BKV;
  static constexpr uint32_t kOCol = BKV + BKV / 2;
  static constexpr uint32_t kTileCols = (kOCol + D) <= 128 ? 128u : 256u;
  static constexpr uint32_t kTmemCols = kTileCols * NQ;
  static constexpr int kMinCtas = (512 / (int)kTmemCols) < 4 ? (512 / (int)kTmemCols) : 4;
  static_assert(kTmemCols <= 512, "tensor memory holds 512 columns");
};

// POLY8 != 0: of the sixteen pairs of scores of a half tile, pairs 4, 9 and 14 take their exponential from poly_exp2_pair
// (FMA pipe) and the rest from ex2.approx (special-function unit), so that both pipes work on every row.  Share and
// placement are measured choices (D = 32, W = 4096): none 439, two adjacent pairs of every eight 476, every fourth pair
// 484, every fifth pair 497 TFLOP/s; larger shares cost more issue slots than the special-function slots they free.
template <int D, int BKV, int NQ, int POLY8, bool F16>
__global__ void __launch_bounds__((AttnCfg<D, BKV, NQ>::kThreads), (AttnCfg<D, BKV, NQ>::kMinCtas))
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, AttnFwdArgs a) {
  using C = AttnCfg<D, BKV, NQ>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char *sq = smem;
  unsigned char *skv = smem + NQ * C::kQBytes;
  uint64_t *bars = reinterpret_cast<uint64_t *>(skv + kKvStages * C::kStageBytes);
  uint64_t *q_full = bars, *kv_full = bars + 1;
  uint64_t *s_full = kv_full + kKvStages, *p_full = s_full + NQ, *o_full = p_full + NQ, *s_free = o_full + NQ;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(s_free + NQ);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // which group of NQ query tiles: tiles of a scope are numbered in scope order, bucket slot major
  const int tiles_per_scope = a.k * a.q_blocks_per_bucket;
  const int groups_per_scope = tiles_per_scope / NQ;
  const int scope = blockIdx.x / groups_per_scope;
  const int tile0 = (blockIdx.x % groups_per_scope) * NQ;
  const int head = blockIdx.y, brow = blockIdx.z;
  const uint32_t *my_scope = a.scopes + (size_t)scope * a.k;
  const int tiles_per_bucket = a.bucket / BKV;
  const int num_tiles = a.k * tiles_per_bucket;
  auto q_token = [&](int t) -> int {                    // first query token of tile t of this CTA (inside batch row)
    const int ti = tile0 + t;
    return (int)my_scope[ti / a.q_blocks_per_bucket] * a.bucket + (ti % a.q_blocks_per_bucket) * kBQ;
  };

  if (threadIdx.x == 0) {
    tc::mbar_init(q_full, 1);
    for (int s = 0; s < kKvStages; ++s) tc::mbar_init(&kv_full[s], 1);
    for (int t = 0; t < NQ; ++t) {
      tc::mbar_init(&s_full[t], 1); tc::mbar_init(&p_full[t], 128); tc::mbar_init(&o_full[t], 1); tc::mbar_init(&s_free[t], 128);
    }
    *abort_flag = 0;
    tc::mbar_fence_init();
  }
  if (warp == 0) { tc::tmem_alloc(tmem_slot, C::kTmemCols); tc::tmem_relinquish(); }
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  tc::WaitCtx wc{abort_flag, a.status};

  if (warp == 0) {
    if (tc::elect_one()) {
      tc::tma_prefetch_desc(&map_q); tc::tma_prefetch_desc(&map_k); tc::tma_prefetch_desc(&map_v);
      tc::mbar_expect_tx(q_full, NQ * C::kQBytes);
#pragma unroll
      for (int t = 0; t < NQ; ++t)
#pragma unroll
        for (int c = 0; c < C::NDCH; ++c)
          tc::tma_load_3d(sq + t * C::kQBytes + c * kBQ * C::RB, &map_q, q_full, c * C::DCH, head, brow * a.L + q_token(t));
      auto load_kv = [&](int j) {
        const int s = j % kKvStages;
        const int key_tok = (int)my_scope[j / tiles_per_bucket] * a.bucket + (j % tiles_per_bucket) * BKV;
        unsigned char *sk = skv + s * C::kStageBytes, *sv = sk + C::kTileBytes;
        tc::mbar_expect_tx(&kv_full[s], C::kStageBytes);
#pragma unroll
        for (int c = 0; c < C::NDCH; ++c) {
          tc::tma_load_3d(sk + c * BKV * C::RB, &map_k, &kv_full[s], c * C::DCH, head, brow * a.L + key_tok);
          tc::tma_load_3d(sv + c * BKV * C::RB, &map_v, &kv_full[s], c * C::DCH, head, brow * a.L + key_tok);
        }
      };
      for (int j = 0; j < kKvStages && j < num_tiles; ++j) load_kv(j);

      constexpr uint32_t idesc_s = tc::make_idesc_f16(kBQ, BKV, !F16, false, false);
      constexpr uint32_t idesc_o = tc::make_idesc_f16(kBQ, C::DCH, !F16, false, true);    // B (= V) is MN-major
      const uint32_t q_addr = tc::smem_u32(sq);
      // S_t = Q_t K^T of key tile j: K-major operands, 8-row groups are 8*RB bytes apart
      auto issue_s = [&](int t, int j) {
        const uint32_t k_addr = tc::smem_u32(skv + (j % kKvStages) * C::kStageBytes);
        const uint32_t s_tmem = tmem_base + t * C::kTileCols;
#pragma unroll
        for (int c = 0; c < C::NDCH; ++c) {
#pragma unroll
          for (int kk = 0; kk < C::DCH / 16; ++kk) {
            uint64_t ad = tc::make_smem_desc(q_addr + t * C::kQBytes + c * kBQ * C::RB + kk * 32, 16, 8 * C::RB, C::SWZ);
            uint64_t bd = tc::make_smem_desc(k_addr + c * BKV * C::RB + kk * 32, 16, 8 * C::RB, C::SWZ);
            tc::mma_f16_ss(s_tmem, ad, bd, idesc_s, (c | kk) != 0 ? 1u : 0u);
          }
        }
        tc::mma_commit(&s_full[t]);
      };
      bool ok = tc::mbar_wait(q_full, 0, wc, 202) && tc::mbar_wait(&kv_full[0], 0, wc, 203);
      if (ok) {
        tc::tc_fence_after_sync();
#pragma unroll
        for (int t = 0; t < NQ; ++t) issue_s(t, 0);
      }
      for (int j = 0; j < num_tiles && ok; ++j) {
        const int s = j % kKvStages;
        if (j + 1 < num_tiles) {
          if (!tc::mbar_wait(&kv_full[(j + 1) % kKvStages], (uint32_t)((j + 1) / kKvStages) & 1u, wc, 203)) { ok = false; break; }
#pragma unroll
          for (int t = 0; t < NQ; ++t) {
            // the next scores may overwrite S once every softmax thread of the tile has read key tile j
            if (!tc::mbar_wait(&s_free[t], (uint32_t)j & 1u, wc, 208)) { ok = false; break; }
            tc::tc_fence_after_sync();
            issue_s(t, j + 1);
          }
          if (!ok) break;
        }
        const uint32_t v_addr = tc::smem_u32(skv + s * C::kStageBytes) + C::kTileBytes;
#pragma unroll
        for (int t = 0; t < NQ; ++t) {
          // O_t += P_t V once the softmax warps of the tile have written P
          if (!tc::mbar_wait(&p_full[t], (uint32_t)j & 1u, wc, 204)) { ok = false; break; }
          tc::tc_fence_after_sync();
          const uint32_t p_tmem = tmem_base + t * C::kTileCols + C::kPCol, o_tmem = tmem_base + t * C::kTileCols + C::kOCol;
#pragma unroll
          for (int c = 0; c < C::NDCH; ++c) {
#pragma unroll
            for (int kk = 0; kk < BKV / 16; ++kk) {
              // 16 keys per MMA: V rows kk*16.. ; P columns kk*8.. (two bf16 per 32-bit column)
              uint64_t bd = tc::make_smem_desc(v_addr + c * BKV * C::RB + kk * 16 * C::RB, 16, 8 * C::RB, C::SWZ);
              tc::mma_f16_ts(o_tmem + c * C::DCH, p_tmem + kk * 8, bd, idesc_o, (j | kk) != 0 ? 1u : 0u);
            }
          }
          tc::mma_commit(&o_full[t]);
        }
        if (!ok) break;
        // every tile has delivered P(j), so every tile had seen O complete up to key tile j-1: stage (j-1) % 4 is free
        if (j >= 1 && j + kKvStages - 1 < num_tiles) load_kv(j + kKvStages - 1);
      }
    }
  } else {
    const int t = (warp - 1) >> 2;                               // query tile of this warp
    const int q = warp & 3;                                      // tensor-memory lane quarter this warp may access
    const int row = q * 32 + lane;                               // query row inside the tile = tensor-memory lane
    const int q_tok = q_token(t);
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const uint32_t tile_tmem = tmem_base + t * C::kTileCols + lane_off;
    const uint32_t s_tmem = tile_tmem, p_tmem = tile_tmem + C::kPCol, o_tmem = tile_tmem + C::kOCol;
    uint64_t *my_s_full = &s_full[t], *my_s_free = &s_free[t], *my_p_full = &p_full[t], *my_o_full = &o_full[t];
    float m_run = -INFINITY, l_run = 0.f;
    const uint64_t c2 = pack2(a.scale_log2, a.scale_log2);
    bool ok = true;
    for (int j = 0; j < num_tiles && ok; ++j) {
      if (!tc::mbar_wait(my_s_full, (uint32_t)j & 1u, wc, 205)) { ok = false; break; }
      tc::tc_fence_after_sync();
      uint32_t r0[32], r1[32];
      tc::tmem_ld_32x32b_x32(s_tmem, r0);
      tc::tmem_ld_32x32b_x32(s_tmem + 32, r1);
      tc::tmem_ld_wait();
      // the scores are in registers: the next key tile's Q K^T may be issued over them
      tc::tc_fence_before_sync();
      tc::mbar_arrive(my_s_free);
      // four independent chains of 3-input maxima instead of one 32 deep
      float mxa = -INFINITY, mxb = -INFINITY, mxc = -INFINITY, mxd = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        mxa = max3(mxa, __uint_as_float(r0[i]), __uint_as_float(r1[i]));
        mxb = max3(mxb, __uint_as_float(r0[i + 1]), __uint_as_float(r1[i + 1]));
        mxc = max3(mxc, __uint_as_float(r0[i + 2]), __uint_as_float(r1[i + 2]));
        mxd = max3(mxd, __uint_as_float(r0[i + 3]), __uint_as_float(r1[i + 3]));
      }
      const float mx = fmaxf(max3(mxa, mxb, mxc), mxd) * a.scale_log2;
      // The reference point m_run of the exponentials follows the row maximum lazily: it moves only when the tile's
      // maximum exceeds it by more than kMaxSlack (base-2 units), so probabilities stay below 2^kMaxSlack, which bf16 /
      // fp16 and the fp32 sums hold without loss, and the result O / l does not depend on the choice.  On typical
      // rows the maximum settles within the first tile or two; afterwards no thread of the warp rescales anything:
      // no exponential for alpha, no round trip of O through tensor memory.
      constexpr float kMaxSlack = 8.f;
      float alpha = 1.f;
      const bool moved = __any_sync(0xFFFFFFFFu, mx > m_run + kMaxSlack);       // first tile: m_run = -inf
      if (moved) {
        const float m_new = mx > m_run + kMaxSlack ? mx : m_run;
        alpha = fast_exp2(m_run - m_new);                 // 1 for rows that keep their reference, 0 on the first tile
        m_run = m_new;
      }
      // x = s * c - m and the row sum run on packed fp32 pairs; the sum adds the unrounded probabilities (the
      // bf16 rounding of P is unbiased, so the normaliser stays consistent with what the MMA reads)
      const uint64_t m2 = pack2(-m_run, -m_run);
      uint64_t sum2 = pack2(0.f, 0.f);
      uint32_t p[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const uint64_t xx = fma2(pack2(__uint_as_float(r0[2 * i]), __uint_as_float(r0[2 * i + 1])), c2, m2);
        float e0, e1;
        if (POLY8 != 0 && (i % 5) == 4) {
          poly_exp2_pair(xx, e0, e1);
        } else {
          float x0, x1;
          unpack2(xx, x0, x1);
          e0 = fast_exp2(x0); e1 = fast_exp2(x1);
        }
        sum2 = add2(sum2, pack2(e0, e1));
        p[i] = pack_p2<F16>(e0, e1);
      }
      if (j > 0) {
        // P of the previous tile has been consumed and O is complete up to it: P may be overwritten, O rescaled
        if (!tc::mbar_wait(my_o_full, (uint32_t)(j - 1) & 1u, wc, 206)) { ok = false; break; }
        tc::tc_fence_after_sync();
      }
      tc::tmem_st_32x32b_x16(p_tmem, p);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const uint64_t xx = fma2(pack2(__uint_as_float(r1[2 * i]), __uint_as_float(r1[2 * i + 1])), c2, m2);
        float e0, e1;
        if (POLY8 != 0 && (i % 5) == 4) {
          poly_exp2_pair(xx, e0, e1);
        } else {
          float x0, x1;
          unpack2(xx, x0, x1);
          e0 = fast_exp2(x0); e1 = fast_exp2(x1);
        }
        sum2 = add2(sum2, pack2(e0, e1));
        p[i] = pack_p2<F16>(e0, e1);
      }
      tc::tmem_st_32x32b_x16(p_tmem + 16, p);
      float sum, sum_hi;
      unpack2(sum2, sum, sum_hi);
      sum += sum_hi;
      l_run = l_run * alpha + sum;
      if (j > 0 && moved) {
#pragma unroll
        for (int c = 0; c < D; c += 16) {
          uint32_t o[16];
          tc::tmem_ld_32x32b_x16(o_tmem + c, o);
          tc::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tc::tmem_st_32x32b_x16(o_tmem + c, o);
        }
      }
      tc::tmem_st_wait();
      tc::tc_fence_before_sync();
      tc::mbar_arrive(my_p_full);
    }
    if (ok && tc::mbar_wait(my_o_full, (uint32_t)(num_tiles - 1) & 1u, wc, 207) && q_tok + row < a.L) {
      tc::tc_fence_after_sync();
      const float inv = 1.f / l_run;
      const size_t tok = (size_t)brow * a.L + q_tok + row;
      __nv_bfloat16 *op = a.O + (tok * a.H + head) * D;
#pragma unroll
      for (int c = 0; c < D; c += 16) {
        uint32_t o[16];
        tc::tmem_ld_32x32b_x16(o_tmem + c, o);
        tc::tmem_ld_wait();
        uint4 w[2];
        uint32_t *h2 = reinterpret_cast<uint32_t *>(w);
#pragma unroll
        for (int i = 0; i < 8; ++i) h2[i] = pack_p2<F16>(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv);
        *reinterpret_cast<uint4 *>(op + c) = w[0];
        *reinterpret_cast<uint4 *>(op + c + 8) = w[1];
      }
      a.lse[tok * a.H + head] = (m_run + log2f(l_run)) * 0.6931471805599453f;
    }
  }

  tc::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 0) { tc::tc_fence_after_sync(); tc::tmem_dealloc(tmem_base, C::kTmemCols); }
}

template <int D, int BKV, int NQ, int POLY8, bool F16>
static int launch_attn_fwd(const void *Q, const void *K, const void *V, AttnFwdArgs a, int device, cudaStream_t st) {
  using C = AttnCfg<D, BKV, NQ>;
  auto kern = attn_fwd_kernel<D, BKV, NQ, POLY8, F16>;
  const int dt = F16 ? 1 : 0;
  F3D_TRY(ensure_dynamic_smem(reinterpret_cast<const void *>(kern), device, C::kSmem));
  CUtensorMap mq, mk, mv;
  const uint64_t rows = (uint64_t)a.B * a.L;
  const uint64_t s1 = (uint64_t)D * 2, s2 = (uint64_t)a.H * D * 2;
  F3D_TRY(encode_tmap_3d(&mq, dt, Q, D, a.H, rows, s1, s2, C::DCH, 1, kBQ, C::RB));
  F3D_TRY(encode_tmap_3d(&mk, dt, K, D, a.H, rows, s1, s2, C::DCH, 1, BKV, C::RB));
  F3D_TRY(encode_tmap_3d(&mv, dt, V, D, a.H, rows, s1, s2, C::DCH, 1, BKV, C::RB));
  dim3 grid(a.num_scopes * (a.k * a.q_blocks_per_bucket / NQ), a.H, a.B);
  kern<<<grid, C::kThreads, C::kSmem, st>>>(mq, mk, mv, a);
  return check_launch("buck_swin_fwd");
}

// Head sizes up to 32 are bound by the special-function unit: three of every sixteen exponentials go to the FMA pipe
// (measured at D = 32, window 4096, with adjacent pairs: 0 / 12.5 / 25 / 37.5 / 50 % -> 439 / 448 / 462 / 446 / 413
// TFLOP/s; spread out as every fifth pair, 18.75 %: 497).  One query tile per CTA:
// two and four tiles per CTA sharing the K/V stream measured 2 % and 4 % slower (their exponential phases line up).
template <bool F16>
static int launch_attn_fwd_any(int D, const void *Q, const void *K, const void *V, AttnFwdArgs a, int device, cudaStream_t st) {
  switch (D) {
    case 16: return launch_attn_fwd<16, 64, 1, 2, F16>(Q, K, V, a, device, st);
    case 32: return launch_attn_fwd<32, 64, 1, 2, F16>(Q, K, V, a, device, st);
    case 64: return launch_attn_fwd<64, 64, 1, 0, F16>(Q, K, V, a, device, st);
    default: return launch_attn_fwd<128, 64, 1, 0, F16>(Q, K, V, a, device, st);
  }
}

}  // namespace f3d

using namespace f3d;

static int buck_swin_fwd_impl(const void *Q, const void *K, const void *V, void *O, void *LSE, const void *scope_buckets,
                              int B, int L, int H, int D, int num_scopes, int scope_size, uint32_t bucket_size, int dtype,
                              int device, void *stream) {
  if (B <= 0 || L <= 0 || H <= 0) return set_error(F3D_ERR_ARG, "buck_swin_fwd: empty tensor");
  if (dtype != 0 && dtype != 1) return set_error(F3D_ERR_UNSUPPORTED, "buck_swin_fwd: element type %d (0 = bf16 and 1 = fp16 are supported)", dtype);
  if (D != 16 && D != 32 && D != 64 && D != 128) return set_error(F3D_ERR_UNSUPPORTED, "buck_swin_fwd: head_dim %d (16, 32, 64, 128 are supported)", D);
  if (bucket_size == 0 || bucket_size % kBQ) return set_error(F3D_ERR_UNSUPPORTED, "buck_swin_fwd: bucket_size %u must be a positive multiple of %d", bucket_size, kBQ);
  if (L % (int)bucket_size) return set_error(F3D_ERR_ARG, "buck_swin_fwd: sequence length %d is not a multiple of bucket_size %u", L, bucket_size);
  if (num_scopes < 0 || scope_size <= 0) return set_error(F3D_ERR_ARG, "buck_swin_fwd: Scope_buckets must be [S,k] with k > 0");
  if ((long long)H > 65535 || (long long)B > 65535) return set_error(F3D_ERR_UNSUPPORTED, "buck_swin_fwd: H and B must fit a grid dimension");
  if (num_scopes == 0) return F3D_OK;
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  F3D_TRY(maybe_sync(st, "buck_swin_fwd"));
  AttnFwdArgs a{static_cast<__nv_bfloat16 *>(O), static_cast<float *>(LSE), static_cast<const uint32_t *>(scope_buckets),
                B, L, H, num_scopes, scope_size, (int)bucket_size, (int)bucket_size / kBQ,
                1.4426950408889634f / sqrtf((float)D), status_word(device)};
  if (!a.status) return F3D_ERR_CUDA;
  F3D_TRY(dtype == 1 ? launch_attn_fwd_any<true>(D, Q, K, V, a, device, st) : launch_attn_fwd_any<false>(D, Q, K, V, a, device, st));
  return maybe_sync(st, "buck_swin_fwd");
}

extern "C" int f3d_buck_swin_fwd(const void *Q, const void *K, const void *V, void *O, void *LSE, const void *scope_buckets,
                                 int B, int L, int H, int D, int num_scopes, int scope_size, uint32_t bucket_size,
                                 int device, void *stream) {
  return buck_swin_fwd_impl(Q, K, V, O, LSE, scope_buckets, B, L, H, D, num_scopes, scope_size, bucket_size, 0, device, stream);
}

extern "C" int f3d_buck_swin_fwd_dtype(const void *Q, const void *K, const void *V, void *O, void *LSE, const void *scope_buckets,
                                       int B, int L, int H, int D, int num_scopes, int scope_size, uint32_t bucket_size,
                                       int dtype, int device, void *stream) {
  return buck_swin_fwd_impl(Q, K, V, O, LSE, scope_buckets, B, L, H, D, num_scopes, scope_size, bucket_size, dtype, device, stream);
}
