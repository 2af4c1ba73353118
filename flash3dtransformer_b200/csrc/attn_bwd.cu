// Bucketed self-attention backward on tcgen05 tensor cores, sm_100a.
//
// Implements buck_swin_bwd(Q, K, V, O, dO, LSE, Delta, dQ, dK, dV, Scope_buckets, bucket_size), which the reference's
// Python layer calls (flash3dxfmr/layers/buck_swin.py:91) but whose kernel and binding are absent from the reference
// snapshot (declaration src/f3d_frontend.cu:94-97, binding commented out :137).  Semantics follow the reference's
// tests (tests/test_attn_bwd.py:24-27,54-62,79-441): Delta[b,t,h] = sum_d dO*O is written to the caller's buffer;
// with P = exp(S - LSE), dV = P^T dO, dP = dO V^T, dS = P o (dP - Delta), dQ = dS K / sqrt(D), dK = dS^T Q / sqrt(D).
// O and LSE may come from any forward implementation (the tests pass FlashAttention's).
//
// Kernels:
//   attn_bwd_delta_kernel   Delta = rowsum(dO o O), one thread per (token, head)
//   attn_bwd_kernel<D>      one CTA per (scope, 128-key block, head, batch row); it loops over the query tiles of the
//                           scope and keeps dK, dV for its keys in tensor memory.  D = 64 / 128: 576 threads, one CTA
//                           per SM, 512 tensor-memory columns.  D <= 32 (32 is the backbone's head size): 320-352 threads,
//                           TWO CTAs per SM with 256 columns each and 64-query tiles, so that one CTA computes while the
//                           other waits for its products
//       warp 0      TMA producer: K_j, V_j once; Q_i, dO_i through a 2- or 3-stage ring
//       warp 1      issues S^T = K Q^T and dP^T = V dO^T into tensor memory (keys on the lanes); once the compute
//                   warps have published P^T and dS^T it first issues the NEXT tile's S^T / dP^T, then dV += P^T dO
//                   and dK += dS^T Q (A from tensor memory where the columns allow it, else K-major shared-memory
//                   tiles) and dQ_i = dS K (the dS^T shared-memory tile read as an MN-major A operand)
//       compute     16 warps (8 at D <= 32): a thread owns one key row and a share of the query columns;
//                   p = exp2(s*c - lse), ds = p*(dp - delta) in packed fp32 pairs.  Except at D = 64 the score products
//                   deliver s - lse/scale and dp - delta themselves (an extra k-step carries the per-query constants,
//                   BwdCfg::kFold); otherwise -lse / -delta of the tile are staged in shared memory one tile ahead
//                   and fetched per column.  Afterwards the warps read dQ of the previous tile from tensor memory
//                   (queries on the lanes) and add it to an fp32 scratch: with vector reductions, or at D = 32 by
//                   staging the tile in shared memory for
//       drain warp  (D = 32) one thread hands each staged dQ tile to the copy engine as a single add-reduce
//                   (cp.reduce.async.bulk.tensor) and recycles the two staging buffers
// What bounds the kernel at D = 32 is the shared-memory pipe: dS^T stores, the tensor cores' operand reads and, before
// the constants moved into the products, one broadcast load per query constant and warp (a third of all wavefronts).
//   attn_bwd_dq_convert     dQ = bf16(scratch / sqrt(D))
// dQ needs the scratch because every key block of a scope contributes to every query; dK and dV are written once.
//   attn_bwd_window_kernel<D>   windows of at most 512 tokens at D <= 32: one CTA per (scope, head) walks key blocks
//                           and query tiles and keeps every dQ tile in tensor memory, so nothing goes through the
//                           scratch (see the comment at the kernel)
#include "f3d_common.cuh"
#include "tc_sm100.cuh"
#include "../../include/f3d_b200.h"

namespace f3d {

int *status_word(int device);

constexpr int kBwdComputeWarps = 16;
constexpr int kBwdThreads = 64 + 32 * kBwdComputeWarps;       // producer warp, MMA warp, compute warps
constexpr int kBK = 128;               // keys per CTA (tensor-memory lanes)

struct AttnBwdArgs {
  const float *lse; const float *delta; float *dq_acc; __nv_bfloat16 *dK; __nv_bfloat16 *dV; const uint32_t *scopes;
  int B, L, H, num_scopes, k, bucket, kblocks_per_bucket;
  float scale_log2, scale, inv_scale;       // log2(e) / sqrt(D), 1 / sqrt(D), sqrt(D)
  int *status;
};

__device__ __forceinline__ float bwd_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// packed fp32 pairs
__device__ __forceinline__ uint64_t bpack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void bunpack2(uint64_t v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t bfma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t badd2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t bmul2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

template <int D> struct BwdCfg {
  // D <= 32 (32 is the backbone's head size) runs as TWO CTAs per SM: tiles of 64 queries, eight compute warps and 256
  // tensor-memory columns per CTA.  A CTA's tile is a chain of hand-offs (score products -> compute warps -> gradient
  // products -> dQ read-out) in which the compute warps, the busiest part, work less than half of the time; with two
  // CTAs on the SM one computes while the other waits.
  static constexpr bool kTwo = D <= 32;
  static constexpr int kMinCtas = kTwo ? 2 : 1;
  static constexpr int kCW = kTwo ? 8 : kBwdComputeWarps;        // compute warps: kCW / 4 per tensor-memory lane quadrant
  static constexpr int BQ = (D == 128 || kTwo) ? 64 : 128;       // queries per inner tile
  static constexpr int QCOLS = BQ / (kCW / 4);                   // query columns per compute thread
  static constexpr int kChunk = kTwo ? 16 : QCOLS;               // of which are held in registers at a time
  static constexpr int DCH = D < 64 ? D : 64;
  static constexpr int NDCH = D / DCH;
  static constexpr int RB = DCH * 2;
  static constexpr uint64_t SWZ = RB == 128 ? tc::kSwizzle128 : (RB == 64 ? tc::kSwizzle64 : tc::kSwizzle32);
  static constexpr int kKVBytes = kBK * D * 2;                   // one of K_j, V_j
  static constexpr int kQBytes = BQ * D * 2;                     // one of Q_i, dO_i
  static constexpr int kQStage = 2 * kQBytes;
  static constexpr int QS = D <= 32 ? 3 : 2;                     // Q / dO stages
  static constexpr int PB = D == 64 ? 1 : 2;                     // P^T / dS^T shared-memory buffers (what fits in 227 KB)
  static constexpr int kPBytes = kBK * BQ * 2;                   // P^T or dS^T tile
  // With D <= 32 the bf16 P^T and dS^T tiles also fit in tensor memory (64 columns each): dV and dK then take
  // their A operand from there and only dS^T, which dQ = dS K reads transposed, goes through shared memory.  That
  // halves the shared-memory traffic per tile, which was what bounded the kernel.
  static constexpr bool kTS = D <= 32;
  // dS^T goes through shared memory in any case (dQ = dS K reads it transposed).  With 512 columns it is also kept in
  // tensor memory for dK; with 256 columns per CTA dK reads the shared-memory tile.
  static constexpr bool kDsT = kTS && !kTwo;
  static constexpr int kBufBytes = kTS ? kPBytes : 2 * kPBytes;  // per buffer: dS^T (| P^T)
  // kFold: -lse and -delta enter the score products themselves.  S^T = K Q^T gets one more k-step of 16 whose K side is
  // a constant tile of ones and whose Q side holds -lse * sqrt(D) of each query as three bf16 terms (hi + mid + lo, exact
  // to 2^-24), so the product comes out as s - lse / scale; dP^T = V dO^T likewise comes out as dp - delta.  Otherwise
  // every compute thread has to fetch both per-query constants for each of its columns from shared memory: broadcast
  // loads that cost a wavefront per value and warp and were a third of all shared-memory traffic of a kernel whose
  // shared-memory pipe (those loads, the dS^T stores, the tensor cores' operand reads) was saturated.
  // (measured per head size: D = 16 200 -> 243 (264 with two CTAs per SM), D = 32 426 -> 485-512, D = 128 579-600 -> 618 TFLOP/s; D = 64, whose
  // compute threads are short of registers, 549 -> 509, so it keeps the per-column loads)
  static constexpr bool kFold = D != 64;
  static constexpr int kOnesBytes = kFold ? kBK * 32 : 0;          // [128 keys][16] bf16, ones in three columns of each half
  static constexpr int kXBytes = kFold ? BQ * 32 : 0;              // [BQ queries][16] bf16: the three terms, then zeros
  static constexpr int kLsdBytes = kFold ? 0 : 2 /*stages*/ * 2 * BQ * 4;
  // D = 32: the dQ tile (128 rows of 128 bytes) leaves through shared memory and ONE add-reduce of the copy engine
  // instead of 1024 vector reductions issued by the compute warps; two staging buffers
  static constexpr bool kTmaDq = D == 32;
  static constexpr int kDqStageBytes = kTmaDq ? BQ * D * 4 : 0;
  static constexpr int kSmem = 2 * kKVBytes + QS * kQStage + PB * kBufBytes + 2 * kDqStageBytes + kOnesBytes + QS * 2 * kXBytes +
                               kLsdBytes + 256 + 1024;
  static constexpr int kThreads = 64 + 32 * kCW + (kTmaDq ? 32 : 0);  // producer, MMA, compute warps (+ one warp that feeds the copy engine)
  static_assert(kSmem <= 227 * 1024, "shared memory budget");
  // tensor-memory columns: S^T, dP^T, (P^T, dS^T as bf16 pairs), dV, dK, dQ
  static constexpr uint32_t kSCol = 0, kDpCol = BQ, kPtCol = 2 * BQ, kDsCol = 2 * BQ + BQ / 2;
  static constexpr uint32_t kDvCol = kTS ? (kDsT ? 3 * BQ : 2 * BQ + BQ / 2) : 2 * BQ, kDkCol = kDvCol + D, kDqCol = kDkCol + D;
  static constexpr uint32_t kTmemCols = kTwo ? 256 : 512;
  static_assert(kDqCol + D <= kTmemCols, "tensor-memory budget");
};

template <int D>
__global__ void __launch_bounds__(BwdCfg<D>::kThreads, BwdCfg<D>::kMinCtas)
attn_bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                const __grid_constant__ CUtensorMap map_dq, AttnBwdArgs a) {
  using C = BwdCfg<D>;
  constexpr int BQ = C::BQ, QS = C::QS, PB = C::PB;
  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char *sk = smem, *sv = sk + C::kKVBytes;
  unsigned char *sqdo = sv + C::kKVBytes;                         // [QS stages][Q | dO]
  // per buffer dS^T sits in front of P^T: with 64-query tiles the dQ MMA (M = 128) reads one 64-row atom past the
  // dS^T tile, which then falls inside the P^T tile of the same buffer (rows 64..127 of that product are never used)
  unsigned char *spds = sqdo + QS * C::kQStage;                   // [PB buffers][dS^T | P^T]
  unsigned char *sdq = spds + PB * C::kBufBytes;                  // [2][BQ rows of 128 bytes] dQ staging (1 KB aligned)
  unsigned char *sones = sdq + 2 * C::kDqStageBytes;             // kFold: the constant k-step of K and V
  unsigned char *sx = sones + C::kOnesBytes;                     // kFold: [QS stages][Q side | dO side] of that k-step
  float *slsd = reinterpret_cast<float *>(sx + QS * 2 * C::kXBytes);      // else: [stage][-lse2 | -delta][BQ]
  uint64_t *bars = reinterpret_cast<uint64_t *>(reinterpret_cast<unsigned char *>(slsd) + C::kLsdBytes);
  uint64_t *kv_full = bars, *qdo_full = bars + 1, *qdo_empty = qdo_full + QS, *s_full = qdo_empty + QS, *dp_full = s_full + 1;
  uint64_t *pds_full = dp_full + 1, *pds_empty = pds_full + 1 /*[PB]*/, *dq_full = pds_empty + PB, *dq_read = dq_full + 1;
  uint64_t *dkv_full = dq_read + 1, *lsd_full = dkv_full + 1 /*[2]*/;
  uint64_t *pt_free = lsd_full + 2;
  uint64_t *dqs_written = pt_free + 1, *dqs_free = dqs_written + 1 /*[2]*/;
  uint64_t *x_full = dqs_free + 2 /*[QS]*/;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(x_full + QS);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb_lin = blockIdx.x;
  const int kb = kb_lin % a.kblocks_per_bucket;
  const int bj = (kb_lin / a.kblocks_per_bucket) % a.k;
  const int scope = kb_lin / (a.kblocks_per_bucket * a.k);
  const int head = blockIdx.y, brow = blockIdx.z;
  const uint32_t *my_scope = a.scopes + (size_t)scope * a.k;
  const int qtiles_per_bucket = a.bucket / BQ;
  const int num_qtiles = a.k * qtiles_per_bucket;
  const int key_tok = (int)my_scope[bj] * a.bucket + kb * kBK;

  if (threadIdx.x == 0) {
    tc::mbar_init(kv_full, 1);
    for (int s = 0; s < QS; ++s) { tc::mbar_init(&qdo_full[s], 1); tc::mbar_init(&qdo_empty[s], 1); }
    tc::mbar_init(s_full, 1); tc::mbar_init(dp_full, 1); tc::mbar_init(pds_full, 32 * C::kCW);
    for (int b = 0; b < PB; ++b) tc::mbar_init(&pds_empty[b], 1);
    tc::mbar_init(dq_full, 1); tc::mbar_init(dq_read, 32 * C::kCW); tc::mbar_init(dkv_full, 1);
    tc::mbar_init(dqs_written, 256); tc::mbar_init(&dqs_free[0], 1); tc::mbar_init(&dqs_free[1], 1);
    tc::mbar_init(&lsd_full[0], BQ); tc::mbar_init(&lsd_full[1], BQ); tc::mbar_init(pt_free, 1);
    for (int s = 0; s < QS; ++s) tc::mbar_init(&x_full[s], BQ);
    *abort_flag = 0;
    tc::mbar_fence_init();
  }
  if (C::kFold) {
    // the constant k-step: every 16-byte half of every row is (1, 1, 1, 0, 0, 0, 0, 0), so that the product with a row
    // that carries its three terms in one half and zeros in the other does not depend on where the swizzle puts the
    // halves; the query-side rows start as zeros and only their first half is rewritten per tile
    for (int c = threadIdx.x; c < C::kOnesBytes / 16; c += C::kThreads)
      tc::sts128(tc::smem_u32(sones) + c * 16, make_uint4(0x3F803F80u, 0x00003F80u, 0u, 0u));
    for (int c = threadIdx.x; c < QS * 2 * C::kXBytes / 16; c += C::kThreads)
      tc::sts128(tc::smem_u32(sx) + c * 16, make_uint4(0u, 0u, 0u, 0u));
    tc::fence_proxy_async();
  }
  if (warp == 1) { tc::tmem_alloc(tmem_slot, C::kTmemCols); tc::tmem_relinquish(); }
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  tc::WaitCtx wc{abort_flag, a.status};

  if (warp == 0) {
    if (tc::elect_one()) {
      tc::tma_prefetch_desc(&map_q); tc::tma_prefetch_desc(&map_k); tc::tma_prefetch_desc(&map_v); tc::tma_prefetch_desc(&map_do);
      tc::mbar_expect_tx(kv_full, 2 * C::kKVBytes);
#pragma unroll
      for (int c = 0; c < C::NDCH; ++c) {
        tc::tma_load_3d(sk + c * kBK * C::RB, &map_k, kv_full, c * C::DCH, head, brow * a.L + key_tok);
        tc::tma_load_3d(sv + c * kBK * C::RB, &map_v, kv_full, c * C::DCH, head, brow * a.L + key_tok);
      }
      for (int i = 0; i < num_qtiles; ++i) {
        const int s = i % QS;
        const uint32_t ph = (uint32_t)(i / QS) & 1u;
        if (!tc::mbar_wait(&qdo_empty[s], ph ^ 1u, wc, 301, 200)) break;
        const int q_tok = (int)my_scope[i / qtiles_per_bucket] * a.bucket + (i % qtiles_per_bucket) * BQ;
        unsigned char *sq = sqdo + s * C::kQStage, *sdo = sq + C::kQBytes;
        tc::mbar_expect_tx(&qdo_full[s], C::kQStage);
#pragma unroll
        for (int c = 0; c < C::NDCH; ++c) {
          tc::tma_load_3d(sq + c * BQ * C::RB, &map_q, &qdo_full[s], c * C::DCH, head, brow * a.L + q_tok);
          tc::tma_load_3d(sdo + c * BQ * C::RB, &map_do, &qdo_full[s], c * C::DCH, head, brow * a.L + q_tok);
        }
      }
    }
  } else if (warp == 1) {
    if (tc::elect_one()) {
      constexpr uint32_t idesc_s = tc::make_idesc_f16(kBK, BQ, true, false, false);          // S^T, dP^T
      constexpr uint32_t idesc_kv = tc::make_idesc_f16(kBK, C::DCH, true, false, true);      // dV, dK: B MN-major
      constexpr uint32_t idesc_dq = tc::make_idesc_f16(128, C::DCH, true, true, true);       // dQ: A and B MN-major
      const uint32_t k_addr = tc::smem_u32(sk), v_addr = tc::smem_u32(sv);
      bool ok = tc::mbar_wait(kv_full, 0, wc, 302);

      auto issue_s_dp = [&](int i) -> bool {
        const int s = i % QS;
        if (!tc::mbar_wait(&qdo_full[s], (uint32_t)(i / QS) & 1u, wc, 303)) return false;
        if (C::kFold && !tc::mbar_wait(&x_full[s], (uint32_t)(i / QS) & 1u, wc, 315)) return false;
        tc::tc_fence_after_sync();
        const uint32_t q_addr = tc::smem_u32(sqdo + s * C::kQStage), do_addr = q_addr + C::kQBytes;
        const uint32_t ones_addr = tc::smem_u32(sones), qx_addr = tc::smem_u32(sx + s * 2 * C::kXBytes), dox_addr = qx_addr + C::kXBytes;
#pragma unroll
        for (int c = 0; c < C::NDCH; ++c)
#pragma unroll
          for (int kk = 0; kk < C::DCH / 16; ++kk)
            tc::mma_f16_ss(tmem_base + C::kSCol, tc::make_smem_desc(k_addr + c * kBK * C::RB + kk * 32, 16, 8 * C::RB, C::SWZ),
                           tc::make_smem_desc(q_addr + c * BQ * C::RB + kk * 32, 16, 8 * C::RB, C::SWZ), idesc_s, (c | kk) != 0);
        if (C::kFold)      // + 1 * (-lse * sqrt(D)) in three terms
          tc::mma_f16_ss(tmem_base + C::kSCol, tc::make_smem_desc(ones_addr, 16, 256, tc::kSwizzle32),
                         tc::make_smem_desc(qx_addr, 16, 256, tc::kSwizzle32), idesc_s, 1u);
        tc::mma_commit(s_full);
#pragma unroll
        for (int c = 0; c < C::NDCH; ++c)
#pragma unroll
          for (int kk = 0; kk < C::DCH / 16; ++kk)
            tc::mma_f16_ss(tmem_base + C::kDpCol, tc::make_smem_desc(v_addr + c * kBK * C::RB + kk * 32, 16, 8 * C::RB, C::SWZ),
                           tc::make_smem_desc(do_addr + c * BQ * C::RB + kk * 32, 16, 8 * C::RB, C::SWZ), idesc_s, (c | kk) != 0);
        if (C::kFold)      // + 1 * (-delta) in three terms
          tc::mma_f16_ss(tmem_base + C::kDpCol, tc::make_smem_desc(ones_addr, 16, 256, tc::kSwizzle32),
                         tc::make_smem_desc(dox_addr, 16, 256, tc::kSwizzle32), idesc_s, 1u);
        tc::mma_commit(dp_full);
        return true;
      };

      if (ok) ok = issue_s_dp(0);
      constexpr uint32_t idesc_kv_ts = tc::make_idesc_f16(kBK, C::DCH, true, false, true);   // A from tensor memory
      for (int i = 0; i < num_qtiles && ok; ++i) {
        const int s = i % QS, pb = i % PB;
        // P^T and dS^T of tile i are published, and every compute thread has read S^T and dP^T
        if (!tc::mbar_wait(pds_full, (uint32_t)i & 1u, wc, 305)) { ok = false; break; }
        // the next tile's scores first: the compute warps work on them while the tensor pipe runs this tile's
        // three gradient products
        if (i + 1 < num_qtiles && !issue_s_dp(i + 1)) { ok = false; break; }
        tc::tc_fence_after_sync();
        const uint32_t q_addr = tc::smem_u32(sqdo + s * C::kQStage), do_addr = q_addr + C::kQBytes;
        const uint32_t ds_addr = tc::smem_u32(spds + pb * C::kBufBytes), pt_addr = ds_addr + C::kPBytes;
        // dV += P^T dO and dK += dS^T Q, 16 queries per instruction.  A = [keys x queries]: tensor memory (two
        // bf16 per column) when it fits, else shared-memory tiles with 128-byte rows of 64 queries
#pragma unroll
        for (int c = 0; c < C::NDCH; ++c) {
#pragma unroll
          for (int qk = 0; qk < BQ / 16; ++qk) {
            const uint32_t b_off = c * BQ * C::RB + qk * 16 * C::RB;
            const uint64_t b_do = tc::make_smem_desc(do_addr + b_off, 16, 8 * C::RB, C::SWZ);
            const uint64_t b_q = tc::make_smem_desc(q_addr + b_off, 16, 8 * C::RB, C::SWZ);
            if (C::kDsT) {
              tc::mma_f16_ts(tmem_base + C::kDvCol + c * C::DCH, tmem_base + C::kPtCol + qk * 8, b_do, idesc_kv_ts, (i | qk) != 0);
              tc::mma_f16_ts(tmem_base + C::kDkCol + c * C::DCH, tmem_base + C::kDsCol + qk * 8, b_q, idesc_kv_ts, (i | qk) != 0);
            } else if (C::kTS) {
              const uint32_t a_off = (qk / 4) * (kBK * 128) + (qk % 4) * 32;
              tc::mma_f16_ts(tmem_base + C::kDvCol + c * C::DCH, tmem_base + C::kPtCol + qk * 8, b_do, idesc_kv_ts, (i | qk) != 0);
              tc::mma_f16_ss(tmem_base + C::kDkCol + c * C::DCH, tc::make_smem_desc(ds_addr + a_off, 16, 1024, tc::kSwizzle128), b_q, idesc_kv, (i | qk) != 0);
            } else {
              const uint32_t a_off = (qk / 4) * (kBK * 128) + (qk % 4) * 32;
              tc::mma_f16_ss(tmem_base + C::kDvCol + c * C::DCH, tc::make_smem_desc(pt_addr + a_off, 16, 1024, tc::kSwizzle128), b_do, idesc_kv, (i | qk) != 0);
              tc::mma_f16_ss(tmem_base + C::kDkCol + c * C::DCH, tc::make_smem_desc(ds_addr + a_off, 16, 1024, tc::kSwizzle128), b_q, idesc_kv, (i | qk) != 0);
            }
          }
        }
        tc::mma_commit(&qdo_empty[s]);
        if (C::kTS) tc::mma_commit(pt_free);
        // dQ_i = dS K_j: A = the dS^T tile read M-major (queries contiguous), K = keys in steps of 16 rows
        if (i > 0 && !tc::mbar_wait(dq_read, (uint32_t)(i - 1) & 1u, wc, 306)) { ok = false; break; }
        tc::tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < C::NDCH; ++c)
#pragma unroll
          for (int ks = 0; ks < kBK / 16; ++ks)
            tc::mma_f16_ss(tmem_base + C::kDqCol + c * C::DCH,
                           tc::make_smem_desc(ds_addr + ks * 16 * 128, kBK * 128, 1024, tc::kSwizzle128),
                           tc::make_smem_desc(k_addr + c * kBK * C::RB + ks * 16 * C::RB, 16, 8 * C::RB, C::SWZ), idesc_dq, ks != 0);
        tc::mma_commit(dq_full);
        tc::mma_commit(&pds_empty[pb]);
        if (i + 1 == num_qtiles) tc::mma_commit(dkv_full);
      }
    }
  } else if (warp < 2 + C::kCW) {
    // Compute warps: kCW / 4 per tensor-memory lane quadrant; a thread owns one key row and, per query tile, the
    // BQ / 4 query columns of its warp.  After publishing tile i the warps read out dQ of tile i - 1 (queries on
    // the lanes) and add it to the fp32 scratch with vector reductions.
    const int cw = warp - 2;                          // 0..kCW-1
    const int q4 = warp & 3;                          // tensor-memory lane quadrant of this warp
    const int cidx = cw >> 2;                         // which part of the query columns
    const int ctid = cw * 32 + lane;                  // 0..32*kCW-1
    const int row = q4 * 32 + lane;                   // key row (S^T, dP^T, dK, dV) or query row (dQ)
    const uint32_t lane_off = (uint32_t)(q4 * 32) << 16;
    constexpr int QCOLS = C::QCOLS;                   // query columns per compute thread (32 or 16)
    constexpr int CH = C::kChunk;                     // of which one tensor-memory load brings in
    const int col0 = cidx * QCOLS;
    const uint64_t c2 = bpack2(a.scale_log2, a.scale_log2);
    bool ok = true;
    // -lse2 and -delta of a query tile are staged in shared memory one tile ahead: the global loads for tile
    // i + 1 are issued before the arithmetic of tile i and land in registers while it runs
    auto lsd_index = [&](int i) {
      const int q_tok = (int)my_scope[i / qtiles_per_bucket] * a.bucket + (i % qtiles_per_bucket) * BQ;
      return ((size_t)brow * a.L + q_tok + ctid) * a.H + head;
    };
    // v as three bf16 terms whose sum is v to 2^-24: (hi | mid << 16, lo)
    auto split3 = [](float v, uint32_t &w0, uint32_t &w1) {
      const __nv_bfloat16 h0 = __float2bfloat16_rn(v);
      const float r1 = v - __bfloat162float(h0);
      const __nv_bfloat16 h1 = __float2bfloat16_rn(r1);
      const __nv_bfloat16 h2 = __float2bfloat16_rn(r1 - __bfloat162float(h1));
      w0 = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
      w1 = (uint32_t)__bfloat16_as_ushort(h2);
    };
    auto lsd_publish = [&](int i, float l, float d) {
      if constexpr (C::kFold) {
        // query ctid of tile i: the first half of its row of the extra k-step, for S^T and for dP^T.  The stage last held
        // tile i - QS, whose score products finished before this thread's previous tile began.
        const int s = i % QS;
        const uint32_t base = tc::smem_u32(sx + s * 2 * C::kXBytes) + (uint32_t)ctid * 32u;
        uint32_t w0, w1;
        split3(-l * a.inv_scale, w0, w1);
        tc::sts128(base, make_uint4(w0, w1, 0u, 0u));
        split3(-d, w0, w1);
        tc::sts128(base + C::kXBytes, make_uint4(w0, w1, 0u, 0u));
        tc::fence_proxy_async();
        tc::mbar_arrive(&x_full[s]);
      } else {
        const uint32_t base = tc::smem_u32(slsd + (i & 1) * 2 * BQ);
        tc::sts32(base + ctid * 4, l * -1.4426950408889634f);
        tc::sts32(base + BQ * 4 + ctid * 4, -d);
        tc::mbar_arrive(&lsd_full[i & 1]);
      }
    };
    // dQ of tile i: two warps per quadrant take half of the D columns each
    auto read_out_dq = [&](int i) -> bool {
      if (!tc::mbar_wait(dq_full, (uint32_t)i & 1u, wc, 310)) return false;
      tc::tc_fence_after_sync();
      const int q_tok = (int)my_scope[i / qtiles_per_bucket] * a.bucket + (i % qtiles_per_bucket) * BQ;
      if constexpr (C::kTmaDq) {
        // The eight warps with cidx < 2 pull the tile out of tensor memory, release it, and write it to a staging
        // buffer in the 128-byte-swizzled layout of the scratch's tensor map; the drain warp hands the whole tile to
        // the copy engine as one add-reduce.  The compute warps issue no global reductions, so their next loads no
        // longer queue behind them (all sixteen warps sharing the read-out measured 1 % slower).
        if (cidx < 2) {
          const int buf = i & 1, use = i >> 1;
          // the add-reduce that last read this buffer (tile i - 2) has finished reading it
          if (use > 0 && !tc::mbar_wait(&dqs_free[buf], (uint32_t)(use - 1) & 1u, wc, 313)) return false;
          __syncwarp();
          const uint32_t stg = tc::smem_u32(sdq + buf * C::kDqStageBytes) + (uint32_t)row * 128u;
          // with 64-query tiles the lanes of quadrants 2 and 3 hold no query (the dQ product has M = 128 rows)
#pragma unroll
          for (int h = 0; h < 2 && q4 * 32 < BQ; ++h) {
            uint32_t o[8];
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                         : "=r"(o[0]), "=r"(o[1]), "=r"(o[2]), "=r"(o[3]), "=r"(o[4]), "=r"(o[5]), "=r"(o[6]), "=r"(o[7])
                         : "r"(tmem_base + lane_off + C::kDqCol + cidx * 16 + h * 8) : "memory");
            tc::tmem_ld_wait();
            const int ch = cidx * 4 + h * 2;
            tc::sts128(stg + (uint32_t)((ch ^ (row & 7)) * 16), make_uint4(o[0], o[1], o[2], o[3]));
            tc::sts128(stg + (uint32_t)(((ch + 1) ^ (row & 7)) * 16), make_uint4(o[4], o[5], o[6], o[7]));
          }
        }
        tc::tc_fence_before_sync();
        tc::mbar_arrive(dq_read);
        if (cidx < 2) {
          const int buf = i & 1;
          tc::fence_proxy_async();
          tc::mbar_arrive(dqs_written);
        }
        return true;
      }
      if (cidx < 2) {
        float *dst = a.dq_acc + (((size_t)brow * a.L + q_tok + row) * a.H + head) * D + cidx * (D / 2);
        const bool live = row < BQ && q_tok + row < a.L;
#pragma unroll
        for (int c = 0; c < D / 2; c += 8) {
          uint32_t o[8];
          asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                       : "=r"(o[0]), "=r"(o[1]), "=r"(o[2]), "=r"(o[3]), "=r"(o[4]), "=r"(o[5]), "=r"(o[6]), "=r"(o[7])
                       : "r"(tmem_base + lane_off + C::kDqCol + cidx * (D / 2) + c) : "memory");
          tc::tmem_ld_wait();
          if (live) {
            atomicAdd(reinterpret_cast<float4 *>(dst + c), make_float4(__uint_as_float(o[0]), __uint_as_float(o[1]), __uint_as_float(o[2]), __uint_as_float(o[3])));
            atomicAdd(reinterpret_cast<float4 *>(dst + c + 4), make_float4(__uint_as_float(o[4]), __uint_as_float(o[5]), __uint_as_float(o[6]), __uint_as_float(o[7])));
          }
        }
      }
      tc::tc_fence_before_sync();
      tc::mbar_arrive(dq_read);
      return true;
    };
    if (ctid < BQ) { const size_t idx = lsd_index(0); lsd_publish(0, a.lse[idx], a.delta[idx]); }
    for (int i = 0; i < num_qtiles && ok; ++i) {
      const int s2 = i & 1, pb = i % PB;
      const uint32_t nlse2 = tc::smem_u32(slsd + s2 * 2 * BQ), ndl = nlse2 + BQ * 4;       // negated: used as addends
      float next_l = 0.f, next_d = 0.f;
      const bool prefetch = ctid < BQ && i + 1 < num_qtiles;
      if (prefetch) { const size_t idx = lsd_index(i + 1); next_l = a.lse[idx]; next_d = a.delta[idx]; }
      if (!C::kFold && !tc::mbar_wait(&lsd_full[s2], (uint32_t)(i >> 1) & 1u, wc, 312)) { ok = false; break; }
      if (!tc::mbar_wait(s_full, (uint32_t)i & 1u, wc, 307) || !tc::mbar_wait(dp_full, (uint32_t)i & 1u, wc, 308)) { ok = false; break; }
      // the MMAs that read this shared-memory buffer (tile i - PB) must have finished
      if (i >= PB && !tc::mbar_wait(&pds_empty[pb], (uint32_t)(i / PB - 1) & 1u, wc, 309)) { ok = false; break; }
      tc::tc_fence_after_sync();
      const uint32_t sds = tc::smem_u32(spds + pb * C::kBufBytes), spt = sds + C::kPBytes;
      const uint32_t prow = spt + (col0 / 64) * (kBK * 128) + row * 128;
      const uint32_t drow = sds + (col0 / 64) * (kBK * 128) + row * 128;
      // CH of the thread's QCOLS columns at a time (all of them, or 16 where two CTAs share the register file)
#pragma unroll
      for (int h0 = 0; h0 < QCOLS; h0 += CH) {
        const int colh = col0 + h0;
        uint32_t sr[CH], dr[CH];
        if (CH == 32) {
          tc::tmem_ld_32x32b_x32(tmem_base + lane_off + C::kSCol + colh, reinterpret_cast<uint32_t (&)[32]>(sr));
          tc::tmem_ld_32x32b_x32(tmem_base + lane_off + C::kDpCol + colh, reinterpret_cast<uint32_t (&)[32]>(dr));
        } else {
          tc::tmem_ld_32x32b_x16(tmem_base + lane_off + C::kSCol + colh, reinterpret_cast<uint32_t (&)[16]>(sr));
          tc::tmem_ld_32x32b_x16(tmem_base + lane_off + C::kDpCol + colh, reinterpret_cast<uint32_t (&)[16]>(dr));
        }
        // -lse2 and -delta of the first 8 queries (the same for every key row: broadcast reads); the next group's are
        // fetched while the current one is worked on
        uint64_t nl[4] = {0, 0, 0, 0}, nd[4] = {0, 0, 0, 0};
        if (!C::kFold) {
          tc::lds64x2(nlse2 + colh * 4, nl[0], nl[1]);
          tc::lds64x2(nlse2 + (colh + 4) * 4, nl[2], nl[3]);
          tc::lds64x2(ndl + colh * 4, nd[0], nd[1]);
          tc::lds64x2(ndl + (colh + 4) * 4, nd[2], nd[3]);
        }
        tc::tmem_ld_wait();
        if (C::kTS && i > 0 && h0 == 0) {
          // the previous tile's dV / dK MMAs must have consumed the tensor-memory copies of P^T and dS^T
          if (!tc::mbar_wait(pt_free, (uint32_t)(i - 1) & 1u, wc, 313)) { ok = false; break; }
          tc::tc_fence_after_sync();
        }
#pragma unroll
        for (int v8 = 0; v8 < CH / 8; ++v8) {
          uint64_t nl_next[4] = {0, 0, 0, 0}, nd_next[4] = {0, 0, 0, 0};
          if (!C::kFold && v8 + 1 < CH / 8) {
            tc::lds64x2(nlse2 + (colh + v8 * 8 + 8) * 4, nl_next[0], nl_next[1]);
            tc::lds64x2(nlse2 + (colh + v8 * 8 + 12) * 4, nl_next[2], nl_next[3]);
            tc::lds64x2(ndl + (colh + v8 * 8 + 8) * 4, nd_next[0], nd_next[1]);
            tc::lds64x2(ndl + (colh + v8 * 8 + 12) * 4, nd_next[2], nd_next[3]);
          }
          uint4 pw, dw;
          uint32_t *pw32 = reinterpret_cast<uint32_t *>(&pw), *dw32 = reinterpret_cast<uint32_t *>(&dw);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            // p = 2^(s c - lse2), ds = p (dp - delta), two queries per instruction
            float x0, x1;
            const uint64_t s2v = bpack2(__uint_as_float(sr[v8 * 8 + 2 * e]), __uint_as_float(sr[v8 * 8 + 2 * e + 1]));
            const uint64_t d2v = bpack2(__uint_as_float(dr[v8 * 8 + 2 * e]), __uint_as_float(dr[v8 * 8 + 2 * e + 1]));
            // kFold: the products already hold s - lse / scale and dp - delta
            bunpack2(C::kFold ? bmul2(s2v, c2) : bfma2(s2v, c2, nl[e]), x0, x1);
            const float p0 = bwd_exp2(x0), p1 = bwd_exp2(x1);
            const uint64_t t = C::kFold ? d2v : badd2(d2v, nd[e]);
            float g0, g1;
            bunpack2(bmul2(bpack2(p0, p1), t), g0, g1);
            const __nv_bfloat162 ph = __floats2bfloat162_rn(p0, p1), gh = __floats2bfloat162_rn(g0, g1);
            pw32[e] = *reinterpret_cast<const uint32_t *>(&ph);
            dw32[e] = *reinterpret_cast<const uint32_t *>(&gh);
          }
          const int chunk16 = ((colh % 64) / 8 + v8) ^ (row & 7);
          tc::sts128(drow + chunk16 * 16, dw);
          if (C::kTS) {
            tc::tmem_st_32x32b_x4(tmem_base + lane_off + C::kPtCol + colh / 2 + v8 * 4, pw.x, pw.y, pw.z, pw.w);
            if (C::kDsT) tc::tmem_st_32x32b_x4(tmem_base + lane_off + C::kDsCol + colh / 2 + v8 * 4, dw.x, dw.y, dw.z, dw.w);
          } else {
            tc::sts128(prow + chunk16 * 16, pw);
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) { nl[e] = nl_next[e]; nd[e] = nd_next[e]; }
        }
      }
      if (!ok) break;
      if (C::kTS) tc::tmem_st_wait();
      // the other stage was last read in tile i - 1, which every thread has left (S^T of tile i was issued only
      // after all of them had signalled pds_full for tile i - 1)
      if (prefetch) lsd_publish(i + 1, next_l, next_d);
      tc::fence_proxy_async();
      tc::tc_fence_before_sync();
      tc::mbar_arrive(pds_full);
      if (i > 0 && !read_out_dq(i - 1)) { ok = false; break; }
    }
    if (ok) ok = read_out_dq(num_qtiles - 1);
    if (ok && tc::mbar_wait(dkv_full, 0, wc, 311) && cidx < 2 && key_tok + row < a.L) {
      tc::tc_fence_after_sync();
      const int wg = cidx;
      const size_t base = (((size_t)brow * a.L + key_tok + row) * a.H + head) * D + wg * (D / 2);
#pragma unroll
      for (int c = 0; c < D / 2; c += 8) {
        uint32_t kk[8], vv[8];
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                     : "=r"(kk[0]), "=r"(kk[1]), "=r"(kk[2]), "=r"(kk[3]), "=r"(kk[4]), "=r"(kk[5]), "=r"(kk[6]), "=r"(kk[7])
                     : "r"(tmem_base + lane_off + C::kDkCol + wg * (D / 2) + c) : "memory");
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                     : "=r"(vv[0]), "=r"(vv[1]), "=r"(vv[2]), "=r"(vv[3]), "=r"(vv[4]), "=r"(vv[5]), "=r"(vv[6]), "=r"(vv[7])
                     : "r"(tmem_base + lane_off + C::kDvCol + wg * (D / 2) + c) : "memory");
        tc::tmem_ld_wait();
        uint4 kw, vw;
        __nv_bfloat162 *k2 = reinterpret_cast<__nv_bfloat162 *>(&kw), *v2 = reinterpret_cast<__nv_bfloat162 *>(&vw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          k2[e] = __floats2bfloat162_rn(__uint_as_float(kk[2 * e]) * a.scale, __uint_as_float(kk[2 * e + 1]) * a.scale);
          v2[e] = __floats2bfloat162_rn(__uint_as_float(vv[2 * e]), __uint_as_float(vv[2 * e + 1]));
        }
        *reinterpret_cast<uint4 *>(a.dK + base + c) = kw;
        *reinterpret_cast<uint4 *>(a.dV + base + c) = vw;
      }
    }
  } else if (C::kTmaDq && lane == 0) {
    // Drain warp: one thread hands every staged dQ tile to the copy engine as an add-reduce into the fp32 scratch and
    // returns the staging buffer once the engine has read it, so no compute warp ever waits for the engine.
    bool ok = true;
    for (int i = 0; i < num_qtiles && ok; ++i) {
      const int buf = i & 1;
      if (!tc::mbar_wait(dqs_written, (uint32_t)i & 1u, wc, 314, 200)) { ok = false; break; }
      const int q_tok = (int)my_scope[i / qtiles_per_bucket] * a.bucket + (i % qtiles_per_bucket) * BQ;
      tc::tma_reduce_add_2d(&map_dq, sdq + buf * C::kDqStageBytes, head * D, brow * a.L + q_tok);
      tc::tma_commit();
      if (i > 0) {
        tc::tma_wait_read<1>();                         // the reduce of tile i - 1 has read its buffer
        tc::mbar_arrive(&dqs_free[buf ^ 1]);
      }
    }
    tc::tma_wait_all<0>();                              // every add-reduce of this CTA has landed
  }

  tc::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) { tc::tc_fence_after_sync(); tc::tmem_dealloc(tmem_base, C::kTmemCols); }
}

// ---------------------------------------------------------------------------------------------------------
// Small windows: when all query tiles of a scope fit in tensor memory as dQ accumulators (W / 128 * D <= 128
// columns, i.e. W <= 512 at D = 32), one CTA takes a whole (scope, head): it walks the key blocks j and, inside,
// the query tiles i, keeps dV_j / dK_j for the current block and dQ_i for every tile in tensor memory, and writes
// all three once as bf16.  No fp32 scratch, no reductions, no conversion pass, and K / V of the next block are
// prefetched into a second shared-memory buffer.
template <int D> struct BwdWinCfg {
  static constexpr int BQ = 128;
  static constexpr int RB = D * 2;
  static constexpr uint64_t SWZ = RB == 64 ? tc::kSwizzle64 : tc::kSwizzle32;
  static constexpr int kKVBytes = kBK * D * 2;
  static constexpr int kQBytes = BQ * D * 2;
  static constexpr int kQStage = 2 * kQBytes;
  static constexpr int QS = 3;
  static constexpr int kPBytes = kBK * BQ * 2;                  // dS^T tile
  static constexpr int kMaxTiles = 4;                           // query tiles (and key blocks) per scope
  // -lse / scale and -delta of every query of the scope enter the score products as an extra k-step of 16 (three bf16
  // terms per query against a tile of ones, see BwdCfg::kFold): written once per CTA, one row pair per query
  static constexpr int kOnesBytes = kBK * 32;
  static constexpr int kXBytes = BQ * 32;                       // per query tile and side (Q side | dO side)
  static constexpr int kSmem = 2 * 2 * kKVBytes + QS * kQStage + 2 * kPBytes + kOnesBytes + kMaxTiles * 2 * kXBytes + 256 + 1024;
  static constexpr uint32_t kSCol = 0, kDpCol = 128, kPtCol = 256, kDvCol = 320, kDkCol = 352, kDqCol = 384;
  static_assert(D <= 32 && kDqCol + kMaxTiles * D <= 512, "tensor-memory budget");
};

template <int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_window_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do, AttnBwdArgs a,
                       __nv_bfloat16 *__restrict__ dQ) {
  using C = BwdWinCfg<D>;
  constexpr int BQ = C::BQ, QS = C::QS;
  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char *skv = smem;                                      // [2 buffers][K | V]
  unsigned char *sqdo = skv + 2 * 2 * C::kKVBytes;                // [QS stages][Q | dO]
  unsigned char *sdsb = sqdo + QS * C::kQStage;                   // [2 buffers] dS^T
  unsigned char *sones = sdsb + 2 * C::kPBytes;                   // the constant k-step of K and V
  unsigned char *sx = sones + C::kOnesBytes;                      // [query tile][Q side | dO side] of that k-step
  uint64_t *bars = reinterpret_cast<uint64_t *>(sx + C::kMaxTiles * 2 * C::kXBytes);
  uint64_t *kv_full = bars /*[2]*/, *kv_empty = bars + 2 /*[2]*/, *qdo_full = bars + 4, *qdo_empty = qdo_full + QS;
  uint64_t *s_full = qdo_empty + QS, *dp_full = s_full + 1, *pds_full = dp_full + 1, *pds_empty = pds_full + 1 /*[2]*/;
  uint64_t *pt_free = pds_empty + 2, *dkv_full = pt_free + 1, *dkv_read = dkv_full + 1, *x_full = dkv_read + 1;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(x_full + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int scope = blockIdx.x, head = blockIdx.y, brow = blockIdx.z;
  const uint32_t *my_scope = a.scopes + (size_t)scope * a.k;
  const int tiles_per_bucket = a.bucket / 128;
  const int nt = a.k * tiles_per_bucket;                          // query tiles = key blocks of the scope (<= 4)
  const int total = nt * nt;                                      // iterations t = j * nt + i
  auto tile_tok = [&](int x) { return (int)my_scope[x / tiles_per_bucket] * a.bucket + (x % tiles_per_bucket) * 128; };

  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; ++b) { tc::mbar_init(&kv_full[b], 1); tc::mbar_init(&kv_empty[b], 1); tc::mbar_init(&pds_empty[b], 1); }
    for (int s = 0; s < QS; ++s) { tc::mbar_init(&qdo_full[s], 1); tc::mbar_init(&qdo_empty[s], 1); }
    tc::mbar_init(s_full, 1); tc::mbar_init(dp_full, 1); tc::mbar_init(pds_full, 32 * kBwdComputeWarps);
    tc::mbar_init(pt_free, 1); tc::mbar_init(dkv_full, 1); tc::mbar_init(dkv_read, 32 * kBwdComputeWarps);
    tc::mbar_init(x_full, 32 * kBwdComputeWarps);
    *abort_flag = 0;
    tc::mbar_fence_init();
  }
  // every 16-byte half of every row of the constant tile is (1, 1, 1, 0, ...): the product with a row that carries its
  // three terms in one half and zeros in the other does not depend on where the swizzle puts the halves
  for (int c = threadIdx.x; c < C::kOnesBytes / 16; c += kBwdThreads)
    tc::sts128(tc::smem_u32(sones) + c * 16, make_uint4(0x3F803F80u, 0x00003F80u, 0u, 0u));
  tc::fence_proxy_async();
  if (warp == 1) { tc::tmem_alloc(tmem_slot, 512); tc::tmem_relinquish(); }
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  tc::WaitCtx wc{abort_flag, a.status};

  if (warp == 0) {
    if (tc::elect_one()) {
      tc::tma_prefetch_desc(&map_q); tc::tma_prefetch_desc(&map_k); tc::tma_prefetch_desc(&map_v); tc::tma_prefetch_desc(&map_do);
      auto load_kv = [&](int j) -> bool {
        const int b = j & 1;
        if (!tc::mbar_wait(&kv_empty[b], ((uint32_t)(j >> 1) & 1u) ^ 1u, wc, 321, 200)) return false;
        unsigned char *sk = skv + b * 2 * C::kKVBytes, *sv = sk + C::kKVBytes;
        tc::mbar_expect_tx(&kv_full[b], 2 * C::kKVBytes);
        tc::tma_load_3d(sk, &map_k, &kv_full[b], 0, head, brow * a.L + tile_tok(j));
        tc::tma_load_3d(sv, &map_v, &kv_full[b], 0, head, brow * a.L + tile_tok(j));
        return true;
      };
      bool ok = load_kv(0);
      for (int t = 0; t < total && ok; ++t) {
        const int j = t / nt, i = t % nt, s = t % QS;
        if (!tc::mbar_wait(&qdo_empty[s], ((uint32_t)(t / QS) & 1u) ^ 1u, wc, 322, 200)) break;
        unsigned char *sq = sqdo + s * C::kQStage, *sdo = sq + C::kQBytes;
        tc::mbar_expect_tx(&qdo_full[s], C::kQStage);
        tc::tma_load_3d(sq, &map_q, &qdo_full[s], 0, head, brow * a.L + tile_tok(i));
        tc::tma_load_3d(sdo, &map_do, &qdo_full[s], 0, head, brow * a.L + tile_tok(i));
        // the next block's K / V go into the other buffer while this block is being worked on
        if (i == 0 && j + 1 < nt) ok = load_kv(j + 1);
      }
    }

  } else if (warp == 1) {
    if (tc::elect_one()) {
      constexpr uint32_t idesc_s = tc::make_idesc_f16(kBK, BQ, true, false, false);          // S^T, dP^T
      constexpr uint32_t idesc_kv = tc::make_idesc_f16(kBK, D, true, false, true);           // dV (A in TMEM), dK: B MN-major
      constexpr uint32_t idesc_dq = tc::make_idesc_f16(128, D, true, true, true);            // dQ: A and B MN-major
      auto issue_s_dp = [&](int t) -> bool {
        const int j = t / nt, i = t % nt, s = t % QS;
        if (i == 0 && !tc::mbar_wait(&kv_full[j & 1], (uint32_t)(j >> 1) & 1u, wc, 323)) return false;
        if (!tc::mbar_wait(&qdo_full[s], (uint32_t)(t / QS) & 1u, wc, 324)) return false;
        tc::tc_fence_after_sync();
        const uint32_t k_addr = tc::smem_u32(skv + (j & 1) * 2 * C::kKVBytes), v_addr = k_addr + C::kKVBytes;
        const uint32_t q_addr = tc::smem_u32(sqdo + s * C::kQStage), do_addr = q_addr + C::kQBytes;
        const uint32_t ones_addr = tc::smem_u32(sones), qx_addr = tc::smem_u32(sx + i * 2 * C::kXBytes), dox_addr = qx_addr + C::kXBytes;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          tc::mma_f16_ss(tmem_base + C::kSCol, tc::make_smem_desc(k_addr + kk * 32, 16, 8 * C::RB, C::SWZ),
                         tc::make_smem_desc(q_addr + kk * 32, 16, 8 * C::RB, C::SWZ), idesc_s, kk != 0);
        tc::mma_f16_ss(tmem_base + C::kSCol, tc::make_smem_desc(ones_addr, 16, 256, tc::kSwizzle32),
                       tc::make_smem_desc(qx_addr, 16, 256, tc::kSwizzle32), idesc_s, 1u);          // - lse / scale
        tc::mma_commit(s_full);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          tc::mma_f16_ss(tmem_base + C::kDpCol, tc::make_smem_desc(v_addr + kk * 32, 16, 8 * C::RB, C::SWZ),
                         tc::make_smem_desc(do_addr + kk * 32, 16, 8 * C::RB, C::SWZ), idesc_s, kk != 0);
        tc::mma_f16_ss(tmem_base + C::kDpCol, tc::make_smem_desc(ones_addr, 16, 256, tc::kSwizzle32),
                       tc::make_smem_desc(dox_addr, 16, 256, tc::kSwizzle32), idesc_s, 1u);         // - delta
        tc::mma_commit(dp_full);
        return true;
      };
      bool ok = tc::mbar_wait(x_full, 0, wc, 327) && issue_s_dp(0);
      for (int t = 0; t < total && ok; ++t) {
        const int j = t / nt, i = t % nt, s = t % QS, pb = t & 1;
        // P^T (tensor memory) and dS^T (shared memory) of iteration t are published, S^T / dP^T have been read
        if (!tc::mbar_wait(pds_full, (uint32_t)t & 1u, wc, 325)) { ok = false; break; }
        if (t + 1 < total && !issue_s_dp(t + 1)) { ok = false; break; }
        // a new key block overwrites dV / dK: the previous block's must have been read out
        if (i == 0 && j > 0 && !tc::mbar_wait(dkv_read, (uint32_t)(j - 1) & 1u, wc, 326)) { ok = false; break; }
        tc::tc_fence_after_sync();
        const uint32_t k_addr = tc::smem_u32(skv + (j & 1) * 2 * C::kKVBytes);
        const uint32_t q_addr = tc::smem_u32(sqdo + s * C::kQStage), do_addr = q_addr + C::kQBytes;
        const uint32_t ds_addr = tc::smem_u32(sdsb + pb * C::kPBytes);
#pragma unroll
        for (int qk = 0; qk < BQ / 16; ++qk) {
          const uint32_t a_off = (qk / 4) * (kBK * 128) + (qk % 4) * 32;
          tc::mma_f16_ts(tmem_base + C::kDvCol, tmem_base + C::kPtCol + qk * 8,
                         tc::make_smem_desc(do_addr + qk * 16 * C::RB, 16, 8 * C::RB, C::SWZ), idesc_kv, (i | qk) != 0);
          tc::mma_f16_ss(tmem_base + C::kDkCol, tc::make_smem_desc(ds_addr + a_off, 16, 1024, tc::kSwizzle128),
                         tc::make_smem_desc(q_addr + qk * 16 * C::RB, 16, 8 * C::RB, C::SWZ), idesc_kv, (i | qk) != 0);
        }
        tc::mma_commit(&qdo_empty[s]);
        tc::mma_commit(pt_free);
        // dQ_i (+)= dS K_j: accumulated over the key blocks in its own tensor-memory columns
#pragma unroll
        for (int ks = 0; ks < kBK / 16; ++ks)
          tc::mma_f16_ss(tmem_base + C::kDqCol + i * D, tc::make_smem_desc(ds_addr + ks * 16 * 128, kBK * 128, 1024, tc::kSwizzle128),
                         tc::make_smem_desc(k_addr + ks * 16 * C::RB, 16, 8 * C::RB, C::SWZ), idesc_dq, (j | ks) != 0);
        tc::mma_commit(&pds_empty[pb]);
        if (i == nt - 1) { tc::mma_commit(dkv_full); tc::mma_commit(&kv_empty[j & 1]); }
      }
    }
  } else {
    const int cw = warp - 2;                          // 0..kCW-1
    const int q4 = warp & 3;                          // tensor-memory lane quadrant of this warp
    const int cidx = cw >> 2;                         // which part of the query columns
    const int ctid = cw * 32 + lane;                  // 0..32*kCW-1
    const int row = q4 * 32 + lane;                   // key row (S^T, dP^T, dK, dV) or query row (dQ)
    const uint32_t lane_off = (uint32_t)(q4 * 32) << 16;
    const int col0 = cidx * 32;
    const uint64_t c2 = bpack2(a.scale_log2, a.scale_log2);
    bool ok = true;
    {
      // thread ctid owns query ctid of the scope (tile ctid / 128): its row pair of the extra k-step, written once
      const int xt = ctid / BQ, xr = ctid % BQ;
      uint4 qrow = make_uint4(0u, 0u, 0u, 0u), drow4 = qrow;
      if (xt < nt) {
        const size_t idx = ((size_t)brow * a.L + tile_tok(xt) + xr) * a.H + head;
        auto split3 = [](float v, uint32_t &w0, uint32_t &w1) {
          const __nv_bfloat16 h0 = __float2bfloat16_rn(v);
          const float r1 = v - __bfloat162float(h0);
          const __nv_bfloat16 h1 = __float2bfloat16_rn(r1);
          const __nv_bfloat16 h2 = __float2bfloat16_rn(r1 - __bfloat162float(h1));
          w0 = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
          w1 = (uint32_t)__bfloat16_as_ushort(h2);
        };
        split3(-a.lse[idx] * a.inv_scale, qrow.x, qrow.y);
        split3(-a.delta[idx], drow4.x, drow4.y);
      }
      const uint32_t base = tc::smem_u32(sx + xt * 2 * C::kXBytes) + (uint32_t)xr * 32u;
      tc::sts128(base, qrow);
      tc::sts128(base + 16, make_uint4(0u, 0u, 0u, 0u));
      tc::sts128(base + C::kXBytes, drow4);
      tc::sts128(base + C::kXBytes + 16, make_uint4(0u, 0u, 0u, 0u));
      tc::fence_proxy_async();
      tc::mbar_arrive(x_full);
    }
    for (int t = 0; t < total && ok; ++t) {
      const int j = t / nt, i = t % nt, pb = t & 1;
      if (!tc::mbar_wait(s_full, (uint32_t)t & 1u, wc, 328) || !tc::mbar_wait(dp_full, (uint32_t)t & 1u, wc, 329)) { ok = false; break; }
      // the dQ MMA that read this shared-memory buffer (iteration t - 2) must have finished
      if (t >= 2 && !tc::mbar_wait(&pds_empty[pb], (uint32_t)(t / 2 - 1) & 1u, wc, 330)) { ok = false; break; }
      tc::tc_fence_after_sync();
      uint32_t sr[32], dr[32];
      tc::tmem_ld_32x32b_x32(tmem_base + lane_off + C::kSCol + col0, sr);
      tc::tmem_ld_32x32b_x32(tmem_base + lane_off + C::kDpCol + col0, dr);
      tc::tmem_ld_wait();
      if (t > 0) {
        // the previous iteration's dV MMAs must have consumed the tensor-memory copy of P^T
        if (!tc::mbar_wait(pt_free, (uint32_t)(t - 1) & 1u, wc, 331)) { ok = false; break; }
        tc::tc_fence_after_sync();
      }
      const uint32_t drow = tc::smem_u32(sdsb + pb * C::kPBytes) + (col0 / 64) * (kBK * 128) + row * 128;
#pragma unroll
      for (int v8 = 0; v8 < 4; ++v8) {
        uint4 pw, dw;
        uint32_t *pw32 = reinterpret_cast<uint32_t *>(&pw), *dw32 = reinterpret_cast<uint32_t *>(&dw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          // the products hold s - lse / scale and dp - delta: p = 2^(c s'), ds = p dp'
          float x0, x1;
          bunpack2(bmul2(bpack2(__uint_as_float(sr[v8 * 8 + 2 * e]), __uint_as_float(sr[v8 * 8 + 2 * e + 1])), c2), x0, x1);
          const float p0 = bwd_exp2(x0), p1 = bwd_exp2(x1);
          const uint64_t tt = bpack2(__uint_as_float(dr[v8 * 8 + 2 * e]), __uint_as_float(dr[v8 * 8 + 2 * e + 1]));
          float g0, g1;
          bunpack2(bmul2(bpack2(p0, p1), tt), g0, g1);
          const __nv_bfloat162 ph = __floats2bfloat162_rn(p0, p1), gh = __floats2bfloat162_rn(g0, g1);
          pw32[e] = *reinterpret_cast<const uint32_t *>(&ph);
          dw32[e] = *reinterpret_cast<const uint32_t *>(&gh);
        }
        const int chunk16 = ((col0 % 64) / 8 + v8) ^ (row & 7);
        tc::sts128(drow + chunk16 * 16, dw);
        tc::tmem_st_32x32b_x4(tmem_base + lane_off + C::kPtCol + col0 / 2 + v8 * 4, pw.x, pw.y, pw.z, pw.w);
      }
      tc::tmem_st_wait();
      tc::fence_proxy_async();
      tc::tc_fence_before_sync();
      tc::mbar_arrive(pds_full);
      if (i == nt - 1) {
        // end of key block j: dK_j and dV_j are complete
        if (!tc::mbar_wait(dkv_full, (uint32_t)j & 1u, wc, 332)) { ok = false; break; }
        tc::tc_fence_after_sync();
        const int key_tok = tile_tok(j);
        if (cidx < 2) {
          const bool live = key_tok + row < a.L;
          const size_t base = (((size_t)brow * a.L + key_tok + (live ? row : 0)) * a.H + head) * D + cidx * (D / 2);
#pragma unroll
          for (int c = 0; c < D / 2; c += 8) {
            uint32_t kk[8], vv[8];
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                         : "=r"(kk[0]), "=r"(kk[1]), "=r"(kk[2]), "=r"(kk[3]), "=r"(kk[4]), "=r"(kk[5]), "=r"(kk[6]), "=r"(kk[7])
                         : "r"(tmem_base + lane_off + C::kDkCol + cidx * (D / 2) + c) : "memory");
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                         : "=r"(vv[0]), "=r"(vv[1]), "=r"(vv[2]), "=r"(vv[3]), "=r"(vv[4]), "=r"(vv[5]), "=r"(vv[6]), "=r"(vv[7])
                         : "r"(tmem_base + lane_off + C::kDvCol + cidx * (D / 2) + c) : "memory");
            tc::tmem_ld_wait();
            uint4 kw, vw;
            __nv_bfloat162 *k2 = reinterpret_cast<__nv_bfloat162 *>(&kw), *v2 = reinterpret_cast<__nv_bfloat162 *>(&vw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              k2[e] = __floats2bfloat162_rn(__uint_as_float(kk[2 * e]) * a.scale, __uint_as_float(kk[2 * e + 1]) * a.scale);
              v2[e] = __floats2bfloat162_rn(__uint_as_float(vv[2 * e]), __uint_as_float(vv[2 * e + 1]));
            }
            if (live) {
              *reinterpret_cast<uint4 *>(a.dK + base + c) = kw;
              *reinterpret_cast<uint4 *>(a.dV + base + c) = vw;
            }
          }
        }
        tc::tc_fence_before_sync();
        tc::mbar_arrive(dkv_read);
      }
    }
    // dQ: the last block's dkv_full also covers the last dQ MMAs; warps of column quarter `cidx` take query tile `cidx`
    if (ok && cidx < nt) {
      tc::tc_fence_after_sync();
      const int q_tok = tile_tok(cidx);
      const bool live = q_tok + row < a.L;
      __nv_bfloat16 *dst = dQ + (((size_t)brow * a.L + q_tok + (live ? row : 0)) * a.H + head) * D;
#pragma unroll
      for (int c = 0; c < D; c += 16) {
        uint32_t o[16];
        tc::tmem_ld_32x32b_x16(tmem_base + lane_off + C::kDqCol + cidx * D + c, o);
        tc::tmem_ld_wait();
        uint4 w[2];
        __nv_bfloat162 *h2 = reinterpret_cast<__nv_bfloat162 *>(w);
#pragma unroll
        for (int e = 0; e < 8; ++e) h2[e] = __floats2bfloat162_rn(__uint_as_float(o[2 * e]) * a.scale, __uint_as_float(o[2 * e + 1]) * a.scale);
        if (live) {
          *reinterpret_cast<uint4 *>(dst + c) = w[0];
          *reinterpret_cast<uint4 *>(dst + c + 8) = w[1];
        }
      }
    }
  }

  tc::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) { tc::tc_fence_after_sync(); tc::tmem_dealloc(tmem_base, 512); }
}

// Delta[b,t,h] = sum_d dO * O  (tests/test_attn_bwd.py:24-27)
__global__ void attn_bwd_delta_kernel(const __nv_bfloat16 *__restrict__ O, const __nv_bfloat16 *__restrict__ dO,
                                      float *__restrict__ delta, size_t rows, int D) {
  size_t r = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const uint4 *po = reinterpret_cast<const uint4 *>(O + r * D), *pd = reinterpret_cast<const uint4 *>(dO + r * D);
  float acc = 0.f;
  for (int c = 0; c < D / 8; ++c) {
    uint4 a4 = __ldg(po + c), b4 = __ldg(pd + c);
    const __nv_bfloat162 *x = reinterpret_cast<const __nv_bfloat162 *>(&a4), *y = reinterpret_cast<const __nv_bfloat162 *>(&b4);
#pragma unroll
    for (int e = 0; e < 4; ++e) { float2 f = __bfloat1622float2(x[e]), g = __bfloat1622float2(y[e]); acc = fmaf(f.x, g.x, acc); acc = fmaf(f.y, g.y, acc); }
  }
  delta[r] = acc;
}

__global__ void attn_bwd_dq_convert_kernel(const float *__restrict__ acc, __nv_bfloat16 *__restrict__ dQ, size_t n8, float scale) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  float4 a4 = reinterpret_cast<const float4 *>(acc)[2 * i], b4 = reinterpret_cast<const float4 *>(acc)[2 * i + 1];
  uint4 w;
  __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&w);
  h[0] = __floats2bfloat162_rn(a4.x * scale, a4.y * scale); h[1] = __floats2bfloat162_rn(a4.z * scale, a4.w * scale);
  h[2] = __floats2bfloat162_rn(b4.x * scale, b4.y * scale); h[3] = __floats2bfloat162_rn(b4.z * scale, b4.w * scale);
  reinterpret_cast<uint4 *>(dQ)[i] = w;
}

template <int D>
static int launch_attn_bwd(const void *Q, const void *K, const void *V, const void *dO, AttnBwdArgs a, int device, cudaStream_t st) {
  using C = BwdCfg<D>;
  auto kern = attn_bwd_kernel<D>;
  F3D_TRY(ensure_dynamic_smem(reinterpret_cast<const void *>(kern), device, C::kSmem));
  CUtensorMap mq, mk, mv, mdo;
  const uint64_t rows = (uint64_t)a.B * a.L;
  const uint64_t s1 = (uint64_t)D * 2, s2 = (uint64_t)a.H * D * 2;
  F3D_TRY(encode_tmap_3d(&mq, 0, Q, D, a.H, rows, s1, s2, C::DCH, 1, C::BQ, C::RB));
  F3D_TRY(encode_tmap_3d(&mdo, 0, dO, D, a.H, rows, s1, s2, C::DCH, 1, C::BQ, C::RB));
  F3D_TRY(encode_tmap_3d(&mk, 0, K, D, a.H, rows, s1, s2, C::DCH, 1, kBK, C::RB));
  F3D_TRY(encode_tmap_3d(&mv, 0, V, D, a.H, rows, s1, s2, C::DCH, 1, kBK, C::RB));
  // fp32 dQ scratch [B*L, H*D] as a tensor map for the add-reduce of a 128-row x 32-column tile (D = 32 only; the
  // other head sizes keep vector reductions and get a map they never use)
  CUtensorMap mdq = mq;
  if (C::kTmaDq)
    F3D_TRY(encode_tmap_2d(&mdq, 2, a.dq_acc, (uint64_t)a.H * D, rows, (uint64_t)a.H * D * 4, D, C::BQ, 128));
  dim3 grid(a.num_scopes * a.k * a.kblocks_per_bucket, a.H, a.B);
  kern<<<grid, C::kThreads, C::kSmem, st>>>(mq, mk, mv, mdo, mdq, a);
  return check_launch("buck_swin_bwd");
}

template <int D>
static int launch_attn_bwd_window(const void *Q, const void *K, const void *V, const void *dO, void *dQ, AttnBwdArgs a, int device,
                                  cudaStream_t st) {
  using C = BwdWinCfg<D>;
  auto kern = attn_bwd_window_kernel<D>;
  F3D_TRY(ensure_dynamic_smem(reinterpret_cast<const void *>(kern), device, C::kSmem));
  CUtensorMap mq, mk, mv, mdo;
  const uint64_t rows = (uint64_t)a.B * a.L;
  const uint64_t s1 = (uint64_t)D * 2, s2 = (uint64_t)a.H * D * 2;
  F3D_TRY(encode_tmap_3d(&mq, 0, Q, D, a.H, rows, s1, s2, D, 1, 128, C::RB));
  F3D_TRY(encode_tmap_3d(&mdo, 0, dO, D, a.H, rows, s1, s2, D, 1, 128, C::RB));
  F3D_TRY(encode_tmap_3d(&mk, 0, K, D, a.H, rows, s1, s2, D, 1, 128, C::RB));
  F3D_TRY(encode_tmap_3d(&mv, 0, V, D, a.H, rows, s1, s2, D, 1, 128, C::RB));
  dim3 grid(a.num_scopes, a.H, a.B);
  kern<<<grid, kBwdThreads, C::kSmem, st>>>(mq, mk, mv, mdo, a, static_cast<__nv_bfloat16 *>(dQ));
  return check_launch("buck_swin_bwd (window)");
}

}  // namespace f3d

using namespace f3d;

extern "C" int f3d_buck_swin_bwd(const void *Q, const void *K, const void *V, const void *O, const void *dO, const void *LSE,
                                 void *Delta, void *dQ, void *dK, void *dV, const void *scope_buckets, int B, int L, int H,
                                 int D, int num_scopes, int scope_size, uint32_t bucket_size, int device, void *stream) {
  if (B <= 0 || L <= 0 || H <= 0) return set_error(F3D_ERR_ARG, "buck_swin_bwd: empty tensor");
  if (D != 16 && D != 32 && D != 64 && D != 128) return set_error(F3D_ERR_UNSUPPORTED, "buck_swin_bwd: head_dim %d (16, 32, 64, 128 are supported)", D);
  if (bucket_size == 0 || bucket_size % 128) return set_error(F3D_ERR_UNSUPPORTED, "buck_swin_bwd: bucket_size %u must be a positive multiple of 128", bucket_size);
  if (L % (int)bucket_size) return set_error(F3D_ERR_ARG, "buck_swin_bwd: sequence length %d is not a multiple of bucket_size %u", L, bucket_size);
  if (num_scopes < 0 || scope_size <= 0) return set_error(F3D_ERR_ARG, "buck_swin_bwd: Scope_buckets must be [S,k] with k > 0");
  if ((long long)H > 65535 || (long long)B > 65535) return set_error(F3D_ERR_UNSUPPORTED, "buck_swin_bwd: H and B must fit a grid dimension");
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  F3D_TRY(maybe_sync(st, "buck_swin_bwd"));
  const size_t rows = (size_t)B * L * H;
  attn_bwd_delta_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(O), static_cast<const __nv_bfloat16 *>(dO),
                                                                       static_cast<float *>(Delta), rows, D);
  F3D_TRY(check_launch("buck_swin_bwd (delta)"));
  if (num_scopes == 0) {          // no bucket is listed: dQ is all zero, dK and dV have no listed rows
    F3D_CUDA_TRY(cudaMemsetAsync(dQ, 0, rows * D * sizeof(__nv_bfloat16), st));
    return maybe_sync(st, "buck_swin_bwd");
  }
  const long long window_tiles = (long long)scope_size * (bucket_size / 128);
  if (D <= 32 && window_tiles <= BwdWinCfg<32>::kMaxTiles) {
    // small windows: one CTA per (scope, head) keeps every dQ tile in tensor memory, no scratch and no reductions
    const float scale = 1.f / sqrtf((float)D);
    AttnBwdArgs a{static_cast<const float *>(LSE), static_cast<const float *>(Delta), nullptr,
                  static_cast<__nv_bfloat16 *>(dK), static_cast<__nv_bfloat16 *>(dV), static_cast<const uint32_t *>(scope_buckets),
                  B, L, H, num_scopes, scope_size, (int)bucket_size, (int)bucket_size / kBK, 1.4426950408889634f * scale, scale, sqrtf((float)D),
                  status_word(device)};
    if (!a.status) return F3D_ERR_CUDA;
    // this kernel writes dQ only for the tokens of listed buckets; the general path below writes every row (zero where
    // no scope lists the bucket).  Both give the same dQ: rows of unlisted buckets are cleared here when the table is too
    // short to list every bucket once.
    if ((long long)num_scopes * scope_size * (long long)bucket_size < (long long)L)
      F3D_CUDA_TRY(cudaMemsetAsync(dQ, 0, rows * D * sizeof(__nv_bfloat16), st));
    F3D_TRY(D == 16 ? launch_attn_bwd_window<16>(Q, K, V, dO, dQ, a, device, st) : launch_attn_bwd_window<32>(Q, K, V, dO, dQ, a, device, st));
    return maybe_sync(st, "buck_swin_bwd");
  }
  void *acc = nullptr;
  F3D_TRY(workspace(device, 2, rows * D * sizeof(float), st, &acc));
  F3D_CUDA_TRY(cudaMemsetAsync(acc, 0, rows * D * sizeof(float), st));
  const float scale = 1.f / sqrtf((float)D);
  AttnBwdArgs a{static_cast<const float *>(LSE), static_cast<const float *>(Delta), static_cast<float *>(acc),
                static_cast<__nv_bfloat16 *>(dK), static_cast<__nv_bfloat16 *>(dV), static_cast<const uint32_t *>(scope_buckets),
                B, L, H, num_scopes, scope_size, (int)bucket_size, (int)bucket_size / kBK, 1.4426950408889634f * scale, scale, sqrtf((float)D),
                status_word(device)};
  if (!a.status) return F3D_ERR_CUDA;
  int rc;
  switch (D) {
    case 16: rc = launch_attn_bwd<16>(Q, K, V, dO, a, device, st); break;
    case 32: rc = launch_attn_bwd<32>(Q, K, V, dO, a, device, st); break;
    case 64: rc = launch_attn_bwd<64>(Q, K, V, dO, a, device, st); break;
    default: rc = launch_attn_bwd<128>(Q, K, V, dO, a, device, st); break;
  }
  F3D_TRY(rc);
  const size_t n8 = rows * D / 8;
  attn_bwd_dq_convert_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, st>>>(static_cast<const float *>(acc), static_cast<__nv_bfloat16 *>(dQ), n8, scale);
  F3D_TRY(check_launch("buck_swin_bwd (dq convert)"));
  return maybe_sync(st, "buck_swin_bwd");
}
