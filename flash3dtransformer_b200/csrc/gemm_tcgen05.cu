// bf16 (or fp16) GEMM for the per-token projections: C[M,N] = A[M,K] . W[N,K]^T (+ bias) (+ residual), fp32
// accumulation.  The element type is a template switch: it sets the operand format of the MMA instruction descriptor
// and the conversions of the epilogue; A, W, the residual and C share it.
//
// Replaces the cuBLAS calls behind nn.Linear in the reference's attention block (qkv and proj,
// flash3dxfmr/layers/buck_swin.py:159,163,185-194) and the toy mma.sync kernel gemm_sm_bf16_ker
// (src/psh/gemm.cuh:30-85, host src/psh/gemm_dispatcher.cu:26-80, which demands M == 128 and synchronises).
//
// Structure (one persistent CTA per SM, 448 threads):
//   warp 0      TMA producer: A tile 128x64 and W tile BNx64 per stage, 128-byte swizzle, mbarrier completion
//   warp 1      owns tensor memory; one elected lane issues tcgen05.mma (M=128, N=BN, K=16) four times per
//               stage and commits the stage's "empty" barrier; after the last k-block it commits "accumulator full"
//   warps 2-13  epilogue: three warps per 32-lane quadrant of the 128xBN fp32 accumulator; a warp takes 32 columns at
//               a time (tcgen05.ld), adds bias / residual, applies GELU / SwiGLU, converts to bf16, stages the
//               32x32 block in swizzled shared memory and writes it with a TMA store
// Up to four accumulators (at most 512 tensor-memory columns) let the epilogues of earlier tiles overlap the MMAs of
// the following ones.
// LayerNorm folded into the projection (optional): with W' = W diag(gamma), s[n] = sum_k W'[n,k] and
// b'[n] = b[n] + sum_k beta[k] W[n,k] prepared by the host, LayerNorm(x) W^T + b = rstd (x W'^T - mean s) + b'.  The
// MMAs run on the raw rows; the epilogue reads each row's (sum, sum of squares) from `ln_stats`, and applies
// rstd * acc - (mean * rstd) * s + b' per column.  Those row sums are themselves a by-product of the GEMM that wrote x:
// with `stats_out` the epilogue adds up each output row and its squares, so a chain projection -> LayerNorm ->
// projection needs neither a LayerNorm kernel nor a pass over x for statistics.  The sums are the same bits on every
// run: a warp adds its tasks of a tile in column order, the three warps of a lane quadrant leave their partial sums in
// shared memory and the last one to finish adds them in a fixed order and stores the row's pair (with more than one
// column tile per row, N > 256, the tiles' pairs meet in an atomic add: two addends commute, so N <= 512 stays exact).
// Outputs may be split column-wise into `nsplit` separate [M, N/nsplit] matrices (Q, K, V written directly in
// the [L, H*D] layout the attention kernel reads, instead of three .contiguous() copies,
// flash3dxfmr/layers/buck_swin.py:188-190).
#include "f3d_common.cuh"
#include "tc_sm100.cuh"
#include "../../include/f3d_b200.h"

namespace f3d {

// Three epilogue warps per tensor-memory lane quadrant: with 16 the register file caps a thread at 96 registers and the
// epilogue spills; 12 warps get 128 registers, spill nothing and execute fewer control instructions per tile (the
// epilogue is bound by instruction issue): 16.4 ms for the backbone's GEMM mix against 17.3 (16 warps) and 17.9 (8).
// The kernel comes in two builds.  The general one (LEAN = false) has every epilogue (SwiGLU, GELU, folded LayerNorm, row
// sums, direct stores) and 12 epilogue warps.  The lean one serves the plain projections (bias, residual, column splits)
// and SwiGLU without a folded LayerNorm:
// without the other epilogues' code a thread needs fewer registers, so 16 epilogue warps fit, and the epilogue, a chain
// of latencies per 32-column task, is what bounds those projections.
constexpr int epi_warps(bool lean) { return lean ? 16 : 12; }
constexpr int gemm_threads(bool lean) { return 64 + 32 * epi_warps(lean); }     // TMA warp, MMA warp, epilogue warps
constexpr int BM = 128;
constexpr int BK = 64;

enum GemmEpilogue : int { EPI_NONE = 0, EPI_GELU = 1, EPI_SWIGLU = 2 };

struct GemmArgs {
  int M, N, K;
  int nsplit;            // output column splits
  int split_n;           // N / nsplit (columns per split; for SWIGLU: output columns = N/2)
  const float *bias;     // [N] fp32 or null
  const __nv_bfloat16 *residual;   // [M, ldr] bf16 or null (added after bias; only with nsplit == 1)
  int ldr;
  int epilogue;
  int direct_store;      // 1: plain 16-byte global stores instead of TMA stores (split rows shorter than a 64-column chunk)
  __nv_bfloat16 *c_ptr;
  long long split_stride;
  int *status;
  int ksplit;            // > 1: A is [ksplit, M, K], W is [ksplit, N, K] and the products of the slices are summed
  const float2 *ln_stats;   // [M] (sum, sum of squares) of every row of A over its K channels, or null: folded LayerNorm
  const float *ln_colsum;   // [N] column sums s of the scaled weight (with ln_stats)
  float ln_eps, ln_inv_k;
  float2 *stats_out;        // [M] or null: (sum, sum of squares) of every output row, accumulated with atomic adds
};

template <int BN, bool LEAN> struct GemmSmem {
  static constexpr int kEpiWarps = epi_warps(LEAN);
  static constexpr int kStages = BN >= 256 ? 3 : 4;
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kOutBytes = kEpiWarps * 2 /*buffers*/ * 32 * 64;    // 32 rows x 32 bf16 per buffer
  static constexpr int kAcc = BN >= 256 ? 2 : 4;        // accumulator buffers in tensor memory (kAcc * BN <= 512 columns)
  static constexpr int kBarBytes = 256;
  // partial row sums of the epilogue warps: [accumulator][quadrant][warp of the quadrant][32 rows] pairs + counters
  static constexpr int kStatBytes = LEAN ? 16 : kAcc * 4 * (kEpiWarps / 4) * 32 * 8 + kAcc * 4 * 4;     // (the lean build has no row sums)
  // bias inside the product: one more k-step of 16 whose A side is a tile of ones [BM][16] and whose W side holds every
  // column's bias as three 16-bit terms [BN][16] (single column tile only, where the W side never changes)
  static constexpr int kFoldBytes = (BM + BN) * 32;
  static constexpr int kTotal = kStages * kStageBytes + kOutBytes + kBarBytes + kStatBytes + kFoldBytes + 1024 /*alignment slack*/;
};

__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  return 0.5f * x * (1.f + tanhf(u));
}

// packed fp32 pairs: one instruction works on two values (halves the issue slots of the epilogue arithmetic)
__device__ __forceinline__ uint64_t gpack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void gunpack2(uint64_t v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t gadd2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t gmul2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t gfma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
// silu(gate) * up for two columns with one special-function instruction each: sigmoid(x) = 0.5 + 0.5 * tanh(x / 2),
// so with h = gate / 2, silu = h + h * tanh(h); tanh.approx has a relative error near 5e-4, an order of magnitude below
// the bf16 rounding of the result
__device__ __forceinline__ void swiglu_pair(uint64_t gate2, uint64_t up2, float &o0, float &o1) {
  const uint64_t h2 = gmul2(gate2, gpack2(0.5f, 0.5f));
  float h0, h1, t0, t1;
  gunpack2(h2, h0, h1);
  asm("tanh.approx.f32 %0, %1;" : "=f"(t0) : "f"(h0));
  asm("tanh.approx.f32 %0, %1;" : "=f"(t1) : "f"(h1));
  gunpack2(gmul2(gfma2(h2, gpack2(t0, t1), h2), up2), o0, o1);
}

// two fp32 values to a packed pair of 16-bit outputs, and back, in the kernel's element type
template <bool F16> __device__ __forceinline__ uint32_t pack_out2(float a, float b) {
  if (F16) { __half2 h = __floats2half2_rn(a, b); return *reinterpret_cast<uint32_t *>(&h); }
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&h);
}
template <bool F16> __device__ __forceinline__ float2 unpack_in2(uint32_t w) {
  if (F16) return __half22float2(*reinterpret_cast<const __half2 *>(&w));
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&w));
}
template <bool F16> __device__ __forceinline__ float unpack_in1(const __nv_bfloat16 *p) {
  if (F16) return __half2float(*reinterpret_cast<const __half *>(p));
  return __bfloat162float(*p);
}

template <int BN, bool F16, bool LEAN>
__global__ void __launch_bounds__(gemm_threads(LEAN), 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const __grid_constant__ CUtensorMap map_c, GemmArgs g) {
  using S = GemmSmem<BN, LEAN>;
  constexpr int kEpiWarps = S::kEpiWarps, kGemmThreads = gemm_threads(LEAN);
  constexpr int kStages = S::kStages;
  constexpr int kAcc = S::kAcc;
  constexpr uint32_t kTmemCols = kAcc * BN < 32 ? 32 : kAcc * BN;
  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char *stage_base = smem;
  unsigned char *out_base = smem + kStages * S::kStageBytes;
  unsigned char *fold_base = out_base + S::kOutBytes;             // [BM][16] ones, then [BN][16] bias terms (1 KB aligned)
  uint64_t *bars = reinterpret_cast<uint64_t *>(fold_base + S::kFoldBytes);
  uint64_t *full = bars, *empty = bars + kStages, *acc_full = bars + 2 * kStages, *acc_empty = bars + 2 * kStages + kAcc;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kStages + 2 * kAcc);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  float2 *stat_slots = reinterpret_cast<float2 *>(fold_base + S::kFoldBytes + S::kBarBytes);
  int *stat_cnt = reinterpret_cast<int *>(stat_slots + kAcc * 4 * (kEpiWarps / 4) * 32);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (g.M + BM - 1) / BM, n_tiles = (g.N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  const int kb_per_split = (g.K + BK - 1) / BK;
  const int kb_count = kb_per_split * g.ksplit;
  // The bias enters the product itself when the kernel has one column tile: the tile of ones times the columns' bias
  // terms (hi + mid + lo in the element type, exact to 2^-24) adds b[n] to every accumulator in fp32, and the epilogue
  // neither loads nor adds it.  Every 16-byte half of the ones rows is (1, 1, 1, 0, ...), the bias rows carry their terms
  // in the first half and zeros in the second, so the sum does not depend on where the 32-byte swizzle puts the halves.
  const bool fold_bias = g.bias != nullptr && g.ln_stats == nullptr && n_tiles == 1 && g.ksplit == 1;
  if (fold_bias) {
    const uint32_t one2 = F16 ? 0x3C003C00u : 0x3F803F80u, one1 = F16 ? 0x00003C00u : 0x00003F80u;
    for (int c = threadIdx.x; c < BM * 2; c += kGemmThreads) tc::sts128(tc::smem_u32(fold_base) + c * 16, make_uint4(one2, one1, 0u, 0u));
    for (int r = threadIdx.x; r < BN; r += kGemmThreads) {
      // row r of the W tile is output column r, or for SwiGLU gate column r | up column r - BN / 2
      int col = r;
      if (g.epilogue == EPI_SWIGLU) col = r < BN / 2 ? r : g.N / 2 + (r - BN / 2);
      const bool live = g.epilogue == EPI_SWIGLU ? (r < BN / 2 ? r < g.N / 2 : r - BN / 2 < g.N / 2) : r < g.N;
      const float b = live ? __ldg(g.bias + col) : 0.f;
      uint32_t w0, w1;
      if (F16) {
        const __half h0 = __float2half_rn(b);
        const float r1 = b - __half2float(h0);
        const __half h1 = __float2half_rn(r1);
        const __half h2 = __float2half_rn(r1 - __half2float(h1));
        w0 = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
        w1 = (uint32_t)__half_as_ushort(h2);
      } else {
        const __nv_bfloat16 h0 = __float2bfloat16_rn(b);
        const float r1 = b - __bfloat162float(h0);
        const __nv_bfloat16 h1 = __float2bfloat16_rn(r1);
        const __nv_bfloat16 h2 = __float2bfloat16_rn(r1 - __bfloat162float(h1));
        w0 = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
        w1 = (uint32_t)__bfloat16_as_ushort(h2);
      }
      const uint32_t base = tc::smem_u32(fold_base) + BM * 32 + r * 32;
      tc::sts128(base, make_uint4(w0, w1, 0u, 0u));
      tc::sts128(base + 16, make_uint4(0u, 0u, 0u, 0u));
    }
    tc::fence_proxy_async();
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { tc::mbar_init(&full[s], 1); tc::mbar_init(&empty[s], 1); }
    for (int a = 0; a < kAcc; ++a) { tc::mbar_init(&acc_full[a], 1); tc::mbar_init(&acc_empty[a], kEpiWarps); }
    if (!LEAN) for (int a = 0; a < kAcc * 4; ++a) stat_cnt[a] = 0;
    *abort_flag = 0;
    tc::mbar_fence_init();
  }
  if (warp == 1) { tc::tmem_alloc(tmem_slot, kTmemCols); tc::tmem_relinquish(); }
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  tc::WaitCtx wc{abort_flag, g.status};

  if (warp == 0) {
    if (tc::elect_one()) {
      tc::tma_prefetch_desc(&map_a); tc::tma_prefetch_desc(&map_b); tc::tma_prefetch_desc(&map_c);
      uint32_t it = 0;
      bool ok = true;
      // With a single column tile and a k-block count that divides the ring, stage s always carries k-block
      // s % kb_count, so its W tile never changes: it is loaded on the stage's first use and stays resident.
      // (A TMA tile load costs about 7 cycles per box row whatever the row length; reloading a 128- or 256-row W
      // tile for every 128 rows of A took a third of the time of the narrow-K shapes.)
      const bool w_resident = n_tiles == 1 && kStages % kb_count == 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int mt = n_tiles == 1 ? tile : tile / n_tiles;      // a single column tile is the common case: no division
        const int m0 = mt * BM, n0 = (tile - mt * n_tiles) * BN;
        for (int kb = 0; kb < kb_count; ++kb, ++it) {
          const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
          if (!tc::mbar_wait(&empty[s], ph ^ 1u, wc, 101)) { ok = false; break; }
          unsigned char *sa = stage_base + s * S::kStageBytes;
          // k-block kb of slice sp starts at column kx of rows [sp * M + m0, ...) of A and [sp * N + n0, ...) of W;
          // columns past K are zero-filled by the copy, rows past a slice's end land in rows or columns never stored
          int kx = kb * BK, ya = m0, yb = n0;
          if (g.ksplit > 1) {
            const int sp = kb / kb_per_split;
            kx = (kb - sp * kb_per_split) * BK;
            ya += sp * g.M;
            yb += sp * g.N;
          }
          if (w_resident && it >= (uint32_t)kStages) {
            // this stage already holds the W tile of k-block kb from its first use: only A moves
            tc::mbar_expect_tx(&full[s], S::kABytes);
            tc::tma_load_2d(sa, &map_a, &full[s], kx, ya);
            continue;
          }
          tc::mbar_expect_tx(&full[s], S::kStageBytes);
          tc::tma_load_2d(sa, &map_a, &full[s], kx, ya);
          if (g.epilogue == EPI_SWIGLU) {
            // gate rows [n0/2, n0/2 + BN/2) and up rows [N/2 + n0/2, ...) of W share one tile
            tc::tma_load_2d(sa + S::kABytes, &map_b, &full[s], kb * BK, n0 / 2);
            tc::tma_load_2d(sa + S::kABytes + S::kBBytes / 2, &map_b, &full[s], kb * BK, g.N / 2 + n0 / 2);
          } else {
            tc::tma_load_2d(sa + S::kABytes, &map_b, &full[s], kx, yb);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (tc::elect_one()) {
      constexpr uint32_t idesc = tc::make_idesc_f16(BM, BN, !F16, false, false);
      uint32_t it = 0, t_local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++t_local) {
        const uint32_t acc = t_local % kAcc, aph = (t_local / kAcc) & 1u;
        if (!tc::mbar_wait(&acc_empty[acc], aph ^ 1u, wc, 102)) { ok = false; break; }
        tc::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kb_count; ++kb, ++it) {
          const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
          if (!tc::mbar_wait(&full[s], ph, wc, 103)) { ok = false; break; }
          tc::tc_fence_after_sync();
          const uint32_t sa = tc::smem_u32(stage_base + s * S::kStageBytes);
          const uint64_t adesc = tc::kmajor_sw128_desc(sa), bdesc = tc::kmajor_sw128_desc(sa + S::kABytes);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            tc::mma_f16_ss(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
          tc::mma_commit(&empty[s]);
        }
        if (ok && fold_bias)
          tc::mma_f16_ss(d_tmem, tc::make_smem_desc(tc::smem_u32(fold_base), 16, 256, tc::kSwizzle32),
                         tc::make_smem_desc(tc::smem_u32(fold_base) + BM * 32, 16, 256, tc::kSwizzle32), idesc, 1u);
        if (ok) tc::mma_commit(&acc_full[acc]);
      }
    }
  } else {
    // Epilogue warps: kEpiWarps / 4 per tensor-memory lane quadrant.  A task is 32 output columns of the warp's 32
    // rows; the tasks of a quadrant are numbered across tiles and dealt round-robin to its warps, so narrow
    // tiles (one or two tasks) still keep all warps busy, each on a different accumulator buffer.
    const int q = warp & 3;                       // tensor-memory lane quadrant this warp may read
    const uint32_t sub = (uint32_t)(warp - 2) >> 2;     // which of the quadrant's warps
    constexpr uint32_t kSub = kEpiWarps / 4;
    unsigned char *my_out = out_base + (warp - 2) * 2 * 32 * 64;
    uint32_t t_local = 0, obuf = 0, task = 0;
    bool ok = true;
    const int tile_cols = g.epilogue == EPI_SWIGLU ? BN / 2 : BN;    // output columns a tile can produce
    const int total_cols = g.epilogue == EPI_SWIGLU ? g.N / 2 : g.N; // output columns there are
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++t_local) {
      const uint32_t acc = t_local % kAcc, aph = (t_local / kAcc) & 1u;
      const int mt = n_tiles == 1 ? tile : tile / n_tiles;
      const int m0 = mt * BM, n0 = (tile - mt * n_tiles) * BN;
      if (!tc::mbar_wait(&acc_full[acc], aph, wc, 104)) { ok = false; break; }
      tc::tc_fence_after_sync();
      const uint32_t t_row = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
      const int row = m0 + q * 32 + lane;
      // folded LayerNorm: this thread's row contributes rstd and -mean * rstd to every column
      float ln_rstd = 1.f, ln_nmr = 0.f;
      if (!LEAN && g.ln_stats) {
        const float2 st = row < g.M ? __ldg(g.ln_stats + row) : make_float2(0.f, 0.f);
        const float mean = st.x * g.ln_inv_k;
        const float var = fmaxf(fmaf(-mean, mean, st.y * g.ln_inv_k), 0.f);
        ln_rstd = rsqrtf(var + g.ln_eps);
        ln_nmr = -mean * ln_rstd;
      }
      const uint64_t rstd2 = gpack2(ln_rstd, ln_rstd), nmr2 = gpack2(ln_nmr, ln_nmr);
      uint64_t tile_sum2 = gpack2(0.f, 0.f), tile_sq2 = gpack2(0.f, 0.f);     // row sums over this warp's tasks of the tile
      // this warp's tasks of the tile: numbers congruent to `sub` modulo kSub, `task` being the tile's first
      // tasks of this tile: only the 32-column groups that hold output columns (N = 96 fills three of a 128-column
      // tile's four groups; the fourth would be computed and then clipped by the store)
      const int first_col = g.epilogue == EPI_SWIGLU ? n0 / 2 : n0;
      const int out_cols = min(tile_cols, (total_cols - first_col + 31) & ~31);
      for (int c0 = (int)((sub + kSub - task % kSub) % kSub) * 32; c0 < out_cols; c0 += 32 * (int)kSub) {
        float v[32];
        const int oc0 = (g.epilogue == EPI_SWIGLU ? n0 / 2 : n0) + c0;      // first output column of the task
        // runtime switches (bias, activation) are tested once per task, never per element
        if (LEAN && g.epilogue == EPI_SWIGLU) {
          // lean build: gate and up accumulators of 16 output columns at a time, so that a thread stays within the
          // registers that 16 epilogue warps leave it
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            uint32_t r[16], u[16];
            tc::tmem_ld_32x32b_x16(t_row + c0 + hh * 16, r);
            tc::tmem_ld_32x32b_x16(t_row + BN / 2 + c0 + hh * 16, u);
            tc::tmem_ld_wait();
            if (g.bias && !fold_bias) {
              const float4 *pg = reinterpret_cast<const float4 *>(g.bias + oc0 + hh * 16);
              const float4 *pu = reinterpret_cast<const float4 *>(g.bias + g.N / 2 + oc0 + hh * 16);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float4 a4 = __ldg(pg + j), b4 = __ldg(pu + j);
                swiglu_pair(gadd2(gpack2(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1])), gpack2(a4.x, a4.y)),
                            gadd2(gpack2(__uint_as_float(u[4 * j]), __uint_as_float(u[4 * j + 1])), gpack2(b4.x, b4.y)),
                            v[hh * 16 + 4 * j], v[hh * 16 + 4 * j + 1]);
                swiglu_pair(gadd2(gpack2(__uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])), gpack2(a4.z, a4.w)),
                            gadd2(gpack2(__uint_as_float(u[4 * j + 2]), __uint_as_float(u[4 * j + 3])), gpack2(b4.z, b4.w)),
                            v[hh * 16 + 4 * j + 2], v[hh * 16 + 4 * j + 3]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                swiglu_pair(gpack2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1])),
                            gpack2(__uint_as_float(u[2 * j]), __uint_as_float(u[2 * j + 1])), v[hh * 16 + 2 * j], v[hh * 16 + 2 * j + 1]);
            }
          }
        } else if (!LEAN && g.epilogue == EPI_SWIGLU) {
          uint32_t r[32], u[32];
          tc::tmem_ld_32x32b_x32(t_row + c0, r);
          tc::tmem_ld_32x32b_x32(t_row + BN / 2 + c0, u);
          tc::tmem_ld_wait();
          if (g.ln_stats) {
            // gate = rstd * acc_g + nmr * s_g + b'_g (likewise up); the host always supplies b' in this mode
            const float4 *pg = reinterpret_cast<const float4 *>(g.bias + oc0), *pu = reinterpret_cast<const float4 *>(g.bias + g.N / 2 + oc0);
            const float4 *sg = reinterpret_cast<const float4 *>(g.ln_colsum + oc0), *su = reinterpret_cast<const float4 *>(g.ln_colsum + g.N / 2 + oc0);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 a4 = __ldg(pg + j), b4 = __ldg(pu + j), c4 = __ldg(sg + j), d4 = __ldg(su + j);
              swiglu_pair(gfma2(gpack2(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1])), rstd2, gfma2(gpack2(c4.x, c4.y), nmr2, gpack2(a4.x, a4.y))),
                          gfma2(gpack2(__uint_as_float(u[4 * j]), __uint_as_float(u[4 * j + 1])), rstd2, gfma2(gpack2(d4.x, d4.y), nmr2, gpack2(b4.x, b4.y))),
                          v[4 * j], v[4 * j + 1]);
              swiglu_pair(gfma2(gpack2(__uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])), rstd2, gfma2(gpack2(c4.z, c4.w), nmr2, gpack2(a4.z, a4.w))),
                          gfma2(gpack2(__uint_as_float(u[4 * j + 2]), __uint_as_float(u[4 * j + 3])), rstd2, gfma2(gpack2(d4.z, d4.w), nmr2, gpack2(b4.z, b4.w))),
                          v[4 * j + 2], v[4 * j + 3]);
            }
          } else if (g.bias && !fold_bias) {
            const float4 *pg = reinterpret_cast<const float4 *>(g.bias + oc0);
            const float4 *pu = reinterpret_cast<const float4 *>(g.bias + g.N / 2 + oc0);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 a4 = __ldg(pg + j), b4 = __ldg(pu + j);
              swiglu_pair(gadd2(gpack2(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1])), gpack2(a4.x, a4.y)),
                          gadd2(gpack2(__uint_as_float(u[4 * j]), __uint_as_float(u[4 * j + 1])), gpack2(b4.x, b4.y)), v[4 * j], v[4 * j + 1]);
              swiglu_pair(gadd2(gpack2(__uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])), gpack2(a4.z, a4.w)),
                          gadd2(gpack2(__uint_as_float(u[4 * j + 2]), __uint_as_float(u[4 * j + 3])), gpack2(b4.z, b4.w)), v[4 * j + 2], v[4 * j + 3]);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              swiglu_pair(gpack2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1])),
                          gpack2(__uint_as_float(u[2 * j]), __uint_as_float(u[2 * j + 1])), v[2 * j], v[2 * j + 1]);
          }
        } else {
          uint32_t r[32];
          tc::tmem_ld_32x32b_x32(t_row + c0, r);
          tc::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          if (!LEAN && g.ln_stats) {
            // v = rstd * acc + (nmr * s + b'); columns past N are never stored, so only the loads are guarded
            const float4 *bp = reinterpret_cast<const float4 *>(g.bias + oc0), *sp4 = reinterpret_cast<const float4 *>(g.ln_colsum + oc0);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (oc0 + 4 * j < g.N) {
                const float4 b4 = __ldg(bp + j), c4 = __ldg(sp4 + j);
                gunpack2(gfma2(gpack2(v[4 * j], v[4 * j + 1]), rstd2, gfma2(gpack2(c4.x, c4.y), nmr2, gpack2(b4.x, b4.y))), v[4 * j], v[4 * j + 1]);
                gunpack2(gfma2(gpack2(v[4 * j + 2], v[4 * j + 3]), rstd2, gfma2(gpack2(c4.z, c4.w), nmr2, gpack2(b4.z, b4.w))), v[4 * j + 2], v[4 * j + 3]);
              }
            }
          } else if (g.bias && !fold_bias) {
            const float4 *bp = reinterpret_cast<const float4 *>(g.bias + oc0);
            if (oc0 + 32 <= g.N) {                               // common case: no guards inside the loop
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float4 b4 = __ldg(bp + j);
                gunpack2(gadd2(gpack2(v[4 * j], v[4 * j + 1]), gpack2(b4.x, b4.y)), v[4 * j], v[4 * j + 1]);
                gunpack2(gadd2(gpack2(v[4 * j + 2], v[4 * j + 3]), gpack2(b4.z, b4.w)), v[4 * j + 2], v[4 * j + 3]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                if (oc0 + 4 * j < g.N) {                          // N is a multiple of 8: groups of 4 are all in or all out
                  const float4 b4 = __ldg(bp + j);
                  v[4 * j] += b4.x; v[4 * j + 1] += b4.y; v[4 * j + 2] += b4.z; v[4 * j + 3] += b4.w;
                }
              }
            }
          }
          if (!LEAN && g.epilogue == EPI_GELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
          }
        }
        if (g.residual && row < g.M) {
          const __nv_bfloat16 *rp = g.residual + (size_t)row * g.ldr + oc0;
          if (oc0 + 32 <= g.N && (reinterpret_cast<uintptr_t>(rp) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              const uint4 w = __ldg(reinterpret_cast<const uint4 *>(rp + j));
              const uint32_t *h2 = reinterpret_cast<const uint32_t *>(&w);
#pragma unroll
              for (int e = 0; e < 4; ++e) { const float2 f = unpack_in2<F16>(h2[e]); gunpack2(gadd2(gpack2(v[j + 2 * e], v[j + 2 * e + 1]), gpack2(f.x, f.y)), v[j + 2 * e], v[j + 2 * e + 1]); }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) if (oc0 + j < g.N) v[j] += unpack_in1<F16>(rp + j);
          }
        }
        if (!LEAN && g.stats_out) {
          // row sums of this task's columns for the LayerNorm that follows (the next projection folds it in)
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            if (oc0 + j < g.N) {
              const uint64_t v2 = gpack2(v[j], v[j + 1]);
              tile_sum2 = gadd2(tile_sum2, v2);
              tile_sq2 = gfma2(v2, v2, tile_sq2);
            }
          }
        }
        if (!LEAN && g.direct_store) {
          if (row < g.M) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              const int oc = oc0 + j;
              if (oc >= g.N) continue;
              uint4 w;
              uint32_t *h2 = reinterpret_cast<uint32_t *>(&w);
#pragma unroll
              for (int e = 0; e < 4; ++e) h2[e] = pack_out2<F16>(v[j + 2 * e], v[j + 2 * e + 1]);
              *reinterpret_cast<uint4 *>(g.c_ptr + (size_t)(oc / g.split_n) * g.split_stride + (size_t)row * g.split_n + oc % g.split_n) = w;
            }
          }
          continue;
        }
        // stage 32 rows x 32 columns (64 bytes per row) in the layout the 64-byte-swizzled TMA store reads:
        // 16-byte chunk j of row r sits at chunk j ^ ((r >> 1) & 3)
        unsigned char *ob = my_out + obuf * 32 * 64;
        if (lane == 0) tc::tma_wait_read<1>();    // the store issued two tasks ago has drained this buffer
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 w;
          uint32_t *h2 = reinterpret_cast<uint32_t *>(&w);
#pragma unroll
          for (int e = 0; e < 4; ++e) h2[e] = pack_out2<F16>(v[j * 8 + 2 * e], v[j * 8 + 2 * e + 1]);
          tc::sts128(tc::smem_u32(ob) + lane * 64 + ((j ^ ((lane >> 1) & 3)) * 16), w);
        }
        tc::fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          const int sp = g.nsplit == 1 ? 0 : oc0 / g.split_n;     // which output matrix (no division without splits)
          tc::tma_store_3d(&map_c, ob, oc0 - sp * g.split_n, m0 + q * 32, sp);
          tc::tma_commit();
        }
        obuf ^= 1u;
      }
      task += (uint32_t)(out_cols / 32);
      if (!LEAN && g.stats_out) {
        // leave this warp's partial sums in its slot; the last warp of the quadrant to get here adds the slots in a
        // fixed order.  The slots of an accumulator are free again before its next tile: every epilogue warp arrives
        // on acc_empty only after this block.
        float s0, s1, q0, q1;
        gunpack2(tile_sum2, s0, s1);
        gunpack2(tile_sq2, q0, q1);
        float2 *slots = stat_slots + ((size_t)(acc * 4 + q) * kSub) * 32;
        slots[sub * 32 + lane] = make_float2(s0 + s1, q0 + q1);
        __threadfence_block();
        __syncwarp();
        int last = 0;
        if (lane == 0) last = atomicAdd(&stat_cnt[acc * 4 + q], 1) == (int)kSub - 1;
        last = __shfl_sync(0xFFFFFFFFu, last, 0);
        if (last) {
          __threadfence_block();
          float2 tot = make_float2(0.f, 0.f);
#pragma unroll
          for (uint32_t w = 0; w < kSub; ++w) { const float2 pw = slots[w * 32 + lane]; tot.x += pw.x; tot.y += pw.y; }
          if (row < g.M) {
            if (n_tiles == 1) {
              g.stats_out[row] = tot;
            } else {
              atomicAdd(&g.stats_out[row].x, tot.x);
              atomicAdd(&g.stats_out[row].y, tot.y);
            }
          }
          __syncwarp();
          if (lane == 0) stat_cnt[acc * 4 + q] = 0;
        }
      }
      tc::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&acc_empty[acc]);
    }
    if (lane == 0) tc::tma_wait_all<0>();
  }

  __syncthreads();
  if (*abort_flag) {
    // a wait was abandoned: give copies that may still be in flight time to land before the CTA retires
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) { tc::tc_fence_after_sync(); tc::tmem_dealloc(tmem_base, kTmemCols); }
}

int *status_word(int device);   // device word, zero until a kernel reports an abandoned wait

template <int BN, bool F16, bool LEAN>
static int launch_gemm_build(const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &mc, const GemmArgs &g, int device,
                             cudaStream_t st) {
  auto kern = gemm_bf16_tcgen05_kernel<BN, F16, LEAN>;
  F3D_TRY(ensure_dynamic_smem(reinterpret_cast<const void *>(kern), device, GemmSmem<BN, LEAN>::kTotal));
  int tiles = ((g.M + BM - 1) / BM) * ((g.N + BN - 1) / BN);
  int grid = tiles < sm_count(device) ? tiles : sm_count(device);
  kern<<<grid, gemm_threads(LEAN), GemmSmem<BN, LEAN>::kTotal, st>>>(ma, mb, mc, g);
  return check_launch("gemm_bf16_tcgen05");
}

template <int BN, bool F16>
static int launch_gemm(const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &mc, const GemmArgs &g, int device,
                       cudaStream_t st) {
  // the plain projections (bias, residual, column splits, TMA stores) take the lean build
  const bool lean = (g.epilogue == EPI_NONE || g.epilogue == EPI_SWIGLU) && !g.ln_stats && !g.stats_out && !g.direct_store;
  if (lean) return launch_gemm_build<BN, F16, true>(ma, mb, mc, g, device, st);
  return launch_gemm_build<BN, F16, false>(ma, mb, mc, g, device, st);
}

struct LinearFusion {
  const void *ln_stats = nullptr;    // folded LayerNorm: row sums of A, with the column sums of the scaled weight
  const void *ln_colsum = nullptr;
  float ln_eps = 1e-5f;
  void *stats_out = nullptr;         // row sums of the output
};

// C (nsplit matrices of [M, split_n] with leading dimension split_n, `split_stride` elements apart); dtype 0 = bf16,
// 1 = fp16 for A, W, residual and C
int linear_bf16(const void *A, int lda, const void *W, int ldw, const void *bias, const void *residual, int ldr, void *C,
                long long split_stride, int M, int N, int K, int nsplit, int epilogue, int device, cudaStream_t st, int ksplit = 1,
                int dtype = 0, LinearFusion fu = LinearFusion()) {
  if (dtype != 0 && dtype != 1) return set_error(F3D_ERR_UNSUPPORTED, "gemm: element type %d (0 = bf16 and 1 = fp16 are supported)", dtype);
  if (M <= 0 || N <= 0 || K <= 0) return set_error(F3D_ERR_ARG, "gemm: M, N, K must be positive (got %d, %d, %d)", M, N, K);
  if (K % 8 || lda % 8 || ldw % 8) return set_error(F3D_ERR_ARG, "gemm: K and the leading dimensions must be multiples of 8 (TMA 16-byte rule)");
  if (nsplit < 1 || N % nsplit) return set_error(F3D_ERR_ARG, "gemm: N=%d is not divisible into %d splits", N, nsplit);
  if (epilogue < 0 || epilogue > 2) return set_error(F3D_ERR_ARG, "gemm: unknown epilogue %d", epilogue);
  int out_n = epilogue == EPI_SWIGLU ? N / 2 : N;
  if (epilogue == EPI_SWIGLU && (nsplit != 1 || N % 128)) return set_error(F3D_ERR_ARG, "gemm: swiglu needs nsplit == 1 and N %% 128 == 0");
  int split_n = out_n / nsplit;
  if (split_n % 8) return set_error(F3D_ERR_ARG, "gemm: output row length %d is not a multiple of 8", split_n);
  if (residual && nsplit != 1) return set_error(F3D_ERR_ARG, "gemm: residual needs nsplit == 1");
  if (ksplit < 1 || (ksplit > 1 && (epilogue == EPI_SWIGLU || lda != K || ldw != K)))
    return set_error(F3D_ERR_ARG, "gemm: %d slices along K need dense operands and no SwiGLU epilogue", ksplit);
  if ((long long)ksplit * M > 0x7FFFFFFFll) return set_error(F3D_ERR_UNSUPPORTED, "gemm: %d slices of %d rows exceed the copy coordinates", ksplit, M);
  if (fu.ln_stats && (!fu.ln_colsum || !bias || ksplit != 1 || N % 4))
    return set_error(F3D_ERR_ARG, "gemm: a folded LayerNorm needs the column sums, the folded bias, one K slice and N %% 4 == 0");
  if (fu.stats_out && (nsplit != 1 || epilogue == EPI_SWIGLU))
    return set_error(F3D_ERR_ARG, "gemm: output row sums need a single plain output matrix");

  int BN = 256;
  if (epilogue == EPI_SWIGLU) BN = (N % 256 == 0) ? 256 : 128;
  else if (N <= 32) BN = 32;
  else if (N <= 64) BN = 64;
  else if (N <= 128 || (nsplit > 1 && split_n % 256)) BN = 128;
  const int direct = (nsplit > 1 && split_n % 32) ? 1 : 0;      // a 32-column task must not straddle two outputs
  // rows that span several column tiles add their tiles' sums into a cleared buffer; one tile stores them
  if (fu.stats_out && N > BN) F3D_CUDA_TRY(cudaMemsetAsync(fu.stats_out, 0, (size_t)M * sizeof(float2), st));
  if (reinterpret_cast<uintptr_t>(C) % 16) return set_error(F3D_ERR_ARG, "gemm: output pointer is not 16-byte aligned");
  CUtensorMap ma, mb, mc;
  F3D_TRY(encode_tmap_2d(&ma, dtype, A, (uint64_t)K, (uint64_t)M * ksplit, (uint64_t)lda * 2, BK, BM, 128));
  int b_box_rows = epilogue == EPI_SWIGLU ? BN / 2 : BN;
  F3D_TRY(encode_tmap_2d(&mb, dtype, W, (uint64_t)K, (uint64_t)N * ksplit, (uint64_t)ldw * 2, BK, b_box_rows, 128));
  F3D_TRY(encode_tmap_3d(&mc, dtype, C, (uint64_t)split_n, (uint64_t)M, (uint64_t)nsplit, (uint64_t)split_n * 2,
                         (uint64_t)split_stride * 2, 32, 32, 1, 64));
  GemmArgs g{M, N, K, nsplit, split_n, static_cast<const float *>(bias), static_cast<const __nv_bfloat16 *>(residual), ldr,
             epilogue, direct, static_cast<__nv_bfloat16 *>(C), split_stride, status_word(device), ksplit,
             static_cast<const float2 *>(fu.ln_stats), static_cast<const float *>(fu.ln_colsum), fu.ln_eps, 1.f / (float)K,
             static_cast<float2 *>(fu.stats_out)};
  if (!g.status) return F3D_ERR_CUDA;
  if (dtype == 1) {
    switch (BN) {
      case 32: return launch_gemm<32, true>(ma, mb, mc, g, device, st);
      case 64: return launch_gemm<64, true>(ma, mb, mc, g, device, st);
      case 128: return launch_gemm<128, true>(ma, mb, mc, g, device, st);
      default: return launch_gemm<256, true>(ma, mb, mc, g, device, st);
    }
  }
  switch (BN) {
    case 32: return launch_gemm<32, false>(ma, mb, mc, g, device, st);
    case 64: return launch_gemm<64, false>(ma, mb, mc, g, device, st);
    case 128: return launch_gemm<128, false>(ma, mb, mc, g, device, st);
    default: return launch_gemm<256, false>(ma, mb, mc, g, device, st);
  }
}

}  // namespace f3d

using namespace f3d;

extern "C" int f3d_linear_bf16(const void *A, const void *W, const void *bias, const void *residual, void *C, int M, int N,
                               int K, int nsplit, int epilogue, int device, void *stream) {
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  F3D_TRY(maybe_sync(st, "linear_bf16"));
  int out_n = epilogue == EPI_SWIGLU ? N / 2 : N;
  F3D_TRY(linear_bf16(A, K, W, K, bias, residual, out_n, C, (long long)M * (out_n / (nsplit > 0 ? nsplit : 1)), M, N, K, nsplit,
                      epilogue, device, st));
  return maybe_sync(st, "linear_bf16");
}

extern "C" int f3d_linear_dtype(const void *A, const void *W, const void *bias, const void *residual, void *C, int M, int N,
                                int K, int nsplit, int epilogue, int dtype, int device, void *stream) {
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  F3D_TRY(maybe_sync(st, "linear"));
  int out_n = epilogue == EPI_SWIGLU ? N / 2 : N;
  F3D_TRY(linear_bf16(A, K, W, K, bias, residual, out_n, C, (long long)M * (out_n / (nsplit > 0 ? nsplit : 1)), M, N, K, nsplit,
                      epilogue, device, st, 1, dtype));
  return maybe_sync(st, "linear");
}

extern "C" int f3d_linear_fused(const void *A, const void *W, const void *bias, const void *residual, void *C, int M, int N,
                                int K, int nsplit, int epilogue, int dtype, const void *ln_stats, const void *ln_colsum,
                                float ln_eps, void *stats_out, int device, void *stream) {
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  F3D_TRY(maybe_sync(st, "linear_fused"));
  int out_n = epilogue == EPI_SWIGLU ? N / 2 : N;
  LinearFusion fu;
  fu.ln_stats = ln_stats; fu.ln_colsum = ln_colsum; fu.ln_eps = ln_eps; fu.stats_out = stats_out;
  F3D_TRY(linear_bf16(A, K, W, K, bias, residual, out_n, C, (long long)M * (out_n / (nsplit > 0 ? nsplit : 1)), M, N, K, nsplit,
                      epilogue, device, st, 1, dtype, fu));
  return maybe_sync(st, "linear_fused");
}

extern "C" int f3d_linear_ksplit_bf16(const void *A, const void *W, const void *bias, const void *residual, void *C, int M, int N,
                                      int K, int ksplit, int device, void *stream) {
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  F3D_TRY(maybe_sync(st, "linear_ksplit_bf16"));
  F3D_TRY(linear_bf16(A, K, W, K, bias, residual, N, C, (long long)M * N, M, N, K, 1, EPI_NONE, device, st, ksplit));
  return maybe_sync(st, "linear_ksplit_bf16");
}

// O[M,N] = A[M,K] . B[K,N]: the reference's gemm_sm_bf16 export (src/psh/gemm_dispatcher.cu:26-80).  B is
// transposed into a scratch [N,K] matrix first so that both operands are K-major for the tensor cores.
namespace f3d {
__global__ void transpose_bf16_kernel(const __nv_bfloat16 *in, __nv_bfloat16 *out, int rows, int cols) {
  __shared__ __nv_bfloat16 t[32][33];
  int x = blockIdx.x * 32 + threadIdx.x, y = blockIdx.y * 32 + threadIdx.y;
  for (int j = 0; j < 32; j += 8) if (x < cols && y + j < rows) t[threadIdx.y + j][threadIdx.x] = in[(size_t)(y + j) * cols + x];
  __syncthreads();
  x = blockIdx.y * 32 + threadIdx.x; y = blockIdx.x * 32 + threadIdx.y;
  for (int j = 0; j < 32; j += 8) if (x < rows && y + j < cols) out[(size_t)(y + j) * rows + x] = t[threadIdx.x][threadIdx.y + j];
}
}  // namespace f3d

extern "C" int f3d_gemm_sm_bf16(const void *A, const void *B, void *O, int M, int N, int K, int device, void *stream) {
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (M <= 0 || N <= 0 || K <= 0) return set_error(F3D_ERR_ARG, "gemm_sm_bf16: empty operand");
  void *bt = nullptr;
  F3D_TRY(workspace(device, 1, (size_t)N * K * 2, st, &bt));
  dim3 grid((N + 31) / 32, (K + 31) / 32), block(32, 8);
  transpose_bf16_kernel<<<grid, block, 0, st>>>(static_cast<const __nv_bfloat16 *>(B), static_cast<__nv_bfloat16 *>(bt), K, N);
  F3D_TRY(check_launch("transpose"));
  F3D_TRY(linear_bf16(A, K, bt, K, nullptr, nullptr, 0, O, (long long)M * N, M, N, K, 1, EPI_NONE, device, st));
  // the reference synchronises here (src/psh/gemm_dispatcher.cu:77)
  F3D_CUDA_TRY(cudaStreamSynchronize(st));
  return F3D_OK;
}
