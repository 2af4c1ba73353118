// Weight and bias gradient of a projection y = x W^T + b on the sm_100a tensor cores:
//     grad_W [N, K] = g^T x      grad_b [N] = column sums of g        g bf16 [M, N], x bf16 [M, K], M = tokens
// The reduction runs over the tokens, hundreds of thousands of rows against an output of a few thousand elements, so the
// work is split over row slabs: a CTA owns one 128 x BKT output tile and one slab, streams its rows of g and x through a
// TMA ring, and accumulates in tensor memory.  Both operands are read "MN-major" (the reduction index is the slow one
// in memory), so neither g nor x is transposed: A = 128 columns of g as two 64-column panels of 128-byte rows, B = up to
// four 64-column panels of x.  While the tensor cores work on a stage, four warps add up the columns of the g tile from
// shared memory - the bias gradient costs no second pass over g.  Partial tiles go to a scratch and a second kernel adds
// the slabs in a fixed order: no atomics, the same bits on every run.
//
// Stands in for the library GEMM g^T x and the separate column-sum pass of the backward of nn.Linear / te.Linear in
// flash3dxfmr/layers/buck_swin.py:159,163 and the MLP of flash3dxfmr/layers/elem_wise.py.
#include "f3d_common.cuh"
#include "tc_sm100.cuh"
#include "../../include/f3d_b200.h"

namespace f3d {

int *status_word(int device);

constexpr int kWgThreads = 192;          // producer warp, MMA warp, four column-sum / epilogue warps
constexpr int kWgRows = 64;              // rows (tokens) per stage
constexpr int kWgStages = 4;
constexpr int kWgPanelBytes = kWgRows * 128;      // 64 rows of 128 bytes

struct WgradArgs {
  int M, N, K;
  int rb;                 // bytes of one x row inside a panel: 128, or 64 when K == 32
  int x_panels;           // 64-column panels of x per k-tile (1..4)
  int k_tiles, n_tiles, slabs, blocks_per_slab;
  float *partial_w;       // slab s: partial_w + s * slab_stride, [N][K]
  float *partial_b;       // slab s: partial_b + s * slab_stride, [N]; or null
  size_t slab_stride;     // floats per slab record (N * K weight sums, then N bias sums when wanted)
  int *status;
};

__global__ void __launch_bounds__(kWgThreads, 1)
wgrad_tcgen05_kernel(const __grid_constant__ CUtensorMap map_g, const __grid_constant__ CUtensorMap map_x, WgradArgs a) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stage_bytes = (2 + a.x_panels) * kWgPanelBytes;
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kWgStages * stage_bytes);
  uint64_t *full = bars, *empty = bars + kWgStages, *acc_full = bars + 2 * kWgStages;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_full + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, slab = blockIdx.y;
  const int nt = tile / a.k_tiles, kt = tile - nt * a.k_tiles;
  const int n0 = nt * 128, k0 = kt * a.x_panels * 64;
  const int total_blocks = (a.M + kWgRows - 1) / kWgRows;
  const int b0 = slab * a.blocks_per_slab;
  const int b1 = b0 + a.blocks_per_slab < total_blocks ? b0 + a.blocks_per_slab : total_blocks;
  const int nblk = b1 > b0 ? b1 - b0 : 0;
  const bool want_bias = a.partial_b != nullptr && kt == 0;
  const uint32_t ncols = (uint32_t)a.x_panels * 64u;                 // accumulator columns (K == 32: half of them unused)
  const uint32_t tmem_cols = ncols <= 64 ? 64 : (ncols <= 128 ? 128 : 256);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kWgStages; ++s) { tc::mbar_init(&full[s], 1); tc::mbar_init(&empty[s], 1 + 4); }
    tc::mbar_init(acc_full, 1);
    *abort_flag = 0;
    tc::mbar_fence_init();
  }
  if (warp == 1) { tc::tmem_alloc(tmem_slot, tmem_cols); tc::tmem_relinquish(); }
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  tc::WaitCtx wc{abort_flag, a.status};

  if (warp == 0) {
    if (tc::elect_one()) {
      tc::tma_prefetch_desc(&map_g); tc::tma_prefetch_desc(&map_x);
      for (int i = 0; i < nblk; ++i) {
        const uint32_t s = i % kWgStages, ph = (i / kWgStages) & 1u;
        if (!tc::mbar_wait(&empty[s], ph ^ 1u, wc, 401, 100)) break;
        unsigned char *st = smem + s * stage_bytes;
        const int r0 = (b0 + i) * kWgRows;
        // rows past M and columns past N or K are zero-filled by the copies and add nothing
        // (a tile load costs the copy engine about 7 cycles per box row: the second g panel is skipped when it lies
        // past N; tensor-memory lanes 64..127 then hold products of stale shared memory and are never stored)
        const bool two = n0 + 64 < a.N;
        tc::mbar_expect_tx(&full[s], (uint32_t)((two ? 2 : 1) * kWgPanelBytes + a.x_panels * kWgRows * a.rb));
        tc::tma_load_2d(st, &map_g, &full[s], n0, r0);
        if (two) tc::tma_load_2d(st + kWgPanelBytes, &map_g, &full[s], n0 + 64, r0);
        for (int p = 0; p < a.x_panels; ++p)
          tc::tma_load_2d(st + (2 + p) * kWgPanelBytes, &map_x, &full[s], k0 + p * 64, r0);
      }
    }
  } else if (warp == 1) {
    if (tc::elect_one()) {
      const uint32_t npanel = a.rb == 64 ? 32u : 64u;                // N of one MMA: the columns of one x panel
      const uint32_t idesc = tc::make_idesc_f16(128, npanel, true, true, true);
      const uint64_t swz = a.rb == 64 ? tc::kSwizzle64 : tc::kSwizzle128;
      bool ok = true;
      for (int i = 0; i < nblk && ok; ++i) {
        const uint32_t s = i % kWgStages, ph = (i / kWgStages) & 1u;
        if (!tc::mbar_wait(&full[s], ph, wc, 402)) { ok = false; break; }
        tc::tc_fence_after_sync();
        const uint32_t g_addr = tc::smem_u32(smem + s * stage_bytes), x_addr = g_addr + 2 * kWgPanelBytes;
        for (int p = 0; p < a.x_panels; ++p) {
#pragma unroll
          for (int ks = 0; ks < kWgRows / 16; ++ks) {
            // A: 16 rows of the g tile, its 128 columns in two panels kWgPanelBytes apart (leading offset); B: the
            // same 16 rows of one x panel
            const uint64_t ad = tc::make_smem_desc(g_addr + ks * 16 * 128, kWgPanelBytes, 1024, tc::kSwizzle128);
            const uint64_t bd = tc::make_smem_desc(x_addr + p * kWgPanelBytes + ks * 16 * a.rb, 16, 8 * a.rb, swz);
            tc::mma_f16_ss(tmem_base + p * 64, ad, bd, idesc, (i | ks) != 0 ? 1u : 0u);
          }
        }
        tc::mma_commit(&empty[s]);
      }
      if (ok) tc::mma_commit(acc_full);
    }
  } else {
    // column sums of the g tile while the tensor cores run.  A warp may read the tensor-memory lanes of quadrant
    // warp % 4 only, so thread (q, lane) owns output row n0 + q * 32 + lane in the sums and in the epilogue alike.
    const int q = warp & 3;
    const int t = q * 32 + lane;                            // 0..127, row of the output tile
    const int n = n0 + t;
    const uint32_t col_off = (uint32_t)(t >> 6) * kWgPanelBytes + (uint32_t)(t & 7) * 2u;
    const uint32_t chunk = (uint32_t)(t & 63) >> 3;
    float bsum = 0.f;
    bool ok = true;
    for (int i = 0; i < nblk && ok; ++i) {
      const uint32_t s = i % kWgStages, ph = (i / kWgStages) & 1u;
      // also without a bias gradient the warps follow the ring stage by stage: the stage's release counts them
      if (!tc::mbar_wait(&full[s], ph, wc, 403)) { ok = false; break; }
      if (want_bias) {
        const uint32_t g_addr = tc::smem_u32(smem + s * stage_bytes) + col_off;
#pragma unroll 16
        for (int r = 0; r < kWgRows; ++r) {
          uint16_t h;
          asm volatile("ld.shared.u16 %0, [%1];" : "=h"(h) : "r"(g_addr + (uint32_t)r * 128u + ((chunk ^ ((uint32_t)r & 7u)) << 4)));
          bsum += __uint_as_float((uint32_t)h << 16);
        }
      }
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&empty[s]);
    }
    // epilogue: lane of tensor memory = output row; the partial tile goes to the slab's scratch as fp32
    if (ok && tc::mbar_wait(acc_full, 0, wc, 404)) {
      __syncwarp();
      tc::tc_fence_after_sync();
      const bool live = n < a.N;
      if (want_bias && live) a.partial_b[(size_t)slab * a.slab_stride + n] = bsum;
      float *dst = a.partial_w + (size_t)slab * a.slab_stride + (size_t)(live ? n : 0) * a.K + k0;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16);
      const uint32_t width = a.rb == 64 ? 32u : 64u;        // K == 32: only the first 32 columns of the panel hold results
      for (uint32_t c = 0; c < ncols; c += 64) {
        for (uint32_t cc = 0; cc < width; cc += 16) {
          uint32_t v[16];
          tc::tmem_ld_32x32b_x16(t_row + c + cc, v);        // warp-wide: rows past N load too, only their stores are skipped
          tc::tmem_ld_wait();
          if (live) {
#pragma unroll
            for (int e = 0; e < 16; e += 4)
              *reinterpret_cast<float4 *>(dst + c + cc + e) = make_float4(__uint_as_float(v[e]), __uint_as_float(v[e + 1]),
                                                                          __uint_as_float(v[e + 2]), __uint_as_float(v[e + 3]));
          }
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
  if (warp == 1) { tc::tc_fence_after_sync(); tc::tmem_dealloc(tmem_base, tmem_cols); }
}

// out[i] = sum over the slabs of partial[s][i], in slab order; a slab's record is its weight tile sums followed by its
// bias sums
__global__ void __launch_bounds__(256) wgrad_reduce_kernel(const float *__restrict__ partial, float *__restrict__ out_w, float *__restrict__ out_b,
                                                           uint32_t slabs, size_t nw, size_t nb) {
  // 32 x 8 threads: thread (tx, ty) adds slabs ty, ty + 8, ... of four consecutive elements, then the eight strands
  // are added in order (a fixed order, with eight loads in flight per element instead of one)
  __shared__ float4 red[8][32];
  const uint32_t tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const size_t i = ((size_t)blockIdx.x * 32 + tx) * 4;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (i < nw + nb)
    for (uint32_t s = ty; s < slabs; s += 8) {
      const float4 v = __ldg(reinterpret_cast<const float4 *>(partial + (size_t)s * (nw + nb) + i));
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
  red[ty][tx] = acc;
  __syncthreads();
  if (ty == 0 && i < nw + nb) {
    float4 t = red[0][tx];
#pragma unroll
    for (int k = 1; k < 8; ++k) { t.x += red[k][tx].x; t.y += red[k][tx].y; t.z += red[k][tx].z; t.w += red[k][tx].w; }
    *reinterpret_cast<float4 *>(i < nw ? out_w + i : out_b + (i - nw)) = t;
  }
}

}  // namespace f3d

using namespace f3d;

extern "C" int f3d_linear_wgrad_bf16(const void *grad_out, const void *x, void *grad_weight, void *grad_bias, int M, int N, int K,
                                     int device, void *stream) {
  if (M <= 0 || N <= 0 || K <= 0) return set_error(F3D_ERR_ARG, "linear_wgrad: M, N, K must be positive (got %d, %d, %d)", M, N, K);
  if (N % 8) return set_error(F3D_ERR_ARG, "linear_wgrad: N = %d must be a multiple of 8", N);
  if (K != 32 && K % 64) return set_error(F3D_ERR_UNSUPPORTED, "linear_wgrad: K = %d must be 32 or a multiple of 64", K);
  if (N % 4 || (reinterpret_cast<uintptr_t>(grad_weight) % 16) || (grad_bias && reinterpret_cast<uintptr_t>(grad_bias) % 16))
    return set_error(F3D_ERR_ARG, "linear_wgrad: outputs must be 16-byte aligned");
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  WgradArgs a{};
  a.M = M; a.N = N; a.K = K;
  a.rb = K == 32 ? 64 : 128;
  const int panels_total = K == 32 ? 1 : K / 64;
  a.x_panels = panels_total < 4 ? panels_total : 4;
  if (panels_total % a.x_panels) a.x_panels = panels_total % 2 == 0 ? 2 : 1;
  a.k_tiles = panels_total / a.x_panels;
  a.n_tiles = (N + 127) / 128;
  const int tiles = a.n_tiles * a.k_tiles;
  const int total_blocks = (M + kWgRows - 1) / kWgRows;
  // one CTA per SM (a CTA's fixed costs - tensor-memory allocation, filling the ring, writing its partial tile - are
  // paid once per slab): as many slabs as fit one wave, at least four row blocks each
  int slabs = sm_count(device) / tiles;
  if (slabs > (total_blocks + 3) / 4) slabs = (total_blocks + 3) / 4;
  if (slabs < 1) slabs = 1;
  a.blocks_per_slab = (total_blocks + slabs - 1) / slabs;
  a.slabs = (total_blocks + a.blocks_per_slab - 1) / a.blocks_per_slab;
  void *scratch = nullptr;
  const size_t nw = (size_t)N * K, nb = grad_bias ? (size_t)N : 0;
  a.slab_stride = nw + nb;
  F3D_TRY(workspace(device, 5, (size_t)a.slabs * a.slab_stride * sizeof(float), st, &scratch));
  a.partial_w = static_cast<float *>(scratch);
  a.partial_b = grad_bias ? a.partial_w + nw : nullptr;
  a.status = status_word(device);
  if (!a.status) return F3D_ERR_CUDA;
  CUtensorMap mg, mx;
  F3D_TRY(encode_tmap_2d(&mg, 0, grad_out, (uint64_t)N, (uint64_t)M, (uint64_t)N * 2, 64, kWgRows, 128));
  F3D_TRY(encode_tmap_2d(&mx, 0, x, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, K == 32 ? 32 : 64, kWgRows, K == 32 ? 64 : 128));
  const int smem = kWgStages * (2 + a.x_panels) * kWgPanelBytes + 256 + 1024;
  F3D_TRY(ensure_dynamic_smem(reinterpret_cast<const void *>(wgrad_tcgen05_kernel), device, kWgStages * 6 * kWgPanelBytes + 256 + 1024));
  dim3 grid(tiles, a.slabs);
  wgrad_tcgen05_kernel<<<grid, kWgThreads, smem, st>>>(mg, mx, a);
  F3D_TRY(check_launch("linear_wgrad"));
  wgrad_reduce_kernel<<<(unsigned)(((nw + nb) / 4 + 31) / 32), 256, 0, st>>>(a.partial_w, static_cast<float *>(grad_weight),
                                                                               static_cast<float *>(grad_bias), (uint32_t)a.slabs, nw, nb);
  F3D_TRY(check_launch("linear_wgrad (reduce)"));
  return F3D_OK;
}
