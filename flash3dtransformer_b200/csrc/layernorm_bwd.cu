// LayerNorm backward over the channel dimension for bf16 activations: dx, and the gradients of the fp32 weight and
// bias.  With xhat = (x - mean) * rstd and ghat = g * weight:
//     dx      = rstd * (ghat - mean_c(ghat) - xhat * mean_c(ghat * xhat))
//     dweight = sum_rows g * xhat            dbias = sum_rows g
// Backward of the native LayerNorm that stands in for te.LayerNorm / nn.LayerNorm in XFMR and the pooling wrappers
// (flash3dxfmr/layers/stage.py:67,95; flash3dxfmr/layers/hourglass.py:76-79).  One read of x and g, one write of dx:
// a group of LPR lanes owns a row (16-byte chunks in registers, statistics recomputed from x with shuffles); the CTAs
// stride over the rows so that a lane keeps its channels and accumulates their dweight / dbias in registers; the
// per-CTA sums go to a scratch and a second small kernel adds them in a fixed order (no atomics, same bits every run).
#include "f3d_common.cuh"
#include "../../include/f3d_b200.h"

namespace f3d {

constexpr int kLnbThreads = 256;

template <int LPR, int CHUNKS>
__global__ void __launch_bounds__(kLnbThreads) layernorm_bwd_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ g,
                                                                    const float *__restrict__ w, __nv_bfloat16 *__restrict__ dx,
                                                                    float *__restrict__ partial, uint32_t rows, uint32_t C, float eps) {
  constexpr uint32_t kRowsPerWarp = 32 / LPR;
  constexpr uint32_t kRowsPerBlock = (kLnbThreads / 32) * kRowsPerWarp;
  __shared__ float red[kLnbThreads / 32][LPR * CHUNKS * 8];      // one warp row per warp, used for dweight then dbias
  const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t sub = lane / LPR, sl = lane % LPR;
  const uint32_t nchunk = C / 8;
  const float inv_c = 1.f / (float)C;
  float ww[CHUNKS][8], dw[CHUNKS][8], db[CHUNKS][8];
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const uint32_t ch = sl + i * LPR;
#pragma unroll
    for (int e = 0; e < 8; ++e) { ww[i][e] = ch < nchunk ? __ldg(w + ch * 8 + e) : 0.f; dw[i][e] = 0.f; db[i][e] = 0.f; }
  }
  for (uint32_t r0 = blockIdx.x * kRowsPerBlock; r0 < rows; r0 += gridDim.x * kRowsPerBlock) {
    const uint32_t row = r0 + warp * kRowsPerWarp + sub;
    const bool live = row < rows;
    float xv[CHUNKS][8], gv[CHUNKS][8];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) {
      const uint32_t ch = sl + i * LPR;
      if (live && ch < nchunk) {
        const uint4 qx = __ldg(reinterpret_cast<const uint4 *>(x + (size_t)row * C) + ch);
        const uint4 qg = __ldg(reinterpret_cast<const uint4 *>(g + (size_t)row * C) + ch);
        const __nv_bfloat162 *hx = reinterpret_cast<const __nv_bfloat162 *>(&qx), *hg = reinterpret_cast<const __nv_bfloat162 *>(&qg);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 fx = __bfloat1622float2(hx[e]), fg = __bfloat1622float2(hg[e]);
          xv[i][2 * e] = fx.x; xv[i][2 * e + 1] = fx.y; gv[i][2 * e] = fg.x; gv[i][2 * e + 1] = fg.y;
          sum += fx.x + fx.y;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) { xv[i][e] = 0.f; gv[i][e] = 0.f; }
      }
    }
#pragma unroll
    for (uint32_t d = LPR >> 1; d; d >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, d);
    const float mean = sum * inv_c;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) {
      const uint32_t ch = sl + i * LPR;
      if (ch < nchunk) {
#pragma unroll
        for (int e = 0; e < 8; ++e) { xv[i][e] -= mean; sq = fmaf(xv[i][e], xv[i][e], sq); }
      }
    }
#pragma unroll
    for (uint32_t d = LPR >> 1; d; d >>= 1) sq += __shfl_xor_sync(0xFFFFFFFFu, sq, d);
    const float rstd = rsqrtf(sq * inv_c + eps);
    // xv <- xhat; row sums of ghat and ghat * xhat; parameter gradients of this lane's channels
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        xv[i][e] *= rstd;
        const float gh = gv[i][e] * ww[i][e];
        s1 += gh;
        s2 = fmaf(gh, xv[i][e], s2);
        dw[i][e] = fmaf(gv[i][e], xv[i][e], dw[i][e]);       // rows beyond the end and chunks beyond C hold zeros
        db[i][e] += gv[i][e];
      }
    }
#pragma unroll
    for (uint32_t d = LPR >> 1; d; d >>= 1) { s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, d); s2 += __shfl_xor_sync(0xFFFFFFFFu, s2, d); }
    const float m1 = s1 * inv_c, m2 = s2 * inv_c;
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) {
      const uint32_t ch = sl + i * LPR;
      if (live && ch < nchunk) {
        uint4 q;
        __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&q);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float o0 = rstd * (gv[i][2 * e] * ww[i][2 * e] - m1 - xv[i][2 * e] * m2);
          const float o1 = rstd * (gv[i][2 * e + 1] * ww[i][2 * e + 1] - m1 - xv[i][2 * e + 1] * m2);
          h[e] = __floats2bfloat162_rn(o0, o1);
        }
        *(reinterpret_cast<uint4 *>(dx + (size_t)row * C) + ch) = q;
      }
    }
  }
  // fold the row groups of a warp (lanes with equal sl), then the warps, in a fixed order
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e)
#pragma unroll
      for (uint32_t d = LPR; d < 32; d <<= 1) { dw[i][e] += __shfl_xor_sync(0xFFFFFFFFu, dw[i][e], d); db[i][e] += __shfl_xor_sync(0xFFFFFFFFu, db[i][e], d); }
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    if (sub == 0) {
#pragma unroll
      for (int i = 0; i < CHUNKS; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) red[warp][(i * LPR + sl) * 8 + e] = pass == 0 ? dw[i][e] : db[i][e];
    }
    __syncthreads();
    for (uint32_t c = threadIdx.x; c < C; c += kLnbThreads) {
      // channel c belongs to chunk c / 8 = i * LPR + sl, stored at that index
      float acc = 0.f;
#pragma unroll
      for (int wq = 0; wq < kLnbThreads / 32; ++wq) acc += red[wq][c];
      partial[((size_t)blockIdx.x * 2 + pass) * C + c] = acc;
    }
    __syncthreads();
  }
}

// dweight[c] / dbias[c] = sum over the per-CTA partial rows.  A block of 32 x 32 threads takes 32 channels: thread
// (tx, ty) adds rows ty, ty + 32, ... in order, then the 32 strands are added in order (fixed summation order; with
// up to 1184 partial rows, eight strands left every thread a chain of 148 dependent loads and additions).
constexpr int kLnbStrands = 32;
__global__ void __launch_bounds__(32 * kLnbStrands) layernorm_bwd_reduce_kernel(const float *__restrict__ partial, float *__restrict__ dweight,
                                                                                float *__restrict__ dbias, uint32_t blocks, uint32_t C) {
  __shared__ float red[2][kLnbStrands][32];
  const uint32_t tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const uint32_t c = blockIdx.x * 32 + tx;
  float a = 0.f, b = 0.f;
  if (c < C)
    for (uint32_t p = ty; p < blocks; p += kLnbStrands) { a += partial[((size_t)p * 2) * C + c]; b += partial[((size_t)p * 2 + 1) * C + c]; }
  red[0][ty][tx] = a; red[1][ty][tx] = b;
  __syncthreads();
  if (ty == 0 && c < C) {
    float sa = 0.f, sb = 0.f;
#pragma unroll
    for (int q = 0; q < kLnbStrands; ++q) { sa += red[0][q][tx]; sb += red[1][q][tx]; }
    dweight[c] = sa;
    dbias[c] = sb;
  }
}

template <int LPR, int CHUNKS>
static void launch_lnb(const __nv_bfloat16 *x, const __nv_bfloat16 *g, const float *w, __nv_bfloat16 *dx, float *partial, uint32_t rows,
                       uint32_t C, float eps, uint32_t grid, cudaStream_t st) {
  layernorm_bwd_kernel<LPR, CHUNKS><<<grid, kLnbThreads, 0, st>>>(x, g, w, dx, partial, rows, C, eps);
}

}  // namespace f3d

using namespace f3d;

extern "C" int f3d_layernorm_bwd_bf16(const void *x, const void *grad_out, const void *weight, void *grad_x, void *grad_weight,
                                      void *grad_bias, uint32_t rows, uint32_t C, float eps, int device, void *stream) {
  if (C == 0 || C % 8 || C > 1024) return set_error(F3D_ERR_ARG, "layernorm_bwd: channel count %u must be a multiple of 8, at most 1024", C);
  if (reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(grad_out) % 16 || reinterpret_cast<uintptr_t>(grad_x) % 16)
    return set_error(F3D_ERR_ARG, "layernorm_bwd: pointers must be 16-byte aligned");
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (rows == 0) {
    F3D_CUDA_TRY(cudaMemsetAsync(grad_weight, 0, C * sizeof(float), st));
    F3D_CUDA_TRY(cudaMemsetAsync(grad_bias, 0, C * sizeof(float), st));
    return F3D_OK;
  }
  const uint32_t nchunk = C / 8;
  uint32_t lpr = 1;
  while (lpr < 32 && lpr < nchunk) lpr <<= 1;
  const uint32_t chunks = (nchunk + lpr - 1) / lpr;
  const uint32_t rows_per_block = (kLnbThreads / 32) * (32 / lpr);
  uint32_t grid = (rows + rows_per_block - 1) / rows_per_block;
  if (grid > 148u * 8u) grid = 148u * 8u;
  void *partial = nullptr;
  F3D_TRY(workspace(device, 3, (size_t)grid * 2 * C * sizeof(float), st, &partial));
  auto xp = static_cast<const __nv_bfloat16 *>(x), gp = static_cast<const __nv_bfloat16 *>(grad_out);
  auto dxp = static_cast<__nv_bfloat16 *>(grad_x);
  auto wp = static_cast<const float *>(weight);
  auto pp = static_cast<float *>(partial);
  if (lpr < 32) {
    switch (lpr) {
      case 1: launch_lnb<1, 1>(xp, gp, wp, dxp, pp, rows, C, eps, grid, st); break;
      case 2: launch_lnb<2, 1>(xp, gp, wp, dxp, pp, rows, C, eps, grid, st); break;
      case 4: launch_lnb<4, 1>(xp, gp, wp, dxp, pp, rows, C, eps, grid, st); break;
      case 8: launch_lnb<8, 1>(xp, gp, wp, dxp, pp, rows, C, eps, grid, st); break;
      default: launch_lnb<16, 1>(xp, gp, wp, dxp, pp, rows, C, eps, grid, st); break;
    }
  } else {
    switch (chunks) {
      case 1: launch_lnb<32, 1>(xp, gp, wp, dxp, pp, rows, C, eps, grid, st); break;
      case 2: launch_lnb<32, 2>(xp, gp, wp, dxp, pp, rows, C, eps, grid, st); break;
      default: launch_lnb<32, 4>(xp, gp, wp, dxp, pp, rows, C, eps, grid, st); break;
    }
  }
  F3D_TRY(check_launch("layernorm_bwd_bf16"));
  layernorm_bwd_reduce_kernel<<<(C + 31) / 32, 32 * kLnbStrands, 0, st>>>(pp, static_cast<float *>(grad_weight), static_cast<float *>(grad_bias), grid, C);
  return check_launch("layernorm_bwd_bf16 (reduce)");
}
