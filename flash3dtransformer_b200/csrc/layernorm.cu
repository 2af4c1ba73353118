// LayerNorm over the channel dimension for bf16 token features (fp32 statistics and parameters), with an optional
// fused GELU.  The reference normalises with te.LayerNorm / nn.LayerNorm inside XFMR and the pooling wrappers
// (flash3dxfmr/layers/stage.py:67,95; flash3dxfmr/layers/hourglass.py:76-79,152-154); this kernel keeps that step
// at one read and one write of the activations: a group of min(32, C/8) lanes owns a row, every lane holds its
// 16-byte chunks in registers, mean and variance are reduced with shuffles (two-pass, so no cancellation), and
// narrow rows share a warp.
#include "f3d_common.cuh"
#include "../../include/f3d_b200.h"

namespace f3d {

// GELU with the error function, x * Phi(x): erf by the five-term rational approximation of Abramowitz & Stegun 7.1.26
// (one reciprocal, one exponential and six multiply-adds; absolute error of erf below 5e-7, of the result below 5e-7,
// three orders of magnitude under the bf16 rounding of the output).  The library erff made the fused LayerNorm + GELU
// compute-bound at a quarter of the memory bandwidth.
__device__ __forceinline__ float gelu_erf(float x) {
  const float z = fabsf(x) * 0.7071067811865476f;
  float t, e;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, z, 1.f)));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-z * z * 1.4426950408889634f));
  float p = fmaf(1.061405429f, t, -1.453152027f);
  p = fmaf(p, t, 1.421413741f);
  p = fmaf(p, t, -0.284496736f);
  p = fmaf(p, t, 0.254829592f);
  const float erf_abs = fmaf(-p * t, e, 1.f);
  return 0.5f * x * (1.f + copysignf(erf_abs, x));
}

constexpr int kLnThreads = 256;
constexpr int kLnMaxChunks = 8;     // chunks of 8 channels per lane -> C <= 2048

// LPR (lanes per row) and the GELU switch are compile-time so that the shuffle trees unroll and no integer division
// or per-element branch is left in the loop (worth 1.7x on rows of up to 256 channels).  A lane group can take
// ROWS rows at once with all loads issued first; measured, that only pays for rows wider than a warp's 512 bytes.
// MODE 0: LayerNorm, 1: LayerNorm + GELU, 2: statistics only - stats[row] = (sum, sum of squares) over the C channels, the
// input of a LayerNorm that the following projection folds in (f3d_linear_fused); the squares are taken around the row
// mean and the mean's share added back, so the pair carries no cancellation error of its own.
template <int LPR, int CHUNKS, int ROWS, int MODE>
__global__ void __launch_bounds__(kLnThreads) layernorm_bf16_kernel(const __nv_bfloat16 *__restrict__ x, const float *__restrict__ w,
                                                                    const float *__restrict__ b, __nv_bfloat16 *__restrict__ y,
                                                                    uint32_t rows, uint32_t C, float eps, float2 *__restrict__ stats) {
  constexpr bool GELU = MODE == 1;
  constexpr uint32_t kRowsPerWarp = 32 / LPR;
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t warp_global = (blockIdx.x * kLnThreads + threadIdx.x) >> 5;
  const uint32_t sub = lane / LPR, sl = lane % LPR;
  const uint32_t row0 = warp_global * ROWS * kRowsPerWarp + sub;      // this lane group's rows: row0 + r * kRowsPerWarp
  const uint32_t nchunk = C / 8;
  const float inv_c = 1.f / (float)C;
  float v[ROWS][CHUNKS][8];
  float sum[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const uint32_t row = row0 + r * kRowsPerWarp;
    sum[r] = 0.f;
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) {
      const uint32_t ch = sl + i * LPR;
      if (row < rows && ch < nchunk) {
        uint4 q = __ldg(reinterpret_cast<const uint4 *>(x + (size_t)row * C) + ch);
        const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&q);
#pragma unroll
        for (int e = 0; e < 4; ++e) { float2 f = __bfloat1622float2(h[e]); v[r][i][2 * e] = f.x; v[r][i][2 * e + 1] = f.y; sum[r] += f.x + f.y; }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[r][i][e] = 0.f;
      }
    }
  }
  float rstd[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
#pragma unroll
    for (uint32_t d = LPR >> 1; d; d >>= 1) sum[r] += __shfl_xor_sync(0xFFFFFFFFu, sum[r], d);
    const float mean = sum[r] * inv_c;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) {
      const uint32_t ch = sl + i * LPR;
      if (ch < nchunk) {
#pragma unroll
        for (int e = 0; e < 8; ++e) { v[r][i][e] -= mean; sq = fmaf(v[r][i][e], v[r][i][e], sq); }
      }
    }
#pragma unroll
    for (uint32_t d = LPR >> 1; d; d >>= 1) sq += __shfl_xor_sync(0xFFFFFFFFu, sq, d);
    rstd[r] = rsqrtf(sq * inv_c + eps);
    if (MODE == 2) {
      const uint32_t row = row0 + r * kRowsPerWarp;
      if (row < rows && sl == 0) stats[row] = make_float2(sum[r], fmaf(mean, sum[r], sq));     // centred part + C mean^2
    }
  }
  if (MODE == 2) return;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const uint32_t ch = sl + i * LPR;
    if (ch >= nchunk) continue;
    float4 w0 = __ldg(reinterpret_cast<const float4 *>(w) + 2 * ch), w1 = __ldg(reinterpret_cast<const float4 *>(w) + 2 * ch + 1);
    float4 b0 = __ldg(reinterpret_cast<const float4 *>(b) + 2 * ch), b1 = __ldg(reinterpret_cast<const float4 *>(b) + 2 * ch + 1);
    const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const uint32_t row = row0 + r * kRowsPerWarp;
      if (row >= rows) continue;
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float t = fmaf(v[r][i][e] * rstd[r], ww[e], bb[e]);
        if (GELU) t = gelu_erf(t);
        o[e] = t;
      }
      uint4 q;
      __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&q);
#pragma unroll
      for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(o[2 * e], o[2 * e + 1]);
      *(reinterpret_cast<uint4 *>(y + (size_t)row * C) + ch) = q;
    }
  }
}

template <int LPR, int CHUNKS, int ROWS>
static void launch_ln(const __nv_bfloat16 *x, const float *w, const float *b, __nv_bfloat16 *y, uint32_t rows, uint32_t C, float eps,
                      int gelu, cudaStream_t st) {
  const uint32_t rows_per_block = (kLnThreads / 32) * (32 / LPR) * ROWS;
  const uint32_t grid = (rows + rows_per_block - 1) / rows_per_block;
  if (gelu == 2) layernorm_bf16_kernel<LPR, CHUNKS, ROWS, 2><<<grid, kLnThreads, 0, st>>>(x, w, b, y, rows, C, eps, reinterpret_cast<float2 *>(y));
  else if (gelu) layernorm_bf16_kernel<LPR, CHUNKS, ROWS, 1><<<grid, kLnThreads, 0, st>>>(x, w, b, y, rows, C, eps, nullptr);
  else layernorm_bf16_kernel<LPR, CHUNKS, ROWS, 0><<<grid, kLnThreads, 0, st>>>(x, w, b, y, rows, C, eps, nullptr);
}

}  // namespace f3d

using namespace f3d;

// mode 0 / 1: LayerNorm (+ GELU) into y; mode 2: row statistics, y is the float2 [rows] output and weight / bias are unused
static int layernorm_dispatch(const void *x, const void *weight, const void *bias, void *y, uint32_t rows, uint32_t C, float eps,
                              int gelu, int device, void *stream) {
  if (C == 0 || C % 8) return set_error(F3D_ERR_ARG, "layernorm: channel count %u must be a positive multiple of 8", C);
  if (C > 8u * 32u * kLnMaxChunks) return set_error(F3D_ERR_UNSUPPORTED, "layernorm: channel count %u exceeds %d", C, 8 * 32 * kLnMaxChunks);
  if (reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(y) % 16 || reinterpret_cast<uintptr_t>(weight) % 16 ||
      reinterpret_cast<uintptr_t>(bias) % 16)
    return set_error(F3D_ERR_ARG, "layernorm: pointers must be 16-byte aligned");
  if (rows == 0) return F3D_OK;
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  uint32_t nchunk = C / 8;
  uint32_t lpr = 1;
  while (lpr < 32 && lpr < nchunk) lpr <<= 1;
  uint32_t chunks = (nchunk + lpr - 1) / lpr;
  auto xp = static_cast<const __nv_bfloat16 *>(x);
  auto yp = static_cast<__nv_bfloat16 *>(y);
  auto wp = static_cast<const float *>(weight), bp = static_cast<const float *>(bias);
  if (nchunk >= 2 && nchunk <= 32 && (nchunk & (nchunk - 1)) == 0) {
    // rows of 16..256 channels: two 16-byte chunks per lane (one shuffle level fewer: 6-13 % faster than one chunk)
    // and two rows per lane group, so a thread has four loads in flight (another 10-14 %; four rows: 30 % slower)
    switch (nchunk / 2) {
      case 1: launch_ln<1, 2, 2>(xp, wp, bp, yp, rows, C, eps, gelu, st); break;
      case 2: launch_ln<2, 2, 2>(xp, wp, bp, yp, rows, C, eps, gelu, st); break;
      case 4: launch_ln<4, 2, 2>(xp, wp, bp, yp, rows, C, eps, gelu, st); break;
      case 8: launch_ln<8, 2, 2>(xp, wp, bp, yp, rows, C, eps, gelu, st); break;
      default: launch_ln<16, 2, 2>(xp, wp, bp, yp, rows, C, eps, gelu, st); break;
    }
    return check_launch("layernorm_bf16");
  }
  if (lpr < 32) {
    switch (lpr) {
      case 1: launch_ln<1, 1, 1>(xp, wp, bp, yp, rows, C, eps, gelu, st); break;
      case 2: launch_ln<2, 1, 1>(xp, wp, bp, yp, rows, C, eps, gelu, st); break;
      case 4: launch_ln<4, 1, 1>(xp, wp, bp, yp, rows, C, eps, gelu, st); break;
      case 8: launch_ln<8, 1, 1>(xp, wp, bp, yp, rows, C, eps, gelu, st); break;
      default: launch_ln<16, 1, 1>(xp, wp, bp, yp, rows, C, eps, gelu, st); break;
    }
  } else {
    switch (chunks) {
      case 1: launch_ln<32, 1, 1>(xp, wp, bp, yp, rows, C, eps, gelu, st); break;
      case 2: launch_ln<32, 2, 2>(xp, wp, bp, yp, rows, C, eps, gelu, st); break;
      case 3: case 4: launch_ln<32, 4, 1>(xp, wp, bp, yp, rows, C, eps, gelu, st); break;
      default: launch_ln<32, 8, 1>(xp, wp, bp, yp, rows, C, eps, gelu, st); break;
    }
  }
  return check_launch("layernorm_bf16");
}

extern "C" int f3d_layernorm_bf16(const void *x, const void *weight, const void *bias, void *y, uint32_t rows, uint32_t C,
                                  float eps, int gelu, int device, void *stream) {
  return layernorm_dispatch(x, weight, bias, y, rows, C, eps, gelu ? 1 : 0, device, stream);
}

extern "C" int f3d_row_stats_bf16(const void *x, void *stats, uint32_t rows, uint32_t C, int device, void *stream) {
  return layernorm_dispatch(x, nullptr, nullptr, stats, rows, C, 0.f, 2, device, stream);
}
