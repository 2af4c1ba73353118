// LayerNorm over the channel dimension for bf16 token features (fp32 statistics and parameters), with an optional
// fused GELU.  The reference normalises with te.LayerNorm / nn.LayerNorm inside XFMR and the pooling wrappers
// (flash3dxfmr/layers/stage.py:67,95; flash3dxfmr/layers/hourglass.py:76-79,152-154); this kernel keeps that step
// at one read and one write of the activations: a group of min(32, C/8) lanes owns a row, every lane holds its
// 16-byte chunks in registers, mean and variance are reduced with shuffles (two-pass, so no cancellation), and
// narrow rows share a warp.
#include "f3d_common.cuh"
#include "../../include/f3d_b200.h"

namespace f3d {

constexpr int kLnThreads = 256;
constexpr int kLnMaxChunks = 8;     // chunks of 8 channels per lane -> C <= 2048

template <int CHUNKS>
__global__ void __launch_bounds__(kLnThreads) layernorm_bf16_kernel(const __nv_bfloat16 *__restrict__ x, const float *__restrict__ w,
                                                                    const float *__restrict__ b, __nv_bfloat16 *__restrict__ y,
                                                                    uint32_t rows, uint32_t C, uint32_t lanes_per_row, float eps, int gelu) {
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t rows_per_warp = 32 / lanes_per_row;
  const uint32_t warp_global = (blockIdx.x * kLnThreads + threadIdx.x) >> 5;
  const uint32_t sub = lane / lanes_per_row, sl = lane % lanes_per_row;
  const uint32_t row = warp_global * rows_per_warp + sub;
  const bool live = row < rows;
  const uint32_t nchunk = C / 8;
  float v[CHUNKS][8];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const uint32_t ch = sl + i * lanes_per_row;
    if (live && ch < nchunk) {
      uint4 q = __ldg(reinterpret_cast<const uint4 *>(x + (size_t)row * C) + ch);
      const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&q);
#pragma unroll
      for (int e = 0; e < 4; ++e) { float2 f = __bfloat1622float2(h[e]); v[i][2 * e] = f.x; v[i][2 * e + 1] = f.y; sum += f.x + f.y; }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[i][e] = 0.f;
    }
  }
  for (uint32_t d = lanes_per_row >> 1; d; d >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, d);
  const float mean = sum / (float)C;
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const uint32_t ch = sl + i * lanes_per_row;
    if (ch < nchunk) {
#pragma unroll
      for (int e = 0; e < 8; ++e) { float d = v[i][e] - mean; sq += d * d; }
    }
  }
  for (uint32_t d = lanes_per_row >> 1; d; d >>= 1) sq += __shfl_xor_sync(0xFFFFFFFFu, sq, d);
  const float rstd = rsqrtf(sq / (float)C + eps);
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const uint32_t ch = sl + i * lanes_per_row;
    if (live && ch < nchunk) {
      float4 w0 = __ldg(reinterpret_cast<const float4 *>(w) + 2 * ch), w1 = __ldg(reinterpret_cast<const float4 *>(w) + 2 * ch + 1);
      float4 b0 = __ldg(reinterpret_cast<const float4 *>(b) + 2 * ch), b1 = __ldg(reinterpret_cast<const float4 *>(b) + 2 * ch + 1);
      const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
      const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float t = (v[i][e] - mean) * rstd * ww[e] + bb[e];
        if (gelu) t = 0.5f * t * (1.f + erff(t * 0.7071067811865476f));
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

}  // namespace f3d

using namespace f3d;

extern "C" int f3d_layernorm_bf16(const void *x, const void *weight, const void *bias, void *y, uint32_t rows, uint32_t C,
                                  float eps, int gelu, int device, void *stream) {
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
  uint32_t rows_per_block = (kLnThreads / 32) * (32 / lpr);
  uint32_t grid = (rows + rows_per_block - 1) / rows_per_block;
  auto xp = static_cast<const __nv_bfloat16 *>(x);
  auto yp = static_cast<__nv_bfloat16 *>(y);
  auto wp = static_cast<const float *>(weight), bp = static_cast<const float *>(bias);
  switch (chunks) {
    case 1: layernorm_bf16_kernel<1><<<grid, kLnThreads, 0, st>>>(xp, wp, bp, yp, rows, C, lpr, eps, gelu); break;
    case 2: layernorm_bf16_kernel<2><<<grid, kLnThreads, 0, st>>>(xp, wp, bp, yp, rows, C, lpr, eps, gelu); break;
    case 3: case 4: layernorm_bf16_kernel<4><<<grid, kLnThreads, 0, st>>>(xp, wp, bp, yp, rows, C, lpr, eps, gelu); break;
    default: layernorm_bf16_kernel<8><<<grid, kLnThreads, 0, st>>>(xp, wp, bp, yp, rows, C, lpr, eps, gelu); break;
  }
  return check_launch("layernorm_bf16");
}
