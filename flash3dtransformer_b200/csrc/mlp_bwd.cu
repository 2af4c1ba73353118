// Element-wise helpers of the MLP / projection backward passes (bf16 activations, fp32 arithmetic):
//   swiglu_bwd   gradient of out = silu(gate) * up with respect to the pre-activation [gate | up] that the fc1 GEMM
//                produced (flash3dxfmr's LayerNormMLP comes from TransformerEngine with activation "swiglu",
//                flash3dxfmr/layers/elem_wise.py; its backward is TransformerEngine's):
//                    d_gate = g * up * s * (1 + gate * (1 - s)),  d_up = g * gate * s,  s = sigmoid(gate)
//   gelu_bwd     gradient of out = gelu(y) with respect to y, exact (error function; the LayerNorm + GELU of the pooling
//                and unpooling wrappers, flash3dxfmr/layers/hourglass.py:101-103, 181-185) or tanh form (the GELU
//                epilogue of the projection GEMM)
//   colsum       bias gradient: fp32 column sums of a bf16 [rows, C] matrix, added in a fixed order
// All are HBM-bound streams: 16-byte loads and stores, one thread per 8 channels.
#include "f3d_common.cuh"
#include "../../include/f3d_b200.h"

namespace f3d {

__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const __nv_bfloat16 *__restrict__ y, const __nv_bfloat16 *__restrict__ g,
                                                         __nv_bfloat16 *__restrict__ dy, size_t rows, uint32_t F) {
  const uint32_t chunks = F / 8;
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * chunks) return;
  const size_t r = idx / chunks;
  const uint32_t c = (uint32_t)(idx % chunks);
  const uint4 qg = __ldg(reinterpret_cast<const uint4 *>(y + r * 2 * F) + c);
  const uint4 qu = __ldg(reinterpret_cast<const uint4 *>(y + r * 2 * F + F) + c);
  const uint4 qo = __ldg(reinterpret_cast<const uint4 *>(g + r * F) + c);
  const __nv_bfloat162 *hg = reinterpret_cast<const __nv_bfloat162 *>(&qg), *hu = reinterpret_cast<const __nv_bfloat162 *>(&qu);
  const __nv_bfloat162 *ho = reinterpret_cast<const __nv_bfloat162 *>(&qo);
  uint4 wg, wu;
  __nv_bfloat162 *og = reinterpret_cast<__nv_bfloat162 *>(&wg), *ou = reinterpret_cast<__nv_bfloat162 *>(&wu);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 a = __bfloat1622float2(hg[e]), u = __bfloat1622float2(hu[e]), o = __bfloat1622float2(ho[e]);
    const float s0 = 1.f / (1.f + __expf(-a.x)), s1 = 1.f / (1.f + __expf(-a.y));
    og[e] = __floats2bfloat162_rn(o.x * u.x * s0 * (1.f + a.x * (1.f - s0)), o.y * u.y * s1 * (1.f + a.y * (1.f - s1)));
    ou[e] = __floats2bfloat162_rn(o.x * a.x * s0, o.y * a.y * s1);
  }
  *(reinterpret_cast<uint4 *>(dy + r * 2 * F) + c) = wg;
  *(reinterpret_cast<uint4 *>(dy + r * 2 * F + F) + c) = wu;
}

template <bool TANH> __device__ __forceinline__ float gelu_grad(float x) {
  if (TANH) {
    // gelu(x) = x/2 (1 + tanh(u)), u = k (x + 0.044715 x^3), k = sqrt(2/pi)
    const float k = 0.7978845608028654f, x2 = x * x;
    const float t = tanhf(k * x * fmaf(0.044715f, x2, 1.f));
    return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k * fmaf(3.f * 0.044715f, x2, 1.f);
  }
  // gelu(x) = x Phi(x): Phi(x) + x phi(x)
  return 0.5f * (1.f + erff(x * 0.7071067811865476f)) + x * 0.3989422804014327f * __expf(-0.5f * x * x);
}

template <bool TANH>
__global__ void __launch_bounds__(256) gelu_bwd_kernel(const __nv_bfloat16 *__restrict__ y, const __nv_bfloat16 *__restrict__ g,
                                                       __nv_bfloat16 *__restrict__ dy, size_t chunks) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= chunks) return;
  const uint4 qy = __ldg(reinterpret_cast<const uint4 *>(y) + idx), qg = __ldg(reinterpret_cast<const uint4 *>(g) + idx);
  const __nv_bfloat162 *hy = reinterpret_cast<const __nv_bfloat162 *>(&qy), *hg = reinterpret_cast<const __nv_bfloat162 *>(&qg);
  uint4 w;
  __nv_bfloat162 *o = reinterpret_cast<__nv_bfloat162 *>(&w);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 a = __bfloat1622float2(hy[e]), b = __bfloat1622float2(hg[e]);
    o[e] = __floats2bfloat162_rn(b.x * gelu_grad<TANH>(a.x), b.y * gelu_grad<TANH>(a.y));
  }
  *(reinterpret_cast<uint4 *>(dy) + idx) = w;
}

// partial[b][c] = sum over the rows of block b; blocks stride over the rows
__global__ void __launch_bounds__(256) colsum_partial_kernel(const __nv_bfloat16 *__restrict__ x, float *__restrict__ partial, size_t rows,
                                                             uint32_t C, uint32_t ld, uint32_t rows_per_block) {
  const uint32_t chunks = C / 8;                      // threads of a block: [row slots][chunks]
  const uint32_t ch = threadIdx.x % chunks, slot = threadIdx.x / chunks, slots = blockDim.x / chunks;
  __shared__ float red[256 * 8];
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (slot < slots) {
    const size_t r0 = (size_t)blockIdx.x * rows_per_block;
    const size_t r1 = r0 + rows_per_block < rows ? r0 + rows_per_block : rows;
    // four rows per step: the loads are issued together (64 bytes in flight per thread), the additions keep the row order
    size_t r = r0 + slot;
    for (; r + 3 * (size_t)slots < r1; r += 4 * (size_t)slots) {
      uint4 q[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) q[k] = __ldg(reinterpret_cast<const uint4 *>(x + (r + (size_t)k * slots) * ld) + ch);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&q[k]);
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(h[e]); acc[2 * e] += f.x; acc[2 * e + 1] += f.y; }
      }
    }
    for (; r < r1; r += slots) {
      const uint4 q = __ldg(reinterpret_cast<const uint4 *>(x + r * ld) + ch);
      const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&q);
#pragma unroll
      for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(h[e]); acc[2 * e] += f.x; acc[2 * e + 1] += f.y; }
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) red[threadIdx.x * 8 + e] = slot < slots ? acc[e] : 0.f;
  __syncthreads();
  for (uint32_t c = threadIdx.x; c < C; c += blockDim.x) {
    float s = 0.f;
    for (uint32_t sl = 0; sl < slots; ++sl) s += red[(sl * chunks + c / 8) * 8 + (c & 7)];
    partial[(size_t)blockIdx.x * C + c] = s;
  }
}

// out[c] = sum over the partial rows: 32 x 8 threads per 32 channels, rows ty, ty + 8, ... in order, then the eight
// slices in order (fixed summation order)
__global__ void __launch_bounds__(256) colsum_reduce_kernel(const float *__restrict__ partial, float *__restrict__ out, uint32_t blocks,
                                                            uint32_t C) {
  __shared__ float red[8][32];
  const uint32_t tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const uint32_t c = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (c < C)
    for (uint32_t b = ty; b < blocks; b += 8) s += partial[(size_t)b * C + c];
  red[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && c < C) {
    float t = 0.f;
#pragma unroll
    for (int q = 0; q < 8; ++q) t += red[q][tx];
    out[c] = t;
  }
}

}  // namespace f3d

using namespace f3d;

extern "C" int f3d_swiglu_bwd_bf16(const void *pre_act, const void *grad_out, void *grad_pre_act, uint64_t rows, uint32_t F,
                                   int device, void *stream) {
  if (F == 0 || F % 8) return set_error(F3D_ERR_ARG, "swiglu_bwd: feature count %u must be a positive multiple of 8", F);
  if (reinterpret_cast<uintptr_t>(pre_act) % 16 || reinterpret_cast<uintptr_t>(grad_out) % 16 || reinterpret_cast<uintptr_t>(grad_pre_act) % 16)
    return set_error(F3D_ERR_ARG, "swiglu_bwd: pointers must be 16-byte aligned");
  if (rows == 0) return F3D_OK;
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const size_t n = (size_t)rows * (F / 8);
  if ((n + 255) / 256 > 0x7FFFFFFFull) return set_error(F3D_ERR_UNSUPPORTED, "swiglu_bwd: tensor too large");
  swiglu_bwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(pre_act), static_cast<const __nv_bfloat16 *>(grad_out),
                                                                static_cast<__nv_bfloat16 *>(grad_pre_act), (size_t)rows, F);
  return check_launch("swiglu_bwd_bf16");
}

extern "C" int f3d_gelu_bwd_bf16(const void *pre_act, const void *grad_out, void *grad_pre_act, uint64_t elems, int tanh_form,
                                 int device, void *stream) {
  if (elems % 8) return set_error(F3D_ERR_ARG, "gelu_bwd: element count %llu must be a multiple of 8", (unsigned long long)elems);
  if (reinterpret_cast<uintptr_t>(pre_act) % 16 || reinterpret_cast<uintptr_t>(grad_out) % 16 || reinterpret_cast<uintptr_t>(grad_pre_act) % 16)
    return set_error(F3D_ERR_ARG, "gelu_bwd: pointers must be 16-byte aligned");
  if (elems == 0) return F3D_OK;
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const size_t n = (size_t)(elems / 8);
  if ((n + 255) / 256 > 0x7FFFFFFFull) return set_error(F3D_ERR_UNSUPPORTED, "gelu_bwd: tensor too large");
  const unsigned grid = (unsigned)((n + 255) / 256);
  const __nv_bfloat16 *y = static_cast<const __nv_bfloat16 *>(pre_act), *g = static_cast<const __nv_bfloat16 *>(grad_out);
  if (tanh_form) gelu_bwd_kernel<true><<<grid, 256, 0, st>>>(y, g, static_cast<__nv_bfloat16 *>(grad_pre_act), n);
  else gelu_bwd_kernel<false><<<grid, 256, 0, st>>>(y, g, static_cast<__nv_bfloat16 *>(grad_pre_act), n);
  return check_launch("gelu_bwd_bf16");
}

extern "C" int f3d_colsum_bf16(const void *x, void *out, uint64_t rows, uint32_t C, int device, void *stream) {
  if (C == 0 || C % 8) return set_error(F3D_ERR_ARG, "colsum: column count %u must be a positive multiple of 8", C);
  if (reinterpret_cast<uintptr_t>(x) % 16) return set_error(F3D_ERR_ARG, "colsum: input pointer must be 16-byte aligned");
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (rows == 0) { F3D_CUDA_TRY(cudaMemsetAsync(out, 0, C * sizeof(float), st)); return F3D_OK; }
  uint32_t blocks = 148u * 4u;
  uint32_t rows_per_block = (uint32_t)((rows + blocks - 1) / blocks);
  if (rows_per_block < 64) rows_per_block = 64;
  blocks = (uint32_t)((rows + rows_per_block - 1) / rows_per_block);
  // column blocks of at most 2048 (256 threads x 8 channels), one after the other through the same scratch
  for (uint32_t c0 = 0; c0 < C; c0 += 2048) {
    const uint32_t cb = C - c0 < 2048 ? C - c0 : 2048;
    void *partial = nullptr;
    F3D_TRY(workspace(device, 4, (size_t)blocks * 2048 * sizeof(float), st, &partial));
    // a block is [row slots][chunks of 8 channels]
    const uint32_t chunks = cb / 8;
    const uint32_t threads = 256 / chunks * chunks;
    colsum_partial_kernel<<<blocks, threads, 0, st>>>(static_cast<const __nv_bfloat16 *>(x) + c0, static_cast<float *>(partial), (size_t)rows, cb, C,
                                                      rows_per_block);
    F3D_TRY(check_launch("colsum_bf16"));
    colsum_reduce_kernel<<<(cb + 31) / 32, 256, 0, st>>>(static_cast<const float *>(partial), static_cast<float *>(out) + c0, blocks, cb);
    F3D_TRY(check_launch("colsum_bf16 (reduce)"));
  }
  return F3D_OK;
}

