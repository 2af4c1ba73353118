// Coordinate embedding: out[n, :] = W x[n, :] + b for fp16 coordinates x [N, 3], fp32 W [C, 3] and b [C], bf16 output.
//
// The reference embeds the bucket-sorted coordinates with te.Linear(3, C) (flash3dxfmr/layers/psh_ops.py:62,77).  With
// an inner dimension of 3 this is not a tensor-core GEMM but three FMAs per output, bounded by the 2*C bytes each row
// writes: a thread produces 8 channels (one 16-byte store) of one row, the row's three coordinates are read once per
// thread (consecutive threads of a row hit the same 8 bytes), and the thread's 24 weights and 8 biases stay in registers
// across the rows it visits.
#include <cuda_fp16.h>
#include "f3d_common.cuh"
#include "../../include/f3d_b200.h"

namespace f3d {

constexpr int kEmbedThreads = 256;

__global__ void __launch_bounds__(kEmbedThreads) coord_embed_kernel(const __half *__restrict__ x, const float *__restrict__ w,
                                                                    const float *__restrict__ b, __nv_bfloat16 *__restrict__ y,
                                                                    uint32_t rows, uint32_t C, uint32_t rows_per_block) {
  const uint32_t chunks = C / 8;                         // 16-byte output chunks per row
  const uint32_t ch = threadIdx.x % chunks, rsub = threadIdx.x / chunks, rstep = kEmbedThreads / chunks;
  if (rsub >= rstep) return;                             // threads beyond a whole number of rows idle
  float wr[8][3], br[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const uint32_t c = ch * 8 + e;
    wr[e][0] = __ldg(w + c * 3); wr[e][1] = __ldg(w + c * 3 + 1); wr[e][2] = __ldg(w + c * 3 + 2);
    br[e] = __ldg(b + c);
  }
  const uint32_t r0 = blockIdx.x * rows_per_block;
  const uint32_t r1 = min(rows, r0 + rows_per_block);
  for (uint32_t r = r0 + rsub; r < r1; r += rstep) {
    const float x0 = __half2float(x[(size_t)r * 3]), x1 = __half2float(x[(size_t)r * 3 + 1]), x2 = __half2float(x[(size_t)r * 3 + 2]);
    uint4 q;
    __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&q);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float o0 = fmaf(x2, wr[2 * e][2], fmaf(x1, wr[2 * e][1], fmaf(x0, wr[2 * e][0], br[2 * e])));
      const float o1 = fmaf(x2, wr[2 * e + 1][2], fmaf(x1, wr[2 * e + 1][1], fmaf(x0, wr[2 * e + 1][0], br[2 * e + 1])));
      h[e] = __floats2bfloat162_rn(o0, o1);
    }
    *(reinterpret_cast<uint4 *>(y + (size_t)r * C) + ch) = q;
  }
}

// Gradients of the embedding's parameters: grad_weight[c][j] = sum_rows g[row][c] * x[row][j], grad_bias[c] = sum_rows
// g[row][c].  A block sums a slab of rows (a thread: 8 channels of every rstep-th row, 32 fp32 accumulators), combines its
// row slots through shared memory in slot order and writes partial[block][4][C]; a second kernel adds the partials in
// block order, so the sums are the same bits on every run.
__global__ void __launch_bounds__(kEmbedThreads) coord_embed_bwd_partial_kernel(const __half *__restrict__ x, const __nv_bfloat16 *__restrict__ g,
                                                                                float *__restrict__ partial, uint32_t rows, uint32_t C,
                                                                                uint32_t rows_per_block) {
  extern __shared__ float red[];                         // [slots][4][C]
  const uint32_t chunks = C / 8;
  const uint32_t ch = threadIdx.x % chunks, rsub = threadIdx.x / chunks, rstep = kEmbedThreads / chunks;
  float acc[4][8];
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[j][e] = 0.f;
  if (rsub < rstep) {
    const uint32_t r0 = blockIdx.x * rows_per_block;
    const uint32_t r1 = min(rows, r0 + rows_per_block);
    for (uint32_t r = r0 + rsub; r < r1; r += rstep) {
      const float x0 = __half2float(x[(size_t)r * 3]), x1 = __half2float(x[(size_t)r * 3 + 1]), x2 = __half2float(x[(size_t)r * 3 + 2]);
      const uint4 q = __ldg(reinterpret_cast<const uint4 *>(g + (size_t)r * C) + ch);
      const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&q);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[0][2 * e] = fmaf(f.x, x0, acc[0][2 * e]); acc[0][2 * e + 1] = fmaf(f.y, x0, acc[0][2 * e + 1]);
        acc[1][2 * e] = fmaf(f.x, x1, acc[1][2 * e]); acc[1][2 * e + 1] = fmaf(f.y, x1, acc[1][2 * e + 1]);
        acc[2][2 * e] = fmaf(f.x, x2, acc[2][2 * e]); acc[2][2 * e + 1] = fmaf(f.y, x2, acc[2][2 * e + 1]);
        acc[3][2 * e] += f.x; acc[3][2 * e + 1] += f.y;
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 8; ++e) red[((size_t)rsub * 4 + j) * C + ch * 8 + e] = acc[j][e];
  }
  __syncthreads();
  for (uint32_t q = threadIdx.x; q < 4 * C; q += kEmbedThreads) {
    float s = 0.f;
    for (uint32_t sl = 0; sl < rstep; ++sl) s += red[(size_t)sl * 4 * C + q];
    partial[(size_t)blockIdx.x * 4 * C + q] = s;
  }
}

__global__ void __launch_bounds__(256) coord_embed_bwd_reduce_kernel(const float *__restrict__ partial, float *__restrict__ gw,
                                                                     float *__restrict__ gb, uint32_t blocks, uint32_t C) {
  const uint32_t q = blockIdx.x * 256 + threadIdx.x;      // q = j * C + c
  if (q >= 4 * C) return;
  float s = 0.f;
  for (uint32_t b = 0; b < blocks; ++b) s += partial[(size_t)b * 4 * C + q];
  const uint32_t j = q / C, c = q % C;
  if (j < 3) gw[c * 3 + j] = s;
  else if (gb) gb[c] = s;
}

}  // namespace f3d

using namespace f3d;

extern "C" int f3d_coord_embed_bwd(const void *coords, const void *grad_out, void *grad_weight, void *grad_bias, uint32_t rows,
                                   uint32_t C, int device, void *stream) {
  if (C == 0 || C % 8 || C > 8u * kEmbedThreads) return set_error(F3D_ERR_ARG, "coord_embed_bwd: channel count %u must be a multiple of 8, at most %d", C, 8 * kEmbedThreads);
  if (reinterpret_cast<uintptr_t>(grad_out) % 16) return set_error(F3D_ERR_ARG, "coord_embed_bwd: gradient pointer is not 16-byte aligned");
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (rows == 0) {
    F3D_CUDA_TRY(cudaMemsetAsync(grad_weight, 0, (size_t)C * 3 * sizeof(float), st));
    if (grad_bias) F3D_CUDA_TRY(cudaMemsetAsync(grad_bias, 0, (size_t)C * sizeof(float), st));
    return F3D_OK;
  }
  const uint32_t chunks = C / 8, rstep = kEmbedThreads / chunks;
  const size_t smem = (size_t)rstep * 4 * C * sizeof(float);          // at most 256 / chunks * 4 * 8 * chunks * 4 = 32 KB
  uint32_t blocks = 148u * 4u;
  uint32_t rows_per_block = (rows + blocks - 1) / blocks;
  if (rows_per_block < 64) rows_per_block = 64;
  blocks = (rows + rows_per_block - 1) / rows_per_block;
  void *partial = nullptr;
  F3D_TRY(workspace(device, 4, (size_t)blocks * 4 * C * sizeof(float), st, &partial));
  coord_embed_bwd_partial_kernel<<<blocks, kEmbedThreads, smem, st>>>(static_cast<const __half *>(coords), static_cast<const __nv_bfloat16 *>(grad_out),
                                                                     static_cast<float *>(partial), rows, C, rows_per_block);
  F3D_TRY(check_launch("coord_embed_bwd"));
  coord_embed_bwd_reduce_kernel<<<(4 * C + 255) / 256, 256, 0, st>>>(static_cast<const float *>(partial), static_cast<float *>(grad_weight),
                                                                    static_cast<float *>(grad_bias), blocks, C);
  return check_launch("coord_embed_bwd (reduce)");
}

extern "C" int f3d_coord_embed_bf16(const void *coords, const void *weight, const void *bias, void *out, uint32_t rows, uint32_t C,
                                    int device, void *stream) {
  if (C == 0 || C % 8 || C > 8u * kEmbedThreads) return set_error(F3D_ERR_ARG, "coord_embed: channel count %u must be a multiple of 8, at most %d", C, 8 * kEmbedThreads);
  if (reinterpret_cast<uintptr_t>(out) % 16) return set_error(F3D_ERR_ARG, "coord_embed: output pointer is not 16-byte aligned");
  if (rows == 0) return F3D_OK;
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const uint32_t rows_per_block = 512;
  const uint32_t grid = (rows + rows_per_block - 1) / rows_per_block;
  coord_embed_kernel<<<grid, kEmbedThreads, 0, st>>>(static_cast<const __half *>(coords), static_cast<const float *>(weight),
                                                    static_cast<const float *>(bias), static_cast<__nv_bfloat16 *>(out), rows, C,
                                                    rows_per_block);
  return check_launch("coord_embed_bf16");
}
