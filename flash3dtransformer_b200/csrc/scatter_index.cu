// Scatter index of the PSH bucket order and row gathers through it.
//
// The reference's batch_psh_cumsum_scatter_feat_index_postpad_ker (src/psh/batch_psh_bucket.cuh:617-753) starts on
// this and stops after writing scatter_idx_out2in: features are never scattered and nothing maps results back to the
// input order (Flash3D.forward drops input_feat and returns bucket order, flash3dxfmr/layers/flash3d.py:148-163).
// Here:
//   scatter_index   out2in[dst] = src and in2out[src] = dst for every point, with dst = scene start + exclusive
//                   cumsum of the scene's bucket sizes at its bucket + its offset inside the bucket - the row the
//                   coordinate scatter wrote (batch_psh_bucket.cuh:722-735); rows [total_N, pad_to) of out2in get
//                   total_N + 3 like the reference's padding mark (:667)
//   gather_rows     out[i, :] = src[index[i], :], zero rows where index[i] is not a valid row: with out2in it scatters
//                   input features into bucket order, with in2out it brings per-token results back to input order (and
//                   each is the other's backward)
// Both are HBM streams: 16-byte chunks, one thread per chunk.
#include "f3d_common.cuh"
#include "../../include/f3d_b200.h"

namespace f3d {

__global__ void __launch_bounds__(256) scatter_index_kernel(const uint16_t *__restrict__ bucket_id, const uint32_t *__restrict__ bucket_offset,
                                                            const uint32_t *__restrict__ cumsum, const uint32_t *__restrict__ batch_sep,
                                                            uint32_t *__restrict__ out2in, uint32_t *__restrict__ in2out, uint32_t total_N,
                                                            uint32_t batch, uint32_t nb, uint32_t pad_to) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= pad_to) return;
  if (i >= total_N) { out2in[i] = total_N + 3u; return; }
  // scene of point i: first separator above i (separators are cumulative point counts, i.e. exclusive scene ends, in ascending order)
  uint32_t lo = 0, hi = batch - 1;
  while (lo < hi) {
    const uint32_t mid = (lo + hi) >> 1;
    if (__ldg(batch_sep + mid) > i) hi = mid; else lo = mid + 1;
  }
  const uint32_t start = lo ? __ldg(batch_sep + lo - 1) : 0u;
  const uint32_t id = bucket_id[i];
  const uint32_t base = id ? __ldg(cumsum + (size_t)lo * nb + id - 1) : 0u;
  const uint32_t dst = start + base + bucket_offset[i];
  if (dst < pad_to) out2in[dst] = i;
  if (in2out) in2out[i] = dst;
}

constexpr int kGatherUnroll = 4;   // 16-byte chunks in flight per thread

template <typename V>
__global__ void __launch_bounds__(256) gather_rows_kernel(const V *__restrict__ src, const uint32_t *__restrict__ index, V *__restrict__ out,
                                                          uint64_t total, uint32_t rows_src, uint32_t vecs_per_row, int shift) {
  const uint64_t t0 = (uint64_t)blockIdx.x * (256 * kGatherUnroll) + threadIdx.x;
  V v[kGatherUnroll];
  uint32_t s[kGatherUnroll], c[kGatherUnroll];
#pragma unroll
  for (int k = 0; k < kGatherUnroll; ++k) {
    const uint64_t t = t0 + k * 256;
    s[k] = 0xFFFFFFFFu;
    if (t < total) {
      // shift >= 0: the row holds a power of two of chunks
      const uint64_t r = shift >= 0 ? (t >> shift) : t / vecs_per_row;
      c[k] = (uint32_t)(t - r * vecs_per_row);
      s[k] = __ldg(index + r);
    }
  }
#pragma unroll
  for (int k = 0; k < kGatherUnroll; ++k) {
    v[k] = V{};
    if (s[k] < rows_src) v[k] = __ldg(src + (size_t)s[k] * vecs_per_row + c[k]);
  }
#pragma unroll
  for (int k = 0; k < kGatherUnroll; ++k) {
    const uint64_t t = t0 + k * 256;
    if (t < total) out[t] = v[k];
  }
}

}  // namespace f3d

using namespace f3d;

extern "C" int f3d_scatter_index(const void *bucket_id, const void *bucket_offset, const void *cumsum_counter, const void *batch_sep,
                                 void *out2in, void *in2out, uint32_t total_N, uint32_t batch_size, uint32_t num_bucket,
                                 uint32_t pad_to_N, int device, void *stream) {
  if (batch_size == 0) return set_error(F3D_ERR_ARG, "scatter_index: batch_sep is empty");
  if (pad_to_N < total_N) return set_error(F3D_ERR_ARG, "scatter_index: pad_to_N (%u) is smaller than the input length (%u)", pad_to_N, total_N);
  if (pad_to_N == 0) return F3D_OK;
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  scatter_index_kernel<<<(pad_to_N + 255) / 256, 256, 0, st>>>(static_cast<const uint16_t *>(bucket_id), static_cast<const uint32_t *>(bucket_offset),
                                                              static_cast<const uint32_t *>(cumsum_counter), static_cast<const uint32_t *>(batch_sep),
                                                              static_cast<uint32_t *>(out2in), static_cast<uint32_t *>(in2out), total_N, batch_size,
                                                              num_bucket, pad_to_N);
  return check_launch("scatter_index");
}

extern "C" int f3d_gather_rows(const void *src, const void *index, void *out, uint64_t rows_out, uint32_t rows_src, uint32_t row_bytes,
                               int device, void *stream) {
  if (row_bytes == 0 || row_bytes % 4) return set_error(F3D_ERR_ARG, "gather_rows: row size %u bytes must be a positive multiple of 4", row_bytes);
  if (rows_out == 0) return F3D_OK;
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool a16 = row_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0;
  const bool a8 = row_bytes % 8 == 0 && reinterpret_cast<uintptr_t>(src) % 8 == 0 && reinterpret_cast<uintptr_t>(out) % 8 == 0;
  const uint32_t vec = a16 ? 16 : (a8 ? 8 : 4);
  const uint32_t vpr = row_bytes / vec;
  const uint64_t n = rows_out * vpr;
  const uint64_t per_cta = 256ull * kGatherUnroll;
  if ((n + per_cta - 1) / per_cta > 0x7FFFFFFFull) return set_error(F3D_ERR_UNSUPPORTED, "gather_rows: tensor too large");
  const unsigned grid = (unsigned)((n + per_cta - 1) / per_cta);
  int shift = -1;
  if ((vpr & (vpr - 1)) == 0) for (shift = 0; (1u << shift) < vpr; ++shift) {}
  auto idx = static_cast<const uint32_t *>(index);
  if (vec == 16) gather_rows_kernel<uint4><<<grid, 256, 0, st>>>(static_cast<const uint4 *>(src), idx, static_cast<uint4 *>(out), n, rows_src, vpr, shift);
  else if (vec == 8) gather_rows_kernel<uint2><<<grid, 256, 0, st>>>(static_cast<const uint2 *>(src), idx, static_cast<uint2 *>(out), n, rows_src, vpr, shift);
  else gather_rows_kernel<uint32_t><<<grid, 256, 0, st>>>(static_cast<const uint32_t *>(src), idx, static_cast<uint32_t *>(out), n, rows_src, vpr, shift);
  return check_launch("gather_rows");
}
