// Front end for raw scans: fp32 point records -> fp16 coordinates (+ the remaining fp32 channels).
//
// LiDAR scan files hold one fp32 record per point (x, y, z, intensity; some formats add a ring index or a time stamp).
// The reference casts and slices them with torch on the host side of collate_coords_flat_sep
// (flash3dxfmr/psh/batching.py:13-28: cat -> .to(dtype) -> [:, :3].contiguous()), three passes over the batch.  Here
// the concatenated records are read once on the device: coords[i] = fp16(rec[i][0..2]) (round to nearest even, the
// conversion torch's .to(float16) applies) and extra[i] = rec[i][3..], both written densely.
// HBM stream: 4 * dim bytes read and 6 + 4 * (dim - 3) bytes written per point.
#include <cuda_fp16.h>

#include "f3d_common.cuh"
#include "../../include/f3d_b200.h"

namespace f3d {

constexpr int kCollateThreads = 256;
constexpr int kCollatePerThread = 4;     // points per thread: independent loads in flight

template <int DIM>
__global__ void __launch_bounds__(kCollateThreads) collate_points_kernel(const float *__restrict__ rec, __half *__restrict__ coords,
                                                                         float *__restrict__ extra, uint64_t rows) {
  const uint64_t base = (uint64_t)blockIdx.x * (kCollateThreads * kCollatePerThread) + threadIdx.x;
  float v[kCollatePerThread][DIM];
#pragma unroll
  for (int k = 0; k < kCollatePerThread; ++k) {
    const uint64_t i = base + (uint64_t)k * kCollateThreads;
    if (i < rows) {
      if constexpr (DIM == 4) {
        const float4 r = __ldg(reinterpret_cast<const float4 *>(rec) + i);
        v[k][0] = r.x; v[k][1] = r.y; v[k][2] = r.z; v[k][3] = r.w;
      } else {
#pragma unroll
        for (int d = 0; d < DIM; ++d) v[k][d] = __ldg(rec + i * DIM + d);
      }
    }
  }
  // coordinates of the CTA's points are packed in shared memory and leave as 16-byte vectors (a CTA's 1024 points are
  // 6144 contiguous bytes of the output); the last, partial CTA and unaligned outputs store halves directly
  constexpr int kPts = kCollateThreads * kCollatePerThread;
  __shared__ __align__(16) __half sc[kPts * 3];
  const uint64_t cta0 = (uint64_t)blockIdx.x * kPts;
  const bool vec = cta0 + kPts <= rows && (reinterpret_cast<uintptr_t>(coords) & 15) == 0;
#pragma unroll
  for (int k = 0; k < kCollatePerThread; ++k) {
    const uint64_t i = base + (uint64_t)k * kCollateThreads;
    if (i < rows) {
      __half *c = vec ? sc + (threadIdx.x + k * kCollateThreads) * 3 : coords + i * 3;
      c[0] = __float2half_rn(v[k][0]); c[1] = __float2half_rn(v[k][1]); c[2] = __float2half_rn(v[k][2]);
      if (extra) {
#pragma unroll
        for (int d = 3; d < DIM; ++d) extra[i * (DIM - 3) + (d - 3)] = v[k][d];
      }
    }
  }
  if (vec) {
    __syncthreads();
    uint4 *dst = reinterpret_cast<uint4 *>(coords + cta0 * 3);
    const uint4 *src = reinterpret_cast<const uint4 *>(sc);
    for (int j = threadIdx.x; j < kPts * 3 * 2 / 16; j += kCollateThreads) dst[j] = src[j];
  }
}

template <int DIM>
static int launch_collate(const void *rec, void *coords, void *extra, uint64_t rows, cudaStream_t st) {
  const uint64_t per_cta = (uint64_t)kCollateThreads * kCollatePerThread;
  collate_points_kernel<DIM><<<(unsigned)((rows + per_cta - 1) / per_cta), kCollateThreads, 0, st>>>(
      static_cast<const float *>(rec), static_cast<__half *>(coords), static_cast<float *>(extra), rows);
  return check_launch("collate_points");
}

}  // namespace f3d

using namespace f3d;

extern "C" int f3d_collate_points_f32(const void *records, void *coords, void *extra, uint64_t rows, uint32_t point_dim, int device,
                                      void *stream) {
  if (point_dim < 3 || point_dim > 6) return set_error(F3D_ERR_ARG, "collate_points: %u floats per point (3 to 6 supported)", point_dim);
  if (rows == 0) return F3D_OK;
  if (rows > 0xFFFFFFFFull) return set_error(F3D_ERR_UNSUPPORTED, "collate_points: more than 2^32 points");
  if (point_dim == 4 && reinterpret_cast<uintptr_t>(records) % 16) return set_error(F3D_ERR_ARG, "collate_points: records are not 16-byte aligned");
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (point_dim) {
    case 3: return launch_collate<3>(records, coords, nullptr, rows, st);
    case 4: return launch_collate<4>(records, coords, extra, rows, st);
    case 5: return launch_collate<5>(records, coords, extra, rows, st);
    default: return launch_collate<6>(records, coords, extra, rows, st);
  }
}
