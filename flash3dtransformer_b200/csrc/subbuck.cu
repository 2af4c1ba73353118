// Sub-bucket construction for stride-S pooling, sm_100a.
//
// Replaces local_subbuck_ker (src/psh/batch_psh_subbuck_reduce.cuh:104-298) and its CumsumCounter
// (src/psh/shmem_cumsum_counter.cuh:25-167).  Per 1024-point block of a scene:
//   block bounding box -> block-normalised voxel -> 13-bit key (16-bit hash / 8, 8192 bins, :130-131,202-203)
//   -> points ordered by (key, index) -> runs of S consecutive points form one sub-bucket
//   -> subbuck_id / subbuck_off / unpool_ind[row, off] = global row, reduced_coord[row] = mean of member coords.
//
// Deliberate, documented differences from the reference, all of which remove run-to-run variation:
//   * no random rotation before the bounding box (the reference draws a fresh quaternion per launch, :193-195);
//   * the block bounding box is the true min/max, broadcast to every thread (the reference consumes a
//     cub::BlockReduce result that is only defined in thread 0, src/common/block_minmax.cuh:43-47);
//   * equal keys are ordered by input index (the reference: shared-memory atomic arrival order);
//   * block k of a scene owns rows [k*ceil(1024/S), ...) of the scene's reduced rows (the reference hands out
//     row ranges with a global atomicAdd in block arrival order, :238);
//   * coordinate means are summed sequentially in sub-bucket order in fp32 (the reference: float shared-memory
//     atomics, :261-270), so the result is bit-reproducible.
#include "f3d_common.cuh"
#include "psh_device.cuh"
#include "../../include/f3d_b200.h"

namespace f3d {

constexpr int kSbThreads = 1024;
constexpr uint32_t kSbBins = 8192;
constexpr uint32_t kSbSegDiv = 65536 / kSbBins;

struct SubbuckArgs {
  const __half *coord; const uint32_t *batch_sep; const uint32_t *red_sep;
  uint32_t *subbuck_id; uint16_t *subbuck_off; uint32_t *unpool_ind; __half *reduced_coord;
  uint32_t total_N, batch, S, num_vox, hash_type, red_rows /* rows of unpool_ind */, red_coord_rows;
};

__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int d = 16; d; d >>= 1) v = fminf(v, __shfl_xor_sync(0xFFFFFFFFu, v, d));
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int d = 16; d; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, d));
  return v;
}

__global__ void __launch_bounds__(kSbThreads) subbuck_build_kernel(SubbuckArgs a) {
  __shared__ uint32_t hist[kSbBins];
  __shared__ uint16_t sorted_tid[kSbThreads];
  __shared__ float sc[3][kSbThreads];
  __shared__ float red[6][32];
  __shared__ uint32_t wsum[33];

  const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t scene = blockIdx.y;
  const uint32_t start = scene ? a.batch_sep[scene - 1] : 0u;
  uint32_t end = min(a.batch_sep[scene], a.total_N);
  const uint32_t n = end > start ? end - start : 0u;
  const uint32_t blk0 = blockIdx.x * kSbThreads;
  if (blk0 >= n) return;
  const uint32_t pts = min((uint32_t)kSbThreads, n - blk0);
  const uint32_t red_start = scene ? a.red_sep[scene - 1] : 0u;
  const uint32_t red_end = a.red_sep[scene];
  const bool valid = tid < pts;
  const uint32_t g = start + blk0 + tid;

  float c[3] = {0.f, 0.f, 0.f};
  if (valid) {
#pragma unroll
    for (int d = 0; d < 3; ++d) c[d] = __half2float(a.coord[(size_t)g * 3 + d]);
  }
  // block bounding box over the valid points
#pragma unroll
  for (int d = 0; d < 3; ++d) {
    float lo = warp_min(valid ? c[d] : INFINITY), hi = warp_max(valid ? c[d] : -INFINITY);
    if (lane == 0) { red[d][warp] = lo; red[3 + d][warp] = hi; }
  }
  for (uint32_t i = tid; i < kSbBins; i += kSbThreads) hist[i] = 0;
  __syncthreads();
  float lo[3], hi[3];
#pragma unroll
  for (int d = 0; d < 3; ++d) {
    lo[d] = warp_min(red[d][lane]);
    hi[d] = warp_max(red[3 + d][lane]);
  }
  uint32_t key = 0, arrival = 0;
  if (valid) {
    uint32_t v[3];
#pragma unroll
    for (int d = 0; d < 3; ++d) v[d] = vox_axis(c[d], lo[d], hi[d], a.num_vox);
    switch (a.hash_type) {
      case H_ZORDER_DIV: key = zorder16(v[0], v[1], v[2]) / kSbSegDiv; break;
      case H_XORSUM_DIV: key = ((v[0] ^ v[1] ^ v[2]) & 0xFFFFu) / kSbSegDiv; break;
      case H_ZORDER_MOD: key = zorder16(v[0], v[1], v[2]) % kSbBins; break;
      default:           key = ((v[0] ^ v[1] ^ v[2]) & 0xFFFFu) % kSbBins; break;
    }
    arrival = atomicAdd(&hist[key], 1u);
  }
  __syncthreads();
  // exclusive scan over the 8192 bins, 8 bins per thread
  uint32_t loc[8], sum = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) { loc[j] = hist[tid * 8 + j]; sum += loc[j]; }
  uint32_t inc = sum;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    uint32_t o = __shfl_up_sync(0xFFFFFFFFu, inc, d);
    if (lane >= d) inc += o;
  }
  if (lane == 31) wsum[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    uint32_t w = wsum[lane], winc = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      uint32_t o = __shfl_up_sync(0xFFFFFFFFu, winc, d);
      if (lane >= d) winc += o;
    }
    wsum[lane] = winc - w;
  }
  __syncthreads();
  uint32_t run = wsum[warp] + inc - sum;
#pragma unroll
  for (int j = 0; j < 8; ++j) { hist[tid * 8 + j] = run; run += loc[j]; }
  __syncthreads();
  uint32_t base = 0, cnt = 0;
  if (valid) {
    base = hist[key];
    cnt = ((key + 1 < kSbBins) ? hist[key + 1] : pts) - base;
    sorted_tid[base + arrival] = (uint16_t)tid;
  }
  __syncthreads();
  uint32_t pt_ind = 0;
  if (valid) {
    uint32_t r = 0;
    for (uint32_t j = 0; j < cnt; ++j) r += (sorted_tid[base + j] < tid) ? 1u : 0u;
    pt_ind = base + r;
    sc[0][pt_ind] = c[0]; sc[1][pt_ind] = c[1]; sc[2][pt_ind] = c[2];
  }
  __syncthreads();
  if (!valid) return;
  const uint32_t per_block = (kSbThreads + a.S - 1) / a.S;
  const uint32_t nb_local = pt_ind / a.S, off = pt_ind % a.S;
  const uint32_t local_row = blockIdx.x * per_block + nb_local;
  const uint32_t row = red_start + local_row;
  a.subbuck_id[g] = local_row;
  a.subbuck_off[g] = (uint16_t)off;
  const bool row_ok = row < red_end && row < a.red_rows;
  if (row_ok) {
    a.unpool_ind[(size_t)row * a.S + off] = g;
    // the last sub-bucket of a block may be short: its first member marks the unfilled slots with the out-of-range
    // index the reference pre-fills the whole table with (flash3dxfmr/psh/subbuck.py:94), so the table needs no pre-fill
    if (off == 0)
      for (uint32_t j = min(a.S, pts - pt_ind); j < a.S; ++j) a.unpool_ind[(size_t)row * a.S + j] = a.total_N + 3u;
  }
  if (off == 0 && row_ok && row < a.red_coord_rows) {
    uint32_t m = min(a.S, pts - pt_ind);
    float s0 = sc[0][pt_ind], s1 = sc[1][pt_ind], s2 = sc[2][pt_ind];
    for (uint32_t j = 1; j < m; ++j) {
      s0 = __fadd_rn(s0, sc[0][pt_ind + j]);
      s1 = __fadd_rn(s1, sc[1][pt_ind + j]);
      s2 = __fadd_rn(s2, sc[2][pt_ind + j]);
    }
    float inv = (float)m;
    a.reduced_coord[(size_t)row * 3 + 0] = __float2half_rn(__fdiv_rn(s0, inv));
    a.reduced_coord[(size_t)row * 3 + 1] = __float2half_rn(__fdiv_rn(s1, inv));
    a.reduced_coord[(size_t)row * 3 + 2] = __float2half_rn(__fdiv_rn(s2, inv));
  }
}

// rows [from, to) of a [rows,3] fp16 array := 0 (alignment padding of reduced_coord)
__global__ void zero_rows3_kernel(__half *p, uint32_t from, uint32_t to) {
  uint64_t i = (uint64_t)from * 3 + blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
  if (i < (uint64_t)to * 3) p[i] = __float2half_rn(0.f);
}

int subbuck_build(const void *coord, const void *batch_sep, const void *red_sep, void *subbuck_id, void *subbuck_off,
                  void *unpool_ind, void *reduced_coord, uint32_t total_N, uint32_t batch, uint32_t max_n, uint32_t S,
                  uint32_t num_vox, uint32_t hash_type, uint32_t red_rows, uint32_t red_coord_rows, cudaStream_t st) {
  SubbuckArgs a{};
  a.coord = static_cast<const __half *>(coord);
  a.batch_sep = static_cast<const uint32_t *>(batch_sep);
  a.red_sep = static_cast<const uint32_t *>(red_sep);
  a.subbuck_id = static_cast<uint32_t *>(subbuck_id);
  a.subbuck_off = static_cast<uint16_t *>(subbuck_off);
  a.unpool_ind = static_cast<uint32_t *>(unpool_ind);
  a.reduced_coord = static_cast<__half *>(reduced_coord);
  a.total_N = total_N; a.batch = batch; a.S = S; a.num_vox = num_vox; a.hash_type = hash_type;
  a.red_rows = red_rows; a.red_coord_rows = red_coord_rows;
  if (max_n > 0 && batch > 0) {
    dim3 grid(cdiv_u32(max_n, kSbThreads), batch);
    subbuck_build_kernel<<<grid, kSbThreads, 0, st>>>(a);
  }
  if (red_coord_rows > red_rows) {
    uint32_t cnt = (red_coord_rows - red_rows) * 3;
    zero_rows3_kernel<<<cdiv_u32(cnt, 256), 256, 0, st>>>(a.reduced_coord, red_rows, red_coord_rows);
  }
  return check_launch("subbuck_build", ((max_n > 0 && batch > 0) ? 1 : 0) + (red_coord_rows > red_rows ? 1 : 0));
}

}  // namespace f3d
