// Feature pooling (sub-bucket reduce) and additive unpooling, forward and backward, sm_100a.
//
// Replaces
//   reduce_feat_ker            src/psh/batch_psh_subbuck_reduce.cuh:300-359
//   reduce_feat_backward_ker   src/psh/batch_psh_subbuck_reduce_bwd.cuh:38-126
//   additive_unpool_fwd_ker    src/psh/additive_unpool.cuh:42-86
//   additive_unpool_bwd_ker    src/psh/additive_unpool.cuh:89-136
// and the host drivers in src/psh/batch_subbuck_pooling_dispatcher.cu:35-144,
// src/psh/batch_subbuck_pooling_bwd_dispatcher.cu:26-85, src/psh/additive_unpool_dispatcher.cu:26-134.
//
// All four are gathers/scatters through unpool_ind [rows, S] and are bound by HBM bandwidth.  The reference
// assigns one warp per reduced row and moves 2 bytes per lane per access; here a thread owns one 16-byte chunk
// (8 bf16/fp16 or 4 fp32 channels) of one reduced row, so a row of C channels is covered by C*esize/16
// neighbouring lanes with 128-bit loads and stores, and rows narrower than a warp share it.  Accumulation is
// fp32 in slot order, as in the reference, so results do not depend on the launch shape.
// Feature dtype is bf16 in the reference (asserted at batch_subbuck_pooling_dispatcher.cu:54); fp16 and fp32 are
// additionally instantiated here.
#include "f3d_common.cuh"
#include "../../include/f3d_b200.h"

namespace f3d {

int subbuck_build(const void *coord, const void *batch_sep, const void *red_sep, void *subbuck_id, void *subbuck_off,
                  void *unpool_ind, void *reduced_coord, uint32_t total_N, uint32_t batch, uint32_t max_n, uint32_t S,
                  uint32_t num_vox, uint32_t hash_type, uint32_t red_rows, uint32_t red_coord_rows, cudaStream_t st);

enum RedOp : uint32_t { O_MEAN = 0, O_SUM = 1, O_MIN = 2, O_MAX = 3 };
constexpr int kMaxS = 8;
constexpr int kPoolThreads = 256;

template <typename T> struct Chunk;   // 16 bytes of channels
template <> struct Chunk<float> {
  static constexpr int N = 4;
  __device__ static void load(const float *p, float (&v)[4]) {
    float4 q = *reinterpret_cast<const float4 *>(p); v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
  }
  __device__ static void store(float *p, const float (&v)[4]) {
    *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
  __device__ static void cvt(const uint4 &q, float (&v)[4]) {
    v[0] = __uint_as_float(q.x); v[1] = __uint_as_float(q.y); v[2] = __uint_as_float(q.z); v[3] = __uint_as_float(q.w);
  }
};
template <> struct Chunk<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16 *p, float (&v)[8]) {
    uint4 q = *reinterpret_cast<const uint4 *>(p);
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  __device__ static void cvt(const uint4 &q, float (&v)[8]) {
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  __device__ static void store(__nv_bfloat16 *p, const float (&v)[8]) {
    uint4 q; __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4 *>(p) = q;
  }
};
template <> struct Chunk<__half> {
  static constexpr int N = 8;
  __device__ static void load(const __half *p, float (&v)[8]) {
    uint4 q = *reinterpret_cast<const uint4 *>(p);
    const __half2 *h = reinterpret_cast<const __half2 *>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  __device__ static void cvt(const uint4 &q, float (&v)[8]) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  __device__ static void store(__half *p, const float (&v)[8]) {
    uint4 q; __half2 *h = reinterpret_cast<__half2 *>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4 *>(p) = q;
  }
};

struct GatherArgs {
  const uint32_t *unpool_ind;
  uint32_t ind_rows;      // rows of unpool_ind
  uint32_t out_rows;      // rows the kernel covers (>= ind_rows: the tail is alignment padding)
  uint32_t valid_N;       // an index < valid_N refers to a real row
  uint32_t C, S, op, chunks_per_row;
};

// ------------------------------------------------------------------------------------------- pooling forward
template <typename T>
__global__ void __launch_bounds__(kPoolThreads) pool_reduce_kernel(const T *__restrict__ in, T *__restrict__ out, GatherArgs a) {
  constexpr int N = Chunk<T>::N;
  // A thread reduces two 16-byte chunks of the output (slots 2 * gid and 2 * gid + 1).  Members are taken two at a
  // time: the indices and then the 16-byte loads of both chunks are issued before the first value is used, so a thread
  // has four loads in flight; every chunk still adds its members in slot order.
  const uint64_t total = (uint64_t)a.out_rows * a.chunks_per_row;
  const uint64_t g0 = ((uint64_t)blockIdx.x * kPoolThreads + threadIdx.x) * 2;
  if (g0 >= total) return;
  uint32_t row[2], ch[2], cnt[2] = {0u, 0u};
  bool live[2];
  float acc[2][N];
  const float init = a.op == O_MIN ? INFINITY : (a.op == O_MAX ? -INFINITY : 0.f);
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const uint64_t g = g0 + k;
    live[k] = g < total;
    row[k] = (uint32_t)((live[k] ? g : g0) / a.chunks_per_row);
    ch[k] = (uint32_t)((live[k] ? g : g0) % a.chunks_per_row);
#pragma unroll
    for (int i = 0; i < N; ++i) acc[k][i] = init;
  }
  for (uint32_t s0 = 0; s0 < a.S; s0 += 2) {
    uint32_t r[2][2];
    bool ok[2][2];
    uint4 q[2][2];
#pragma unroll
    for (int k = 0; k < 2; ++k)
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        const bool has = live[k] && row[k] < a.ind_rows && s0 + m < a.S;
        r[k][m] = has ? __ldg(a.unpool_ind + (size_t)row[k] * a.S + s0 + m) : 0xFFFFFFFFu;
      }
#pragma unroll
    for (int k = 0; k < 2; ++k)
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        ok[k][m] = r[k][m] < a.valid_N;
        q[k][m] = make_uint4(0, 0, 0, 0);
        if (ok[k][m]) q[k][m] = __ldg(reinterpret_cast<const uint4 *>(in + (size_t)r[k][m] * a.C + ch[k] * N));
      }
#pragma unroll
    for (int k = 0; k < 2; ++k)
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        if (ok[k][m]) {
          ++cnt[k];
          float v[N];
          Chunk<T>::cvt(q[k][m], v);
#pragma unroll
          for (int i = 0; i < N; ++i) {
            if (a.op == O_MIN) acc[k][i] = fminf(acc[k][i], v[i]);
            else if (a.op == O_MAX) acc[k][i] = fmaxf(acc[k][i], v[i]);
            else acc[k][i] = __fadd_rn(acc[k][i], v[i]);
          }
        }
      }
  }
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    if (!live[k]) continue;
#pragma unroll
    for (int i = 0; i < N; ++i) {
      if (a.op == O_MEAN && cnt[k]) acc[k][i] = __fdiv_rn(acc[k][i], (float)cnt[k]);
      if (cnt[k] == 0) acc[k][i] = 0.f;
    }
    Chunk<T>::store(out + (size_t)row[k] * a.C + ch[k] * N, acc[k]);
  }
}

// ------------------------------------------------------------------------------------------ pooling backward
template <typename T>
__global__ void __launch_bounds__(kPoolThreads) pool_reduce_bwd_kernel(const T *__restrict__ grad_red, const T *__restrict__ in,
                                                                       T *__restrict__ grad_in, GatherArgs a) {
  constexpr int N = Chunk<T>::N;
  uint64_t gid = (uint64_t)blockIdx.x * kPoolThreads + threadIdx.x;
  uint32_t row = (uint32_t)(gid / a.chunks_per_row), ch = (uint32_t)(gid % a.chunks_per_row);
  if (row >= a.ind_rows) return;
  uint32_t idx[kMaxS];
  uint32_t cnt = 0;
  for (uint32_t s = 0; s < a.S; ++s) {
    idx[s] = __ldg(a.unpool_ind + (size_t)row * a.S + s);
    cnt += idx[s] < a.valid_N ? 1u : 0u;
  }
  if (cnt == 0) return;
  float g[N];
  Chunk<T>::load(grad_red + (size_t)row * a.C + ch * N, g);
  if (a.op == O_SUM || a.op == O_MEAN) {
    if (a.op == O_MEAN) {
#pragma unroll
      for (int i = 0; i < N; ++i) g[i] = __fdiv_rn(g[i], (float)cnt);
    }
    for (uint32_t s = 0; s < a.S; ++s)
      if (idx[s] < a.valid_N) Chunk<T>::store(grad_in + (size_t)idx[s] * a.C + ch * N, g);
    return;
  }
  // min / max: the first strict winner in slot order takes the gradient, the other members get zero
  float best[N];
  uint32_t win[N];
#pragma unroll
  for (int i = 0; i < N; ++i) { best[i] = a.op == O_MIN ? INFINITY : -INFINITY; win[i] = 0; }
  for (uint32_t s = 0; s < a.S; ++s) {
    if (idx[s] >= a.valid_N) continue;
    float v[N];
    Chunk<T>::load(in + (size_t)idx[s] * a.C + ch * N, v);
#pragma unroll
    for (int i = 0; i < N; ++i) {
      bool w = a.op == O_MAX ? (v[i] > best[i]) : (v[i] < best[i]);
      if (w) { best[i] = v[i]; win[i] = s; }
    }
  }
  for (uint32_t s = 0; s < a.S; ++s) {
    if (idx[s] >= a.valid_N) continue;
    float o[N];
#pragma unroll
    for (int i = 0; i < N; ++i) o[i] = (win[i] == s) ? g[i] : 0.f;
    Chunk<T>::store(grad_in + (size_t)idx[s] * a.C + ch * N, o);
  }
}

// --------------------------------------------------------------------------------------------- unpool forward
// up[r] = res[r] + down[i] for r in unpool_ind[i,:]; rows of `up` in [covered_rows, up_rows) := 0
template <typename T>
__global__ void __launch_bounds__(kPoolThreads) unpool_add_kernel(const T *__restrict__ res, const T *__restrict__ down,
                                                                  T *__restrict__ up, GatherArgs a, uint32_t covered_rows,
                                                                  uint32_t up_rows, uint32_t gather_blocks) {
  constexpr int N = Chunk<T>::N;
  if (blockIdx.x >= gather_blocks) {
    uint64_t gid = (uint64_t)(blockIdx.x - gather_blocks) * kPoolThreads + threadIdx.x;
    uint64_t row = covered_rows + gid / a.chunks_per_row;
    uint32_t ch = (uint32_t)(gid % a.chunks_per_row);
    if (row < up_rows) {
      float z[N];
#pragma unroll
      for (int i = 0; i < N; ++i) z[i] = 0.f;
      Chunk<T>::store(up + row * a.C + ch * N, z);
    }
    return;
  }
  uint64_t gid = (uint64_t)blockIdx.x * kPoolThreads + threadIdx.x;
  uint32_t row = (uint32_t)(gid / a.chunks_per_row), ch = (uint32_t)(gid % a.chunks_per_row);
  if (row >= a.ind_rows) return;
  float d[N];
  Chunk<T>::load(down + (size_t)row * a.C + ch * N, d);
  for (uint32_t s = 0; s < a.S; ++s) {
    uint32_t r = __ldg(a.unpool_ind + (size_t)row * a.S + s);
    if (r < a.valid_N) {
      float v[N];
      Chunk<T>::load(res + (size_t)r * a.C + ch * N, v);
#pragma unroll
      for (int i = 0; i < N; ++i) v[i] = __fadd_rn(d[i], v[i]);
      Chunk<T>::store(up + (size_t)r * a.C + ch * N, v);
    }
  }
}

// -------------------------------------------------------------------------------------------- unpool backward
template <typename T>
__global__ void __launch_bounds__(kPoolThreads) unpool_add_bwd_kernel(T *__restrict__ grad_res, T *__restrict__ grad_down,
                                                                      const T *__restrict__ grad_up, GatherArgs a) {
  constexpr int N = Chunk<T>::N;
  uint64_t gid = (uint64_t)blockIdx.x * kPoolThreads + threadIdx.x;
  uint32_t row = (uint32_t)(gid / a.chunks_per_row), ch = (uint32_t)(gid % a.chunks_per_row);
  if (row >= a.ind_rows) return;
  float acc[N];
#pragma unroll
  for (int i = 0; i < N; ++i) acc[i] = 0.f;
  for (uint32_t s = 0; s < a.S; ++s) {
    uint32_t r = __ldg(a.unpool_ind + (size_t)row * a.S + s);
    if (r < a.valid_N) {
      float v[N];
      Chunk<T>::load(grad_up + (size_t)r * a.C + ch * N, v);
      Chunk<T>::store(grad_res + (size_t)r * a.C + ch * N, v);
#pragma unroll
      for (int i = 0; i < N; ++i) acc[i] = __fadd_rn(acc[i], v[i]);
    }
  }
  Chunk<T>::store(grad_down + (size_t)row * a.C + ch * N, acc);
}

// ------------------------------------------------------------------------------------------------------ host
static int esize(int dt) { return dt == F3D_FP32 ? 4 : 2; }

static int check_feat(uint32_t C, uint32_t S, int dt, const void *const *ptrs, int nptr) {
  if (dt < 0 || dt > 2) return set_error(F3D_ERR_ARG, "unsupported feature dtype code %d", dt);
  if (S == 0 || S > (uint32_t)kMaxS) return set_error(F3D_ERR_ARG, "subbuck_size=%u is outside [1,%d]", S, kMaxS);
  if (C == 0 || (C * esize(dt)) % 16 != 0)
    return set_error(F3D_ERR_ARG, "feature dim %u: a row must be a multiple of 16 bytes", C);
  for (int i = 0; i < nptr; ++i)
    if (reinterpret_cast<uintptr_t>(ptrs[i]) % 16 != 0) return set_error(F3D_ERR_ARG, "feature pointer %d is not 16-byte aligned", i);
  return F3D_OK;
}

static uint32_t blocks_for(uint64_t rows, uint32_t cpr) { return (uint32_t)((rows * cpr + kPoolThreads - 1) / kPoolThreads); }

#define F3D_DISPATCH_DT(dt, ...)                                        \
  do {                                                                  \
    if ((dt) == F3D_BF16) { using T = __nv_bfloat16; __VA_ARGS__; }     \
    else if ((dt) == F3D_FP16) { using T = __half; __VA_ARGS__; }       \
    else { using T = float; __VA_ARGS__; }                              \
  } while (0)

}  // namespace f3d

using namespace f3d;

extern "C" int f3d_batch_subbuck_reduce(
    const void *scattered_coord, const void *scattered_feat, const void *batch_sep, uint32_t total_N,
    uint32_t batch_size, uint32_t instance_max_N, uint32_t subbuck_size, uint32_t num_vox, const void *bbox_min,
    const void *bbox_max, void *subbuck_id, void *subbuck_off, const void *reduced_batch_sep, void *reduced_coord,
    void *reduced_feat, void *unpool_ind, uint32_t unpool_rows, uint32_t reduced_rows, uint32_t feat_dim,
    int feat_dtype, uint32_t hash_type, uint32_t red_op, int device, void *stream) {
  (void)bbox_min; (void)bbox_max;   // the sub-bucket hash normalises with the block bounding box (see subbuck.cu)
  const void *ptrs[2] = {scattered_feat, reduced_feat};
  F3D_TRY(check_feat(feat_dim, subbuck_size, feat_dtype, ptrs, 2));
  if (red_op > 3) return set_error(F3D_ERR_ARG, "Unsupported reduction operation id-%u", red_op);
  if (hash_type < 1 || hash_type > 4) return set_error(F3D_ERR_ARG, "Unsupported hash_type=%u", hash_type);
  if (reduced_rows < unpool_rows)
    return set_error(F3D_ERR_ARG, "Reduced feature length(%u) is smaller than unpool_ind length(%u).", reduced_rows, unpool_rows);
  if (batch_size == 0) return set_error(F3D_ERR_ARG, "batch_sep is empty");
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  F3D_TRY(maybe_sync(st, "batch_subbuck_reduce"));
  if (instance_max_N > total_N) instance_max_N = total_N;
  F3D_TRY(subbuck_build(scattered_coord, batch_sep, reduced_batch_sep, subbuck_id, subbuck_off, unpool_ind, reduced_coord,
                        total_N, batch_size, instance_max_N, subbuck_size, num_vox, hash_type, unpool_rows, reduced_rows, st));
  GatherArgs a{static_cast<const uint32_t *>(unpool_ind), unpool_rows, reduced_rows, total_N, feat_dim, subbuck_size, red_op,
               feat_dim * (uint32_t)esize(feat_dtype) / 16};
  if (reduced_rows > 0) {
    F3D_DISPATCH_DT(feat_dtype, pool_reduce_kernel<T><<<(blocks_for(reduced_rows, a.chunks_per_row) + 1) / 2, kPoolThreads, 0, st>>>(
        static_cast<const T *>(scattered_feat), static_cast<T *>(reduced_feat), a));
  }
  F3D_TRY(check_launch("batch_subbuck_reduce"));
  return maybe_sync(st, "batch_subbuck_reduce");
}

extern "C" int f3d_batch_subbuck_reduce_backward(
    const void *grad_red_feat, const void *input_feat, const void *unpool_ind, void *grad_input_feat, uint32_t total_N,
    uint32_t unpool_rows, uint32_t feat_dim, int feat_dtype, uint32_t subbuck_size, uint32_t red_op, int device,
    void *stream) {
  const void *ptrs[3] = {grad_red_feat, input_feat, grad_input_feat};
  F3D_TRY(check_feat(feat_dim, subbuck_size, feat_dtype, ptrs, 3));
  if (red_op > 3) return set_error(F3D_ERR_ARG, "Unsupported reduction_op=%u", red_op);
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  F3D_TRY(maybe_sync(st, "batch_subbuck_reduce_backward"));
  GatherArgs a{static_cast<const uint32_t *>(unpool_ind), unpool_rows, unpool_rows, total_N, feat_dim, subbuck_size, red_op,
               feat_dim * (uint32_t)esize(feat_dtype) / 16};
  if (unpool_rows > 0) {
    F3D_DISPATCH_DT(feat_dtype, pool_reduce_bwd_kernel<T><<<blocks_for(unpool_rows, a.chunks_per_row), kPoolThreads, 0, st>>>(
        static_cast<const T *>(grad_red_feat), static_cast<const T *>(input_feat), static_cast<T *>(grad_input_feat), a));
  }
  F3D_TRY(check_launch("batch_subbuck_reduce_backward"));
  return maybe_sync(st, "batch_subbuck_reduce_backward");
}

extern "C" int f3d_additive_unpool_fwd(
    const void *res_feat, const void *down_feat, void *up_add_feat, const void *unpool_ind, uint32_t up_rows,
    uint32_t unpool_rows, uint32_t covered_rows, uint32_t feat_dim, int feat_dtype, uint32_t subbuck_size, int device,
    void *stream) {
  const void *ptrs[3] = {res_feat, down_feat, up_add_feat};
  F3D_TRY(check_feat(feat_dim, subbuck_size, feat_dtype, ptrs, 3));
  if (covered_rows > up_rows) covered_rows = up_rows;
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  F3D_TRY(maybe_sync(st, "additive_unpool_fwd"));
  GatherArgs a{static_cast<const uint32_t *>(unpool_ind), unpool_rows, unpool_rows, up_rows, feat_dim, subbuck_size, 0,
               feat_dim * (uint32_t)esize(feat_dtype) / 16};
  uint32_t gb = blocks_for(unpool_rows, a.chunks_per_row);
  uint32_t zb = blocks_for(up_rows - covered_rows, a.chunks_per_row);
  if (gb + zb > 0) {
    F3D_DISPATCH_DT(feat_dtype, unpool_add_kernel<T><<<gb + zb, kPoolThreads, 0, st>>>(
        static_cast<const T *>(res_feat), static_cast<const T *>(down_feat), static_cast<T *>(up_add_feat), a, covered_rows,
        up_rows, gb));
  }
  F3D_TRY(check_launch("additive_unpool_fwd"));
  return maybe_sync(st, "additive_unpool_fwd");
}

extern "C" int f3d_additive_unpool_bwd(
    void *grad_res, void *grad_down, const void *grad_up_added, const void *unpool_ind, uint32_t up_rows,
    uint32_t unpool_rows, uint32_t feat_dim, int feat_dtype, uint32_t subbuck_size, int device, void *stream) {
  const void *ptrs[3] = {grad_res, grad_down, grad_up_added};
  F3D_TRY(check_feat(feat_dim, subbuck_size, feat_dtype, ptrs, 3));
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  F3D_TRY(maybe_sync(st, "additive_unpool_bwd"));
  GatherArgs a{static_cast<const uint32_t *>(unpool_ind), unpool_rows, unpool_rows, up_rows, feat_dim, subbuck_size, 0,
               feat_dim * (uint32_t)esize(feat_dtype) / 16};
  if (unpool_rows > 0) {
    F3D_DISPATCH_DT(feat_dtype, unpool_add_bwd_kernel<T><<<blocks_for(unpool_rows, a.chunks_per_row), kPoolThreads, 0, st>>>(
        static_cast<T *>(grad_res), static_cast<T *>(grad_down), static_cast<const T *>(grad_up_added), a));
  }
  F3D_TRY(check_launch("additive_unpool_bwd"));
  return maybe_sync(st, "additive_unpool_bwd");
}
