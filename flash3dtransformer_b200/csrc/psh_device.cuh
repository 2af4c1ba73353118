// Device-side arithmetic of the perfect-spatial-hash (PSH) path: voxelisation, the four first-level hashes,
// the counter-based random generator and the probe perturbation.  Every function here has a line-for-line
// numpy twin in oracle/psh_oracle.py; GPU and oracle must agree bit for bit.
//
// Reference semantics restated here:
//   voxel coordinate          src/psh/hash_fns.cuh:23-33   (fp32, evaluated left to right, clamp to [0, num_vox-1])
//   Z-order hash              src/psh/hash_fns.cuh:79-86,113-135  (48-bit Morton code >> 31, truncated to 16 bits)
//   XOR-sum hash              src/psh/hash_fns.cuh:48-68
//   probe perturbation        src/common/rand.cuh:95-115
// The reference draws from cuRAND states of which only one is initialised (src/common/rand.cuh:122-143);
// here the randomness is Philox4x32-10 keyed by (seed, scene, point, probe), so results are reproducible.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace f3d {

enum HashType : uint32_t { H_ZORDER_DIV = 1, H_XORSUM_DIV = 2, H_ZORDER_MOD = 3, H_XORSUM_MOD = 4 };

constexpr uint32_t kNumProbes = 128;       // rows of the probe table (src/psh/batch_psh_bucket.cuh:39)
constexpr uint32_t kRecycleBucket = 0;     // src/psh/bucket_dispatcher.cuh:83-86
constexpr uint32_t kPending = 0xFFFFFFFFu; // bucket_offset marker for a point whose slot is not final yet

// IEEE fp32 with explicit rounding: no fast-math, no FMA contraction, so numpy float32 reproduces it.
__device__ __forceinline__ uint32_t vox_axis(float c, float lo, float hi, uint32_t num_vox) {
  float t = __fdiv_rn(__fmul_rn(__fsub_rn(c, lo), (float)num_vox), __fsub_rn(hi, lo));
  // clamp(x, 0, top) = max(0, min(x, top)) (src/common/arithmetic.cuh:26-29) with the device rule of min / max: a NaN
  // operand is dropped.  On an axis where every point has the same coordinate the quotient is 0/0 = NaN, min(NaN, top)
  // is top, and the voxel index is num_vox - 1, as in the reference.
  float top = (float)(num_vox - 1u);
  return (uint32_t)fmaxf(0.f, fminf(floorf(t), top));
}

// The same voxel index for many points of one axis: the divisor hi - lo is a constant, so its correctly rounded
// reciprocal is taken once and every quotient costs five FMA-pipe instructions instead of a division.  a * r is
// within two units in the last place of a / d; one residual correction q + (a - q d) r makes it faithful, and the
// second one rounds it correctly (the classical residual-correction division: the residual is exact under FMA and
// r is the correctly rounded reciprocal), so the result has the bits of __fdiv_rn.  A zero divisor (flat axis) takes
// the division itself.
struct AxisScale { float lo, d, r, nv, top; };

__device__ __forceinline__ AxisScale make_axis_scale(float lo, float hi, uint32_t num_vox) {
  AxisScale s;
  s.lo = lo; s.d = __fsub_rn(hi, lo); s.r = __frcp_rn(s.d); s.nv = (float)num_vox; s.top = (float)(num_vox - 1u);
  return s;
}

__device__ __forceinline__ uint32_t vox_axis(float c, const AxisScale &s) {
  const float a = __fmul_rn(__fsub_rn(c, s.lo), s.nv);
  float q;
  if (s.d != 0.f) {
    q = __fmul_rn(a, s.r);
    q = __fmaf_rn(__fmaf_rn(-q, s.d, a), s.r, q);
    q = __fmaf_rn(__fmaf_rn(-q, s.d, a), s.r, q);
  } else {
    q = __fdiv_rn(a, s.d);
  }
  return (uint32_t)fmaxf(0.f, fminf(floorf(q), s.top));
}

// x < 1024: bit i moves to bit 3i
__device__ __forceinline__ uint32_t spread3(uint32_t x) {
  x = (x | (x << 16)) & 0x030000FFu;
  x = (x | (x << 8)) & 0x0300F00Fu;
  x = (x | (x << 4)) & 0x030C30C3u;
  x = (x | (x << 2)) & 0x09249249u;
  return x;
}

// Bits 31..46 of the 48-bit Morton code of three 16-bit voxel indices (x in bit 3i, y in 3i+1, z in 3i+2).
// Only x[11..15], y[10..15], z[10..14] reach the result, which is what the reference's ">> 31" followed by
// the store into a 16-bit register keeps (src/psh/hash_fns.cuh:120).
__device__ __forceinline__ uint32_t zorder16(uint32_t vx, uint32_t vy, uint32_t vz) {
  uint32_t ax = vx >> 11, ay = vy >> 10, az = (vz >> 10) & 31u;
  return ((ay & 1u) | (spread3(az) << 1) | (spread3(ax) << 2) | (spread3(ay >> 1) << 3)) & 0xFFFFu;
}

__device__ __forceinline__ uint32_t first_hash(uint32_t hash_type, uint32_t vx, uint32_t vy, uint32_t vz,
                                               uint32_t divisor, uint32_t num_bucket) {
  uint32_t h;
  switch (hash_type) {
    case H_ZORDER_DIV: h = zorder16(vx, vy, vz) / divisor; break;
    case H_XORSUM_DIV: h = ((vx ^ vy ^ vz) & 0xFFFFu) / divisor; break;
    case H_ZORDER_MOD: h = zorder16(vx, vy, vz) % num_bucket; break;
    default:           h = ((vx ^ vy ^ vz) & 0xFFFFu) % num_bucket; break;
  }
  return h < num_bucket ? h : num_bucket - 1u;   // guard for divisors that do not cover the range
}

// The same hash with the division / remainder turned into a shift / mask when the divisor (div hashes) or the bucket
// count (mod hashes) is a power of two, which is what the host's plan always produces (num_bucket is rounded to a
// power of two and the divisor is ceil(65535 / num_bucket)).  `shift` < 0 selects the general path.
struct HashPlan { uint32_t hash_type, divisor, num_bucket; int shift; };

__device__ __forceinline__ HashPlan make_hash_plan(uint32_t hash_type, uint32_t divisor, uint32_t num_bucket) {
  HashPlan p{hash_type, divisor, num_bucket, -1};
  const uint32_t v = (hash_type == H_ZORDER_DIV || hash_type == H_XORSUM_DIV) ? divisor : num_bucket;
  if (v && (v & (v - 1u)) == 0u) p.shift = 31 - __clz(v);
  return p;
}

__device__ __forceinline__ uint32_t first_hash(const HashPlan &p, uint32_t vx, uint32_t vy, uint32_t vz) {
  if (p.shift < 0) return first_hash(p.hash_type, vx, vy, vz, p.divisor, p.num_bucket);
  const bool zorder = p.hash_type == H_ZORDER_DIV || p.hash_type == H_ZORDER_MOD;
  const uint32_t code = zorder ? zorder16(vx, vy, vz) : ((vx ^ vy ^ vz) & 0xFFFFu);
  const bool div = p.hash_type == H_ZORDER_DIV || p.hash_type == H_XORSUM_DIV;
  const uint32_t h = div ? (code >> p.shift) : (code & (p.num_bucket - 1u));
  return h < p.num_bucket ? h : p.num_bucket - 1u;
}

// Philox4x32-10 (Salmon et al., SC'11): counter (c0..c3), key (k0,k1) -> four 32-bit words.
__device__ __forceinline__ void philox4x32(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                           uint32_t k0, uint32_t k1, uint32_t (&out)[4]) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

struct RngKey { uint32_t k0, k1; };

// Random words for (scene, point-in-scene, tag): tags 128..130 are the draws of the recycle redistribution, tag 200
// seeds the probe walk of the rebalance.
__device__ __forceinline__ void psh_rand(RngKey key, uint32_t scene, uint32_t point, uint32_t tag, uint32_t (&out)[4]) {
  philox4x32(point, scene, tag, 0u, key.k0, key.k1, out);
}

// Random words of the 128-probe walk of one point.  One Philox call (tag 200) seeds four linear congruential
// streams; every probe advances each stream once (s <- s * 1664525 + 1013904223) and uses s ^ (s >> 15).  The walk
// needs four draws per probe for up to 128 probes per overflowing point; a full Philox call per probe made the
// walk the most expensive part of the whole bucketing.
struct ProbeStream { uint32_t s[4]; };

__device__ __forceinline__ void probe_stream_init(RngKey key, uint32_t scene, uint32_t point, ProbeStream &st) {
  psh_rand(key, scene, point, 200u, st.s);
}

__device__ __forceinline__ void probe_stream_next(ProbeStream &st, uint32_t (&r)[4]) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    st.s[k] = st.s[k] * 1664525u + 1013904223u;
    r[k] = st.s[k] ^ (st.s[k] >> 15);
  }
}

// Shifted voxel for one probe: segment length = round(U(2.56,5.12) * num_vox / divisor), the voxel moves by
// probe[d] segments plus a uniform jitter of +-half a segment, and wraps by |v| mod num_vox
// (src/common/rand.cuh:95-115).  `ratio` = fp32(num_vox) / fp32(divisor), computed once by the caller; the jitter
// maps a 32-bit draw to [0, span) with a multiply-high instead of a division.
__device__ __forceinline__ void perturb_vox(const uint32_t (&r)[4], uint32_t num_vox, float ratio,
                                            const int16_t *__restrict__ probe_row, const uint32_t (&vox)[3],
                                            uint32_t (&nvox)[3]) {
  float u = (float)(r[0] >> 8) * (1.0f / 16777216.0f);
  float scaling = __fadd_rn(2.56f, __fmul_rn(u, 2.56f));
  int32_t seg = (int32_t)floorf(__fadd_rn(__fmul_rn(scaling, ratio), 0.5f));
  int32_t half_seg = seg / 2;
  uint32_t span = (uint32_t)(2 * half_seg + 1);
#pragma unroll
  for (int d = 0; d < 3; ++d) {
    int32_t jitter = (int32_t)__umulhi(r[1 + d], span) - half_seg;
    int32_t shifted = (int32_t)vox[d] + (int32_t)probe_row[d] * seg + jitter;
    uint32_t mag = (uint32_t)(shifted < 0 ? -shifted : shifted);
    if (mag >= num_vox) mag %= num_vox;
    nvox[d] = mag;
  }
}

__device__ __forceinline__ float probe_ratio(uint32_t num_vox, uint32_t divisor) { return __fdiv_rn((float)num_vox, (float)divisor); }

}  // namespace f3d
