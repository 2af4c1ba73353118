// Host build of the REFERENCE's own first-level hash arithmetic, for pinning oracle/psh_oracle.py.
// TEST INFRASTRUCTURE ONLY.  This file holds no hash code: it includes the reference's headers from the reference
// checkout at build time (src/common/arithmetic.cuh for clamp, src/psh/hash_fns.cuh:23-33,48-68,79-86,113-135 for
// vox_coord, h1_xorsum_{div,mod}, space_out_bit_3d, h1_zorder_{div,mod}_3d) with the CUDA qualifiers defined away, and
// exports one C function that runs their register overloads over an array of points.
//
// Two things differ from the reference's device build and are stated here because they bound what this pin proves:
//  * `min` / `max` on floats: device code resolves them to the PTX min.f32 / max.f32, which return the other operand
//    when one is NaN; fminf / fmaxf below have the same rule, so clamp() treats a NaN voxel (degenerate bounding box,
//    0/0) like the device does;
//  * the reference compiles with --use_fast_math (CMakeLists.txt:50), which replaces the IEEE division of vox_coord by
//    an approximate one; this host build divides exactly, so a point that sits within an ulp of a voxel boundary can
//    land in the neighbouring voxel in a reference GPU binary.
#include <math.h>
#include <stdint.h>

#define __device__
#define __forceinline__ inline
static inline float max(float a, float b) { return fmaxf(a, b); }
static inline float min(float a, float b) { return fminf(a, b); }

#include "common/arithmetic.cuh"
#include "psh/hash_fns.cuh"

extern "C" {

// coord: n x 3 floats holding fp16 values (float(half) is exact); bbox_min / bbox_max: 3 floats each.
// vox_out: n x 3 u16; hash_out: 4 x n u16 in the order of the reference's HASHTYPE enum (1 Z-order div, 2 XOR-sum div,
// 3 Z-order mod, 4 XOR-sum mod).
void f3d_ref_vox_hash(const float *coord, const float *bbox_min, const float *bbox_max, uint32_t num_vox, uint64_t n,
                      uint16_t divisor, uint16_t num_bucket, uint16_t *vox_out, uint16_t *hash_out) {
  float lo[3] = {bbox_min[0], bbox_min[1], bbox_min[2]};
  float hi[3] = {bbox_max[0], bbox_max[1], bbox_max[2]};
  for (uint64_t i = 0; i < n; ++i) {
    float c[3] = {coord[3 * i], coord[3 * i + 1], coord[3 * i + 2]};
    uint16_t v[3];
    f3d::vox_coord<float, uint16_t, 3>(c, v, lo, hi, num_vox);
    vox_out[3 * i] = v[0]; vox_out[3 * i + 1] = v[1]; vox_out[3 * i + 2] = v[2];
    uint16_t h;
    f3d::h1_zorder_div_3d<uint16_t>(v, h, divisor);      hash_out[0 * n + i] = h;
    f3d::h1_xorsum_div<uint16_t, 3>(v, h, divisor);       hash_out[1 * n + i] = h;
    f3d::h1_zorder_mod_3d<uint16_t>(v, h, num_bucket);    hash_out[2 * n + i] = h;
    f3d::h1_xorsum_mod<uint16_t, 3>(v, h, num_bucket);    hash_out[3 * n + i] = h;
  }
}

// The hashes of given voxel triples (n x 3 u16), so that every bit pattern can be fed without going through floats.
void f3d_ref_hash_of_vox(const uint16_t *vox, uint64_t n, uint16_t divisor, uint16_t num_bucket, uint16_t *hash_out) {
  for (uint64_t i = 0; i < n; ++i) {
    uint16_t v[3] = {vox[3 * i], vox[3 * i + 1], vox[3 * i + 2]};
    uint16_t h;
    f3d::h1_zorder_div_3d<uint16_t>(v, h, divisor);      hash_out[0 * n + i] = h;
    f3d::h1_xorsum_div<uint16_t, 3>(v, h, divisor);       hash_out[1 * n + i] = h;
    f3d::h1_zorder_mod_3d<uint16_t>(v, h, num_bucket);    hash_out[2 * n + i] = h;
    f3d::h1_xorsum_mod<uint16_t, 3>(v, h, num_bucket);    hash_out[3 * n + i] = h;
  }
}

}  // extern "C"
