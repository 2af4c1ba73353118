// Host-side construction of TMA tensor maps.  cuTensorMapEncodeTiled is looked up through
// cudaGetDriverEntryPoint so that the library carries no link-time dependency on the driver library.
#include "f3d_common.cuh"
#include "tc_sm100.cuh"
#include <cudaTypedefs.h>
#include <mutex>

namespace f3d {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

static CUtensorMapDataType dt_of(int code) {
  return code == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : (code == 1 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
}
static CUtensorMapSwizzle sw_of(int bytes) {
  switch (bytes) {
    case 128: return CU_TENSOR_MAP_SWIZZLE_128B;
    case 64: return CU_TENSOR_MAP_SWIZZLE_64B;
    case 32: return CU_TENSOR_MAP_SWIZZLE_32B;
    default: return CU_TENSOR_MAP_SWIZZLE_NONE;
  }
}

int encode_tmap_2d(CUtensorMap *map, int dtype_code, const void *base, uint64_t inner, uint64_t outer,
                   uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return set_error(F3D_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0) return set_error(F3D_ERR_ARG, "TMA base pointer is not 16-byte aligned");
  if (row_stride_bytes % 16 != 0) return set_error(F3D_ERR_ARG, "TMA row stride (%llu bytes) is not a multiple of 16", (unsigned long long)row_stride_bytes);
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt_of(dtype_code), 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  sw_of(swizzle_bytes), CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(F3D_ERR_CUDA, "cuTensorMapEncodeTiled(2d) failed with code %d", (int)r);
  return F3D_OK;
}

int encode_tmap_3d(CUtensorMap *map, int dtype_code, const void *base, uint64_t d0, uint64_t d1, uint64_t d2,
                   uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1, uint32_t b2, int swizzle_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return set_error(F3D_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0) return set_error(F3D_ERR_ARG, "TMA base pointer is not 16-byte aligned");
  if (stride1_bytes % 16 != 0 || stride2_bytes % 16 != 0) return set_error(F3D_ERR_ARG, "TMA strides must be multiples of 16 bytes");
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, dt_of(dtype_code), 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  sw_of(swizzle_bytes), CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(F3D_ERR_CUDA, "cuTensorMapEncodeTiled(3d) failed with code %d", (int)r);
  return F3D_OK;
}

}  // namespace f3d
