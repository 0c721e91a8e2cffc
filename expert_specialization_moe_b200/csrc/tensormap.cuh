// Host-side construction of TMA tensor maps (cuTensorMapEncodeTiled fetched through the runtime's driver entry
// point lookup, so the library links against cudart only).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace es_b200 {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline int get_encode_fn(EncodeTiledFn* out) {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    ES_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    if (q != cudaDriverEntryPointSuccess || !p)
      return fail(ES_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the installed driver");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  *out = fn;
  return ES_B200_OK;
}

// Row-major byte matrix [rows, row_bytes] (row_bytes % 16 == 0, base 16-byte aligned); box = box_rows x 128 bytes,
// 128-byte swizzle, out-of-range elements read as zero.
inline int make_tensormap_u8_sw128(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                                   uint32_t box_rows) {
  EncodeTiledFn fn;
  int rc = get_encode_fn(&fn);
  if (rc != ES_B200_OK) return rc;
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(ES_B200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return ES_B200_OK;
}

// Array of 512-byte records (the swizzled scale-factor atoms) viewed as [count, 128] uint32; box = one record,
// no swizzle: a load places the 512 bytes contiguously in shared memory.
inline int make_tensormap_records512(CUtensorMap* map, const void* base, uint64_t count) {
  EncodeTiledFn fn;
  int rc = get_encode_fn(&fn);
  if (rc != ES_B200_OK) return rc;
  cuuint64_t dims[2] = {128, count};
  cuuint64_t strides[1] = {512};
  cuuint32_t box[2] = {128, 1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(ES_B200_ERR_CUDA, "cuTensorMapEncodeTiled (records) failed with CUresult %d", (int)r);
  return ES_B200_OK;
}

}  // namespace es_b200
