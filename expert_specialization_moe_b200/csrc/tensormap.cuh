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

// A tensor map is a pure function of (base, extents, box): the encodings are kept in a small per-thread cache so that a
// call on operands seen before (weights never move; activation buffers of a serving loop are reused) costs a lookup
// instead of a driver call per map.
struct MapCacheEntry {
  const void* base;
  uint64_t rows, row_bytes;
  uint32_t box_rows, kind;      // kind 0: byte matrix with 128-byte swizzle, 1: 512-byte records, 2: columns of such records
  bool valid;
  CUtensorMap map;
};
constexpr int MAP_CACHE_SLOTS = 128;
inline MapCacheEntry* map_cache_slot(const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows,
                                     uint32_t kind) {
  static thread_local MapCacheEntry cache[MAP_CACHE_SLOTS] = {};
  uint64_t h = reinterpret_cast<uintptr_t>(base) * 0x9E3779B97F4A7C15ull;
  h ^= (rows + 0x7F4A7C15ull) * 0xC2B2AE3D27D4EB4Full;
  h ^= (row_bytes * 31 + box_rows * 7 + kind) * 0x165667B19E3779F9ull;
  return &cache[(h >> 40) % MAP_CACHE_SLOTS];
}
inline bool map_cache_hit(const MapCacheEntry* e, const void* base, uint64_t rows, uint64_t row_bytes,
                          uint32_t box_rows, uint32_t kind) {
  return e->valid && e->base == base && e->rows == rows && e->row_bytes == row_bytes && e->box_rows == box_rows &&
         e->kind == kind;
}

// Row-major byte matrix [rows, row_bytes] (row_bytes % 16 == 0, base 16-byte aligned); box = box_rows x 128 bytes,
// 128-byte swizzle, out-of-range elements read as zero.
inline int make_tensormap_u8_sw128(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                                   uint32_t box_rows) {
  MapCacheEntry* slot = map_cache_slot(base, rows, row_bytes, box_rows, 0);
  if (map_cache_hit(slot, base, rows, row_bytes, box_rows, 0)) {
    *map = slot->map;
    return ES_B200_OK;
  }
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
  *slot = MapCacheEntry{base, rows, row_bytes, box_rows, 0, true, *map};
  return ES_B200_OK;
}

// Array of 512-byte records (the swizzled scale-factor atoms) viewed as [count, 128] uint32; box = one record,
// no swizzle: a load places the 512 bytes contiguously in shared memory.
inline int make_tensormap_records512(CUtensorMap* map, const void* base, uint64_t count) {
  MapCacheEntry* slot = map_cache_slot(base, count, 512, 1, 1);
  if (map_cache_hit(slot, base, count, 512, 1, 1)) {
    *map = slot->map;
    return ES_B200_OK;
  }
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
  *slot = MapCacheEntry{base, count, 512, 1, 1, true, *map};
  return ES_B200_OK;
}

// The same records viewed as [rows, per_row x 128] uint32 — record (r, j) at index r * per_row + j — with a box of one
// record in j and `box_rows` rows: ONE load fetches the records (r .. r + box_rows - 1, j), 512 bytes each,
// contiguous in shared memory (rows past the end read as zero).
inline int make_tensormap_record_columns(CUtensorMap* map, const void* base, uint64_t rows, uint64_t per_row,
                                         uint32_t box_rows) {
  MapCacheEntry* slot = map_cache_slot(base, rows, 512 * per_row, box_rows, 2);
  if (map_cache_hit(slot, base, rows, 512 * per_row, box_rows, 2)) {
    *map = slot->map;
    return ES_B200_OK;
  }
  EncodeTiledFn fn;
  int rc = get_encode_fn(&fn);
  if (rc != ES_B200_OK) return rc;
  cuuint64_t dims[2] = {128 * per_row, rows};
  cuuint64_t strides[1] = {512 * per_row};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(ES_B200_ERR_CUDA, "cuTensorMapEncodeTiled (record columns) failed with CUresult %d", (int)r);
  *slot = MapCacheEntry{base, rows, 512 * per_row, box_rows, 2, true, *map};
  return ES_B200_OK;
}

}  // namespace es_b200
