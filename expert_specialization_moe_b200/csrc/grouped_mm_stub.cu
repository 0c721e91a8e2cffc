// temporary stubs
#include "common.cuh"
extern "C" size_t es_b200_grouped_mm_scratch_bytes(int, int64_t, int, int) { return 256; }
extern "C" int es_b200_mxfp8_grouped_mm(const void*, const void*, const uint8_t*, const uint8_t*, void*, int, const int32_t*, const int32_t*, const int32_t*, int, int64_t, int, int, int64_t, void*, size_t, void*) { return es_b200::fail(ES_B200_ERR_UNSUPPORTED_DEVICE, "not built yet"); }
extern "C" int es_b200_fp8_blockwise_grouped_mm(const void*, const void*, const float*, const float*, void*, int, const int32_t*, const int32_t*, int, int64_t, int, int, void*, size_t, void*) { return es_b200::fail(ES_B200_ERR_UNSUPPORTED_DEVICE, "not built yet"); }
extern "C" int es_b200_check_status(const void*, void*, uint32_t*) { return 0; }
