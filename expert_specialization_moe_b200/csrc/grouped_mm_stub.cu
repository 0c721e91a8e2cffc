// temporary stub
#include "common.cuh"
extern "C" int es_b200_fp8_blockwise_grouped_mm(const void*, const void*, const float*, const float*, void*, int, const int32_t*, const int32_t*, int, int64_t, int, int, void*, size_t, void*) { return es_b200::fail(ES_B200_ERR_UNSUPPORTED_DEVICE, "not built yet"); }
