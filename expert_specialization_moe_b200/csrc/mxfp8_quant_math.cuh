// MXFP8 quantisation arithmetic shared by the grouped quant kernel and the expert-parallel dispatch kernel.
//
// Arithmetic contract (bit-exact with the reference kernel, es_sm100_mxfp8_blockscaled_group_quant.cuh:36-134):
//   amax  = max |x_i| over the 32-block, NaN members dropped (max.bf16x2 / max.f16x2 semantics)
//   s     = fp32(amax) * rcp.approx.ftz.f32(448.0f)
//   sf    = cvt.rp.satfinite.ue8m0x2.f32(s)
//   inv   = amax != 0 ? rcp.approx.ftz.f32(float(sf)) : 0
//   code  = cvt.rn.satfinite.e4m3x2.f32(fp32(x_i) * inv)
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace es_b200 {

__device__ __forceinline__ float rcp_approx_ftz(float a) {
  float b;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(b) : "f"(a));   // pure: may be hoisted / scheduled freely
  return b;
}

__device__ __forceinline__ uint4 ld_stream_16B(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void st_stream_8B(void* p, uint2 v) {
  asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

template <typename T>
struct Vec2;
template <>
struct Vec2<__nv_bfloat16> {
  using type = __nv_bfloat162;
  static __device__ __forceinline__ float2 to_float2(type v) { return __bfloat1622float2(v); }
  static __device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ type from_floats(float a, float b) { return __floats2bfloat162_rn(a, b); }
};
template <>
struct Vec2<__half> {
  using type = __half2;
  static __device__ __forceinline__ float2 to_float2(type v) { return __half22float2(v); }
  static __device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
  static __device__ __forceinline__ type from_floats(float a, float b) { return __floats2half2_rn(a, b); }
};

// Quantise the 8 elements this lane holds; the four lanes of a quad share one 32-element block.
// Returns the block's UE8M0 byte (same value in all four lanes); writes the 8 codes to `codes`.
template <typename T>
__device__ __forceinline__ uint32_t quantize8(const uint4& raw, uint2& codes) {
  using V2 = typename Vec2<T>::type;
  V2 v[4];
  v[0] = *reinterpret_cast<const V2*>(&raw.x);
  v[1] = *reinterpret_cast<const V2*>(&raw.y);
  v[2] = *reinterpret_cast<const V2*>(&raw.z);
  v[3] = *reinterpret_cast<const V2*>(&raw.w);
  V2 mx = __hmax2(__hmax2(__habs2(v[0]), __habs2(v[1])), __hmax2(__habs2(v[2]), __habs2(v[3])));
  {
    uint32_t bits = *reinterpret_cast<uint32_t*>(&mx);
    uint32_t o = __shfl_xor_sync(0xffffffffu, bits, 1);
    mx = __hmax2(mx, *reinterpret_cast<V2*>(&o));
    bits = *reinterpret_cast<uint32_t*>(&mx);
    o = __shfl_xor_sync(0xffffffffu, bits, 2);
    mx = __hmax2(mx, *reinterpret_cast<V2*>(&o));
  }
  const float block_max = Vec2<T>::to_float(__hmax(mx.x, mx.y));
  float sf_val = block_max * rcp_approx_ftz(448.0f);
  __nv_fp8_e8m0 sf;
  sf.__x = __nv_cvt_float_to_e8m0(sf_val, __NV_SATFINITE, cudaRoundPosInf);
  sf_val = static_cast<float>(sf);
  const float inv = block_max != 0.f ? rcp_approx_ftz(sf_val) : 0.0f;

  uint32_t out[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    float2 lo = Vec2<T>::to_float2(v[2 * i]);
    float2 hi = Vec2<T>::to_float2(v[2 * i + 1]);
    lo.x *= inv; lo.y *= inv; hi.x *= inv; hi.y *= inv;
    uint32_t p0 = __nv_cvt_float2_to_fp8x2(lo, __NV_SATFINITE, __NV_E4M3);
    uint32_t p1 = __nv_cvt_float2_to_fp8x2(hi, __NV_SATFINITE, __NV_E4M3);
    out[i] = p0 | (p1 << 16);
  }
  codes.x = out[0];
  codes.y = out[1];
  return sf.__x;
}

// Byte offset, inside one operand's swizzled scale buffer, of the 32-bit scale word of (row r, K tile 0): 512-byte
// atoms of 128 rows x 4 K blocks, atoms K-fastest (kt = K / 128 atoms per 128 rows); the word of K tile q is q * 512
// further on.
__device__ __host__ __forceinline__ int64_t scale_word_offset(int r, int kt) {
  return (int64_t)(r >> 7) * kt * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4;
}

}  // namespace es_b200
