// MXFP8 grouped quantisation for sm_100a: bf16/fp16 rows -> e4m3 codes + UE8M0 scale per 32 elements, scales
// written straight into the SM100 swizzled layout (512-byte atoms of 128 rows x 4 K-blocks) at per-expert offsets.
//
// Arithmetic contract (bit-exact with the reference kernel, es_sm100_mxfp8_blockscaled_group_quant.cuh:36-134):
//   amax  = max |x_i| over the 32-block, NaN members dropped (max.bf16x2 / max.f16x2 semantics)
//   s     = fp32(amax) * rcp.approx.ftz.f32(448.0f)
//   sf    = cvt.rp.satfinite.ue8m0x2.f32(s)
//   inv   = amax != 0 ? rcp.approx.ftz.f32(float(sf)) : 0
//   code  = cvt.rn.satfinite.e4m3x2.f32(fp32(x_i) * inv)
//
// Schedule: the reference walks the experts one after another and strides its CTAs over one expert's 128x128
// tiles at a time.  Here all experts form one flat list of 8-row chunks (one row per warp, whole K per row), found
// with a per-CTA prefix scan over the experts' row counts, so every CTA streams long contiguous rows with 128-bit
// loads regardless of how the rows are split between experts.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "common.cuh"
#include "mxfp8_quant_math.cuh"

namespace es_b200 {

constexpr int QUANT_THREADS = 256;
constexpr int QUANT_ROWS_PER_CHUNK = QUANT_THREADS / 32;   // one row per warp
constexpr int QUANT_UNROLL = 4;                             // 16-byte loads in flight per lane
// the fused SiLU variant is bound by its arithmetic (exact expf and division): one load per lane in flight keeps the
// register count low and every lane busy when k is not a multiple of 1024 (k = 768: 0.23 -> 0.16 ms for 131072 rows)
constexpr int QUANT_UNROLL_SILU = 1;

// act = round_to_T( silu(gate) * up ) on 8 elements, computed in fp32: x / (1 + exp(-x)) with the accurate expf, one
// IEEE multiply, round to nearest even — the arithmetic of an unfused silu(gate.float()) * up.float() -> T.
template <typename T>
__device__ __forceinline__ uint4 silu_mul8(const uint4& g, const uint4& u) {
  using V2 = typename Vec2<T>::type;
  const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
  uint32_t out[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 gf = Vec2<T>::to_float2(*reinterpret_cast<const V2*>(&gw[i]));
    const float2 uf = Vec2<T>::to_float2(*reinterpret_cast<const V2*>(&uw[i]));
    const float a0 = (gf.x / (1.0f + expf(-gf.x))) * uf.x;
    const float a1 = (gf.y / (1.0f + expf(-gf.y))) * uf.y;
    const V2 r = Vec2<T>::from_floats(a0, a1);
    out[i] = *reinterpret_cast<const uint32_t*>(&r);
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}

// kSiluMul = false: input [rows, k].  kSiluMul = true: input [rows, 2k] = gate | up, quantises silu(gate) * up.
template <typename T, bool kSiluMul>
__global__ void __launch_bounds__(QUANT_THREADS)
mxfp8_group_quant_kernel(const T* __restrict__ input, const int* __restrict__ problem_sizes,
                         const int* __restrict__ expert_offsets, const int* __restrict__ blockscale_offsets,
                         uint8_t* __restrict__ quant_output, uint8_t* __restrict__ scale_factor, int num_experts,
                         int k) {
  __shared__ int chunk_prefix[ES_B200_MAX_EXPERTS + 1];
  __shared__ int warp_sums[32];

  pdl_wait_prior_grid();
  block_exclusive_scan(num_experts, chunk_prefix, warp_sums, [&](int e) {
    int m = problem_sizes[e * 3];
    return m > 0 ? (m + QUANT_ROWS_PER_CHUNK - 1) / QUANT_ROWS_PER_CHUNK : 0;
  });
  pdl_launch_dependents();
  const int total_chunks = chunk_prefix[num_experts];

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int kt = k >> 7;                 // 128-element K tiles = scale words per row
  const int64_t kb = k >> 5;             // scale bytes per row

  for (int u = blockIdx.x; u < total_chunks; u += gridDim.x) {
    const int e = upper_bound_expert(chunk_prefix, num_experts, u);
    const int chunk = u - chunk_prefix[e];
    const int m = problem_sizes[e * 3];
    const int r = chunk * QUANT_ROWS_PER_CHUNK + warp;      // row inside the expert
    uint8_t* sf_expert = scale_factor + (int64_t)blockscale_offsets[e] * kb;

    if (r < m) {
      const int64_t grow = (int64_t)expert_offsets[e] + r;
      const T* in_row = input + grow * (kSiluMul ? 2 * (int64_t)k : (int64_t)k);
      uint8_t* out_row = quant_output + grow * k;
      // scale word of (row r, K tile q): atom (r/128, q), inside the atom (r%32)*16 + ((r%128)/32)*4
      uint8_t* sf_row = sf_expert + (int64_t)(r >> 7) * kt * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4;

      constexpr int U = kSiluMul ? QUANT_UNROLL_SILU : QUANT_UNROLL;
      for (int c0 = 0; c0 < k; c0 += 256 * U) {
        uint4 raw[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
          const int col = c0 + j * 256 + lane * 8;
          raw[j] = col < k ? ld_stream_16B(in_row + col) : make_uint4(0, 0, 0, 0);
        }
        if constexpr (kSiluMul) {
          uint4 up[U];
#pragma unroll
          for (int j = 0; j < U; ++j) {
            const int col = c0 + j * 256 + lane * 8;
            up[j] = col < k ? ld_stream_16B(in_row + k + col) : make_uint4(0, 0, 0, 0);
          }
#pragma unroll
          for (int j = 0; j < U; ++j) raw[j] = silu_mul8<T>(raw[j], up[j]);
        }
#pragma unroll
        for (int j = 0; j < U; ++j) {
          const int cbase = c0 + j * 256;
          if (cbase >= k) break;                        // warp-uniform
          const int col = cbase + lane * 8;
          uint2 codes;
          uint32_t sf = quantize8<T>(raw[j], codes);
          if (col < k) st_stream_8B(out_row + col, codes);
          // pack the four scale bytes of one K tile (lanes 0-15 / 16-31) into one aligned 32-bit word
          uint32_t w = sf << (((lane >> 2) & 3) * 8);
          w |= __shfl_xor_sync(0xffffffffu, w, 4);
          w |= __shfl_xor_sync(0xffffffffu, w, 8);
          if ((lane & 15) == 0 && col < k) {
            const int q = col >> 7;
            *reinterpret_cast<uint32_t*>(sf_row + (int64_t)q * 512) = w;
          }
        }
      }
    }

    // the chunk holding the expert's last row also clears the scale bytes of the padding rows m..align128(m)-1
    if (chunk == chunk_prefix[e + 1] - chunk_prefix[e] - 1) {
      const int mp = (m + 127) & ~127;
      const int npad = mp - m;
      for (int i = threadIdx.x; i < npad * kt; i += QUANT_THREADS) {
        const int pr = m + i / kt;
        const int q = i - (i / kt) * kt;
        uint8_t* p = sf_expert + (int64_t)(pr >> 7) * kt * 512 + (int64_t)q * 512 + (pr & 31) * 16 + ((pr & 127) >> 5) * 4;
        *reinterpret_cast<uint32_t*>(p) = 0u;
      }
    }
  }
}

template <bool kSiluMul>
static int quant_impl(const void* input, int input_dtype, const int32_t* problem_sizes, const int32_t* expert_offsets,
                      const int32_t* blockscale_offsets, void* quant_output, uint8_t* scale_factor, int num_experts,
                      int64_t num_rows, int k, void* stream) {
  ES_REQUIRE(input_dtype == ES_B200_BF16 || input_dtype == ES_B200_FP16, "dtype must be kFloat16 or kBFloat16");
  ES_REQUIRE(k > 0 && k % 128 == 0, "k must align to 128");
  ES_REQUIRE(num_experts >= 0 && num_experts <= ES_B200_MAX_EXPERTS,
             "Number of experts cannot exceed %d", ES_B200_MAX_EXPERTS);
  ES_REQUIRE(num_rows >= 0, "num_rows must be non-negative");
  if (num_experts == 0 || num_rows == 0) return ES_B200_OK;
  ES_REQUIRE(input && quant_output && scale_factor && problem_sizes && expert_offsets && blockscale_offsets,
             "null pointer argument");
  ES_REQUIRE(aligned16(input) && aligned16(quant_output), "input and quant_output must be 16-byte aligned");
  ES_REQUIRE((reinterpret_cast<uintptr_t>(scale_factor) & 3u) == 0, "scale_factor must be 4-byte aligned");

  DeviceInfo info;
  int rc = get_device_info(&info);
  if (rc != ES_B200_OK) return rc;

  // at most one partial chunk per expert on top of the full chunks of num_rows rows
  const int64_t max_chunks = (num_rows + QUANT_ROWS_PER_CHUNK - 1) / QUANT_ROWS_PER_CHUNK + num_experts;
  static int blocks_per_sm[2] = {0, 0};   // per input type (and per instantiation); same on every device of a box
  int& occ = blocks_per_sm[input_dtype == ES_B200_BF16 ? 0 : 1];
  if (occ == 0) {
    int v = 0;
    if (input_dtype == ES_B200_BF16)
      ES_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&v, mxfp8_group_quant_kernel<__nv_bfloat16, kSiluMul>, QUANT_THREADS, 0));
    else
      ES_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&v, mxfp8_group_quant_kernel<__half, kSiluMul>, QUANT_THREADS, 0));
    occ = v > 0 ? v : 1;
  }
  const int64_t resident = (int64_t)info.sm_count * occ;
  const int grid = (int)(max_chunks < resident ? max_chunks : resident);

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (input_dtype == ES_B200_BF16) {
    mxfp8_group_quant_kernel<__nv_bfloat16, kSiluMul><<<grid, QUANT_THREADS, 0, s>>>(
        static_cast<const __nv_bfloat16*>(input), problem_sizes, expert_offsets, blockscale_offsets,
        static_cast<uint8_t*>(quant_output), scale_factor, num_experts, k);
  } else {
    mxfp8_group_quant_kernel<__half, kSiluMul><<<grid, QUANT_THREADS, 0, s>>>(
        static_cast<const __half*>(input), problem_sizes, expert_offsets, blockscale_offsets,
        static_cast<uint8_t*>(quant_output), scale_factor, num_experts, k);
  }
  ES_CUDA_TRY(cudaGetLastError());
  return ES_B200_OK;
}
}  // namespace es_b200

extern "C" int es_b200_mxfp8_grouped_quant(const void* input, int input_dtype, const int32_t* problem_sizes,
                                           const int32_t* expert_offsets, const int32_t* blockscale_offsets,
                                           void* quant_output, uint8_t* scale_factor, int num_experts,
                                           int64_t num_rows, int k, void* stream) {
  es_b200::NvtxRange nvtx_range("es_b200_mxfp8_grouped_quant");
  return es_b200::quant_impl<false>(input, input_dtype, problem_sizes, expert_offsets, blockscale_offsets, quant_output,
                                    scale_factor, num_experts, num_rows, k, stream);
}

extern "C" int es_b200_mxfp8_silu_mul_grouped_quant(const void* gate_up, int input_dtype, const int32_t* problem_sizes,
                                                    const int32_t* expert_offsets, const int32_t* blockscale_offsets,
                                                    void* quant_output, uint8_t* scale_factor, int num_experts,
                                                    int64_t num_rows, int k, void* stream) {
  es_b200::NvtxRange nvtx_range("es_b200_mxfp8_silu_mul_grouped_quant");
  return es_b200::quant_impl<true>(gate_up, input_dtype, problem_sizes, expert_offsets, blockscale_offsets, quant_output,
                                   scale_factor, num_experts, num_rows, k, stream);
}
