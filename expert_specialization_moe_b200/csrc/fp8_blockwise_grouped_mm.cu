// FP8-blockwise grouped GEMM for sm_100a: e4m3 x e4m3 with fp32 scales (one per 1x128 of a, one per 128x128 of b).
//
// Per expert e:  d[off_e + i, n] = sum_kb sa[off_e + i, kb] * sb[e, n/128, kb] * sum_{k in kb} a[off_e + i, k] * b[e, n, k]
//
// The reference runs this op on Hopper only (wgmma templates).  Here every 128-wide K block is one unscaled
// tcgen05.mma.kind::f8f6f4 group (4 MMAs of K=32) into a TMEM partial buffer; the four epilogue warps pull each
// partial out of TMEM (tcgen05.ld), multiply by the block's scale product and accumulate in fp32 registers, while
// the tensor core already works on the next K block in the second partial buffer (two-stage promotion).
// Same mapping as the MXFP8 kernels: 128 weight rows on the MMA M axis, the expert's tokens on the runtime-sized
// MMA N axis (multiple of 16, <= 128), work list from a per-CTA prefix scan, persistent grid of one CTA per SM.
//
//   warp 0    producer: TMA loads of the weight tile and the token tile per K block (5-stage ring)
//   warp 1    TMEM allocation, MMA issue (one lane)
//   warps 2-5 scale staging (sa * sb for the tile, transposed into shared memory), promotion, output
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "tensormap.cuh"

namespace es_b200 {
namespace bw {

constexpr int THREADS = 192;
constexpr int TILE_N = 128;
constexpr int TILE_K = 128;
constexpr int TOK_TILE = 128;
constexpr int STAGES = 5;
constexpr int W_BYTES = TILE_N * TILE_K;
constexpr int X_BYTES = TOK_TILE * TILE_K;
constexpr int STAGE_BYTES = W_BYTES + X_BYTES;     // 32 KB
constexpr uint32_t TMEM_COLS = 256;                // two partial buffers of 128 columns
constexpr int MAX_KT = 112;                        // K <= 14336: the per-tile scale table must fit shared memory

constexpr uint32_t ERR_PRODUCER = 0x100u, ERR_MMA = 0x200u, ERR_EPILOGUE = 0x400u;

struct SharedCtl {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t part_full[2];
  uint64_t part_empty[2];
  uint64_t epi_sync;            // 128 arrivals: rendezvous of the epilogue threads (bounded, unlike bar.sync)
  uint32_t tmem_base;
  int abort_flag;
  int warp_sums[32];
  int tile_prefix[ES_B200_MAX_EXPERTS + 1];
};

__device__ uint32_t g_status = 0;

struct TileInfo {
  int e, tt, nt, valid, n_mma, row0;
};

__device__ __forceinline__ TileInfo decode_tile(int t, const int* prefix, int num_experts, const int* problem_sizes,
                                                const int* expert_offsets) {
  TileInfo ti;
  ti.e = upper_bound_expert(prefix, num_experts, t);
  const int i = t - prefix[ti.e];
  const int m = problem_sizes[ti.e * 3];
  const int token_tiles = (m + TOK_TILE - 1) / TOK_TILE;
  ti.nt = i / token_tiles;
  ti.tt = i - ti.nt * token_tiles;
  const int rem = m - ti.tt * TOK_TILE;
  ti.valid = rem < TOK_TILE ? rem : TOK_TILE;
  ti.n_mma = (ti.valid + 15) & ~15;
  ti.row0 = expert_offsets[ti.e] + ti.tt * TOK_TILE;
  return ti;
}

template <typename OutT>
__device__ __forceinline__ OutT from_f32(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// Rendezvous of the 128 epilogue threads on an mbarrier, so that a thread whose partners gave up returns false
// after the wait limit instead of blocking forever.
__device__ __forceinline__ bool epilogue_rendezvous(uint64_t* bar, uint32_t& phase, volatile int* abort_flag) {
  ptx::mbar_arrive(bar);
  const bool ok = ptx::mbar_wait(bar, phase, abort_flag);
  phase ^= 1u;
  return ok;
}

template <typename OutT>
__global__ void __launch_bounds__(THREADS, 1)
fp8_blockwise_grouped_mm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x16,
                                const __grid_constant__ CUtensorMap map_x32, const __grid_constant__ CUtensorMap map_x64,
                                const __grid_constant__ CUtensorMap map_x128, const float* __restrict__ scales_a,
                                const float* __restrict__ scales_b, OutT* __restrict__ d,
                                const int* __restrict__ problem_sizes, const int* __restrict__ expert_offsets,
                                int num_experts, int n, int k) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int kt_count = k / TILE_K;
  float* s_tile = reinterpret_cast<float*>(smem + (size_t)STAGES * STAGE_BYTES);          // [kt_count][128]
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(smem + (size_t)STAGES * STAGE_BYTES + (size_t)kt_count * 512);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&ctl->full[s], 1);
      ptx::mbar_init(&ctl->empty[s], 1);
    }
    for (int p = 0; p < 2; ++p) {
      ptx::mbar_init(&ctl->part_full[p], 1);
      ptx::mbar_init(&ctl->part_empty[p], 4);
    }
    ptx::mbar_init(&ctl->epi_sync, 128);
    ctl->abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&map_w);
    ptx::prefetch_tensormap(&map_x16);
    ptx::prefetch_tensormap(&map_x32);
    ptx::prefetch_tensormap(&map_x64);
    ptx::prefetch_tensormap(&map_x128);
  }
  if (warp == 1) {
    ptx::tmem_alloc(&ctl->tmem_base, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  pdl_wait_prior_grid();
  const int n_tiles = n / TILE_N;
  block_exclusive_scan(num_experts, ctl->tile_prefix, ctl->warp_sums, [&](int e) {
    const int m = problem_sizes[e * 3];
    return m > 0 ? ((m + TOK_TILE - 1) / TOK_TILE) * n_tiles : 0;
  });
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  pdl_launch_dependents();

  const uint32_t tmem_base = ctl->tmem_base;
  const int total_tiles = ctl->tile_prefix[num_experts];
  volatile int* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        const TileInfo ti = decode_tile(t, ctl->tile_prefix, num_experts, problem_sizes, expert_offsets);
        const CUtensorMap* xm = ti.n_mma <= 16 ? &map_x16 : ti.n_mma <= 32 ? &map_x32 : ti.n_mma <= 64 ? &map_x64 : &map_x128;
        const uint32_t box_rows = ti.n_mma <= 16 ? 16u : ti.n_mma <= 32 ? 32u : ti.n_mma <= 64 ? 64u : 128u;
        const uint32_t tx = W_BYTES + box_rows * TILE_K;
        const int w_row = ti.e * n + ti.nt * TILE_N;
        for (int kt = 0; kt < kt_count; ++kt) {
          if (!ptx::mbar_wait(&ctl->empty[s], ph ^ 1u, abort_flag)) {
            ok = false;
            *abort_flag = 1;
            atomicOr(&g_status, ERR_PRODUCER);
            break;
          }
          uint8_t* stage = smem + (size_t)s * STAGE_BYTES;
          ptx::mbar_arrive_expect_tx(&ctl->full[s], tx);
          ptx::tma_load_2d(stage, &map_w, &ctl->full[s], kt * TILE_K, w_row);
          ptx::tma_load_2d(stage + W_BYTES, xm, &ctl->full[s], kt * TILE_K, ti.row0);
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      int p = 0;
      uint32_t p_ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        const TileInfo ti = decode_tile(t, ctl->tile_prefix, num_experts, problem_sizes, expert_offsets);
        const uint32_t idesc = ptx::make_idesc_f8(TILE_N, ti.n_mma);
        for (int kt = 0; kt < kt_count; ++kt) {
          if (!ptx::mbar_wait(&ctl->part_empty[p], p_ph ^ 1u, abort_flag)) { ok = false; break; }
          if (!ptx::mbar_wait(&ctl->full[s], ph, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const uint32_t stage = ptx::smem_u32(smem + (size_t)s * STAGE_BYTES);
          const uint64_t a_desc = ptx::make_desc_k_sw128(stage);
          const uint64_t b_desc = ptx::make_desc_k_sw128(stage + W_BYTES);
          const uint32_t d_tmem = tmem_base + p * 128;
#pragma unroll
          for (uint32_t j = 0; j < 4; ++j)
            ptx::tc_mma_f8(d_tmem, a_desc + 2 * j, b_desc + 2 * j, idesc, j != 0 ? 1u : 0u);
          ptx::tc_commit(&ctl->empty[s]);
          ptx::tc_commit(&ctl->part_full[p]);
          if (++s == STAGES) { s = 0; ph ^= 1u; }
          p ^= 1;
          if (p == 0) p_ph ^= 1u;
        }
        if (!ok) {
          *abort_flag = 1;
          atomicOr(&g_status, ERR_MMA);
        }
      }
    }
  } else {
    const int q = warp & 3;
    const int etid = threadIdx.x - 64;     // 0..127 among the epilogue threads
    int p = 0;
    uint32_t p_ph = 0;
    bool alive = true;
    uint32_t sync_ph = 0;
    for (int t = blockIdx.x; alive && t < total_tiles; t += gridDim.x) {
      const TileInfo ti = decode_tile(t, ctl->tile_prefix, num_experts, problem_sizes, expert_offsets);
      // scale table of the tile: s_tile[kt][tok] = sa[row0 + tok, kt] * sb[e, nt, kt]
      if (!epilogue_rendezvous(&ctl->epi_sync, sync_ph, abort_flag)) break;   // all done with the previous table
      {
        const float* sb_row = scales_b + ((int64_t)ti.e * n_tiles + ti.nt) * kt_count;
        if (etid < ti.valid) {
          const float* sa_row = scales_a + (int64_t)(ti.row0 + etid) * kt_count;
          for (int kt = 0; kt < kt_count; ++kt) s_tile[kt * 128 + etid] = __ldg(sa_row + kt) * __ldg(sb_row + kt);
        } else {
          for (int kt = 0; kt < kt_count; ++kt) s_tile[kt * 128 + etid] = 0.f;
        }
      }
      if (!epilogue_rendezvous(&ctl->epi_sync, sync_ph, abort_flag)) break;

      float acc[128];
#pragma unroll
      for (int j = 0; j < 128; ++j) acc[j] = 0.f;

      for (int kt = 0; kt < kt_count; ++kt) {
        const bool got = ptx::mbar_wait(&ctl->part_full[p], p_ph, abort_flag);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0) {
            *abort_flag = 1;
            atomicOr(&g_status, ERR_EPILOGUE);
          }
          alive = false;
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t taddr = tmem_base + p * 128 + ((uint32_t)(q * 32) << 16);
        const float4* srow = reinterpret_cast<const float4*>(s_tile + kt * 128);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          if (c * 16 < ti.n_mma) {     // warp-uniform
            uint32_t v[16];
            ptx::tc_ld_32x32b_x16(taddr + c * 16, v);
            ptx::tc_wait_ld();
            if ((c + 1) * 16 >= ti.n_mma) {
              // last read of this partial buffer by this warp: the tensor core may overwrite it
              ptx::tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) ptx::mbar_arrive(&ctl->part_empty[p]);
            }
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const float4 sc = srow[c * 4 + g];      // same address in every lane: broadcast
              acc[c * 16 + g * 4 + 0] = fmaf(__uint_as_float(v[g * 4 + 0]), sc.x, acc[c * 16 + g * 4 + 0]);
              acc[c * 16 + g * 4 + 1] = fmaf(__uint_as_float(v[g * 4 + 1]), sc.y, acc[c * 16 + g * 4 + 1]);
              acc[c * 16 + g * 4 + 2] = fmaf(__uint_as_float(v[g * 4 + 2]), sc.z, acc[c * 16 + g * 4 + 2]);
              acc[c * 16 + g * 4 + 3] = fmaf(__uint_as_float(v[g * 4 + 3]), sc.w, acc[c * 16 + g * 4 + 3]);
            }
          }
        }
        p ^= 1;
        if (p == 0) p_ph ^= 1u;
      }
      if (!alive) break;
      OutT* dcol = d + (int64_t)ti.row0 * n + (ti.nt * TILE_N + q * 32 + lane);
#pragma unroll
      for (int j = 0; j < 128; ++j)
        if (j < ti.valid) dcol[(int64_t)j * n] = from_f32<OutT>(acc[j]);
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <typename OutT>
int launch(const void* a, const void* b, const float* sa, const float* sb, void* d, const int32_t* ps,
           const int32_t* eo, int num_experts, int64_t num_rows, int n, int k, cudaStream_t stream) {
  DeviceInfo info;
  int rc = get_device_info(&info);
  if (rc != ES_B200_OK) return rc;
  const int kt_count = k / TILE_K;
  if (kt_count > MAX_KT)
    return fail(ES_B200_ERR_INVALID_ARGUMENT, "fp8 blockwise grouped GEMM supports k <= %d (got %d)", MAX_KT * TILE_K, k);

  CUtensorMap map_w, map_x[4];
  rc = make_tensormap_u8_sw128(&map_w, b, (uint64_t)num_experts * n, (uint64_t)k, TILE_N);
  if (rc != ES_B200_OK) return rc;
  const uint32_t boxes[4] = {16, 32, 64, 128};
  for (int i = 0; i < 4; ++i) {
    rc = make_tensormap_u8_sw128(&map_x[i], a, (uint64_t)num_rows, (uint64_t)k, boxes[i]);
    if (rc != ES_B200_OK) return rc;
  }
  auto kernel = fp8_blockwise_grouped_mm_kernel<OutT>;
  const size_t smem_bytes = 1024 + (size_t)STAGES * STAGE_BYTES + (size_t)kt_count * 512 + sizeof(SharedCtl);
  static size_t configured[64] = {0};   // largest dynamic shared memory size set so far, per device
  int dev = 0;
  ES_CUDA_TRY(cudaGetDevice(&dev));
  if (configured[dev & 63] < smem_bytes) {
    ES_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
    configured[dev & 63] = smem_bytes;
  }
  const int64_t max_tiles = ((num_rows + TOK_TILE - 1) / TOK_TILE + num_experts) * (int64_t)(n / TILE_N);
  const int grid = (int)(max_tiles < info.sm_count ? max_tiles : info.sm_count);

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  ES_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, map_w, map_x[0], map_x[1], map_x[2], map_x[3], sa, sb,
                                 static_cast<OutT*>(d), ps, eo, num_experts, n, k));
  return ES_B200_OK;
}

int read_and_clear_status(uint32_t* out) {
  uint32_t v = 0;
  ES_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_status, sizeof(v)));
  if (v != 0) {
    uint32_t zero = 0;
    ES_CUDA_TRY(cudaMemcpyToSymbol(g_status, &zero, sizeof(zero)));
  }
  *out = v;
  return ES_B200_OK;
}

}  // namespace bw
}  // namespace es_b200

extern "C" int es_b200_fp8_blockwise_grouped_mm(const void* a, const void* b, const float* scales_a,
                                                const float* scales_b, void* d, int out_dtype,
                                                const int32_t* problem_sizes, const int32_t* expert_offsets,
                                                int num_experts, int64_t num_rows, int n, int k, void* scratch,
                                                size_t scratch_bytes, void* stream) {
  using namespace es_b200;
  (void)scratch; (void)scratch_bytes;
  ES_REQUIRE(out_dtype == ES_B200_BF16 || out_dtype == ES_B200_FP16, "output must be bfloat16 or half");
  ES_REQUIRE(k > 0 && k % 128 == 0, "k should align 128");
  ES_REQUIRE(n > 0 && n % 128 == 0, "n should align 128");
  ES_REQUIRE(num_experts >= 0 && num_experts <= ES_B200_MAX_EXPERTS, "Number of experts cannot exceed %d",
             ES_B200_MAX_EXPERTS);
  ES_REQUIRE(num_rows >= 0 && num_rows < (int64_t)1 << 31, "num_rows out of range");
  ES_REQUIRE((int64_t)num_experts * n < (int64_t)1 << 31, "num_experts * n out of range");
  if (num_experts == 0 || num_rows == 0) return ES_B200_OK;
  ES_REQUIRE(a && b && scales_a && scales_b && d && problem_sizes && expert_offsets, "null pointer argument");
  ES_REQUIRE(aligned16(a) && aligned16(b), "a and b must be 16-byte aligned");
  ES_REQUIRE((reinterpret_cast<uintptr_t>(scales_a) & 3u) == 0 && (reinterpret_cast<uintptr_t>(scales_b) & 3u) == 0,
             "scales must be 4-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (out_dtype == ES_B200_BF16)
    return bw::launch<__nv_bfloat16>(a, b, scales_a, scales_b, d, problem_sizes, expert_offsets, num_experts, num_rows,
                                     n, k, s);
  return bw::launch<__half>(a, b, scales_a, scales_b, d, problem_sizes, expert_offsets, num_experts, num_rows, n, k, s);
}
