// MXFP8 block-scaled grouped GEMM for sm_100a, hand-written around tcgen05.mma.kind::mxf8f6f4.block_scale.
//
// Per expert e:  d[off_e + i, n] = sum_k a[off_e + i, k] * 2^(sfa-127) * b[e, n, k] * 2^(sfb-127), fp32 accumulate.
//
// Mapping ("swap-AB"): the 128 rows of the tensor-core tile are 128 WEIGHT rows (output columns n), the token rows
// of the expert sit on the MMA N axis.  N of tcgen05.mma can be any multiple of 16 up to 256, so a tile of an expert
// with 3 tokens issues N=16 MMAs, one with 100 tokens N=112: the ragged dimension costs no padding to 128 and the
// tail of an expert never needs a clipped tensor-map store.  Every tile streams a [128 x K] slab of the expert's
// weights exactly once through a TMA ring (10 stages for tiles of at most 32 tokens, 6 stages for tiles of up to 128),
// which is what bounds the layer (weights dominate the bytes).
//
//   warp 0    producer: TMA loads (weights tile, token tile, two 512-byte scale atoms) per 128-wide K step
//   warp 1    tensor memory allocation + MMA issue (one elected lane): scale atoms smem -> TMEM (tcgen05.cp),
//             4 x tcgen05.mma (K=32 each) per K step, tcgen05.commit to free the stage / publish the accumulator
//   warps 2-5 epilogue: tcgen05.ld accumulator (lane = output column, column = token) -> bf16/fp16 -> global,
//             each warp store writes 64 contiguous bytes of one output row; double-buffered against the MMAs
//
// Work list: tiles (expert, token tile of <=128, weight tile of 128) found with a per-CTA prefix scan over the
// problem sizes (device resident: no host round trip).  The producer lane takes tile indices from the bucket's work
// counter in the caller's scratch (atomicAdd; round-robin over the grid when the caller gave no scratch) and hands
// each one to the MMA lane and the epilogue warps through a small shared-memory queue, so a CTA that starts late —
// behind another kernel of the same call — just takes what is left.  Within an expert the token tile index runs
// fastest so that CTAs working at the same time read the same weight slab (L2 reuse).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdlib>

#include "bucket_table.cuh"
#include "common.cuh"
#include "epilogue.cuh"
#include "grouped_mm_call.cuh"
#include "sm100_ptx.cuh"
#include "tensormap.cuh"

namespace es_b200 {
namespace mm {

constexpr int THREADS = 192;
constexpr int TILE_N = 128;     // weight rows per tile  (tcgen05.mma M)
constexpr int TILE_K = 128;     // bytes of K per pipeline stage (one 128-byte swizzle atom)
constexpr int W_BYTES = TILE_N * TILE_K;
constexpr int SF_BYTES = 512;
constexpr int MAX_STAGES = 10;

// Two tile shapes of the same kernel.  What bounds a streaming expert is how many weight bytes each SM keeps in
// flight, i.e. the number of ring stages that fit the 227 KB of shared memory: experts with at most 32 rows need a
// 4 KB token slot per stage and get 10 stages (160 KB of weights in flight), experts with up to 128 rows a 16 KB
// slot and 6 stages.
template <int TOK_TILE_, int STAGES_>
struct Shape {
  static constexpr int TOK_TILE = TOK_TILE_;     // token rows per tile (tcgen05.mma N, runtime multiple of 16)
  static constexpr int STAGES = STAGES_;
  static constexpr int X_BYTES = TOK_TILE * TILE_K;
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES + 2 * SF_BYTES;   // a multiple of 1024
  static_assert(STAGE_BYTES % 1024 == 0 && STAGES <= MAX_STAGES, "stage layout");
};
using ShapeTiny = Shape<32, 10>;     // 21 KB stages
using ShapeMid = Shape<128, 6>;      // 33 KB stages
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t ACC_COLS = 128;      // two accumulators: columns [0,128) and [128,256)
constexpr uint32_t SFW_COL = 256;       // 4 columns: scales of the weight tile
constexpr uint32_t SFX_COL = 260;       // 4 columns: scales of the token tile

constexpr uint32_t ERR_PRODUCER = 1u, ERR_MMA = 2u, ERR_EPILOGUE = 4u;
constexpr int QUEUE_DEPTH = 4;          // tile indices in flight between the producer lane and the other roles

struct SharedCtl {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t q_full[QUEUE_DEPTH];         // 1 arrival: the producer lane has written q_tile[slot]
  uint64_t q_empty[QUEUE_DEPTH];        // 5 arrivals: the MMA lane and the four epilogue warps have read it
  int q_tile[QUEUE_DEPTH];              // tile index, or -1: no more work
  uint32_t tmem_base;
  int abort_flag;
  int warp_sums[32];
  int tile_prefix[ES_B200_MAX_EXPERTS + 1];
};

template <class S>
constexpr size_t smem_bytes() {
  return 1024 /*alignment slack*/ + (size_t)S::STAGES * S::STAGE_BYTES + 4 * EPI_STAGE_BYTES_PER_WARP + sizeof(SharedCtl);
}

__device__ uint32_t g_status = 0;   // sticky error bits of the grouped GEMM kernels (bounded waits that gave up)

struct TileInfo {
  int e, tt, nt;
  int valid;     // token rows of this tile that belong to the expert
  int n_mma;     // valid rounded up to 16
  int row0;      // first token row in a / d
};

template <int TOK_TILE>
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

template <typename OutT, class S>
__global__ void __launch_bounds__(THREADS, 1)
mxfp8_grouped_mm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x16,
                        const __grid_constant__ CUtensorMap map_x32, const __grid_constant__ CUtensorMap map_x64,
                        const __grid_constant__ CUtensorMap map_x128, const uint8_t* __restrict__ sf_tokens,
                        const uint8_t* __restrict__ sf_weights, OutT* __restrict__ d,
                        const int* __restrict__ problem_sizes, const int* __restrict__ expert_offsets,
                        const int* __restrict__ blockscale_offsets, int num_experts, int n, int k, int min_rows,
                        int max_rows, int wait_at_start, const __grid_constant__ RowScatter scatter,
                        uint32_t* counters, int bucket, int last_of_call, uint32_t earlier_ctas) {
  constexpr int TOK_TILE = S::TOK_TILE, STAGES = S::STAGES, X_BYTES = S::X_BYTES, STAGE_BYTES = S::STAGE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_stage = smem + (size_t)STAGES * STAGE_BYTES;      // 4 x 2 KB, one per epilogue warp
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(epi_stage + 4 * EPI_STAGE_BYTES_PER_WARP);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&ctl->full[s], 1);
      ptx::mbar_init(&ctl->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&ctl->tmem_full[a], 1);
      ptx::mbar_init(&ctl->tmem_empty[a], 4);   // one arrival per epilogue warp
    }
    for (int q = 0; q < QUEUE_DEPTH; ++q) {
      ptx::mbar_init(&ctl->q_full[q], 1);
      ptx::mbar_init(&ctl->q_empty[q], 5);
    }
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
  // Everything above is independent of the previous kernel's output; problem sizes may not be.  The first kernel
  // of a call waits here for whatever precedes the call; the later kernels of the same call are launched (programmatic
  // dependent launch) only after every CTA of the first has passed this point, so their operands are final: they
  // start on SMs as they become free; stream order for what follows the call is kept at the end (end_of_kernel).
  if (wait_at_start) pdl_wait_prior_grid();
  const int n_tiles = n / TILE_N;
  // this launch owns the experts with min_rows <= rows <= max_rows
  // (an expert whose scales do not start on a 128-row atom cannot be addressed: reported and skipped)
  block_exclusive_scan(num_experts, ctl->tile_prefix, ctl->warp_sums, [&](int e) {
    const int m = problem_sizes[e * 3];
    if (!(m > 0 && m >= min_rows && m <= max_rows)) return 0;
    if ((blockscale_offsets[e] & 127) != 0) {
      atomicOr(&g_status, ERR_SCALE_OFFSET_BIT);
      return 0;
    }
    return ((m + TOK_TILE - 1) / TOK_TILE) * n_tiles;
  });
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  pdl_launch_dependents();

  const uint32_t tmem_base = ctl->tmem_base;
  const int total_tiles = ctl->tile_prefix[num_experts];
  const int kt_count = k / TILE_K;
  const int64_t sf_row_bytes = k / 32;
  volatile int* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      int s = 0, qs = 0;
      uint32_t ph = 0, qph = 0;
      bool ok = true;
      uint32_t* counter = counters ? counters + bucket : nullptr;
      int t = counter ? (int)atomicAdd(counter, 1u) : (int)blockIdx.x;
      while (ok) {
        // hand the tile index (or the end mark) to the other roles
        if (!ptx::mbar_wait(&ctl->q_empty[qs], qph ^ 1u, abort_flag)) {
          *abort_flag = 1;
          atomicOr(&g_status, ERR_PRODUCER);
          break;
        }
        const bool live = t < total_tiles;
        ctl->q_tile[qs] = live ? t : -1;
        ptx::mbar_arrive(&ctl->q_full[qs]);
        if (++qs == QUEUE_DEPTH) { qs = 0; qph ^= 1u; }
        if (!live) break;
        // the next index is requested now; its round trip to L2 hides behind this tile's loads
        const int t_next = counter ? (int)atomicAdd(counter, 1u) : t + (int)gridDim.x;
        const TileInfo ti = decode_tile<TOK_TILE>(t, ctl->tile_prefix, num_experts, problem_sizes, expert_offsets);
        const CUtensorMap* xm = ti.n_mma <= 16 ? &map_x16 : ti.n_mma <= 32 ? &map_x32 : ti.n_mma <= 64 ? &map_x64 : &map_x128;
        const uint32_t box_rows = ti.n_mma <= 16 ? 16u : ti.n_mma <= 32 ? 32u : ti.n_mma <= 64 ? 64u : 128u;
        const uint32_t tx = W_BYTES + box_rows * TILE_K + 2 * SF_BYTES;
        const uint8_t* sfw = sf_weights + (int64_t)ti.e * n * sf_row_bytes + (int64_t)ti.nt * kt_count * SF_BYTES;
        const uint8_t* sfx = sf_tokens + (int64_t)blockscale_offsets[ti.e] * sf_row_bytes + (int64_t)ti.tt * kt_count * SF_BYTES;
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
          ptx::bulk_load(stage + W_BYTES + X_BYTES, sfw + (int64_t)kt * SF_BYTES, SF_BYTES, &ctl->full[s]);
          ptx::bulk_load(stage + W_BYTES + X_BYTES + SF_BYTES, sfx + (int64_t)kt * SF_BYTES, SF_BYTES, &ctl->full[s]);
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        t = t_next;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      int s = 0, qs = 0;
      uint32_t ph = 0, qph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      const uint32_t sfw_t = tmem_base + SFW_COL;
      const uint32_t sfx_t = tmem_base + SFX_COL;
      while (ok) {
        if (!ptx::mbar_wait(&ctl->q_full[qs], qph, abort_flag)) {
          *abort_flag = 1;
          atomicOr(&g_status, ERR_MMA);
          break;
        }
        const int t = ctl->q_tile[qs];
        ptx::mbar_arrive(&ctl->q_empty[qs]);
        if (++qs == QUEUE_DEPTH) { qs = 0; qph ^= 1u; }
        if (t < 0) break;
        const TileInfo ti = decode_tile<TOK_TILE>(t, ctl->tile_prefix, num_experts, problem_sizes, expert_offsets);
        if (!ptx::mbar_wait(&ctl->tmem_empty[acc], acc_ph ^ 1u, abort_flag)) { ok = false; }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
        for (int kt = 0; ok && kt < kt_count; ++kt) {
          if (!ptx::mbar_wait(&ctl->full[s], ph, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const uint32_t stage = ptx::smem_u32(smem + (size_t)s * STAGE_BYTES);
          ptx::tc_cp_sf(sfw_t, ptx::make_desc_sf(stage + W_BYTES + X_BYTES));
          ptx::tc_cp_sf(sfx_t, ptx::make_desc_sf(stage + W_BYTES + X_BYTES + SF_BYTES));
          const uint64_t a_desc = ptx::make_desc_k_sw128(stage);
          const uint64_t b_desc = ptx::make_desc_k_sw128(stage + W_BYTES);
#pragma unroll
          for (uint32_t j = 0; j < 4; ++j) {
            ptx::tc_mma_mxf8(d_tmem, a_desc + 2 * j, b_desc + 2 * j, ptx::make_idesc_mxf8(TILE_N, ti.n_mma, j, j),
                             sfw_t | (j << 30), sfx_t | (j << 30), (kt | j) != 0 ? 1u : 0u);
          }
          ptx::tc_commit(&ctl->empty[s]);      // stage reusable once these MMAs have read it
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (!ok) {
          *abort_flag = 1;
          atomicOr(&g_status, ERR_MMA);
          break;
        }
        ptx::tc_commit(&ctl->tmem_full[acc]);  // accumulator complete
        acc ^= 1;
        if (acc == 0) acc_ph ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;   // TMEM lane quadrant this warp may access
    int acc = 0, qs = 0;
    uint32_t acc_ph = 0, qph = 0;
    while (true) {
      const bool have = ptx::mbar_wait(&ctl->q_full[qs], qph, abort_flag);
      if (!__all_sync(0xffffffffu, have)) {
        if (lane == 0) {
          *abort_flag = 1;
          atomicOr(&g_status, ERR_EPILOGUE);
        }
        break;
      }
      const int t = ctl->q_tile[qs];
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&ctl->q_empty[qs]);
      if (++qs == QUEUE_DEPTH) { qs = 0; qph ^= 1u; }
      if (t < 0) break;
      const TileInfo ti = decode_tile<TOK_TILE>(t, ctl->tile_prefix, num_experts, problem_sizes, expert_offsets);
      const bool got = ptx::mbar_wait(&ctl->tmem_full[acc], acc_ph, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) {
          *abort_flag = 1;
          atomicOr(&g_status, ERR_EPILOGUE);
        }
        break;
      }
      ptx::tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * ACC_COLS + ((uint32_t)(q * 32) << 16);
      OutT* dst = d + (int64_t)ti.row0 * n + (ti.nt * TILE_N + q * 32);
      drain_accumulator<OutT>(taddr, ti.n_mma, ti.valid, reinterpret_cast<OutT*>(epi_stage) + (warp - 2) * 1024, dst, n,
                              true, lane, [&] {
                                // all of this warp's accumulator reads are done: hand the buffer back to the MMA warp
                                ptx::tc_fence_before_sync();
                                __syncwarp();
                                if (lane == 0) ptx::mbar_arrive(&ctl->tmem_empty[acc]);
                              }, scatter, ti.row0, ti.nt * TILE_N + q * 32, &g_status);
      acc ^= 1;
      if (acc == 0) acc_ph ^= 1u;
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
  end_of_kernel(counters, wait_at_start != 0, last_of_call != 0, earlier_ctas, scatter.meta != nullptr, &g_status);
}

// earlier_ctas: in/out — CTAs launched so far by this call; the last kernel of the call waits for that many reports
template <typename OutT, class S>
int launch(const CallArgs& c, int min_rows, int max_rows, bool first_of_call, bool last_of_call, int bucket,
           uint32_t* earlier_ctas) {
  constexpr int TOK_TILE = S::TOK_TILE;
  constexpr size_t SMEM_BYTES = smem_bytes<S>();
  DeviceInfo info;
  int rc = get_device_info(&info);
  if (rc != ES_B200_OK) return rc;

  CUtensorMap map_w, map_x[4];
  rc = make_tensormap_u8_sw128(&map_w, c.b, (uint64_t)c.num_experts * c.n, (uint64_t)c.k, TILE_N);
  if (rc != ES_B200_OK) return rc;
  const uint32_t boxes[4] = {16, 32, 64, 128};
  for (int i = 0; i < 4; ++i) {
    rc = make_tensormap_u8_sw128(&map_x[i], c.a, (uint64_t)c.num_rows, (uint64_t)c.k, boxes[i]);
    if (rc != ES_B200_OK) return rc;
  }

  auto kernel = mxfp8_grouped_mm_kernel<OutT, S>;
  static bool configured[64] = {false};   // per device (one static per instantiation)
  int dev = 0;
  ES_CUDA_TRY(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    ES_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
    configured[dev & 63] = true;
  }
  // upper bound of the tile count known on the host: full token tiles of num_rows plus one partial per expert
  const int64_t max_tiles = ((c.num_rows + TOK_TILE - 1) / TOK_TILE + c.num_experts) * (int64_t)(c.n / TILE_N);
  int grid = (int)(max_tiles < info.sm_count ? max_tiles : info.sm_count);
  const int cap = tunables().mm_stream_max_ctas;
  if (cap > 0 && grid > cap) grid = cap;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = c.stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  ES_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, map_w, map_x[0], map_x[1], map_x[2], map_x[3], c.sfa, c.sfb,
                                 static_cast<OutT*>(c.d), c.ps, c.eo, c.bo, c.num_experts, c.n, c.k, min_rows, max_rows,
                                 first_of_call ? 1 : 0, *c.scatter, c.counters, bucket, last_of_call ? 1 : 0,
                                 *earlier_ctas));
  *earlier_ctas += (uint32_t)grid;
  return ES_B200_OK;
}

}  // namespace mm

namespace ep {    // expert-parallel dispatch / combine kernels (ep_dispatch_combine.cu)
int read_and_clear_status(uint32_t* out);
}
namespace route {  // expert-parallel routing tables (ep_route.cu)
int read_and_clear_status(uint32_t* out);
}
namespace bw {    // FP8-blockwise kernel (fp8_blockwise_grouped_mm.cu)
int read_and_clear_status(uint32_t* out);
}
}  // namespace es_b200

extern "C" size_t es_b200_grouped_mm_scratch_bytes(int, int64_t, int, int) {
  return es_b200::GROUPED_MM_SCRATCH_BYTES;
}

namespace es_b200 {
static int grouped_mm_impl(const void* a, const void* b, const uint8_t* sfa, const uint8_t* sfb, void* d, int out_dtype,
                           const int32_t* problem_sizes, const int32_t* expert_offsets,
                           const int32_t* blockscale_offsets, int num_experts, int64_t num_rows, int n, int k,
                           int64_t sfa_rows, const RowScatter& scatter, void* scratch, size_t scratch_bytes,
                           void* stream) {
  ES_REQUIRE(out_dtype == ES_B200_BF16 || out_dtype == ES_B200_FP16, "dtype must be kFloat16 or kBFloat16");
  ES_REQUIRE(k > 0 && k % 128 == 0, "k should align 128");
  ES_REQUIRE(n > 0 && n % 128 == 0, "n should align 128");
  ES_REQUIRE(num_experts >= 0 && num_experts <= ES_B200_MAX_EXPERTS, "Number of experts cannot exceed %d",
             ES_B200_MAX_EXPERTS);
  ES_REQUIRE(num_rows >= 0 && num_rows < (int64_t)1 << 31, "num_rows out of range");
  ES_REQUIRE((int64_t)num_experts * n < (int64_t)1 << 31, "num_experts * n out of range");
  if (num_experts == 0 || num_rows == 0) return ES_B200_OK;
  ES_REQUIRE(a && b && sfa && sfb && (d || scatter.meta) && problem_sizes && expert_offsets && blockscale_offsets,
             "null pointer argument");
  ES_REQUIRE(aligned16(a) && aligned16(b) && aligned16(sfa) && aligned16(sfb), "a, b, sfa, sfb must be 16-byte aligned");
  ES_REQUIRE(aligned16(d), "d must be 16-byte aligned");
  ES_REQUIRE(sfa_rows >= 0, "sfa_rows must be non-negative");
  if (scratch != nullptr) {
    if (scratch_bytes < GROUPED_MM_SCRATCH_BYTES)
      return fail(ES_B200_ERR_SCRATCH_TOO_SMALL, "scratch holds %zu bytes, es_b200_grouped_mm_scratch_bytes asks for %zu",
                  scratch_bytes, GROUPED_MM_SCRATCH_BYTES);
    ES_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 15u) == 0, "scratch must be 16-byte aligned");
  }
  // Tile-shape specialisation.  Problem sizes live on the device, so the host cannot bucket the experts; instead
  // one kernel per row-count bucket is launched, back to back on the caller's stream with programmatic dependent
  // launch, and each one filters the experts by row count inside its own work-list scan:
  //   rows <= tiny_max  : single-CTA kernel, 128 weights x <=32 tokens, 10-stage ring  \  these experts stream their
  //   rows <  heavy_min : single-CTA kernel, 128 weights x <=128 tokens, 6-stage ring  /  weights from HBM exactly
  //                       once; what counts is weight bytes in flight;
  //   rows >= heavy_min : CTA-pair kernel, 256 weights x <=384 tokens, weight-stationary K step — these experts
  //                       re-read operands from L2, what counts is operand bytes per FLOP.
  // A kernel whose bucket is empty exits after its scan.  A bucket that even the host-known upper bound of rows per
  // expert (num_rows) cannot reach is not launched at all.  The thresholds come from a per-(n, k) table
  // (bucket_table.cuh) unless a tunable overrides them.
  //
  // With scratch (work counters) a large call is SPLIT: a pair launch capped to a few CTA pairs goes first, then the
  // two streaming kernels on the SMs it leaves, then a second pair launch that takes the SMs the streaming kernels
  // free and drains the same counter.  The streaming buckets are bound by HBM and leave the tensor pipe idle, the pair
  // bucket is bound by the tensor pipe and leaves HBM idle: side by side the call costs about max() of the two
  // instead of their sum.  Every kernel is persistent and takes tiles from its bucket's counter, and no kernel of the
  // call waits for its predecessor (see end_of_kernel), so whichever side runs out first hands its SMs to the
  // kernels queued behind it.
  const Tunables& tn = tunables();
  const BucketThresholds table = bucket_thresholds(n, k);
  int heavy_min = tn.mm_heavy_min_rows > 0 ? tn.mm_heavy_min_rows : tn.mm_heavy_min_rows < 0 ? 0x7fffffff : table.heavy_min_rows;
  int tiny_max = tn.mm_tiny_max_rows > 0 ? tn.mm_tiny_max_rows : table.tiny_max_rows;
  if (tiny_max > 32) tiny_max = 32;
  if (tiny_max > heavy_min - 1) tiny_max = heavy_min - 1;
  const bool bf16 = out_dtype == ES_B200_BF16;
  mm::CallArgs c = {a, b, sfa, sfb, d, problem_sizes, expert_offsets, blockscale_offsets, num_experts, num_rows, n, k,
                    sfa_rows, &scatter, (tn.mm_dynamic && scratch) ? static_cast<uint32_t*>(scratch) : nullptr,
                    static_cast<cudaStream_t>(stream)};

  const bool want_tiny = tiny_max >= 1;
  const bool want_mid = heavy_min - 1 > tiny_max && num_rows > tiny_max;
  const bool want_pair = num_rows >= heavy_min;
  const bool split = want_pair && c.counters != nullptr && (want_tiny || want_mid) &&
                     num_rows >= tn.mm_split_min_rows && tn.mm_pair_first_clusters > 0;
  int rc = ES_B200_OK;
  bool first = true;
  uint32_t ctas = 0;       // CTAs launched so far by this call
  auto pair = [&](int max_clusters, bool last) {
    const int r = bf16 ? mm2::launch_bf16(c, heavy_min, max_clusters, first, last, &ctas)
                       : mm2::launch_fp16(c, heavy_min, max_clusters, first, last, &ctas);
    first = false;
    return r;
  };
  if (split) {
    rc = pair(tn.mm_pair_first_clusters, false);
    if (rc != ES_B200_OK) return rc;
  }
  if (want_tiny) {
    const bool last = !want_mid && !want_pair;
    rc = bf16 ? mm::launch<__nv_bfloat16, mm::ShapeTiny>(c, 1, tiny_max, first, last, 0, &ctas)
              : mm::launch<__half, mm::ShapeTiny>(c, 1, tiny_max, first, last, 0, &ctas);
    if (rc != ES_B200_OK) return rc;
    first = false;
  }
  if (want_mid) {
    const bool last = !want_pair;
    rc = bf16 ? mm::launch<__nv_bfloat16, mm::ShapeMid>(c, tiny_max + 1, heavy_min - 1, first, last, 1, &ctas)
              : mm::launch<__half, mm::ShapeMid>(c, tiny_max + 1, heavy_min - 1, first, last, 1, &ctas);
    if (rc != ES_B200_OK) return rc;
    first = false;
  }
  if (want_pair) rc = pair(tn.mm_pair_max_clusters, true);
  return rc;
}
}  // namespace es_b200

extern "C" int es_b200_mxfp8_grouped_mm(const void* a, const void* b, const uint8_t* sfa, const uint8_t* sfb, void* d,
                                        int out_dtype, const int32_t* problem_sizes, const int32_t* expert_offsets,
                                        const int32_t* blockscale_offsets, int num_experts, int64_t num_rows, int n,
                                        int k, int64_t sfa_rows, void* scratch, size_t scratch_bytes, void* stream) {
  es_b200::NvtxRange nvtx_range("es_b200_mxfp8_grouped_mm");
  es_b200::RowScatter dense = {};
  return es_b200::grouped_mm_impl(a, b, sfa, sfb, d, out_dtype, problem_sizes, expert_offsets, blockscale_offsets,
                                  num_experts, num_rows, n, k, sfa_rows, dense, scratch, scratch_bytes, stream);
}

extern "C" int es_b200_mxfp8_grouped_mm_scatter(const void* a, const void* b, const uint8_t* sfa, const uint8_t* sfb,
                                                int out_dtype, const int32_t* problem_sizes,
                                                const int32_t* expert_offsets, const int32_t* blockscale_offsets,
                                                int num_experts, int64_t num_rows, int n, int k, int64_t sfa_rows,
                                                const int32_t* row_meta, const void* const* peer_out, int world,
                                                int64_t slots_per_gpu, void* scratch, size_t scratch_bytes,
                                                void* stream) {
  es_b200::NvtxRange nvtx_range("es_b200_mxfp8_grouped_mm_scatter");
  using namespace es_b200;
  ES_REQUIRE(world >= 1 && world <= SCATTER_MAX_GPUS, "world size must be in [1, %d]", SCATTER_MAX_GPUS);
  ES_REQUIRE(row_meta && peer_out, "null pointer argument");
  ES_REQUIRE((reinterpret_cast<uintptr_t>(row_meta) & 7u) == 0, "row_meta must be 8-byte aligned");
  ES_REQUIRE(slots_per_gpu >= 0, "slots_per_gpu out of range");
  RowScatter sc = {};
  sc.meta = reinterpret_cast<const int2*>(row_meta);
  sc.gpus = world;
  sc.slots = slots_per_gpu;
  for (int i = 0; i < world; ++i) {
    ES_REQUIRE(peer_out[i] != nullptr && aligned16(peer_out[i]), "peer output %d must be a 16-byte aligned pointer", i);
    sc.base[i] = const_cast<void*>(peer_out[i]);
  }
  return grouped_mm_impl(a, b, sfa, sfb, nullptr, out_dtype, problem_sizes, expert_offsets, blockscale_offsets,
                         num_experts, num_rows, n, k, sfa_rows, sc, scratch, scratch_bytes, stream);
}

extern "C" int es_b200_check_status(void* stream, uint32_t* raw_status) {
  using namespace es_b200;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint32_t v = 0;
  ES_CUDA_TRY(cudaStreamSynchronize(s));
  ES_CUDA_TRY(cudaMemcpyFromSymbol(&v, mm::g_status, sizeof(v)));
  if (v != 0) {
    uint32_t zero = 0;
    ES_CUDA_TRY(cudaMemcpyToSymbol(mm::g_status, &zero, sizeof(zero)));
  }
  uint32_t v2 = 0;
  int rc2 = mm2::read_and_clear_status(&v2);
  if (rc2 != ES_B200_OK) return rc2;
  v |= v2;
  rc2 = bw::read_and_clear_status(&v2);
  if (rc2 != ES_B200_OK) return rc2;
  v |= v2;
  rc2 = ep::read_and_clear_status(&v2);
  if (rc2 != ES_B200_OK) return rc2;
  v |= v2;
  rc2 = route::read_and_clear_status(&v2);
  if (rc2 != ES_B200_OK) return rc2;
  v |= v2;
  if (raw_status) *raw_status = v;
  if (v != 0)
    return fail(ES_B200_ERR_DEVICE_TIMEOUT,
                "a bounded device-side wait gave up or an index was out of range (status bits 0x%x)", v);
  return ES_B200_OK;
}
