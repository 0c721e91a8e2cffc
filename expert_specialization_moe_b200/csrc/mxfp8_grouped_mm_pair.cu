// MXFP8 block-scaled grouped GEMM for sm_100a on CTA PAIRS: tcgen05.mma.cta_group::2 with M = 256.
//
// Same mapping as the single-CTA kernel (weights on the MMA M axis, the expert's token rows on the runtime-sized
// MMA N axis), but two CTAs of a cluster share every tile: each CTA holds 128 of the 256 weight rows and HALF of
// the token rows in its own shared memory, and the pair's tensor cores exchange the token halves.  Per CTA and
// K step that is 16 KB of weights + at most 12 KB of tokens for a 128 x 192 x 128 share of the MMA, i.e. the
// operand bytes each SM has to pull through L2 per FLOP are ~40 % lower than with 128 x 128 single-CTA tiles —
// which is what bounds experts with many tokens — without any multicast load.  Token tiles are 192 rows: two
// 192-column fp32 accumulators (double buffering) plus per-stage scale slots fit the 512 TMEM columns, and a
// 192-row tile starts on a 64-row boundary of the 128-row scale atoms, which a 2-column TMEM offset addresses.
//
//   warp 0    producer (both CTAs): 4 TMA loads per K step (own weight rows, own half of the tokens, own weight
//             scale atom, the tile's token scale atoms); all completion bytes are credited to the leader's barrier
//   warp 1    TMEM allocation (both CTAs); in the leader CTA one lane issues tcgen05.cp (scales smem -> TMEM of
//             both CTAs) and 4 tcgen05.mma per K step, and commits to the barriers of both CTAs
//   warps 2-5 epilogue (both CTAs): own 128 accumulator lanes -> bf16/fp16 -> global
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "tensormap.cuh"

namespace es_b200 {
namespace mm2 {

constexpr int THREADS = 192;
constexpr int TILE_N = 128;      // weight rows per CTA (the pair covers 256)
constexpr int TILE_K = 128;
constexpr int TOK_TILE = 192;    // token rows per tile (MMA N, runtime multiple of 16)
constexpr int STAGES = 7;
constexpr int W_BYTES = TILE_N * TILE_K;               // 16384
constexpr int X_BYTES = (TOK_TILE / 2) * TILE_K;       // 12288: this CTA's half of the token tile
constexpr int SFW_BYTES = 512;
constexpr int SFX_BYTES = 1024;                        // up to two 512-byte atoms
constexpr int STAGE_BYTES = 30720;                     // 30 KB: W | X | SFW | SFX | pad  (multiple of 1024)
static_assert(W_BYTES + X_BYTES + SFW_BYTES + SFX_BYTES <= STAGE_BYTES, "stage layout");
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t ACC_COLS = 192;        // accumulators at columns [0,192) and [192,384)
constexpr uint32_t SF_COL0 = 384;         // per-stage scale slots of 16 columns: 4 (weights) + 8 (tokens) + 4 unused
constexpr uint32_t SF_SLOT_COLS = 16;
static_assert(SF_COL0 + STAGES * SF_SLOT_COLS <= TMEM_COLS, "TMEM budget");

constexpr uint32_t ERR_PRODUCER = 0x10u, ERR_MMA = 0x20u, ERR_EPILOGUE = 0x40u;

struct SharedCtl {
  uint64_t full[STAGES];        // used in the leader CTA only
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];       // used in the leader CTA only (8 arrivals: 4 epilogue warps x 2 CTAs)
  uint32_t tmem_base;
  int abort_flag;
  int warp_sums[32];
  int tile_prefix[2][ES_B200_MAX_EXPERTS + 1];   // [0]: experts with one token tile (weights streamed once from HBM),
                                                 // [1]: experts with several token tiles (weights re-read from L2)
#ifdef ES_PROFILE
  long long t_issue[STAGES];
  long long t_commit[STAGES];
#endif
};

constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES + sizeof(SharedCtl);

__device__ uint32_t g_status = 0;
#ifdef ES_PROFILE
__device__ unsigned long long g_prof[16];
#define PROF_T0() long long _pt = clock64()
#define PROF_ADD(i) do { long long _n = clock64(); _acc[i] += _n - _pt; _pt = _n; } while (0)
#else
#define PROF_T0()
#define PROF_ADD(i)
#endif

struct TileInfo {
  int e, tt, np;
  int valid, n_mma;
  int row0;        // first token row of the tile in a / d
  int atom0;       // first 128-row scale atom of the tile inside the expert
  int n_atoms;     // 1 or 2 atoms exist for this tile
  uint32_t sf_col; // column offset of the tile's first row inside its first atom: 0 or 2
  bool heavy;      // the expert has more than one token tile
};

// Position p of the merged work list -> tile.  The two classes are merged proportionally (a Bresenham walk), so that
// at any time the CTA pairs running side by side are a mix of HBM-streaming tiles and L2-resident, tensor-bound tiles
// and both lists run out together.
__device__ __forceinline__ TileInfo decode_tile(int p, const int (*prefix2)[ES_B200_MAX_EXPERTS + 1], int num_experts,
                                                const int* problem_sizes, const int* expert_offsets) {
  TileInfo ti;
  const int n_light = prefix2[0][num_experts], n_heavy = prefix2[1][num_experts];
  const long long tot = (long long)n_light + n_heavy;
  const int h0 = (int)(((long long)p * n_heavy) / tot);
  const int h1 = (int)(((long long)(p + 1) * n_heavy) / tot);
  ti.heavy = h1 > h0;
  const int t = ti.heavy ? h0 : p - h0;
  const int* prefix = prefix2[ti.heavy ? 1 : 0];
  ti.e = upper_bound_expert(prefix, num_experts, t);
  const int i = t - prefix[ti.e];
  const int m = problem_sizes[ti.e * 3];
  const int token_tiles = (m + TOK_TILE - 1) / TOK_TILE;
  ti.np = i / token_tiles;
  ti.tt = i - ti.np * token_tiles;
  const int r_local = ti.tt * TOK_TILE;
  const int rem = m - r_local;
  ti.valid = rem < TOK_TILE ? rem : TOK_TILE;
  ti.n_mma = (ti.valid + 15) & ~15;
  ti.row0 = expert_offsets[ti.e] + r_local;
  ti.atom0 = r_local >> 7;
  ti.sf_col = (uint32_t)((r_local & 127) >> 5);
  const int last_atom = (r_local + ti.valid - 1) >> 7;
  ti.n_atoms = last_atom - ti.atom0 + 1;
  return ti;
}

template <typename OutT>
__device__ __forceinline__ OutT from_f32(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

struct Maps {
  CUtensorMap w;        // weights  [E*N, K] bytes, box 128 rows x 128 B, 128-byte swizzle
  CUtensorMap x[5];     // tokens   [T, K]   bytes, boxes of 8 / 16 / 32 / 64 / 96 rows
  CUtensorMap sfw;      // weight scale atoms, 512-byte records
  CUtensorMap sfx;      // token scale atoms, 512-byte records
};

template <typename OutT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
mxfp8_grouped_mm_pair_kernel(const __grid_constant__ Maps maps, OutT* __restrict__ d,
                             const int* __restrict__ problem_sizes, const int* __restrict__ expert_offsets,
                             const int* __restrict__ blockscale_offsets, int num_experts, int n, int k) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(smem + (size_t)STAGES * STAGE_BYTES);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();      // 0 = leader (issues the MMAs), 1 = peer
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&ctl->full[s], 1);
      ptx::mbar_init(&ctl->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&ctl->tmem_full[a], 1);
      ptx::mbar_init(&ctl->tmem_empty[a], 8);
    }
    ctl->abort_flag = 0;
#ifdef ES_PROFILE
    for (int s = 0; s < STAGES; ++s) { ctl->t_issue[s] = 0; ctl->t_commit[s] = 0; }
#endif
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&maps.w);
    ptx::prefetch_tensormap(&maps.sfw);
    ptx::prefetch_tensormap(&maps.sfx);
#pragma unroll
    for (int i = 0; i < 5; ++i) ptx::prefetch_tensormap(&maps.x[i]);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(&ctl->tmem_base, TMEM_COLS);
    ptx::tmem_relinquish_pair();
  }
  pdl_wait_prior_grid();
  const int n_tiles = n / TILE_N;
  const int n_pairs = (n_tiles + 1) >> 1;
  block_exclusive_scan(num_experts, ctl->tile_prefix[0], ctl->warp_sums, [&](int e) {
    const int m = problem_sizes[e * 3];
    return (m > 0 && m <= TOK_TILE) ? n_pairs : 0;
  });
  block_exclusive_scan(num_experts, ctl->tile_prefix[1], ctl->warp_sums, [&](int e) {
    const int m = problem_sizes[e * 3];
    return m > TOK_TILE ? ((m + TOK_TILE - 1) / TOK_TILE) * n_pairs : 0;
  });
  // barriers and TMEM of both CTAs must exist before either CTA signals the other
  ptx::tc_fence_before_sync();
  ptx::cluster_sync();
  ptx::tc_fence_after_sync();
  pdl_launch_dependents();

  const uint32_t tmem_base = ctl->tmem_base;
  const int total_tiles = ctl->tile_prefix[0][num_experts] + ctl->tile_prefix[1][num_experts];
  const int kt_count = k / TILE_K;
  const int sfw_atoms_per_expert = n_tiles * kt_count;
  volatile int* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (warp 0 of each CTA)
    // The whole warp walks the work list; per K step lanes 0..4 each issue ONE of the stage's loads in the same
    // instruction (a TMA issue costs the issuing thread ~80 cycles, five in a row would be a third of a stage time).
    int s = 0;
    uint32_t ph = 0;
    const bool mixed = ctl->tile_prefix[1][num_experts] > 0;
#ifdef ES_PROFILE
    long long _acc[4] = {0, 0, 0, 0};
#endif
    PROF_T0();
    for (int t = pair; t < total_tiles; t += num_pairs) {
      const TileInfo ti = decode_tile(t, ctl->tile_prefix, num_experts, problem_sizes, expert_offsets);
      const int half = ti.n_mma >> 1;                       // token rows held by each CTA
      const int xi = half <= 8 ? 0 : half <= 16 ? 1 : half <= 32 ? 2 : half <= 64 ? 3 : 4;
      const uint32_t box_rows = xi == 0 ? 8u : xi == 1 ? 16u : xi == 2 ? 32u : xi == 3 ? 64u : 96u;
      const uint32_t tx = 2u * (W_BYTES + box_rows * TILE_K + SFW_BYTES + (uint32_t)ti.n_atoms * 512u);
      int nt = ti.np * 2 + (int)rank;
      const int w_row = ti.e * n + nt * TILE_N;             // may run past the expert when n/128 is odd: not stored
      if (nt >= n_tiles) nt = n_tiles - 1;                  // keep the scale-atom load inside the buffer
      const int sfw_atom = ti.e * sfw_atoms_per_expert + nt * kt_count;
      const int sfx_atom = ((blockscale_offsets[ti.e] >> 7) + ti.atom0) * kt_count;
      const int x_row = ti.row0 + (int)rank * half;
      // weights of single-tile experts are used once: do not let them push the re-read working set out of L2
      const uint64_t w_hint = ti.heavy ? ptx::kL2EvictLast : (mixed ? ptx::kL2EvictFirst : ptx::kL2EvictNormal);
      // this lane's load: 0 weights, 1 tokens, 2 weight scales, 3 / 4 token scale atoms
      const int n_ops = 4 + (ti.n_atoms > 1 ? 1 : 0);
      const CUtensorMap* my_map = lane == 0 ? &maps.w : lane == 1 ? &maps.x[xi] : lane == 2 ? &maps.sfw : &maps.sfx;
      const uint32_t my_off = lane == 0 ? 0u : lane == 1 ? (uint32_t)W_BYTES : lane == 2 ? (uint32_t)(W_BYTES + X_BYTES)
                              : lane == 3 ? (uint32_t)(W_BYTES + X_BYTES + SFW_BYTES)
                                          : (uint32_t)(W_BYTES + X_BYTES + SFW_BYTES + 512);
      const int my_c1 = lane == 0 ? w_row : lane == 1 ? x_row : lane == 2 ? sfw_atom : lane == 3 ? sfx_atom
                                                                                               : sfx_atom + kt_count;
      const uint64_t my_hint = lane == 0 ? w_hint : lane == 1 ? ptx::kL2EvictLast : ptx::kL2EvictNormal;
      bool ok = true;
      for (int kt = 0; kt < kt_count; ++kt) {
        ok = __all_sync(0xffffffffu, ptx::mbar_wait(&ctl->empty[s], ph ^ 1u, abort_flag));
        if (!ok) break;
        PROF_ADD(0);
#ifdef ES_PROFILE
        if (rank == 0 && lane == 0) { ctl->t_issue[s] = clock64(); if (ctl->t_commit[s]) _acc[2] += ctl->t_issue[s] - ctl->t_commit[s]; }
#endif
        uint8_t* stage = smem + (size_t)s * STAGE_BYTES;
        if (rank == 0 && lane == 0) ptx::mbar_arrive_expect_tx(&ctl->full[s], tx);
        __syncwarp();
        if (lane < n_ops)
          ptx::tma_load_2d_pair_hint(stage + my_off, my_map, &ctl->full[s], lane < 2 ? kt * TILE_K : 0,
                                     lane < 2 ? my_c1 : my_c1 + kt, my_hint);
        if (++s == STAGES) { s = 0; ph ^= 1u; }
        PROF_ADD(1);
      }
      if (!ok) {
        if (lane == 0) {
          *abort_flag = 1;
          atomicOr(&g_status, ERR_PRODUCER);
        }
        break;
      }
    }
#ifdef ES_PROFILE
    if (lane == 0) {
      atomicAdd(&g_prof[0 + 4 * rank], (unsigned long long)_acc[0]);
      atomicAdd(&g_prof[1 + 4 * rank], (unsigned long long)_acc[1]);
      atomicAdd(&g_prof[2 + 4 * rank], (unsigned long long)_acc[2]);
    }
#endif
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issue (leader CTA, one lane)
    if (lane == 0 && rank == 0) {
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
#ifdef ES_PROFILE
      long long _acc[4] = {0, 0, 0, 0};
#endif
      PROF_T0();
      for (int t = pair; ok && t < total_tiles; t += num_pairs) {
        const TileInfo ti = decode_tile(t, ctl->tile_prefix, num_experts, problem_sizes, expert_offsets);
        if (!ptx::mbar_wait(&ctl->tmem_empty[acc], acc_ph ^ 1u, abort_flag)) ok = false;
        PROF_ADD(0);
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
        for (int kt = 0; ok && kt < kt_count; ++kt) {
          if (!ptx::mbar_wait(&ctl->full[s], ph, abort_flag)) { ok = false; break; }
          PROF_ADD(1);
#ifdef ES_PROFILE
          _acc[3] += clock64() - ctl->t_issue[s];
#endif
          ptx::tc_fence_after_sync();
          const uint32_t stage = ptx::smem_u32(smem + (size_t)s * STAGE_BYTES);
          const uint32_t sfw_t = tmem_base + SF_COL0 + s * SF_SLOT_COLS;
          const uint32_t sfx_t = sfw_t + 4;
          ptx::tc_cp_sf_pair(sfw_t, ptx::make_desc_sf(stage + W_BYTES + X_BYTES));
          ptx::tc_cp_sf_pair(sfx_t, ptx::make_desc_sf(stage + W_BYTES + X_BYTES + SFW_BYTES));
          if (ti.n_atoms > 1)
            ptx::tc_cp_sf_pair(sfx_t + 4, ptx::make_desc_sf(stage + W_BYTES + X_BYTES + SFW_BYTES + 512));
          const uint64_t a_desc = ptx::make_desc_k_sw128(stage);
          const uint64_t b_desc = ptx::make_desc_k_sw128(stage + W_BYTES);
#ifndef ES_EXPERIMENT
#define ES_EXPERIMENT 0
#endif
#pragma unroll
          for (uint32_t j = 0; j < ((ES_EXPERIMENT & 1) ? 0u : 4u); ++j) {
            ptx::tc_mma_mxf8_pair(d_tmem, a_desc + 2 * j, b_desc + 2 * j,
                                  ptx::make_idesc_mxf8(2 * TILE_N, ti.n_mma, j, j), sfw_t | (j << 30),
                                  (sfx_t + ti.sf_col) | (j << 30), (kt | j) != 0 ? 1u : 0u);
          }
          ptx::tc_commit_pair(&ctl->empty[s], 3);       // both CTAs may refill the stage
#ifdef ES_PROFILE
          ctl->t_commit[s] = clock64();
#endif
          if (++s == STAGES) { s = 0; ph ^= 1u; }
          PROF_ADD(2);
        }
        if (!ok) {
          *abort_flag = 1;
          atomicOr(&g_status, ERR_MMA);
          break;
        }
        ptx::tc_commit_pair(&ctl->tmem_full[acc], 3);   // accumulators of both CTAs complete
        acc ^= 1;
        if (acc == 0) acc_ph ^= 1u;
      }
#ifdef ES_PROFILE
      atomicAdd(&g_prof[8], (unsigned long long)_acc[0]);
      atomicAdd(&g_prof[9], (unsigned long long)_acc[1]);
      atomicAdd(&g_prof[10], (unsigned long long)_acc[2]);
      atomicAdd(&g_prof[11], 1ull);
      atomicAdd(&g_prof[12], (unsigned long long)_acc[3]);
#endif
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_ph = 0;
    for (int t = pair; t < total_tiles; t += num_pairs) {
      const TileInfo ti = decode_tile(t, ctl->tile_prefix, num_experts, problem_sizes, expert_offsets);
      const bool got = ptx::mbar_wait(&ctl->tmem_full[acc], acc_ph, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) {
          *abort_flag = 1;
          atomicOr(&g_status, ERR_EPILOGUE);
        }
        break;
      }
      ptx::tc_fence_after_sync();
      const int nt = ti.np * 2 + (int)rank;
      const bool store = nt < n_tiles;
      const uint32_t taddr = tmem_base + acc * ACC_COLS + ((uint32_t)(q * 32) << 16);
      OutT* dcol = d + (int64_t)ti.row0 * n + (nt * TILE_N + q * 32 + lane);
      for (int c0 = 0; c0 < ti.n_mma; c0 += 16) {
        uint32_t v[16];
        ptx::tc_ld_32x32b_x16(taddr + c0, v);
        ptx::tc_wait_ld();
        if (c0 + 16 >= ti.n_mma) {
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive_cluster(&ctl->tmem_empty[acc], 0);   // the leader owns this barrier
        }
        if (store) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int tok = c0 + j;
            if (tok < ti.valid) dcol[(int64_t)tok * n] = from_f32<OutT>(__uint_as_float(v[j]));
          }
        }
      }
      acc ^= 1;
      if (acc == 0) acc_ph ^= 1u;
    }
  }

  // neither CTA may leave (or free TMEM) while its partner can still signal it or read its shared memory
  ptx::tc_fence_before_sync();
  ptx::cluster_sync();
  if (warp == 1) {
    __syncwarp();
    ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

template <typename OutT>
int launch(const void* a, const void* b, const uint8_t* sfa, const uint8_t* sfb, void* d, const int32_t* ps,
           const int32_t* eo, const int32_t* bo, int num_experts, int64_t num_rows, int n, int k, int64_t sfa_rows,
           cudaStream_t stream) {
  DeviceInfo info;
  int rc = get_device_info(&info);
  if (rc != ES_B200_OK) return rc;
  const int kt_count = k / TILE_K;

  Maps maps;
  rc = make_tensormap_u8_sw128(&maps.w, b, (uint64_t)num_experts * n, (uint64_t)k, TILE_N);
  if (rc != ES_B200_OK) return rc;
  const uint32_t boxes[5] = {8, 16, 32, 64, 96};
  for (int i = 0; i < 5; ++i) {
    rc = make_tensormap_u8_sw128(&maps.x[i], a, (uint64_t)num_rows, (uint64_t)k, boxes[i]);
    if (rc != ES_B200_OK) return rc;
  }
  rc = make_tensormap_records512(&maps.sfw, sfb, (uint64_t)num_experts * (n / TILE_N) * kt_count);
  if (rc != ES_B200_OK) return rc;
  // whole 128-row atoms only; loads past the end read as zero (a map needs at least one record)
  const uint64_t sfx_records = (uint64_t)(sfa_rows / 128) * kt_count;
  rc = make_tensormap_records512(&maps.sfx, sfa, sfx_records ? sfx_records : 1);
  if (rc != ES_B200_OK) return rc;

  auto kernel = mxfp8_grouped_mm_pair_kernel<OutT>;
  static bool configured[64] = {false};
  int dev = 0;
  ES_CUDA_TRY(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    ES_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
    configured[dev & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;

  // how many CTA pairs can be resident at once (SMs pair up inside a GPC, so this can be below sm_count / 2)
  static int resident_clusters[64] = {0};
  if (resident_clusters[dev & 63] == 0) {
    cfg.gridDim = dim3(info.sm_count & ~1);
    cfg.numAttrs = 1;
    int nc = 0;
    ES_CUDA_TRY(cudaOccupancyMaxActiveClusters(&nc, kernel, &cfg));
    if (nc < 1) return fail(ES_B200_ERR_CUDA, "no CTA pair of the grouped GEMM kernel fits on this device");
    resident_clusters[dev & 63] = nc;
  }
  const int n_pairs = (n / TILE_N + 1) / 2;
  const int64_t max_tiles = ((num_rows + TOK_TILE - 1) / TOK_TILE + num_experts) * (int64_t)n_pairs;
  const int max_clusters = resident_clusters[dev & 63];
  const int clusters = (int)(max_tiles < max_clusters ? max_tiles : max_clusters);
  cfg.gridDim = dim3(2 * clusters);
  cfg.numAttrs = 2;
  ES_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, maps, static_cast<OutT*>(d), ps, eo, bo, num_experts, n, k));
  return ES_B200_OK;
}

int launch_bf16(const void* a, const void* b, const uint8_t* sfa, const uint8_t* sfb, void* d, const int32_t* ps,
                const int32_t* eo, const int32_t* bo, int num_experts, int64_t num_rows, int n, int k,
                int64_t sfa_rows, cudaStream_t stream) {
  return launch<__nv_bfloat16>(a, b, sfa, sfb, d, ps, eo, bo, num_experts, num_rows, n, k, sfa_rows, stream);
}
int launch_fp16(const void* a, const void* b, const uint8_t* sfa, const uint8_t* sfb, void* d, const int32_t* ps,
                const int32_t* eo, const int32_t* bo, int num_experts, int64_t num_rows, int n, int k,
                int64_t sfa_rows, cudaStream_t stream) {
  return launch<__half>(a, b, sfa, sfb, d, ps, eo, bo, num_experts, num_rows, n, k, sfa_rows, stream);
}

#ifdef ES_PROFILE
extern "C" int es_b200_prof_read(unsigned long long* out16) {
  unsigned long long z[16] = {0};
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(out16, g_prof, sizeof(z));
  cudaMemcpyToSymbol(g_prof, z, sizeof(z));
  return 0;
}
#endif

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

}  // namespace mm2
}  // namespace es_b200
