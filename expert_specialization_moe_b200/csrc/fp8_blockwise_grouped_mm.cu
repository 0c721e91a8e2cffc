// FP8-blockwise grouped GEMM for sm_100a: e4m3 x e4m3 with fp32 scales (one per 1x128 of a, one per 128x128 of b).
//
// Per expert e:  d[off_e + i, n] = sum_kb sa[off_e + i, kb] * sb[e, n/128, kb] * sum_{k in kb} a[off_e + i, k] * b[e, n, k]
//
// The reference runs this op on Hopper only (wgmma templates).  Here every 128-wide K block is one unscaled
// tcgen05.mma.kind::f8f6f4 group (4 MMAs of K=32) into one of FOUR TMEM partial buffers; the epilogue warps pull
// each partial out of TMEM (tcgen05.ld), multiply by the block's scale product and accumulate in fp32 registers
// while the tensor core works up to three K blocks ahead (two-stage promotion, as the reference's Hopper kernel
// does in registers).  Same mapping as the MXFP8 kernels: 128 weight rows on the MMA M axis, the expert's tokens on
// the runtime-sized MMA N axis (multiple of 16), work list from a per-CTA prefix scan, persistent grid of one CTA
// per SM, one launch per row-count bucket (<= 32, 33..64, >= 65 rows) chained with programmatic dependent launch.
// The buckets differ in the token tile and therefore in how many stages of weights fit the ring: these shapes are
// HBM-bound on the weights, and bytes in flight per SM are what saturates HBM.
//
//   warp 0     producer: TMA loads of the weight tile and the token tile per K block
//   warps 1, 2 MMA issue, one lane each: warp 1 (which also owns the TMEM allocation) takes the even K blocks, warp 2
//              the odd ones — consecutive K blocks go to different partial buffers, and a tcgen05.mma costs its
//              issuing thread ~90 cycles against 64 cycles of tensor time for a 128 x 128 x 32 MMA
//   warps 3(,4) scale loaders (two of them alternate chunks where registers allow): sa[token, kb] * sb[tile, kb] for
//              8 K blocks at a time, transposed to [kb][token] in a ring of chunks, so that the epilogue reads one broadcast float4 per 4 tokens and
//              never waits on global memory, whatever K is
//   then       promotion (partial * scale -> fp32 registers) and output through a per-warp shared-memory transpose:
//              one set of four warps (the four TMEM lane quadrants) per 32 token columns, so that a warp holds
//              32 accumulators, reads its share of a partial with ONE tcgen05.ld, and the sets hide each other's
//              TMEM latency; for the narrow tiles two such groups take alternate tiles, which hides the per-tile
//              latencies (work-list decode, output) that dominate when K is only 2-4 blocks
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include "common.cuh"
#include "epilogue.cuh"
#include "sm100_ptx.cuh"
#include "tensormap.cuh"

namespace es_b200 {
namespace bw {

constexpr int TILE_N = 128;
constexpr int TILE_K = 128;
constexpr int W_BYTES = TILE_N * TILE_K;
constexpr int NPART = 4;             // TMEM partial buffers
constexpr int CH_KT = 8;             // K blocks per scale chunk
constexpr int MAX_NCH = 4;           // scale chunks in the ring (per shape: 2 or 4)
constexpr int MAX_STAGES = 10;
constexpr int EPI_TOK = 16;                          // tokens per pass through an epilogue warp's transposition tile
constexpr int EPI_TILE_BYTES = EPI_TOK * 32 * 2;     // 1 KB

constexpr uint32_t ERR_PRODUCER = 0x1000u, ERR_MMA = 0x2000u, ERR_EPILOGUE = 0x4000u, ERR_SCALES = 0x8000u;

struct SharedCtl {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t part_full[NPART];
  uint64_t part_empty[NPART];     // one arrival per warp of the epilogue group that owns the tile
  uint64_t chunk_full[MAX_NCH];   // 1 arrival: the chunk's scale loader
  uint64_t chunk_empty[MAX_NCH];  // one arrival per warp of the epilogue group that owns the tile
  uint64_t turn[2];               // turn[x]: epilogue group x may enter the K loop of its next tile
  uint32_t tmem_base;
  int abort_flag;
  int warp_sums[32];
  int tile_prefix[ES_B200_MAX_EXPERTS + 1];   // item prefix [0, E], then the per-expert tables (fill_expert_table)
};

template <int TOK_TILE_, int STAGES_, int NCH_, int LOADERS_, int GROUPS_>
struct Shape {
  static constexpr int GROUPS = GROUPS_;                   // epilogue groups; consecutive tiles alternate between them
  static constexpr int LOADERS = LOADERS_;                 // scale loader warps (1 or 2)
  static constexpr int FIRST_EPI_WARP = 3 + LOADERS;
  static constexpr int TOK_TILE = TOK_TILE_;               // token rows per tile = columns of one TMEM partial
  static constexpr int STAGES = STAGES_;
  static constexpr int NCH = NCH_;
  static constexpr int GROUP_WARPS = 4 * (TOK_TILE / 32);  // 4 lane quadrants x sets of 32 token columns
  static constexpr int EPI_WARPS = GROUPS * GROUP_WARPS;
  static constexpr int THREADS = 32 * (FIRST_EPI_WARP + EPI_WARPS);
  static constexpr int X_BYTES = TOK_TILE * TILE_K;
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  static constexpr uint32_t TMEM_COLS = NPART * TOK_TILE;  // 128 / 256 / 512
  static constexpr int CHUNK_FLOATS = CH_KT * TOK_TILE;
  static constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES + (size_t)NCH * CHUNK_FLOATS * 4 +
                                       (size_t)EPI_WARPS * EPI_TILE_BYTES + sizeof(SharedCtl);
  static_assert(NCH == 2 || NCH == 4, "ring slots are taken modulo a power of two");
  static_assert(LOADERS == 1 || LOADERS == 2, "chunks alternate between at most two loaders");
  static_assert(GROUPS == 1 || GROUPS == 2, "tiles alternate between at most two epilogue groups");
  static_assert(STAGES <= MAX_STAGES, "ring too deep for the control block");
  // A waiter may be at most one phase ahead of its mbarrier.  Each ring barrier therefore has ONE waiting role per
  // revolution: K blocks (and chunks) alternate between two lanes (warps), so ring sizes must be even.
  static_assert(STAGES % 2 == 0 && NPART % 2 == 0, "alternating owners need even rings");
  static_assert(STAGE_BYTES % 1024 == 0, "stages must keep the 1024-byte alignment of the swizzled tiles");
  static_assert(SMEM_BYTES <= 232448, "shared memory of one CTA per SM");
};
// 20 warps = 5 per scheduler leave 96 registers per thread; 21 would leave 80
using ShapeTiny = Shape<32, 10, 4, 2, 2>;    // rows <= 32:   20 KB stages, 200 KB in flight; 13 warps
using ShapeSmall = Shape<64, 8, 4, 1, 2>;    // rows 33..64:  24 KB stages; 20 warps
using ShapeFull = Shape<128, 6, 2, 1, 1>;    // rows >= 65:   32 KB stages; 20 warps

__device__ uint32_t g_status = 0;

struct TileInfo {
  int e, tt, nt, valid, n_mma, row0;
};

// A work item is `group` consecutive weight tiles of one (expert, token tile); CTA `block` of the `blocks` CTAs of its
// shape takes the items block, block + blocks, ... and every role walks their tiles in the same order.  The item is
// decoded once (binary search over the item prefix, a division) and the tiles inside it only advance `nt`: with two
// K blocks per tile (k = 256) every role spent more time per tile finding out what the tile was than working on it
// (measured: the producer lane and both MMA lanes ~2200 cycles per tile, almost none of it waiting).
template <int TOK_TILE>
struct TileWalk {
  TileInfo ti;
  int item, left, blocks;
  __device__ __forceinline__ TileWalk(int block, int blocks_) : item(block - blocks_), left(0), blocks(blocks_) {}
  // advances to this CTA's next tile; false when there is none
  __device__ __forceinline__ bool next(const ExpertTable& tab, int num_experts, int total_items, int n_tiles, int group) {
    if (left > 0) {
      --left;
      ++ti.nt;
      return true;
    }
    item += blocks;
    if (item >= total_items) return false;
    ti.e = upper_bound_expert(tab.prefix, num_experts, item);
    const int i = item - tab.prefix[ti.e];
    const int m = tab.m(ti.e);
    const int token_tiles = (m + TOK_TILE - 1) / TOK_TILE;
    const int ng = i / token_tiles;
    ti.tt = i - ng * token_tiles;
    ti.nt = ng * group;
    const int rem = m - ti.tt * TOK_TILE;
    ti.valid = rem < TOK_TILE ? rem : TOK_TILE;
    ti.n_mma = (ti.valid + 15) & ~15;
    ti.row0 = tab.row0(ti.e) + ti.tt * TOK_TILE;
    const int rest = n_tiles - ti.nt;
    left = (rest < group ? rest : group) - 1;
    return true;
  }
};

// One CTA of shape S: `block` of the `blocks` CTAs that serve the experts with min_rows <= rows <= max_rows.  The tensor
// maps are the kernel's __grid_constant__ parameters.
template <typename OutT, class S>
__device__ __forceinline__ void blockwise_cta(const CUtensorMap& map_w, const CUtensorMap& map_x16,
                                              const CUtensorMap& map_x32, const CUtensorMap& map_x64,
                                              const CUtensorMap& map_x128, const float* __restrict__ scales_a,
                                              const float* __restrict__ scales_b, OutT* __restrict__ d,
                                              const int* __restrict__ problem_sizes,
                                              const int* __restrict__ expert_offsets, int num_experts, int n, int k,
                                              int min_rows, int max_rows, int wait_at_start, int group, int block,
                                              int blocks) {
  constexpr int TOK = S::TOK_TILE;
  constexpr int STAGES = S::STAGES;
  constexpr int NCH = S::NCH;
  if (!wait_at_start) pdl_launch_dependents();   // not the first kernel of its call: the next one may launch at once
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* chunks = reinterpret_cast<float*>(smem + (size_t)STAGES * S::STAGE_BYTES);        // [NCH][CH_KT][TOK]
  uint8_t* epi_stage = reinterpret_cast<uint8_t*>(chunks + NCH * S::CHUNK_FLOATS);        // 1 KB per epilogue warp
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(epi_stage + (size_t)S::EPI_WARPS * EPI_TILE_BYTES);
  const int kt_count = k / TILE_K;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&ctl->full[s], 1);
      ptx::mbar_init(&ctl->empty[s], 1);
    }
    for (int p = 0; p < NPART; ++p) {
      ptx::mbar_init(&ctl->part_full[p], 1);
      ptx::mbar_init(&ctl->part_empty[p], S::GROUP_WARPS);
    }
    for (int c = 0; c < NCH; ++c) {
      ptx::mbar_init(&ctl->chunk_full[c], 1);
      ptx::mbar_init(&ctl->chunk_empty[c], S::GROUP_WARPS);
    }
    ptx::mbar_init(&ctl->turn[0], S::GROUP_WARPS);
    ptx::mbar_init(&ctl->turn[1], S::GROUP_WARPS);
    ctl->abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&map_w);
    ptx::prefetch_tensormap(&map_x16);
    ptx::prefetch_tensormap(&map_x32);
    ptx::prefetch_tensormap(&map_x64);
    ptx::prefetch_tensormap(&map_x128);
  }
  if (warp == 1) {
    ptx::tmem_alloc(&ctl->tmem_base, S::TMEM_COLS);
    ptx::tmem_relinquish();
  }
  // The first kernel of a call waits for the stream's earlier work and then lets the other buckets' kernels start;
  // those write disjoint rows of d and only wait for their predecessor before they exit (stream order).
  if (wait_at_start) pdl_wait_prior_grid();
  const int n_tiles = n / TILE_N;
  block_exclusive_scan(num_experts, ctl->tile_prefix, ctl->warp_sums, [&](int e) {
    const int m = problem_sizes[e * 3];
    return (m > 0 && m >= min_rows && m <= max_rows) ? ((m + TOK - 1) / TOK) * ((n_tiles + group - 1) / group) : 0;
  });
  // a launch without work (the host only knows an upper bound of the rows per expert) ends here
  if (ctl->tile_prefix[num_experts] == 0) {
    if (wait_at_start) pdl_launch_dependents();
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) ptx::tmem_dealloc(ctl->tmem_base, S::TMEM_COLS);
    if (!wait_at_start) pdl_wait_prior_grid();
    return;
  }
  const ExpertTable tab = fill_expert_table(ctl->tile_prefix, num_experts, problem_sizes, expert_offsets, nullptr);
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  if (wait_at_start) pdl_launch_dependents();

  const uint32_t tmem_base = ctl->tmem_base;
  const int total_items = ctl->tile_prefix[num_experts];
  volatile int* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      TileWalk<TOK> walk(block, blocks);
      while (ok && walk.next(tab, num_experts, total_items, n_tiles, group)) {
        const TileInfo& ti = walk.ti;
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
          uint8_t* stage = smem + (size_t)s * S::STAGE_BYTES;
          ptx::mbar_arrive_expect_tx(&ctl->full[s], tx);
          ptx::tma_load_2d(stage, &map_w, &ctl->full[s], kt * TILE_K, w_row);
          ptx::tma_load_2d(stage + W_BYTES, xm, &ctl->full[s], kt * TILE_K, ti.row0);
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp == 1 || warp == 2) {
    // ------------------------------------------------------------------ MMA issue: K blocks alternate between the
    // two lanes; g counts K blocks over all tiles of this CTA (stage = g mod STAGES, partial = g mod 4)
    if (lane == 0) {
      const int mine = warp - 1;
      int g = 0;
      bool ok = true;
      TileWalk<TOK> walk(block, blocks);
      while (ok && walk.next(tab, num_experts, total_items, n_tiles, group)) {
        const TileInfo& ti = walk.ti;
        const uint32_t idesc = ptx::make_idesc_f8(TILE_N, ti.n_mma);
        for (int kt = 0; kt < kt_count; ++kt, ++g) {
          if ((g & 1) != mine) continue;
          const int s = g % STAGES;
          const uint32_t ph = (uint32_t)(g / STAGES) & 1u;
          const int p = g & (NPART - 1);
          const uint32_t p_ph = (uint32_t)(g / NPART) & 1u;
          if (!ptx::mbar_wait(&ctl->part_empty[p], p_ph ^ 1u, abort_flag)) { ok = false; break; }
          if (!ptx::mbar_wait(&ctl->full[s], ph, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const uint32_t stage = ptx::smem_u32(smem + (size_t)s * S::STAGE_BYTES);
          const uint64_t a_desc = ptx::make_desc_k_sw128(stage);
          const uint64_t b_desc = ptx::make_desc_k_sw128(stage + W_BYTES);
          const uint32_t d_tmem = tmem_base + p * TOK;
#pragma unroll
          for (uint32_t j = 0; j < 4; ++j)
            ptx::tc_mma_f8(d_tmem, a_desc + 2 * j, b_desc + 2 * j, idesc, j != 0 ? 1u : 0u);
          ptx::tc_commit(&ctl->empty[s]);
          ptx::tc_commit(&ctl->part_full[p]);
        }
        if (!ok) {
          *abort_flag = 1;
          atomicOr(&g_status, ERR_MMA);
        }
      }
    }
  } else if (warp < S::FIRST_EPI_WARP) {
    // ------------------------------------------------------------------ scale loaders: chunks alternate between the
    // two warps; c counts chunks over all tiles of this CTA (ring slot = c mod NCH)
    constexpr int LMASK = S::LOADERS - 1;     // 0: one loader takes every chunk; 1: the two loaders alternate
    const int mine = warp - 3;
    int c = 0;
    bool ok = true;
    TileWalk<TOK> walk(block, blocks);
    while (ok && walk.next(tab, num_experts, total_items, n_tiles, group)) {
      const int chunks_in_tile = (kt_count + CH_KT - 1) / CH_KT;
      // this warp's chunks of the tile: c, c+1, .. with (c & 1) == mine
      if (chunks_in_tile == 1 && (c & LMASK) != mine) { ++c; continue; }   // common for small K
      const TileInfo& ti = walk.ti;
      const float* sb_row = scales_b + ((int64_t)ti.e * n_tiles + ti.nt) * kt_count;
      for (int kt0 = 0; kt0 < kt_count; kt0 += CH_KT, ++c) {
        if ((c & LMASK) != mine) continue;
        const int cs = c & (NCH - 1);
        const uint32_t c_ph = (uint32_t)(c / NCH) & 1u;
        // the loads do not depend on the ring slot: issue them before waiting for it
        const int nk = kt_count - kt0 < CH_KT ? kt_count - kt0 : CH_KT;
        float sb[CH_KT];
#pragma unroll
        for (int i = 0; i < CH_KT; ++i) sb[i] = i < nk ? __ldg(sb_row + kt0 + i) : 0.f;
        float sa[TOK / 32][CH_KT];
#pragma unroll
        for (int u = 0; u < TOK / 32; ++u) {
          const int tok = u * 32 + lane;
          const float* sa_row = scales_a + (int64_t)(ti.row0 + tok) * kt_count + kt0;
#pragma unroll
          for (int i = 0; i < CH_KT; ++i) sa[u][i] = (tok < ti.valid && i < nk) ? __ldg(sa_row + i) : 0.f;
        }
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctl->chunk_empty[cs], c_ph ^ 1u, abort_flag))) {
          ok = false;
          if (lane == 0) {
            *abort_flag = 1;
            atomicOr(&g_status, ERR_SCALES);
          }
          break;
        }
        float* chunk = chunks + cs * S::CHUNK_FLOATS;
#pragma unroll
        for (int u = 0; u < TOK / 32; ++u) {
          const int tok = u * 32 + lane;
          if (u * 32 < ti.n_mma) {                 // columns past n_mma are never read (warp-uniform)
#pragma unroll
            for (int i = 0; i < CH_KT; ++i) chunk[i * TOK + tok] = sa[u][i] * sb[i];
          }
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&ctl->chunk_full[cs]);
      }
    }
  } else {
    // ------------------------------------------------------------------ promotion and output (warps 5..)
    // Consecutive tiles alternate between the epilogue groups: while one group converts and stores its tile (and
    // decodes the next), the other is already accumulating the following tile's partials.  The K loops themselves
    // are strictly serial (turn barriers): a group that waited on part_full / chunk_full for a tile further ahead
    // would be more than one phase ahead of those barriers, and a parity wait cannot tell phases n and n+2 apart.
    const int q = warp & 3;                           // TMEM lane quadrant of this warp
    const int egroup = (warp - S::FIRST_EPI_WARP) / S::GROUP_WARPS;
    const int col0 = (((warp - S::FIRST_EPI_WARP) % S::GROUP_WARPS) >> 2) * 32;   // this warp's 32 token columns
    OutT* stage_warp = reinterpret_cast<OutT*>(epi_stage) + (warp - S::FIRST_EPI_WARP) * (EPI_TOK * 32);
    const int part = lane & 3;
    int g = 0;                                        // K blocks over all tiles of this CTA
    int c = 0;                                        // scale chunks over all tiles of this CTA
    bool alive = true;
    uint32_t turn_ph = 0;
    int tile_index = 0;
    TileWalk<TOK> walk(block, blocks);
    while (alive && walk.next(tab, num_experts, total_items, n_tiles, group)) {
      const int my_index = tile_index++;
      if ((my_index & (S::GROUPS - 1)) != egroup) {   // the other group's tile
        g += kt_count;
        c += (kt_count + CH_KT - 1) / CH_KT;
        continue;
      }
      const TileInfo& ti = walk.ti;
      const bool has_cols = col0 < ti.n_mma;          // warp-uniform: a set past the tile's tokens only keeps the
                                                      // barriers moving
      float acc[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) acc[j] = 0.f;
      if (S::GROUPS == 2 && my_index > 0) {            // the other group has left the K loop of the previous tile
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctl->turn[egroup], turn_ph, abort_flag))) {
          if (lane == 0) {
            *abort_flag = 1;
            atomicOr(&g_status, ERR_EPILOGUE);
          }
          break;
        }
        turn_ph ^= 1u;
      }

      for (int kt = 0; kt < kt_count; ++kt, ++g) {
        const int ki = kt & (CH_KT - 1);
        const int cs = c & (NCH - 1);
        const int p = g & (NPART - 1);
        bool got = true;
        if (ki == 0) got = ptx::mbar_wait(&ctl->chunk_full[cs], (uint32_t)(c / NCH) & 1u, abort_flag);
        got = got && ptx::mbar_wait(&ctl->part_full[p], (uint32_t)(g / NPART) & 1u, abort_flag);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0) {
            *abort_flag = 1;
            atomicOr(&g_status, ERR_EPILOGUE);
          }
          alive = false;
          break;
        }
        uint32_t v[32];
        if (has_cols) {
          ptx::tc_fence_after_sync();
          ptx::tc_ld_32x32b_x32(tmem_base + p * TOK + col0 + ((uint32_t)(q * 32) << 16), v);
          ptx::tc_wait_ld();
          ptx::tc_fence_before_sync();
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&ctl->part_empty[p]);      // the tensor core may overwrite this partial
        if (has_cols) {
          const float4* srow = reinterpret_cast<const float4*>(chunks + cs * S::CHUNK_FLOATS + ki * TOK + col0);
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            const float4 sc = srow[j4];                // same address in every lane: broadcast
            acc[j4 * 4 + 0] = fmaf(__uint_as_float(v[j4 * 4 + 0]), sc.x, acc[j4 * 4 + 0]);
            acc[j4 * 4 + 1] = fmaf(__uint_as_float(v[j4 * 4 + 1]), sc.y, acc[j4 * 4 + 1]);
            acc[j4 * 4 + 2] = fmaf(__uint_as_float(v[j4 * 4 + 2]), sc.z, acc[j4 * 4 + 2]);
            acc[j4 * 4 + 3] = fmaf(__uint_as_float(v[j4 * 4 + 3]), sc.w, acc[j4 * 4 + 3]);
          }
        }
        if (ki == CH_KT - 1 || kt == kt_count - 1) {          // done with this scale chunk
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&ctl->chunk_empty[cs]);
          ++c;
        }
      }
      if (!alive) break;
      if (S::GROUPS == 2) {
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&ctl->turn[egroup ^ 1]);
      }
      // output: this warp's 32 tokens x 32 n, 16 tokens at a time through its 1 KB tile, 128-bit stores (4 lanes per
      // 64-byte row piece)
      if (col0 < ti.valid) {
        OutT* dst = d + (int64_t)(ti.row0 + col0) * n + (ti.nt * TILE_N + q * 32);
#pragma unroll
        for (int h = 0; h < 32 / EPI_TOK; ++h) {
#pragma unroll
          for (int j = 0; j < EPI_TOK; ++j) stage_warp[j * 32 + lane] = out_from_f32<OutT>(acc[h * EPI_TOK + j]);
          __syncwarp();
#pragma unroll
          for (int it = 0; it < EPI_TOK / 8; ++it) {
            const int tok = it * 8 + (lane >> 2);
            const uint4 val = *reinterpret_cast<const uint4*>(stage_warp + tok * 32 + part * 8);
            const int row = col0 + h * EPI_TOK + tok;
            if (row < ti.valid) *reinterpret_cast<uint4*>(dst + (int64_t)(h * EPI_TOK + tok) * n + part * 8) = val;
          }
          __syncwarp();
        }
      }
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    ptx::tmem_dealloc(tmem_base, S::TMEM_COLS);
  }
  if (!wait_at_start) pdl_wait_prior_grid();   // do not complete before the preceding kernel of this call has
}

template <typename OutT, class S>
__global__ void __launch_bounds__(S::THREADS, 1)
fp8_blockwise_grouped_mm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x16,
                                const __grid_constant__ CUtensorMap map_x32, const __grid_constant__ CUtensorMap map_x64,
                                const __grid_constant__ CUtensorMap map_x128, const float* __restrict__ scales_a,
                                const float* __restrict__ scales_b, OutT* __restrict__ d,
                                const int* __restrict__ problem_sizes, const int* __restrict__ expert_offsets,
                                int num_experts, int n, int k, int min_rows, int max_rows, int wait_at_start, int group) {
  blockwise_cta<OutT, S>(map_w, map_x16, map_x32, map_x64, map_x128, scales_a, scales_b, d, problem_sizes, expert_offsets,
                         num_experts, n, k, min_rows, max_rows, wait_at_start, group, (int)blockIdx.x, (int)gridDim.x);
}

// The 64-token and the 128-token shape in one launch (both run 20 warps): CTAs [0, small_ctas) serve the experts with
// 33..64 rows, the others those with 65 rows and more.  The hardware starts CTAs in index order, so the second shape
// takes the SMs as the first runs out of items — what two chained launches did, for one launch (and, when a bucket is
// empty, one pass of empty CTAs over every SM) less per call.
template <typename OutT>
__global__ void __launch_bounds__(ShapeSmall::THREADS, 1)
fp8_blockwise_two_shapes_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x16,
                                const __grid_constant__ CUtensorMap map_x32, const __grid_constant__ CUtensorMap map_x64,
                                const __grid_constant__ CUtensorMap map_x128, const float* __restrict__ scales_a,
                                const float* __restrict__ scales_b, OutT* __restrict__ d,
                                const int* __restrict__ problem_sizes, const int* __restrict__ expert_offsets,
                                int num_experts, int n, int k, int small_ctas, int wait_at_start, int group) {
  static_assert(ShapeSmall::THREADS == ShapeFull::THREADS, "the two shapes share one block size");
  if ((int)blockIdx.x < small_ctas)
    blockwise_cta<OutT, ShapeSmall>(map_w, map_x16, map_x32, map_x64, map_x128, scales_a, scales_b, d, problem_sizes,
                                    expert_offsets, num_experts, n, k, 33, 64, wait_at_start, group, (int)blockIdx.x,
                                    small_ctas);
  else
    blockwise_cta<OutT, ShapeFull>(map_w, map_x16, map_x32, map_x64, map_x128, scales_a, scales_b, d, problem_sizes,
                                   expert_offsets, num_experts, n, k, 65, 0x7fffffff, wait_at_start, group,
                                   (int)blockIdx.x - small_ctas, (int)gridDim.x - small_ctas);
}

struct LaunchArgs {
  const void* a;
  const void* b;
  const float* sa;
  const float* sb;
  void* d;
  const int32_t* ps;
  const int32_t* eo;
  int num_experts;
  int64_t num_rows;
  int n, k;
  cudaStream_t stream;
};

// weight tiles per work item: the per-item work of every role (decode) is spread over ~8 K blocks
static int tiles_per_item(int k) {
  const int kt_count = k / TILE_K;
  const int group = (8 + kt_count - 1) / kt_count;
  return group < 1 ? 1 : group;
}

static int make_maps(const LaunchArgs& c, CUtensorMap* map_w, CUtensorMap (&map_x)[4]) {
  int rc = make_tensormap_u8_sw128(map_w, c.b, (uint64_t)c.num_experts * c.n, (uint64_t)c.k, TILE_N);
  if (rc != ES_B200_OK) return rc;
  const uint32_t boxes[4] = {16, 32, 64, 128};
  for (int i = 0; i < 4; ++i) {
    rc = make_tensormap_u8_sw128(&map_x[i], c.a, (uint64_t)c.num_rows, (uint64_t)c.k, boxes[i]);
    if (rc != ES_B200_OK) return rc;
  }
  return ES_B200_OK;
}

// CTAs for one shape: one per SM, fewer when the host-known upper bound of its item count is smaller
template <class S>
static int ctas_for(const LaunchArgs& c, int group, int sm_count) {
  const int64_t max_items = ((c.num_rows + S::TOK_TILE - 1) / S::TOK_TILE + c.num_experts) *
                            (int64_t)((c.n / TILE_N + group - 1) / group);
  return (int)(max_items < sm_count ? max_items : sm_count);
}

template <typename Kernel>
static int configure(Kernel kernel, size_t smem_bytes, bool (&configured)[64]) {
  int dev = 0;
  ES_CUDA_TRY(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    ES_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
    configured[dev & 63] = true;
  }
  return ES_B200_OK;
}

static void pdl_config(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr, int grid, int threads, size_t smem,
                       cudaStream_t stream) {
  *cfg = {};
  cfg->gridDim = dim3(grid);
  cfg->blockDim = dim3(threads);
  cfg->dynamicSmemBytes = smem;
  cfg->stream = stream;
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg->attrs = attr;
  cfg->numAttrs = 1;
}

// the <= 32-row shape (13 warps), always the first kernel of a call
template <typename OutT>
int launch_tiny(const LaunchArgs& c) {
  using S = ShapeTiny;
  DeviceInfo info;
  int rc = get_device_info(&info);
  if (rc != ES_B200_OK) return rc;
  CUtensorMap map_w, map_x[4];
  rc = make_maps(c, &map_w, map_x);
  if (rc != ES_B200_OK) return rc;
  auto kernel = fp8_blockwise_grouped_mm_kernel<OutT, S>;
  static bool configured[64] = {false};
  rc = configure(kernel, S::SMEM_BYTES, configured);
  if (rc != ES_B200_OK) return rc;
  const int group = tiles_per_item(c.k);
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[1];
  pdl_config(&cfg, attr, ctas_for<S>(c, group, info.sm_count), S::THREADS, S::SMEM_BYTES, c.stream);
  ES_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, map_w, map_x[0], map_x[1], map_x[2], map_x[3], c.sa, c.sb,
                                 static_cast<OutT*>(c.d), c.ps, c.eo, c.num_experts, c.n, c.k, 1, 32, 1, group));
  return ES_B200_OK;
}

// the 33..64-row and the >= 65-row shapes in one launch; want_full = false leaves the first alone
template <typename OutT>
int launch_small_and_full(const LaunchArgs& c, bool want_full) {
  DeviceInfo info;
  int rc = get_device_info(&info);
  if (rc != ES_B200_OK) return rc;
  CUtensorMap map_w, map_x[4];
  rc = make_maps(c, &map_w, map_x);
  if (rc != ES_B200_OK) return rc;
  auto kernel = fp8_blockwise_two_shapes_kernel<OutT>;
  constexpr size_t SMEM = ShapeSmall::SMEM_BYTES > ShapeFull::SMEM_BYTES ? ShapeSmall::SMEM_BYTES : ShapeFull::SMEM_BYTES;
  static bool configured[64] = {false};
  rc = configure(kernel, SMEM, configured);
  if (rc != ES_B200_OK) return rc;
  const int group = tiles_per_item(c.k);
  const int small_ctas = ctas_for<ShapeSmall>(c, group, info.sm_count);
  const int full_ctas = want_full ? ctas_for<ShapeFull>(c, group, info.sm_count) : 0;
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[1];
  pdl_config(&cfg, attr, small_ctas + full_ctas, ShapeSmall::THREADS, SMEM, c.stream);
  ES_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, map_w, map_x[0], map_x[1], map_x[2], map_x[3], c.sa, c.sb,
                                 static_cast<OutT*>(c.d), c.ps, c.eo, c.num_experts, c.n, c.k, small_ctas, 0, group));
  return ES_B200_OK;
}

template <typename OutT>
int launch_buckets(const void* a, const void* b, const float* sa, const float* sb, void* d, const int32_t* ps,
                   const int32_t* eo, int num_experts, int64_t num_rows, int n, int k, cudaStream_t stream) {
  // The <= 32-row shape first, then the two larger shapes in one launch, chained with programmatic dependent launch;
  // every CTA filters the experts in its own scan.  A bucket that even the host-known upper bound of rows per expert
  // cannot reach gets no CTAs.
  const LaunchArgs c = {a, b, sa, sb, d, ps, eo, num_experts, num_rows, n, k, stream};
  int rc = launch_tiny<OutT>(c);
  if (rc != ES_B200_OK || num_rows <= 32) return rc;
  return launch_small_and_full<OutT>(c, num_rows > 64);
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
  es_b200::NvtxRange nvtx_range("es_b200_fp8_blockwise_grouped_mm");
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
  ES_REQUIRE(aligned16(a) && aligned16(b) && aligned16(d), "a, b and d must be 16-byte aligned");
  ES_REQUIRE((reinterpret_cast<uintptr_t>(scales_a) & 3u) == 0 && (reinterpret_cast<uintptr_t>(scales_b) & 3u) == 0,
             "scales must be 4-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (out_dtype == ES_B200_BF16)
    return bw::launch_buckets<__nv_bfloat16>(a, b, scales_a, scales_b, d, problem_sizes, expert_offsets, num_experts,
                                             num_rows, n, k, s);
  return bw::launch_buckets<__half>(a, b, scales_a, scales_b, d, problem_sizes, expert_offsets, num_experts, num_rows,
                                    n, k, s);
}
