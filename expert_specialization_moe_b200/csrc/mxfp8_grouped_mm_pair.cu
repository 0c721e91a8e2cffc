// MXFP8 block-scaled grouped GEMM for sm_100a on CTA PAIRS, for experts with many token rows:
// tcgen05.mma.cta_group::2 with M = 256 and a weight-stationary K step over up to 384 token rows.
//
// Same mapping as the single-CTA kernel (weights on the MMA M axis, the expert's token rows on the runtime-sized
// MMA N axis).  Two CTAs of a cluster share every work item: each CTA holds 128 of the 256 weight rows and HALF of
// the token rows in its own shared memory, and the pair's tensor cores exchange the token halves (no multicast
// load anywhere).  One work item covers up to 384 token rows as two sub-tiles of <=192 rows with one accumulator
// each: every 16 KB weight stage that a CTA pulls through L2 feeds BOTH sub-tiles' MMAs.  Per CTA and K step that
// is 16 KB of weights + 2 x 12 KB of tokens for 128 x 384 x 128 MACs — 2.4x fewer operand bytes per FLOP than
// 128 x 128 single-CTA tiles, which is what bounds experts with many rows (the operand feed, not the tensor pipe).
// Sub-tiles are 192 rows because two 192-column fp32 accumulators plus per-stage scale slots fit the 512 TMEM
// columns, and the second sub-tile starts on a 64-row boundary of the 128-row scale atoms, which a TMEM column
// offset addresses.
//
//   warp 0    producer (both CTAs): per K step lanes 0..4 each issue one TMA load (own weight rows, own halves of
//             the two token sub-tiles, own weight scale atom, the item's token scale atoms); all completion bytes
//             are credited to the leader CTA's barrier
//   warp 1    TMEM allocation (both CTAs); in the leader CTA one lane issues sub-tile 0's four tcgen05.mma per K step
//   warps 2-17  epilogue (both CTAs): own 128 accumulator lanes -> registers (bf16/fp16) -> accumulators handed back
//               -> global; four warps per TMEM lane quadrant share the 32-column chunks of both accumulators
//   warp 18     leader CTA, one lane: sub-tile 1's four tcgen05.mma per K step
//   warp 19     leader CTA, one lane: the K step's four tcgen05.cp (scales smem -> TMEM of both CTAs)
//
// Work items come from the bucket's work counter in the caller's scratch (atomicAdd by lane 0 of the leader's producer
// warp; round-robin over the clusters without scratch).  The index travels to every other role of BOTH CTAs through a
// four-deep queue: the leader writes it into its own and its partner's shared memory and arrives on both CTAs'
// q_full barriers; every consuming role arrives on the leader's q_empty barrier.  Two launches of this kernel may
// serve one call (a small one in front of the streaming kernels, a full-width one behind them): they drain the same
// counter.
//
// Three issuing lanes instead of one because a tcgen05 instruction costs the thread that issues it ~90 cycles (mma)
// or ~65 cycles (cp) whatever its size (measured: the K step of a single issuing lane took the same ~1000 cycles with
// N = 64 and with N = 256 MMAs), while the tensor pipe needs 96 cycles for a 256 x 192 x 32 MMA.  One lane issuing
// 8 MMAs + 4 copies + a commit per K step is therefore issue-bound at ~1260 cycles for 768 cycles of tensor work;
// split three ways every lane stays below the pipe's time.  The lanes meet only through mbarriers: the copy lane
// commits to sf_ready[stage], both MMA lanes commit to empty[stage] (2 arrivals) and to their accumulator's barrier.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "epilogue.cuh"
#include "grouped_mm_call.cuh"
#include "sm100_ptx.cuh"
#include "tensormap.cuh"

namespace es_b200 {
namespace mm2 {

constexpr int THREADS = 640;
constexpr int TILE_N = 128;      // weight rows per CTA (the pair covers 256)
constexpr int TILE_K = 128;
constexpr int SUB_TILE = 192;    // token rows per accumulator (MMA N, runtime multiple of 16)
constexpr int TOK_TILE = 2 * SUB_TILE;   // token rows per work item
constexpr int STAGES = 5;
constexpr int W_BYTES = TILE_N * TILE_K;               // 16384
constexpr int X_BYTES = (SUB_TILE / 2) * TILE_K;       // 12288: this CTA's half of one token sub-tile
constexpr int SFW_BYTES = 512;
constexpr int SFX_BYTES = 1536;                        // three 512-byte atoms cover 384 rows
constexpr int STAGE_BYTES = 43008;                     // 42 KB: W | X0 | X1 | SFW | SFX  (multiple of 1024)
static_assert(W_BYTES + 2 * X_BYTES + SFW_BYTES + SFX_BYTES <= STAGE_BYTES, "stage layout");
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t ACC_COLS = 192;        // accumulators at columns [0,192) and [192,384)
constexpr uint32_t SF_COL0 = 384;         // per-stage scale slots of 16 columns: 4 (weights) + 12 (tokens)
constexpr uint32_t SF_SLOT_COLS = 16;
static_assert(SF_COL0 + STAGES * SF_SLOT_COLS <= TMEM_COLS, "TMEM budget");

constexpr uint32_t ERR_PRODUCER = 0x10u, ERR_MMA = 0x20u, ERR_EPILOGUE = 0x40u;
constexpr uint32_t ERR_SCALE_COPY = 0x100u;
constexpr int EPI_WARPS = 16;                              // 4 TMEM lane quadrants x 4 warps
constexpr int EPI_BYTES_PER_WARP = 8 * 32 * 2;             // 512 bytes: 8 tokens x 32 n (scattered output only)
constexpr int MMA_B_WARP = 2 + EPI_WARPS;                  // 18
constexpr int COPY_WARP = MMA_B_WARP + 1;                  // 19
constexpr int QUEUE_DEPTH = 4;
// readers of a queue slot: in the leader CTA the two MMA lanes, the copy lane and 16 epilogue warps; in the partner CTA
// the producer warp and 16 epilogue warps
constexpr int Q_CONSUMERS = (3 + EPI_WARPS) + (1 + EPI_WARPS);

struct SharedCtl {
  uint64_t full[STAGES];        // used in the leader CTA only
  uint64_t empty[STAGES];       // 2 arrivals: one commit from each MMA lane
  uint64_t sf_ready[STAGES];    // leader only: the stage's scales are in the TMEM of both CTAs
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];       // used in the leader CTA only (32 arrivals: 16 epilogue warps x 2 CTAs)
                                // index = accumulator (sub-tile 0 / 1)
  uint64_t q_full[QUEUE_DEPTH];   // 1 arrival from the leader's producer lane (in the partner CTA also the 8 bytes of
                                  // the entry, sent with the arrival): q_item[slot] is written
  uint64_t q_empty[QUEUE_DEPTH];  // leader only: Q_CONSUMERS arrivals, every consuming role of both CTAs has read it
  int2 q_item[QUEUE_DEPTH];       // x: work item index, or -1: no more work; y: the item's expert (found once, by
                                  // the leader's producer lane)
  uint32_t tmem_base;
  int abort_flag;
  int warp_sums[32];
  // [0, E]: exclusive prefix of the experts' item counts; behind it the per-expert tables (fill_expert_table)
  int table[ES_B200_MAX_EXPERTS + 1];
};

constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES + EPI_WARPS * EPI_BYTES_PER_WARP + sizeof(SharedCtl);
static_assert(SMEM_BYTES <= 232448, "shared memory of one CTA per SM");

__device__ uint32_t g_status = 0;

struct TileInfo {
  int e, tt, np;
  int valid;       // token rows of this item that belong to the expert (<= 384)
  int n0, n1;      // MMA N of the two sub-tiles (multiples of 16; n1 == 0 when the item has <= 192 rows)
  int v0, v1;      // valid rows of the two sub-tiles
  int row0;        // first token row of the item in a / d
  int atom0;       // first 128-row scale atom of the item inside the expert (items start on atom boundaries)
  int n_atoms;     // 1..3 atoms cover the item's valid rows
};

__device__ __forceinline__ TileInfo decode_tile(int t, int e, const ExpertTable& tab, int n, int n_pairs) {
  TileInfo ti;
  ti.e = e;
  const int i = t - tab.prefix[e];
  const int m = tab.m(e);
  const int token_tiles = (m + TOK_TILE - 1) / TOK_TILE;
  // Consecutive items run at the same time on different CTA pairs and share one operand in L2 while they sweep the
  // other: the swept operand should be the SMALLER one.  Token tile fastest (items share a weight slab and sweep the
  // expert's m x k tokens) unless the expert has more token rows than weight rows; then weight pair fastest (items
  // share a token tile and sweep the n x k weights).
  if (m <= n) {
    ti.np = i / token_tiles;
    ti.tt = i - ti.np * token_tiles;
  } else {
    ti.tt = i / n_pairs;
    ti.np = i - ti.tt * n_pairs;
  }
  const int r_local = ti.tt * TOK_TILE;
  const int rem = m - r_local;
  ti.valid = rem < TOK_TILE ? rem : TOK_TILE;
  ti.v0 = ti.valid < SUB_TILE ? ti.valid : SUB_TILE;
  ti.v1 = ti.valid - ti.v0;
  ti.n0 = (ti.v0 + 15) & ~15;
  ti.n1 = (ti.v1 + 15) & ~15;
  ti.row0 = tab.row0(e) + r_local;
  ti.atom0 = r_local >> 7;
  ti.n_atoms = (ti.valid + 127) >> 7;
  return ti;
}

__device__ __forceinline__ int box_index(int half_rows) {   // token tensor maps: boxes of 8 / 16 / 32 / 64 / 96 rows
  return half_rows <= 8 ? 0 : half_rows <= 16 ? 1 : half_rows <= 32 ? 2 : half_rows <= 64 ? 3 : 4;
}
__device__ __forceinline__ uint32_t box_rows_of(int idx) {
  return idx == 0 ? 8u : idx == 1 ? 16u : idx == 2 ? 32u : idx == 3 ? 64u : 96u;
}

struct Maps {
  CUtensorMap w;        // weights  [E*N, K] bytes, box 128 rows x 128 B, 128-byte swizzle
  CUtensorMap x[5];     // tokens   [T, K]   bytes, boxes of 8 / 16 / 32 / 64 / 96 rows
  CUtensorMap sfw;      // weight scale atoms, 512-byte records
  CUtensorMap sfx;      // token scale atoms as [128-row block][K block] of 512-byte records; box = 3 row blocks
};

template <typename OutT, bool HOLD>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
mxfp8_grouped_mm_pair_kernel(const __grid_constant__ Maps maps, OutT* __restrict__ d,
                             const int* __restrict__ problem_sizes, const int* __restrict__ expert_offsets,
                             const int* __restrict__ blockscale_offsets, int num_experts, int n, int k, int min_rows,
                             int wait_at_start, const __grid_constant__ RowScatter scatter, uint32_t* counters,
                             int last_of_call, uint32_t earlier_ctas) {
  if (!wait_at_start) pdl_launch_dependents();   // not the first kernel of its call: the next one may launch at once
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_stage = smem + (size_t)STAGES * STAGE_BYTES;      // 16 x 512 bytes, one per epilogue warp
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(epi_stage + EPI_WARPS * EPI_BYTES_PER_WARP);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();      // 0 = leader (issues the MMAs), 1 = peer
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&ctl->full[s], 1);
      ptx::mbar_init(&ctl->empty[s], 2);
      ptx::mbar_init(&ctl->sf_ready[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&ctl->tmem_full[a], 1);
      ptx::mbar_init(&ctl->tmem_empty[a], 2 * EPI_WARPS);
    }
    for (int q = 0; q < QUEUE_DEPTH; ++q) {
      ptx::mbar_init(&ctl->q_full[q], 1);
      ptx::mbar_init(&ctl->q_empty[q], Q_CONSUMERS);
    }
    ctl->abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&maps.w);
    ptx::prefetch_tensormap(&maps.sfw);
    ptx::prefetch_tensormap(&maps.sfx);
#pragma unroll
    for (int i = 0; i < 5; ++i) ptx::prefetch_tensormap(&maps.x[i]);
  }
  // This kernel is chained with the single-CTA kernels of the same call by programmatic dependent launch — behind
  // them, and for a large call also in front of them with a capped grid.  The first kernel of the call waits for
  // everything before it (griddepcontrol.wait) before it lets the others start, so the operands are final; the
  // kernels write disjoint rows of d.  A launch that is not first therefore starts on SMs as they become free; stream
  // order for whatever follows the call is kept at the end (end_of_kernel).
  // (a launch that is not first has let the next kernel of the call launch at entry; the first one does so after its
  // prologue, below)
  if (wait_at_start) pdl_wait_prior_grid();
  const int n_tiles = n / TILE_N;
  const int n_pairs = (n_tiles + 1) >> 1;
  // only experts with at least min_rows rows belong to this kernel (the single-CTA kernel takes the others)
  // (an expert whose scales do not start on a 128-row atom cannot be addressed: reported and skipped)
  block_exclusive_scan(num_experts, ctl->table, ctl->warp_sums, [&](int e) {
    const int m = problem_sizes[e * 3];
    if (!(m > 0 && m >= min_rows)) return 0;
    if ((blockscale_offsets[e] & 127) != 0) {
      atomicOr(&g_status, ERR_SCALE_OFFSET_BIT);
      return 0;
    }
    return ((m + TOK_TILE - 1) / TOK_TILE) * n_pairs;
  });
  // A launch without work (the host only knows an upper bound of the rows per expert) ends here, before it holds
  // TMEM or has signalled its partner CTA; both CTAs of a pair see the same total.
  if (ctl->table[num_experts] == 0) {
    if (wait_at_start) pdl_launch_dependents();
    end_of_kernel(counters, wait_at_start != 0, last_of_call != 0, earlier_ctas, scatter.meta != nullptr, &g_status);
    return;
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(&ctl->tmem_base, TMEM_COLS);
    ptx::tmem_relinquish_pair();
  }
  const ExpertTable tab = fill_expert_table(ctl->table, num_experts, problem_sizes, expert_offsets, blockscale_offsets);
  // barriers, TMEM and tables of both CTAs must exist before either CTA signals the other
  ptx::tc_fence_before_sync();
  ptx::cluster_sync();
  ptx::tc_fence_after_sync();
  if (wait_at_start) pdl_launch_dependents();

  const uint32_t tmem_base = ctl->tmem_base;
  const int total_tiles = tab.prefix[num_experts];
  const int kt_count = k / TILE_K;
  const int sfw_atoms_per_expert = n_tiles * kt_count;
  volatile int* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (warp 0 of each CTA)
    // The whole warp walks the work list; per K step lanes 0..4 each issue ONE of the stage's loads in the same
    // instruction (a TMA issue costs the issuing thread ~80 cycles, five in a row would be a third of a stage time).
    int s = 0, qs = 0;
    uint32_t ph = 0, qph = 0;
    uint32_t* counter = counters ? counters + 2 : nullptr;
    int t_mine = 0;                   // leader, lane 0: the index that goes out next
    if (rank == 0 && lane == 0) t_mine = counter ? (int)atomicAdd(counter, 1u) : pair;
    while (true) {
      // the leader publishes the next item (or the end mark) to both CTAs; the partner's producer reads its copy
      int t = -1, e = 0;
      bool q_ok = true;
      if (rank == 0) {
        if (lane == 0) {
          q_ok = ptx::mbar_wait(&ctl->q_empty[qs], qph ^ 1u, abort_flag);
          if (q_ok) {
            t = t_mine < total_tiles ? t_mine : -1;
            e = t >= 0 ? upper_bound_expert(tab.prefix, num_experts, t) : 0;
            ctl->q_item[qs] = make_int2(t, e);
            ptx::mbar_arrive(&ctl->q_full[qs]);
            ptx::send_u64_to_cluster_cta(&ctl->q_item[qs], &ctl->q_full[qs], 1, (uint32_t)t, (uint32_t)e);
            // the following index is requested now; its round trip to L2 hides behind this item's loads
            if (t >= 0) t_mine = counter ? (int)atomicAdd(counter, 1u) : t_mine + num_pairs;
          }
        }
        q_ok = __shfl_sync(0xffffffffu, (int)q_ok, 0) != 0;
        t = __shfl_sync(0xffffffffu, t, 0);
        e = __shfl_sync(0xffffffffu, e, 0);
      } else {
        q_ok = __all_sync(0xffffffffu, ptx::mbar_wait_cluster(&ctl->q_full[qs], qph, abort_flag));
        if (q_ok) {
          t = ctl->q_item[qs].x;
          e = ctl->q_item[qs].y;
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive_cluster(&ctl->q_empty[qs], 0);
        }
      }
      if (++qs == QUEUE_DEPTH) { qs = 0; qph ^= 1u; }
      if (!q_ok) {
        if (lane == 0) {
          *abort_flag = 1;
          atomicOr(&g_status, ERR_PRODUCER);
        }
        break;
      }
      if (t < 0) break;
      const TileInfo ti = decode_tile(t, e, tab, n, n_pairs);
      const int half0 = ti.n0 >> 1, half1 = ti.n1 >> 1;     // token rows of each sub-tile held by each CTA
      const int xi0 = box_index(half0), xi1 = box_index(half1);
      const uint32_t tx = 2u * (W_BYTES + box_rows_of(xi0) * TILE_K + (ti.n1 ? box_rows_of(xi1) * TILE_K : 0u) +
                                SFW_BYTES + SFX_BYTES);
      int nt = ti.np * 2 + (int)rank;
      const int w_row = ti.e * n + nt * TILE_N;             // may run past the expert when n/128 is odd: not stored
      if (nt >= n_tiles) nt = n_tiles - 1;                  // keep the scale-atom load inside the buffer
      const int sfw_atom = ti.e * sfw_atoms_per_expert + nt * kt_count;
      const int bs_off = tab.scale0(ti.e);                  // a multiple of 128 (checked by the scan)
      const int sfx_atom_row = (bs_off >> 7) + ti.atom0;
      // this lane's load: 0 weights, 1 tokens of sub-tile 0, 2 tokens of sub-tile 1, 3 weight scales, 4 the three
      // token scale atoms of the item (one load: the lanes of a warp issue their loads one after the other, ~75
      // cycles each, and the producer's issue time per K step is part of every stage's turnaround)
      const bool active = lane == 0 || lane == 1 || (lane == 2 && ti.n1 > 0) || lane == 3 || lane == 4;
      const CUtensorMap* my_map = lane == 0 ? &maps.w : lane == 1 ? &maps.x[xi0] : lane == 2 ? &maps.x[xi1]
                                  : lane == 3 ? &maps.sfw : &maps.sfx;
      const uint32_t my_off = lane == 0 ? 0u : lane == 1 ? (uint32_t)W_BYTES : lane == 2 ? (uint32_t)(W_BYTES + X_BYTES)
                              : lane == 3 ? (uint32_t)(W_BYTES + 2 * X_BYTES)
                                          : (uint32_t)(W_BYTES + 2 * X_BYTES + SFW_BYTES);
      const int my_c1 = lane == 0 ? w_row : lane == 1 ? ti.row0 + (int)rank * half0
                        : lane == 2 ? ti.row0 + SUB_TILE + (int)rank * half1
                        : lane == 3 ? sfw_atom : sfx_atom_row;
      const uint64_t my_hint = lane < 3 ? ptx::kL2EvictLast : ptx::kL2EvictNormal;
      bool ok = true;
      for (int kt = 0; kt < kt_count; ++kt) {
        ok = __all_sync(0xffffffffu, ptx::mbar_wait(&ctl->empty[s], ph ^ 1u, abort_flag));
        if (!ok) break;
        uint8_t* stage = smem + (size_t)s * STAGE_BYTES;
        if (rank == 0 && lane == 0) ptx::mbar_arrive_expect_tx(&ctl->full[s], tx);
        __syncwarp();
        if (active)
          ptx::tma_load_2d_pair_hint(stage + my_off, my_map, &ctl->full[s],
                                     lane < 3 ? kt * TILE_K : lane == 3 ? 0 : kt * 128,
                                     lane == 3 ? my_c1 + kt : my_c1, my_hint);
        if (++s == STAGES) { s = 0; ph ^= 1u; }
      }
      if (!ok) {
        if (lane == 0) {
          *abort_flag = 1;
          atomicOr(&g_status, ERR_PRODUCER);
        }
        break;
      }
    }
  } else if (warp == 1 || warp == MMA_B_WARP) {
    // ------------------------------------------------------------------ MMA issue (leader CTA): warp 1 issues the
    // MMAs of sub-tile 0 into accumulator 0, warp 18 those of sub-tile 1 into accumulator 1
    if (lane == 0 && rank == 0) {
      const int sub = warp == 1 ? 0 : 1;
      int s = 0, qs = 0;
      uint32_t ph = 0, qph = 0;
      uint32_t acc_ph = 0;             // phase of this accumulator's empty barrier (advances once per use)
      bool ok = true;
      while (ok) {
        if (!ptx::mbar_wait(&ctl->q_full[qs], qph, abort_flag)) {
          *abort_flag = 1;
          atomicOr(&g_status, ERR_MMA);
          break;
        }
        const int t = ctl->q_item[qs].x;
        const int e = ctl->q_item[qs].y;
        ptx::mbar_arrive(&ctl->q_empty[qs]);
        if (++qs == QUEUE_DEPTH) { qs = 0; qph ^= 1u; }
        if (t < 0) break;
        const TileInfo ti = decode_tile(t, e, tab, n, n_pairs);
        const uint32_t n_mma = sub == 0 ? ti.n0 : ti.n1;
        const uint32_t d_acc = tmem_base + sub * ACC_COLS;
        for (int kt = 0; ok && kt < kt_count; ++kt) {
          if (!ptx::mbar_wait(&ctl->full[s], ph, abort_flag)) { ok = false; break; }
          if (n_mma > 0) {
            if (!ptx::mbar_wait(&ctl->sf_ready[s], ph, abort_flag)) { ok = false; break; }
            if (kt == 0) {   // the previous item's epilogue must have drained this accumulator
              if (!ptx::mbar_wait(&ctl->tmem_empty[sub], acc_ph ^ 1u, abort_flag)) { ok = false; break; }
              acc_ph ^= 1u;
            }
            ptx::tc_fence_after_sync();
            const uint32_t stage = ptx::smem_u32(smem + (size_t)s * STAGE_BYTES);
            const uint32_t sfw_t = tmem_base + SF_COL0 + s * SF_SLOT_COLS;
            // sub-tile 1 starts 192 rows = 6 scale columns into the item's block of token scales
            const uint32_t sfx_t = sfw_t + 4 + sub * 6;
            const uint64_t a_desc = ptx::make_desc_k_sw128(stage);
            const uint64_t b_desc = ptx::make_desc_k_sw128(stage + W_BYTES + sub * X_BYTES);
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j)
              ptx::tc_mma_mxf8_pair(d_acc, a_desc + 2 * j, b_desc + 2 * j, ptx::make_idesc_mxf8(2 * TILE_N, n_mma, j, j),
                                    sfw_t | (j << 30), sfx_t | (j << 30), (kt | j) != 0 ? 1u : 0u);
          }
          ptx::tc_commit_pair(&ctl->empty[s], 3);       // this lane's share: both CTAs may refill once both have
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (!ok) {
          *abort_flag = 1;
          atomicOr(&g_status, ERR_MMA);
          break;
        }
        if (n_mma > 0) ptx::tc_commit_pair(&ctl->tmem_full[sub], 3);     // this accumulator is complete in both CTAs
      }
    }
  } else if (warp == COPY_WARP) {
    // ------------------------------------------------------------------ scale copies (leader CTA, one lane)
    // Token rows 0..383 of the item = scale atoms 0..2: sub-tile 0 reads atoms 0 and 1, sub-tile 1 atoms 1 and 2.
    if (lane == 0 && rank == 0) {
      int s = 0, qs = 0;
      uint32_t ph = 0, qph = 0;
      bool ok = true;
      while (ok) {
        if (!ptx::mbar_wait(&ctl->q_full[qs], qph, abort_flag)) {
          *abort_flag = 1;
          atomicOr(&g_status, ERR_SCALE_COPY);
          break;
        }
        const int t = ctl->q_item[qs].x;
        const int e = ctl->q_item[qs].y;
        ptx::mbar_arrive(&ctl->q_empty[qs]);
        if (++qs == QUEUE_DEPTH) { qs = 0; qph ^= 1u; }
        if (t < 0) break;
        const TileInfo ti = decode_tile(t, e, tab, n, n_pairs);
        for (int kt = 0; kt < kt_count; ++kt) {
          if (!ptx::mbar_wait(&ctl->full[s], ph, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const uint32_t sf_smem = ptx::smem_u32(smem + (size_t)s * STAGE_BYTES) + W_BYTES + 2 * X_BYTES;
          const uint32_t sfw_t = tmem_base + SF_COL0 + s * SF_SLOT_COLS;
          ptx::tc_cp_sf_pair(sfw_t, ptx::make_desc_sf(sf_smem));
          ptx::tc_cp_sf_pair(sfw_t + 4, ptx::make_desc_sf(sf_smem + SFW_BYTES));
          if (ti.n_atoms > 1) ptx::tc_cp_sf_pair(sfw_t + 8, ptx::make_desc_sf(sf_smem + SFW_BYTES + 512));
          if (ti.n_atoms > 2) ptx::tc_cp_sf_pair(sfw_t + 12, ptx::make_desc_sf(sf_smem + SFW_BYTES + 1024));
          ptx::tc_commit_pair(&ctl->sf_ready[s], 1);    // leader's barrier, once the copies have landed in both TMEMs
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (!ok) {
          *abort_flag = 1;
          atomicOr(&g_status, ERR_SCALE_COPY);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs), 16 warps: four per
    // TMEM lane quadrant share the twelve 32-column chunks of an item's two accumulators, three each (two of one
    // accumulator and one of the other).  A warp reads its chunks of accumulator 0 into registers (converted), hands
    // accumulator 0 back, does the same for accumulator 1, and stores afterwards: both accumulators of an item
    // complete together, the MMA lanes get them back after ~two TMEM reads each instead of after the stores (which
    // take several thousand cycles per item), and the next item's MMAs run during the stores.
    //   slot 0: accumulator 0, columns 32 idx          slot 1: idx < 2 ? accumulator 0, columns 32 idx + 128
    //   slot 2: idx < 2 ? accumulator 1, columns 32 (idx + 2)              : accumulator 1, columns 32 (idx - 2)
    //                   : accumulator 1, columns 32 (idx - 2) + 128
    const int q = warp & 3;
    const int idx = (warp - 2) >> 2;      // 0..3 within the lane quadrant
    const bool low = idx < 2;
    const int col0 = idx * 32;
    const int col1 = low ? idx * 32 + 128 : (idx - 2) * 32;
    const int col2 = low ? (idx + 2) * 32 : (idx - 2) * 32 + 128;
    OutT* stage_warp = reinterpret_cast<OutT*>(epi_stage) + (warp - 2) * (EPI_BYTES_PER_WARP / 2);
    // HOLD = false (chosen by the host for one or two K steps per item): each chunk is stored right after it is read.
    // Such a call is bound by the output stores themselves (n x k is small against the m x n output) and holding only
    // adds concurrent load traffic to them (measured at k = 256: 1.03 ms held, 0.71 ms not).
    uint32_t full_ph = 0, qph = 0;        // both accumulators' barriers advance once per item that uses them
    uint32_t full1_ph = 0;
    int qs = 0;
    while (true) {
      const bool have = rank == 0 ? ptx::mbar_wait(&ctl->q_full[qs], qph, abort_flag)
                                  : ptx::mbar_wait_cluster(&ctl->q_full[qs], qph, abort_flag);
      if (!__all_sync(0xffffffffu, have)) {
        if (lane == 0) {
          *abort_flag = 1;
          atomicOr(&g_status, ERR_EPILOGUE);
        }
        break;
      }
      const int t = ctl->q_item[qs].x;
      const int e = ctl->q_item[qs].y;
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(&ctl->q_empty[qs], 0);   // leader's barrier
      if (++qs == QUEUE_DEPTH) { qs = 0; qph ^= 1u; }
      if (t < 0) break;
      const TileInfo ti = decode_tile(t, e, tab, n, n_pairs);
      const int nt = ti.np * 2 + (int)rank;
      const bool store = nt < n_tiles;
      const bool store_now = !HOLD && store;
      const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
      uint32_t held0[16], held1[16], held2[16];
      // which of this warp's chunks exist in this item (warp-uniform)
      const bool has0 = col0 < ti.n0;
      const bool has1 = low ? col1 < ti.n0 : col1 < ti.n1;
      const bool has2 = col2 < ti.n1;
      // token row (within the item) of each slot's first column
      const int tok0 = col0;
      const int tok1 = low ? col1 : SUB_TILE + col1;
      const int tok2 = SUB_TILE + col2;
      const int col_off = nt * TILE_N + q * 32;
      auto store_slot = [&](const uint32_t (&held)[16], int tok) {
        if (scatter.meta == nullptr) {
          uint16_t* out = reinterpret_cast<uint16_t*>(d + (int64_t)(ti.row0 + tok) * n + col_off);
          store_held_chunk_dense(held, out, n, ti.valid - tok, lane);
        } else {
          // lane l fetches the destination of token l of the chunk
          OutT* dest = scatter_row_ptr<OutT>(scatter, ti.row0 + tok + lane, tok + lane < ti.valid, n, col_off, &g_status);
          store_held_chunk_scatter<OutT>(held, stage_warp, dest, lane);
        }
      };
      bool got = ptx::mbar_wait(&ctl->tmem_full[0], full_ph, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) {
          *abort_flag = 1;
          atomicOr(&g_status, ERR_EPILOGUE);
        }
        break;
      }
      full_ph ^= 1u;
      ptx::tc_fence_after_sync();
      if (has0) {
        read_held_chunk<OutT>(lane_base + col0, held0);
        if (store_now) store_slot(held0, tok0);
      }
      if (low && has1) {
        read_held_chunk<OutT>(lane_base + col1, held1);
        if (store_now) store_slot(held1, tok1);
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(&ctl->tmem_empty[0], 0);     // leader's barrier
      if (ti.n1 > 0) {                                      // an item of <= 192 rows does not use accumulator 1
        got = ptx::mbar_wait(&ctl->tmem_full[1], full1_ph, abort_flag);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0) {
            *abort_flag = 1;
            atomicOr(&g_status, ERR_EPILOGUE);
          }
          break;
        }
        full1_ph ^= 1u;
        ptx::tc_fence_after_sync();
        if (!low && has1) {
          read_held_chunk<OutT>(lane_base + ACC_COLS + col1, held1);
          if (store_now) store_slot(held1, tok1);
        }
        if (has2) {
          read_held_chunk<OutT>(lane_base + ACC_COLS + col2, held2);
          if (store_now) store_slot(held2, tok2);
        }
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_cluster(&ctl->tmem_empty[1], 0);
      }
      if (HOLD && store) {
        if (has0) store_slot(held0, tok0);
        if (has1) store_slot(held1, tok1);
        if (has2) store_slot(held2, tok2);
      }
    }
  }

  // neither CTA may leave (or free TMEM) while its partner can still signal it or read its shared memory
  ptx::tc_fence_before_sync();
  ptx::cluster_sync();
  if (warp == 1) {
    __syncwarp();
    ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
  end_of_kernel(counters, wait_at_start != 0, last_of_call != 0, earlier_ctas, scatter.meta != nullptr, &g_status);
}

template <typename OutT, bool HOLD>
int launch_as(const mm::CallArgs& c, int min_rows, int cluster_cap, bool first_of_call, bool last_of_call,
              uint32_t* earlier_ctas) {
  DeviceInfo info;
  int rc = get_device_info(&info);
  if (rc != ES_B200_OK) return rc;
  const int kt_count = c.k / TILE_K;

  Maps maps;
  rc = make_tensormap_u8_sw128(&maps.w, c.b, (uint64_t)c.num_experts * c.n, (uint64_t)c.k, TILE_N);
  if (rc != ES_B200_OK) return rc;
  const uint32_t boxes[5] = {8, 16, 32, 64, 96};
  for (int i = 0; i < 5; ++i) {
    rc = make_tensormap_u8_sw128(&maps.x[i], c.a, (uint64_t)c.num_rows, (uint64_t)c.k, boxes[i]);
    if (rc != ES_B200_OK) return rc;
  }
  rc = make_tensormap_records512(&maps.sfw, c.sfb, (uint64_t)c.num_experts * (c.n / TILE_N) * kt_count);
  if (rc != ES_B200_OK) return rc;
  // whole 128-row atoms only; loads past the end read as zero (a map needs at least one row)
  const uint64_t sfx_rows = (uint64_t)(c.sfa_rows / 128);
  rc = make_tensormap_record_columns(&maps.sfx, c.sfa, sfx_rows ? sfx_rows : 1, (uint64_t)kt_count, 3);
  if (rc != ES_B200_OK) return rc;

  auto kernel = mxfp8_grouped_mm_pair_kernel<OutT, HOLD>;
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
  cfg.stream = c.stream;
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
  const int n_pairs = (c.n / TILE_N + 1) / 2;
  const int64_t max_tiles = ((c.num_rows + TOK_TILE - 1) / TOK_TILE + c.num_experts) * (int64_t)n_pairs;
  int max_clusters = resident_clusters[dev & 63];
  if (cluster_cap > 0 && cluster_cap < max_clusters) max_clusters = cluster_cap;
  const int clusters = (int)(max_tiles < max_clusters ? max_tiles : max_clusters);
  cfg.gridDim = dim3(2 * clusters);
  cfg.numAttrs = 2;
  ES_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, maps, static_cast<OutT*>(c.d), c.ps, c.eo, c.bo, c.num_experts, c.n, c.k,
                                 min_rows, first_of_call ? 1 : 0, *c.scatter, c.counters, last_of_call ? 1 : 0,
                                 *earlier_ctas));
  *earlier_ctas += 2u * (uint32_t)clusters;
  return ES_B200_OK;
}

// items of one or two K steps store each chunk as soon as it is read (see the epilogue)
template <typename OutT>
int launch(const mm::CallArgs& c, int min_rows, int cluster_cap, bool first_of_call, bool last_of_call,
           uint32_t* earlier_ctas) {
  return c.k / TILE_K > 2 ? launch_as<OutT, true>(c, min_rows, cluster_cap, first_of_call, last_of_call, earlier_ctas)
                          : launch_as<OutT, false>(c, min_rows, cluster_cap, first_of_call, last_of_call, earlier_ctas);
}

int launch_bf16(const mm::CallArgs& c, int min_rows, int max_clusters, bool first_of_call, bool last_of_call,
                uint32_t* earlier_ctas) {
  return launch<__nv_bfloat16>(c, min_rows, max_clusters, first_of_call, last_of_call, earlier_ctas);
}
int launch_fp16(const mm::CallArgs& c, int min_rows, int max_clusters, bool first_of_call, bool last_of_call,
                uint32_t* earlier_ctas) {
  return launch<__half>(c, min_rows, max_clusters, first_of_call, last_of_call, earlier_ctas);
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

}  // namespace mm2
}  // namespace es_b200
