// MXFP8 block-scaled grouped GEMM for sm_100a, hand-written around tcgen05.mma.kind::mxf8f6f4.block_scale.
//
// Per expert e:  d[off_e + i, n] = sum_k a[off_e + i, k] * 2^(sfa-127) * b[e, n, k] * 2^(sfb-127), fp32 accumulate.
//
// This file: the two STREAMING shapes (experts with few rows, whose weights are read from HBM exactly once and
// dominate the bytes) and the dispatcher that chains them with the CTA-pair kernel (mxfp8_grouped_mm_pair.cu).
//
// Mapping ("swap-AB"): the 128 rows of the tensor-core tile are 128 WEIGHT rows (output columns n), the token rows
// of the expert sit on the MMA N axis.  N of tcgen05.mma can be any multiple of 16 up to 256, so a tile of an expert
// with 3 tokens issues N=16 MMAs, one with 100 tokens N=112: the ragged dimension costs no padding to 128 and the
// tail of an expert never needs a clipped tensor-map store.  Every tile streams a [128 x K] slab of the expert's
// weights once through a ring of 128-byte-wide K steps (10 slots of 21 KB for tiles of at most 32 tokens, 6 slots of
// 31 KB for tiles of up to 112).
//
// What bounds such a tile is not the tensor pipe (a 128 x 32 x 32 MMA is 16 cycles of work) but two per-SM issue
// limits, both measured on B200:
//   * a tcgen05 instruction costs the THREAD that issues it ~180 cycles (mma) / ~65 cycles (cp), whatever its size.
//     One thread issuing the four MMAs of every K step tops out at ~44 GB/s of weights per SM; the rate doubles with
//     a second issuing thread.  Hence LANES threads issue the MMAs, thread l taking the K steps with kt % LANES == l
//     into a partial accumulator of its own (the epilogue adds the partials), and the scale copies have two threads
//     of their own;
//   * what one SM pulls out of HBM through TMA is capped at ~55 GB/s whatever the box shape or the number of slots
//     in flight; cp.async from 128 threads reaches ~63 GB/s, both together ~73-80 GB/s.  Hence the ODD ring slots are
//     filled with cp.async (16-byte pieces written in the 128-byte swizzle pattern TMA would produce).
// With both, ~90-110 SMs saturate HBM instead of all 148, and the rest can run the CTA-pair kernel of the same call
// at the same time.
//
//   warp 0      producer: per K step in an even slot, lanes 0..3 each issue ONE TMA load in the same instruction (weight
//               tile, token tile, the two 512-byte scale atoms as records of their own tensor maps); lane 0 also takes
//               the tile indices from the work counter and hands them to the other roles
//   warp 1, 11-13  MMA issue, one lane each (as many as the shape has LANES): 4 x tcgen05.mma (K=32 each) per own K
//               step, tcgen05.commit to free the slot / publish the accumulator; warp 1 also owns the TMEM allocation
//   warps 2-5   epilogue: tcgen05.ld of the partial accumulators (lane = output column, column = token), fp32 sum,
//               -> bf16/fp16 -> global: a 2-byte store per lane and token row when K is long (no shared memory), a
//               shared-memory transpose and 128-bit stores when K is short or the output is scattered;
//               double-buffered against the MMAs of the next tile
//   warps 6, 14 scale copies, one lane each: the slot's weight / token scale atom smem -> the slot's TMEM columns
//               (tcgen05.cp), tcgen05.commit to the slot's sf_ready barrier
//   warps 7-10  second load path: the odd ring slots by cp.async — or, for the 112-token shape when K is short, a
//               second epilogue group (every slot is then filled by TMA and the two groups take alternate 32-token
//               chunks of a tile)
//
// Work list: items (expert, 1..8 consecutive weight tiles of 128 — one tile when K is long, several when it is short, so
// that an item spans ~16 K steps) found with a per-CTA prefix scan over the problem sizes (device resident: no host
// round trip).  The producer takes item indices from the bucket's work counter in the caller's scratch (atomicAdd;
// round-robin over the shape's CTAs when the caller gave no scratch) and hands each one to the other roles through a
// small shared-memory queue, so a CTA that starts late — behind other CTAs of the same call — just takes what is left.
// Both shapes run in ONE launch (mxfp8_grouped_mm_kernel below picks the shape from the CTA index).
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

constexpr int THREADS = 480;           // 15 warps, see the role table above
constexpr int COPY_WARP0 = 6, COPY_WARP1 = 14;
constexpr int LOADER_WARP0 = 7;        // warps 7..10: cp.async loaders
constexpr int LOADER_THREADS = 128;
constexpr int MMA_WARP1 = 11;          // MMA lanes 1..3 sit in warps 11..13 (lane 0 in warp 1)
constexpr int MAX_LANES = 4;
constexpr int TILE_N = 128;     // weight rows per tile  (tcgen05.mma M)
constexpr int TILE_K = 128;     // bytes of K per ring slot (one 128-byte swizzle atom)
constexpr int W_BYTES = TILE_N * TILE_K;
constexpr int SF_BYTES = 512;
constexpr int MAX_STAGES = 10;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t SF_SLOT_COLS = 8;    // per ring slot: 4 columns of weight scales + 4 of token scales

// A streaming shape: experts with at most TOK_TILE rows (ONE token tile per expert: the tile's token scales are then
// exactly one 128-row atom), STAGES ring slots, LANES MMA-issuing threads = partial accumulators.
template <int TOK_TILE_, int STAGES_, int LANES_, bool SECOND_LOAD_PATH_, bool SECOND_EPILOGUE_>
struct Shape {
  static constexpr int TOK_TILE = TOK_TILE_;     // token rows per tile (tcgen05.mma N, runtime multiple of 16)
  static constexpr int STAGES = STAGES_;
  static constexpr int LANES = LANES_;
  // odd ring slots by cp.async (second load path).  Alone on the GPU the 112-token shape is slower with it (its 128
  // loader threads copy as many token bytes, L2 hits, as weight bytes: 48 vs 52 GB/s per SM) but inside a call, next to
  // the other kernels, the call is faster with it (reference-distribution workload at 32 experts: 0.1938 vs 0.1967 ms)
  static constexpr bool SECOND_LOAD_PATH = SECOND_LOAD_PATH_;
  // With few K steps per tile the four epilogue warps set the pace of a tile of many tokens (partial sums and the store
  // of four 32-token chunks take ~10000 cycles, the loads of three K steps ~1500).  The shape can then run the four
  // loader warps as a second epilogue group instead (every ring slot by TMA; the two groups take alternate chunks).
  // Needs four more 2 KB store tiles, which the 32-token shape has no room for and, with its single chunk, no use for.
  static constexpr bool SECOND_EPILOGUE = SECOND_EPILOGUE_;
  static constexpr int EPILOGUE_TILES = SECOND_EPILOGUE ? 8 : 4;
  static constexpr int X_BYTES = TOK_TILE * TILE_K;
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES + 2 * SF_BYTES;   // W | X | weight scales | token scales
  static constexpr uint32_t ACC_COLS = LANES * TOK_TILE;                 // one accumulator buffer: LANES partials
  static constexpr uint32_t SF_COL0 = 2 * ACC_COLS;                      // two buffers, then the scale slots
  static_assert(STAGE_BYTES % 1024 == 0 && STAGES <= MAX_STAGES && STAGES % 2 == 0, "ring layout");
  static_assert(TOK_TILE % 16 == 0 && TOK_TILE <= 128 && (LANES == 1 || LANES == 2 || LANES == 4), "tile shape");
  static_assert(SF_COL0 + STAGES * SF_SLOT_COLS <= TMEM_COLS, "TMEM budget");
};
using ShapeTiny = Shape<32, 10, 4, true, false>;   // 21 KB slots; TMEM: 2 x 4 x 32 accumulator columns + 80 scale columns
using ShapeMid = Shape<112, 6, 2, true, true>;   // 31 KB slots; TMEM: 2 x 2 x 112 accumulator columns + 48 scale columns

// CTAs of the 112-token shape in front of the 32-token shape's (tunable mm_stream_mid_lead_ctas < 0).  Measured in one
// process, bursts of 20 calls, on the reference benchmark's row distribution: n = 512, E = 256: 0.1980 ms with 0,
// 0.2008 with 32, 0.1912 with 40, 0.1907 with 48, 0.1942 with 64; n = 4096, E = 32: 0.1968 / 0.1892 / 0.1884 / 0.1889 /
// 0.1878; the Zipf decode and prefill workloads do not move (+-0.5 %).
constexpr int kDefaultMidLeadCtas = 48;

constexpr uint32_t ERR_PRODUCER = 1u, ERR_MMA = 2u, ERR_EPILOGUE = 4u, ERR_SCALE_COPY = 8u, ERR_LOADER = 0x400u;
constexpr int QUEUE_DEPTH = 4;          // tile indices in flight between the producer lane and the other roles

struct SharedCtl {
  uint64_t full[MAX_STAGES];            // even slots: 1 arrive.expect_tx + bytes; odd slots: one arrival per loader thread
  uint64_t empty[MAX_STAGES];           // 1 arrival: the commit of the MMA lane that owns the K step
  uint64_t sf_ready[MAX_STAGES];        // 2 arrivals: both scale atoms of the slot are in its TMEM columns
  uint64_t tmem_full[2];                // LANES arrivals: every MMA lane's share of the tile is complete
  uint64_t tmem_empty[2];               // 4 (8 with the second group) arrivals: the epilogue warps have read the buffer
  uint64_t q_full[QUEUE_DEPTH];         // 1 arrival: the producer lane has written q_tile[slot]
  uint64_t q_empty[QUEUE_DEPTH];        // every consuming role has read it
  int q_tile[QUEUE_DEPTH];              // tile index, or -1: no more work
  uint32_t tmem_base;
  int abort_flag;
  int warp_sums[32];
  int tile_prefix[ES_B200_MAX_EXPERTS + 1];   // item prefix [0, E], then the per-expert tables (fill_expert_table)
};

template <class S>
constexpr size_t smem_bytes() {
  return 1024 /*alignment slack*/ + (size_t)S::STAGES * S::STAGE_BYTES + S::EPILOGUE_TILES * EPI_STAGE_BYTES_PER_WARP +
         sizeof(SharedCtl);
}

__device__ uint32_t g_status = 0;   // sticky error bits of the grouped GEMM kernels (bounded waits that gave up)

struct TileInfo {
  int e, nt;     // expert, first weight tile of the work item
  int n_sub;     // weight tiles of the item (1 .. group)
  int valid;     // token rows of the expert (= of this tile)
  int n_mma;     // valid rounded up to 16
  int row0;      // first token row in a / d
};

// Work item t of this launch -> (expert, its weight tiles nt .. nt + n_sub - 1); one token tile per expert.  An item
// is `group` consecutive weight tiles (the last item of an expert may be shorter): with few K steps per tile — k = 256
// is two — every role would otherwise spend more time on the queue hand-over and the decode of a tile than on the
// tile, so the host sizes the items to ~16 K steps, at most 8 tiles (group = 1 from k = 2048 up).  Measured on the
// reference benchmark's row distribution: n = 7168, k = 256, E = 256: 0.257 ms with one tile per item, 0.206 with 4,
// 0.201 with 8; n = 4096, k = 384, E = 128: 0.103 / 0.087 / 0.085.
__device__ __forceinline__ TileInfo decode_tile(int t, const ExpertTable& tab, int num_experts, int n_tiles, int group) {
  TileInfo ti;
  ti.e = upper_bound_expert(tab.prefix, num_experts, t);
  ti.nt = (t - tab.prefix[ti.e]) * group;
  const int rest = n_tiles - ti.nt;
  ti.n_sub = rest < group ? rest : group;
  ti.valid = tab.m(ti.e);
  ti.n_mma = (ti.valid + 15) & ~15;
  ti.row0 = tab.row0(ti.e);
  return ti;
}

// One consumer of the tile queue: waits for the slot, reads the index, reports the slot read.  `whole_warp`: all 32
// lanes call it together (one arrival per warp), otherwise a single lane.
struct QueueReader {
  int qs = 0;
  uint32_t qph = 0;
  template <bool whole_warp>
  __device__ __forceinline__ bool next(SharedCtl* ctl, volatile int* abort_flag, int lane, int* t) {
    bool have = ptx::mbar_wait(&ctl->q_full[qs], qph, abort_flag);
    if (whole_warp) have = __all_sync(0xffffffffu, have);
    if (!have) return false;
    *t = ctl->q_tile[qs];
    if (whole_warp) {
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&ctl->q_empty[qs]);
    } else {
      ptx::mbar_arrive(&ctl->q_empty[qs]);
    }
    if (++qs == QUEUE_DEPTH) { qs = 0; qph ^= 1u; }
    return true;
  }
};

// Arguments that do not depend on the tile shape
struct KernelArgs {
  const uint8_t* a_codes;
  const uint8_t* w_codes;
  const uint8_t* sf_tokens;
  const uint8_t* sf_weights;
  int num_rows;
  long long sf_token_bytes;
  void* d;
  const int* problem_sizes;
  const int* expert_offsets;
  const int* blockscale_offsets;
  int num_experts, n, k;
  int wait_at_start;
  int group;                 // weight tiles per work item
  uint32_t* counters;
  int last_of_call;
  uint32_t earlier_ctas;
};

// One CTA of shape S: `block` of `blocks` CTAs that serve the experts with min_rows <= rows <= max_rows (work counter
// `bucket`).  The tensor maps are the kernel's __grid_constant__ parameters.
template <typename OutT, class S>
__device__ __forceinline__ void grouped_mm_cta(const CUtensorMap& map_w, const CUtensorMap& map_x16,
                                               const CUtensorMap& map_x32, const CUtensorMap& map_x64,
                                               const CUtensorMap& map_xt, const CUtensorMap& map_sfx,
                                               const CUtensorMap& map_sfw, const KernelArgs& args,
                                               const RowScatter& scatter, int min_rows, int max_rows, int bucket,
                                               int load_mode, int block, int blocks) {
  // load_mode 0: every ring slot by TMA; 1: odd slots by cp.async from warps 7..10; 2: every slot by TMA and warps 7..10
  // are a second epilogue group (shapes with SECOND_EPILOGUE only)
  const bool use_lsu = load_mode == 1;
  const bool epi2 = S::SECOND_EPILOGUE && load_mode == 2;
  const uint8_t* __restrict__ a_codes = args.a_codes;
  const uint8_t* __restrict__ w_codes = args.w_codes;
  const uint8_t* __restrict__ sf_tokens = args.sf_tokens;
  const uint8_t* __restrict__ sf_weights = args.sf_weights;
  const int num_rows = args.num_rows;
  const long long sf_token_bytes = args.sf_token_bytes;
  OutT* __restrict__ d = static_cast<OutT*>(args.d);
  const int* __restrict__ problem_sizes = args.problem_sizes;
  const int* __restrict__ expert_offsets = args.expert_offsets;
  const int* __restrict__ blockscale_offsets = args.blockscale_offsets;
  const int num_experts = args.num_experts, n = args.n, k = args.k, group = args.group;
  const int wait_at_start = args.wait_at_start, last_of_call = args.last_of_call;
  // A kernel that is not the first of its call lets the next one launch at once (measured: 1.6 % on a 0.19 ms call,
  // nothing elsewhere); the first one triggers only after its prologue — triggering right after its wait made the
  // decode workload 2 % slower.
  if (!wait_at_start) pdl_launch_dependents();
  uint32_t* counters = args.counters;
  const uint32_t earlier_ctas = args.earlier_ctas;
  constexpr int TOK_TILE = S::TOK_TILE, STAGES = S::STAGES, X_BYTES = S::X_BYTES, STAGE_BYTES = S::STAGE_BYTES;
  constexpr int LANES = S::LANES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_stage = smem + (size_t)STAGES * STAGE_BYTES;      // 2 KB per epilogue warp
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(epi_stage + S::EPILOGUE_TILES * EPI_STAGE_BYTES_PER_WARP);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&ctl->full[s], (use_lsu && (s & 1)) ? LOADER_THREADS : 1);
      ptx::mbar_init(&ctl->empty[s], 1);
      ptx::mbar_init(&ctl->sf_ready[s], 2);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&ctl->tmem_full[a], LANES);
      ptx::mbar_init(&ctl->tmem_empty[a], epi2 ? 8 : 4);
    }
    for (int q = 0; q < QUEUE_DEPTH; ++q) {
      ptx::mbar_init(&ctl->q_full[q], 1);
      // readers: LANES MMA lanes, 2 copy lanes, 4 epilogue warps, and warps 7..10 when they run (as loaders or as the
      // second epilogue group)
      ptx::mbar_init(&ctl->q_empty[q], LANES + 2 + 4 + ((use_lsu || epi2) ? LOADER_THREADS / 32 : 0));
    }
    ctl->abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&map_w);
    ptx::prefetch_tensormap(&map_x16);
    ptx::prefetch_tensormap(&map_x32);
    ptx::prefetch_tensormap(&map_x64);
    ptx::prefetch_tensormap(&map_xt);
    ptx::prefetch_tensormap(&map_sfx);
    ptx::prefetch_tensormap(&map_sfw);
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
  // this launch owns the experts with min_rows <= rows <= max_rows (<= TOK_TILE)
  // (an expert whose scales do not start on a 128-row atom cannot be addressed: reported and skipped)
  block_exclusive_scan(num_experts, ctl->tile_prefix, ctl->warp_sums, [&](int e) {
    const int m = problem_sizes[e * 3];
    if (!(m > 0 && m >= min_rows && m <= max_rows)) return 0;
    if ((blockscale_offsets[e] & 127) != 0) {
      atomicOr(&g_status, ERR_SCALE_OFFSET_BIT);
      return 0;
    }
    return (n_tiles + group - 1) / group;
  });
  // A launch without work (the host only knows an upper bound of the rows per expert) ends here: the kernels of a call
  // run one after the other on every SM, and an empty one that ran its roles through the empty queue cost ~5 us of
  // every call (an empty four-kernel call: 22 us on the GPU, 14 us with this exit).
  if (ctl->tile_prefix[num_experts] == 0) {
    if (wait_at_start) pdl_launch_dependents();
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) ptx::tmem_dealloc(ctl->tmem_base, TMEM_COLS);
    end_of_kernel(counters, wait_at_start != 0, last_of_call != 0, earlier_ctas, scatter.meta != nullptr, &g_status);
    return;
  }
  const ExpertTable tab = fill_expert_table(ctl->tile_prefix, num_experts, problem_sizes, expert_offsets, blockscale_offsets);
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  if (wait_at_start) pdl_launch_dependents();

  const uint32_t tmem_base = ctl->tmem_base;
  const int total_tiles = ctl->tile_prefix[num_experts];
  const int kt_count = k / TILE_K;
  volatile int* abort_flag = &ctl->abort_flag;
  const int mma_lane = warp == 1 ? 0 : (warp >= MMA_WARP1 && warp < MMA_WARP1 + MAX_LANES - 1) ? warp - MMA_WARP1 + 1 : -1;

  // ------------------------------------------------------------------ epilogue: warps 2..5, and warps 7..10 as a second
  // group when the shape runs that way; a group's warp takes the 32-token chunks first_col, first_col + col_stride, ...
  auto run_epilogue = [&](OutT* stage_warp, int first_col, int col_stride) {
    const int quad = warp & 3;   // TMEM lane quadrant this warp may access
    QueueReader q;
    int acc = 0;
    uint32_t acc_ph = 0;
    bool ok = true;
    while (ok) {
      int t;
      if (!q.next<true>(ctl, abort_flag, lane, &t)) { ok = false; break; }
      if (t < 0) break;
      const TileInfo ti = decode_tile(t, tab, num_experts, n_tiles, group);
      for (int sub = 0; ok && sub < ti.n_sub; ++sub) {
      const int nt = ti.nt + sub;
      const bool got = ptx::mbar_wait(&ctl->tmem_full[acc], acc_ph, abort_flag);
      if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
      ptx::tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * S::ACC_COLS + ((uint32_t)(quad * 32) << 16);
      OutT* dst = d + (int64_t)ti.row0 * n + (nt * TILE_N + quad * 32);
      drain_partial_sums<OutT, LANES>(
          taddr, TOK_TILE, kt_count < LANES ? kt_count : LANES, ti.n_mma, ti.valid,
          stage_warp, dst, n, lane,
          [&] {
            // all of this warp's accumulator reads are done: hand the buffer back to the MMA lanes
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&ctl->tmem_empty[acc]);
          },
          scatter, ti.row0, nt * TILE_N + quad * 32, &g_status, kt_count >= 8, first_col, col_stride);
      acc ^= 1;
      if (acc == 0) acc_ph ^= 1u;
      }   // weight tiles of the item
    }
    if (!ok && lane == 0) {
      *abort_flag = 1;
      atomicOr(&g_status, ERR_EPILOGUE);
    }
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (whole warp walks the work list)
    int s = 0, qs = 0;
    uint32_t ph = 0, qph = 0;
    uint32_t* counter = counters ? counters + bucket : nullptr;
    int t_mine = 0;                   // lane 0: the index that goes out next
    if (lane == 0) t_mine = counter ? (int)atomicAdd(counter, 1u) : block;
    while (true) {
      // lane 0 hands the tile index (or the end mark) to the other roles
      int t = -1;
      bool q_ok = true;
      if (lane == 0) {
        q_ok = ptx::mbar_wait(&ctl->q_empty[qs], qph ^ 1u, abort_flag);
        if (q_ok) {
          t = t_mine < total_tiles ? t_mine : -1;
          ctl->q_tile[qs] = t;
          ptx::mbar_arrive(&ctl->q_full[qs]);
          // the next index is requested now; its round trip to L2 hides behind this tile's loads
          if (t >= 0) t_mine = counter ? (int)atomicAdd(counter, 1u) : t_mine + blocks;
        }
      }
      q_ok = __shfl_sync(0xffffffffu, (int)q_ok, 0) != 0;
      t = __shfl_sync(0xffffffffu, t, 0);
      if (++qs == QUEUE_DEPTH) { qs = 0; qph ^= 1u; }
      if (!q_ok) {
        if (lane == 0) {
          *abort_flag = 1;
          atomicOr(&g_status, ERR_PRODUCER);
        }
        break;
      }
      if (t < 0) break;
      const TileInfo ti = decode_tile(t, tab, num_experts, n_tiles, group);
      const CUtensorMap* xm = ti.n_mma <= 16 ? &map_x16 : ti.n_mma <= 32 ? &map_x32 : ti.n_mma <= 64 ? &map_x64 : &map_xt;
      const uint32_t box_rows = ti.n_mma <= 16 ? 16u : ti.n_mma <= 32 ? 32u : ti.n_mma <= 64 ? 64u : (uint32_t)TOK_TILE;
      const uint32_t tx = W_BYTES + box_rows * TILE_K + 2 * SF_BYTES;
      // this lane's load: 0 weight tile (streamed once: evict first), 1 token tile (re-read by every weight tile of
      // the expert: evict last), 2 weight scale atom, 3 token scale atom (512-byte records, index = atom number)
      const int sfw_atom = (ti.e * n_tiles + ti.nt) * kt_count;
      const int sfx_atom = (tab.scale0(ti.e) >> 7) * kt_count;
      const CUtensorMap* my_map = lane == 0 ? &map_w : lane == 1 ? xm : lane == 2 ? &map_sfw : &map_sfx;
      const uint32_t my_off = lane == 0 ? 0u : lane == 1 ? (uint32_t)W_BYTES
                              : lane == 2 ? (uint32_t)(W_BYTES + X_BYTES) : (uint32_t)(W_BYTES + X_BYTES + SF_BYTES);
      const int my_c1_first = lane == 0 ? ti.e * n + ti.nt * TILE_N : lane == 1 ? ti.row0 : lane == 2 ? sfw_atom : sfx_atom;
      const int my_c1_step = lane == 0 ? TILE_N : lane == 2 ? kt_count : 0;     // per weight tile of the item
      const uint64_t my_hint = lane == 0 ? ptx::kL2EvictFirst : lane == 1 ? ptx::kL2EvictLast : ptx::kL2EvictNormal;
      bool ok = true;
      for (int sub = 0; ok && sub < ti.n_sub; ++sub) {
      const int my_c1 = my_c1_first + sub * my_c1_step;
      for (int kt = 0; kt < kt_count; ++kt) {
        if (!(use_lsu && (s & 1))) {          // odd slots belong to the cp.async loaders
          ok = __all_sync(0xffffffffu, ptx::mbar_wait(&ctl->empty[s], ph ^ 1u, abort_flag));
          if (!ok) break;
          uint8_t* stage = smem + (size_t)s * STAGE_BYTES;
          if (lane == 0) ptx::mbar_arrive_expect_tx(&ctl->full[s], tx);
          __syncwarp();
          if (lane < 4)
            ptx::tma_load_2d_hint(stage + my_off, my_map, &ctl->full[s], lane < 2 ? kt * TILE_K : 0,
                                  lane < 2 ? my_c1 : my_c1 + kt, my_hint);
        }
        if (++s == STAGES) { s = 0; ph ^= 1u; }
      }
      }   // weight tiles of the item
      if (!ok) {
        if (lane == 0) {
          *abort_flag = 1;
          atomicOr(&g_status, ERR_PRODUCER);
        }
        break;
      }
    }
  } else if (mma_lane >= 0) {
    // ------------------------------------------------------------------ MMA issue: lane l of LANES takes the K steps
    // with kt % LANES == l and accumulates them in partial accumulator l of the tile's buffer
    if (lane == 0 && mma_lane < LANES) {
      QueueReader q;
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      while (ok) {
        int t;
        if (!q.next<false>(ctl, abort_flag, lane, &t)) { ok = false; break; }
        if (t < 0) break;
        const TileInfo ti = decode_tile(t, tab, num_experts, n_tiles, group);
        for (int sub = 0; ok && sub < ti.n_sub; ++sub) {
        if (!ptx::mbar_wait(&ctl->tmem_empty[acc], acc_ph ^ 1u, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * S::ACC_COLS + mma_lane * TOK_TILE;
        for (int kt = 0; kt < kt_count; ++kt) {
          if ((kt & (LANES - 1)) == mma_lane) {
            if (!ptx::mbar_wait(&ctl->full[s], ph, abort_flag)) { ok = false; break; }
            if (!ptx::mbar_wait(&ctl->sf_ready[s], ph, abort_flag)) { ok = false; break; }
            if (use_lsu && (s & 1)) ptx::fence_proxy_async_shared();   // slot written by cp.async (generic proxy)
            ptx::tc_fence_after_sync();
            const uint32_t stage = ptx::smem_u32(smem + (size_t)s * STAGE_BYTES);
            const uint32_t sfw_t = tmem_base + S::SF_COL0 + s * SF_SLOT_COLS;
            const uint32_t sfx_t = sfw_t + 4;
            const uint64_t a_desc = ptx::make_desc_k_sw128(stage);
            const uint64_t b_desc = ptx::make_desc_k_sw128(stage + W_BYTES);
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j)      // the lane's first MMA of the tile overwrites its partial
              ptx::tc_mma_mxf8(d_tmem, a_desc + 2 * j, b_desc + 2 * j, ptx::make_idesc_mxf8(TILE_N, ti.n_mma, j, j),
                               sfw_t | (j << 30), sfx_t | (j << 30), (kt == mma_lane && j == 0) ? 0u : 1u);
            ptx::tc_commit(&ctl->empty[s]);       // slot reusable once these MMAs have read it
          }
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (!ok) break;
        ptx::tc_commit(&ctl->tmem_full[acc]);     // this lane's share of the accumulator is complete
        acc ^= 1;
        if (acc == 0) acc_ph ^= 1u;
        }   // weight tiles of the item
      }
      if (!ok) {
        *abort_flag = 1;
        atomicOr(&g_status, ERR_MMA);
      }
    }
  } else if (warp == COPY_WARP0 || warp == COPY_WARP1) {
    // ------------------------------------------------------------------ scale copies: warp 6 the weight atom, warp 14
    // the token atom of every slot.  A slot's TMEM columns are rewritten only after the slot was refilled, i.e. after
    // the MMAs that read them have completed (their commit released the slot to the producer).
    if (lane == 0) {
      const int which = warp == COPY_WARP0 ? 0 : 1;
      QueueReader q;
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      while (ok) {
        int t;
        if (!q.next<false>(ctl, abort_flag, lane, &t)) { ok = false; break; }
        if (t < 0) break;
        const int k_steps = decode_tile(t, tab, num_experts, n_tiles, group).n_sub * kt_count;
        for (int kk = 0; kk < k_steps; ++kk) {
          if (!ptx::mbar_wait(&ctl->full[s], ph, abort_flag)) { ok = false; break; }
          if (use_lsu && (s & 1)) ptx::fence_proxy_async_shared();
          ptx::tc_fence_after_sync();
          const uint32_t sf_smem = ptx::smem_u32(smem + (size_t)s * STAGE_BYTES) + W_BYTES + X_BYTES + which * SF_BYTES;
          ptx::tc_cp_sf(tmem_base + S::SF_COL0 + s * SF_SLOT_COLS + which * 4, ptx::make_desc_sf(sf_smem));
          ptx::tc_commit(&ctl->sf_ready[s]);
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
      if (!ok) {
        *abort_flag = 1;
        atomicOr(&g_status, ERR_SCALE_COPY);
      }
    }
  } else if (warp >= LOADER_WARP0 && warp < LOADER_WARP0 + LOADER_THREADS / 32) {
    // ------------------------------------------------------------------ second load path (warps 7..10, cp.async)
    // Fills the odd ring slots.  Per slot a thread copies 8 pieces of the weight tile, its share of the token tile
    // and one piece of the two scale atoms (16 bytes each); the slot's barrier counts one arrival per loader thread,
    // made by the hardware when that thread's copies have landed (cp.async.mbarrier.arrive.noinc), so a thread never
    // waits for its own copies and keeps as many slots in flight as the ring has free.  The consumers of a cp.async
    // slot (MMA lanes, copy lanes) issue a proxy fence after their wait: the data was written through the generic
    // proxy and is read by tcgen05 through the async proxy.
    if (epi2) {
      run_epilogue(reinterpret_cast<OutT*>(epi_stage) + (4 + warp - LOADER_WARP0) * 1024, 32, 64);
    } else if (use_lsu) {
      const int lt = threadIdx.x - LOADER_WARP0 * 32;        // 0..127
      const int c16 = lt & 7, r0 = lt >> 3;                   // this thread's 16-byte column and first row
      QueueReader q;
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      while (ok) {
        int t;
        if (!q.next<true>(ctl, abort_flag, lane, &t)) { ok = false; break; }
        if (t < 0) break;
        const TileInfo ti = decode_tile(t, tab, num_experts, n_tiles, group);
        const uint8_t* w_src = w_codes + ((int64_t)ti.e * n + ti.nt * TILE_N + r0) * k + c16 * 16;
        const uint8_t* x_src = a_codes + ((int64_t)ti.row0 + r0) * k + c16 * 16;
        const int64_t sfw_off = ((int64_t)(ti.e * n_tiles + ti.nt) * kt_count) * SF_BYTES;
        const int64_t sfx_off = ((int64_t)(tab.scale0(ti.e) >> 7) * kt_count) * SF_BYTES;
        // the two scale atoms are 64 pieces: threads 0..31 the weight atom, 32..63 the token atom (zeros past the buffer)
        const uint8_t* sf_src = lt < 32 ? sf_weights + sfw_off + lt * 16 : sf_tokens + sfx_off + (lt - 32) * 16;
        const bool sf_in_range = lt < 32 || sfx_off + (int64_t)kt_count * SF_BYTES <= sf_token_bytes;
        const uint32_t dst_swz = (uint32_t)(r0 * 128 + ((c16 ^ (r0 & 7)) << 4));   // row r0 + 16 j keeps (r & 7)
        for (int sub = 0; ok && sub < ti.n_sub; ++sub) {
        const uint8_t* w_sub = w_src + (int64_t)sub * TILE_N * k;                 // weight tile nt + sub
        const uint8_t* sf_sub = lt < 32 ? sf_src + (int64_t)sub * kt_count * SF_BYTES : sf_src;
        for (int kt = 0; kt < kt_count; ++kt) {
          if (s & 1) {
            ok = __all_sync(0xffffffffu, ptx::mbar_wait(&ctl->empty[s], ph ^ 1u, abort_flag));
            if (!ok) break;
            const uint32_t stage = ptx::smem_u32(smem + (size_t)s * STAGE_BYTES);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              ptx::cp_async_16_hint(stage + dst_swz + j * 2048, w_sub + (int64_t)j * 16 * k + kt * TILE_K,
                                    ptx::kL2EvictFirst);      // weights are read once
#pragma unroll
            for (int j = 0; j < TOK_TILE / 16; ++j) {
              const int r = r0 + 16 * j;
              if (r < ti.n_mma) {
                const bool in_range = ti.row0 + r < num_rows;       // rows past the end of `a` read as zeros
                ptx::cp_async_16(stage + W_BYTES + dst_swz + j * 2048,
                                 in_range ? x_src + (int64_t)j * 16 * k + kt * TILE_K : a_codes, in_range ? 16u : 0u);
              }
            }
            if (lt < 64)
              ptx::cp_async_16(stage + W_BYTES + X_BYTES + lt * 16,
                               sf_in_range ? sf_sub + (int64_t)kt * SF_BYTES : sf_weights, sf_in_range ? 16u : 0u);
            ptx::cp_async_arrive_noinc(&ctl->full[s]);
          }
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        }   // weight tiles of the item
      }
      if (!ok && lane == 0) {
        *abort_flag = 1;
        atomicOr(&g_status, ERR_LOADER);
      }
    }
  } else if (warp >= 2 && warp <= 5) {
    run_epilogue(reinterpret_cast<OutT*>(epi_stage) + (warp - 2) * 1024, 0, epi2 ? 64 : 32);
  }
  // (warps of MMA lanes the shape does not use fall through)

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
  end_of_kernel(counters, wait_at_start != 0, last_of_call != 0, earlier_ctas, scatter.meta != nullptr, &g_status);
}

// One launch for both streaming shapes: tiny_ctas CTAs run the 32-token shape on the experts with 1 .. split_rows rows,
// the others the 112-token shape on split_rows+1 .. max_rows.  The hardware starts CTAs in index order: the first
// mid_lead CTAs of the 112-token shape, then the 32-token shape's, then the rest of the 112-token shape's, which take
// the SMs as the 32-token shape runs out of tiles — what two launches chained by programmatic dependent launch did,
// for one launch less per call (~4 us of host time).  The leading CTAs work through the middle bucket next to the
// small one from the start; tiles are dealt per bucket, so whichever CTAs of a shape are running share its tiles.
// tiny_ctas == gridDim.x or == 0 leaves a single shape.
template <typename OutT>
__global__ void __launch_bounds__(THREADS, 1)
mxfp8_grouped_mm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x16,
                        const __grid_constant__ CUtensorMap map_x32, const __grid_constant__ CUtensorMap map_x64,
                        const __grid_constant__ CUtensorMap map_x112, const __grid_constant__ CUtensorMap map_sfx,
                        const __grid_constant__ CUtensorMap map_sfw, const __grid_constant__ KernelArgs args,
                        const __grid_constant__ RowScatter scatter, int tiny_ctas, int mid_lead, int split_rows,
                        int max_rows, int load_mode_tiny, int load_mode_mid) {
  const int mid_ctas = (int)gridDim.x - tiny_ctas;
  const int b = (int)blockIdx.x;
  if (b >= mid_lead && b < mid_lead + tiny_ctas)
    grouped_mm_cta<OutT, ShapeTiny>(map_w, map_x16, map_x32, map_x64, map_x32, map_sfx, map_sfw, args, scatter, 1,
                                    split_rows, 0, load_mode_tiny, b - mid_lead, tiny_ctas);
  else
    grouped_mm_cta<OutT, ShapeMid>(map_w, map_x16, map_x32, map_x64, map_x112, map_sfx, map_sfw, args, scatter,
                                   split_rows + 1, max_rows, 1, load_mode_mid, b < mid_lead ? b : b - tiny_ctas, mid_ctas);
}

// earlier_ctas: in/out — CTAs launched so far by this call; the last kernel of the call waits for that many reports.
// Experts with 1 .. tiny_max rows go to the 32-token shape (if want_tiny), tiny_max+1 .. mid_max to the 112-token shape
// (if want_mid).
template <typename OutT>
int launch_streaming(const CallArgs& c, int tiny_max, int mid_max, bool want_tiny, bool want_mid, bool first_of_call,
                     bool last_of_call, uint32_t* earlier_ctas) {
  constexpr size_t SMEM_TINY = smem_bytes<ShapeTiny>(), SMEM_MID = smem_bytes<ShapeMid>();
  constexpr size_t SMEM_BYTES = SMEM_TINY > SMEM_MID ? SMEM_TINY : SMEM_MID;
  DeviceInfo info;
  int rc = get_device_info(&info);
  if (rc != ES_B200_OK) return rc;

  CUtensorMap map_w, map_x[4];
  rc = make_tensormap_u8_sw128(&map_w, c.b, (uint64_t)c.num_experts * c.n, (uint64_t)c.k, TILE_N);
  if (rc != ES_B200_OK) return rc;
  const uint32_t boxes[4] = {16, 32, 64, (uint32_t)ShapeMid::TOK_TILE};   // token boxes; 32 and 112 are the full tiles
  static_assert(ShapeTiny::TOK_TILE == 32, "the 32-row token box doubles as the small shape's full tile");
  for (int i = 0; i < 4; ++i) {
    rc = make_tensormap_u8_sw128(&map_x[i], c.a, (uint64_t)c.num_rows, (uint64_t)c.k, boxes[i]);
    if (rc != ES_B200_OK) return rc;
  }

  CUtensorMap map_sfx, map_sfw;
  const int kt_count = c.k / TILE_K;
  rc = make_tensormap_records512(&map_sfw, c.sfb, (uint64_t)c.num_experts * (c.n / TILE_N) * kt_count);
  if (rc != ES_B200_OK) return rc;
  // whole 128-row atoms only; loads past the end read as zero (a map needs at least one record)
  const uint64_t sfx_records = (uint64_t)(c.sfa_rows / 128) * kt_count;
  rc = make_tensormap_records512(&map_sfx, c.sfa, sfx_records ? sfx_records : 1);
  if (rc != ES_B200_OK) return rc;

  auto kernel = mxfp8_grouped_mm_kernel<OutT>;
  static bool configured[64] = {false};   // per device (one static per instantiation)
  int dev = 0;
  ES_CUDA_TRY(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    ES_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
    configured[dev & 63] = true;
  }
  // weight tiles per work item: ~mm_item_k_steps K steps per item
  int item_k_steps = tunables().mm_item_k_steps;
  if (item_k_steps < 1) item_k_steps = 1;
  int group = (item_k_steps + kt_count - 1) / kt_count;
  if (group > 8) group = 8;
  // upper bound of the item count known on the host: one token tile per expert
  const int64_t max_tiles = (int64_t)c.num_experts * ((c.n / TILE_N + group - 1) / group);
  int per_shape = (int)(max_tiles < info.sm_count ? max_tiles : info.sm_count);
  const int cap = tunables().mm_stream_max_ctas;
  if (cap > 0 && per_shape > cap) per_shape = cap;
  const int first_ctas = want_tiny ? per_shape : 0;
  const int mid_ctas = want_mid ? per_shape : 0;
  const int grid = first_ctas + mid_ctas;
  int mid_lead = tunables().mm_stream_mid_lead_ctas;
  if (mid_lead < 0) mid_lead = kDefaultMidLeadCtas;
  if (mid_lead > mid_ctas) mid_lead = mid_ctas;

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
  const int lsu = tunables().mm_stream_lsu ? 1 : 0;
  KernelArgs args = {static_cast<const uint8_t*>(c.a), static_cast<const uint8_t*>(c.b), c.sfa, c.sfb, (int)c.num_rows,
                     (long long)(c.sfa_rows * (c.k / 32)), c.d, c.ps, c.eo, c.bo, c.num_experts, c.n, c.k,
                     first_of_call ? 1 : 0, group, c.counters, last_of_call ? 1 : 0, *earlier_ctas};
  ES_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, map_w, map_x[0], map_x[1], map_x[2], map_x[3], map_sfx, map_sfw, args,
                                 *c.scatter, first_ctas, mid_lead, tiny_max, mid_max,
                                 (ShapeTiny::SECOND_LOAD_PATH && lsu) ? 1 : 0,
                                 (ShapeMid::SECOND_EPILOGUE && kt_count < 8) ? 2 : (ShapeMid::SECOND_LOAD_PATH && lsu) ? 1 : 0));
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
  // the kernels of all row-count buckets are launched, back to back on the caller's stream with programmatic
  // dependent launch (the two single-CTA shapes share one launch), and each CTA filters the experts by row count
  // inside its own work-list scan:
  //   rows <= tiny_max  : single-CTA kernel, 128 weights x <=32 tokens, 10-slot ring   \  these experts stream their
  //   rows <  heavy_min : single-CTA kernel, 128 weights x <=112 tokens, 6-slot ring   /  weights from HBM exactly
  //                       once; what counts is weight bytes per second and SM;
  //   rows >= heavy_min : CTA-pair kernel, 256 weights x <=384 tokens, weight-stationary K step — these experts
  //                       re-read operands from L2, what counts is operand bytes per FLOP.
  // A CTA whose bucket is empty ends after its scan.  A bucket that even the host-known upper bound of rows per
  // expert (num_rows) cannot reach gets no CTAs at all.  The thresholds come from a per-(n, k) table
  // (bucket_table.cuh) unless a tunable overrides them.
  //
  // With scratch (work counters) a large call is SPLIT: a pair launch capped to a few CTA pairs goes first, then the
  // streaming launch on the SMs it leaves, then a second pair launch that takes the SMs the streaming kernels
  // free and drains the same counter.  The streaming buckets are bound by HBM and leave the tensor pipe idle, the pair
  // bucket is bound by the tensor pipe and leaves HBM idle: side by side the call costs about max() of the two
  // instead of their sum.  Every kernel is persistent and takes tiles from its bucket's counter, and no kernel of the
  // call waits for its predecessor (see end_of_kernel), so whichever side runs out first hands its SMs to the
  // kernels queued behind it.
  const Tunables& tn = tunables();
  const BucketThresholds table = bucket_thresholds(n, k);
  // (a streaming shape holds a whole expert in one token tile, so the CTA-pair kernel takes everything above the
  // larger shape's tile)
  int heavy_min = tn.mm_heavy_min_rows > 0 ? tn.mm_heavy_min_rows : table.heavy_min_rows;
  if (heavy_min > mm::ShapeMid::TOK_TILE + 1) heavy_min = mm::ShapeMid::TOK_TILE + 1;
  int tiny_max = tn.mm_tiny_max_rows > 0 ? tn.mm_tiny_max_rows : table.tiny_max_rows;
  if (tiny_max > mm::ShapeTiny::TOK_TILE) tiny_max = mm::ShapeTiny::TOK_TILE;
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
  if (want_tiny || want_mid) {
    const bool last = !want_pair;
    rc = bf16 ? mm::launch_streaming<__nv_bfloat16>(c, tiny_max, heavy_min - 1, want_tiny, want_mid, first, last, &ctas)
              : mm::launch_streaming<__half>(c, tiny_max, heavy_min - 1, want_tiny, want_mid, first, last, &ctas);
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
  if (v != 0) note_device_error();
  if (v != 0)
    return fail(ES_B200_ERR_DEVICE_TIMEOUT,
                "a bounded device-side wait gave up or an index was out of range (status bits 0x%x)", v);
  return ES_B200_OK;
}
