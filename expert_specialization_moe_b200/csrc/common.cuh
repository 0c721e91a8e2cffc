// Shared host/device helpers of the es_b200 library (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include <nvtx3/nvToolsExt.h>

#include "es_b200.h"

namespace es_b200 {

// ---- host: error reporting ------------------------------------------------------------------
char* last_error_buffer();            // thread-local, 512 bytes
int fail(int code, const char* fmt, ...);

#define ES_CUDA_TRY(expr)                                                                   \
  do {                                                                                      \
    cudaError_t _e = (expr);                                                                \
    if (_e != cudaSuccess)                                                                  \
      return ::es_b200::fail(ES_B200_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

#define ES_REQUIRE(cond, ...)                                                        \
  do {                                                                               \
    if (!(cond)) return ::es_b200::fail(ES_B200_ERR_INVALID_ARGUMENT, __VA_ARGS__);  \
  } while (0)

// Cached per-device properties (SM count, compute capability).  Queried once per device.
struct DeviceInfo {
  int sm_count;
  int cc_major;
  int cc_minor;
};
int get_device_info(DeviceInfo* out);   // for the current device

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- host: NVTX range around the launches of one operator call ---------------------------------
// (header-only NVTX: a no-op unless a profiler is attached; makes a tool's launch list attributable per operator, as the
// reference's benchmark does around its call: benchmark_sm100_mxfp8_blockscaled_moe.py:112-114)
struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};

// ---- host: tunables of the tile-shape dispatcher -----------------------------------------------
// One set per process; each has a built-in default, an environment override read once (ES_B200_<NAME in capitals>)
// and can be changed at run time with es_b200_set_tunable.  A per-(n, k) table (bucket_table.cuh) supplies the
// defaults of the two row-count thresholds; an explicit setting (environment or call) wins over the table.
struct Tunables {
  int mm_heavy_min_rows;        // MXFP8 GEMM: experts with at least this many rows go to the CTA-pair kernel; 0 = table
  int mm_tiny_max_rows;         // experts with at most this many rows go to the 32-token streaming shape; 0 = table
  int mm_pair_first_clusters;   // CTA pairs of the leading pair launch when a call is split (see grouped_mm_impl)
  int mm_split_min_rows;        // calls with at least this many rows put a capped pair launch in front
  int mm_stream_max_ctas;       // cap of the streaming kernels' grids (0 = one CTA per SM)
  int mm_pair_max_clusters;     // cap of the trailing pair launch (0 = as many CTA pairs as fit)
  int mm_dynamic;               // 1: tiles are dealt through the work counters in scratch when scratch is given
  int mm_stream_lsu;            // 1: the streaming kernels fill every other ring slot with cp.async instead of TMA
  int mm_item_k_steps;          // streaming kernel: a work item spans enough weight tiles for this many K steps (<= 8 tiles)
  int mm_stream_mid_lead_ctas;  // streaming launch: this many CTAs of the 112-token shape start before the 32-token
                                // shape's (they work through the middle bucket from the start); the rest follow it;
                                // negative = built-in default
};
Tunables& tunables();
void note_device_error();   // es_b200_check_status found status bits set (see es_b200_error_epoch)

// ---- device: programmatic dependent launch ---------------------------------------------------
// Both are no-ops when the kernel was not launched with the programmatic-stream-serialization attribute.
__device__ __forceinline__ void pdl_wait_prior_grid() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- device: work counters of the grouped GEMMs ------------------------------------------------
// The scratch of a grouped GEMM call holds five 32-bit words, zero between calls:
//   [0..2] next tile index of each of the three row-count buckets.  Every kernel of the call takes its tiles with
//          atomicAdd on its bucket's word, so CTAs that start late (behind another kernel of the same call, on SMs
//          that another bucket has just left) simply take what is left;
//   [4]    CTAs of the call's earlier kernels that have finished (all their stores fenced);
//   [3]    CTAs of the call's LAST kernel that have finished and seen [4] reach the number of earlier CTAs.
// The kernels of a call are chained with programmatic dependent launch and only the first one waits for the stream's
// earlier work; none of the others waits for its predecessor — a streaming kernel's CTAs leave their SMs to the next
// kernel as soon as their bucket is empty, while a CTA-pair launch in front of them is still running.  What keeps
// stream order for whatever follows the call is this rendezvous: every CTA of the last kernel, before it exits,
// waits (bounded) until all earlier CTAs of the call have reported.  That wait cannot starve anybody: a dependent
// launch only starts once every CTA of its predecessor is resident and has passed its launch_dependents, so by the
// time a CTA of the last kernel runs, every CTA it waits for is already on an SM.  The last CTA to get through
// clears the five words.
constexpr int WORK_COUNTER_WORDS = 5;
constexpr size_t GROUPED_MM_SCRATCH_BYTES = 256;
constexpr uint32_t ERR_SCALE_OFFSET_BIT = 0x80u;   // a blockscale offset that is not a multiple of 128 rows
constexpr uint32_t ERR_CALL_RENDEZVOUS_BIT = 0x200u;   // the last kernel gave up waiting for the call's earlier CTAs
constexpr unsigned long long kRendezvousLimitNs = 4000000000ull;

// Called by ALL threads of a CTA once its roles are done (in a CTA pair: by each CTA).  Without counters the kernels
// keep stream order the simple way: every kernel but the first waits for its predecessor before it exits.
__device__ __forceinline__ void end_of_kernel(uint32_t* counters, bool waited_at_start, bool last_of_call,
                                              uint32_t earlier_ctas, bool peer_stores, uint32_t* status) {
  if (counters == nullptr) {
    if (!waited_at_start) pdl_wait_prior_grid();
    return;
  }
  if (peer_stores) __threadfence_system(); else __threadfence();     // this thread's output stores
  __syncthreads();
  if (threadIdx.x != 0) return;
  if (!last_of_call) {
    atomicAdd(&counters[4], 1u);
    return;
  }
  unsigned long long t0 = 0;
  uint32_t spins = 0;
  while (true) {
    uint32_t seen;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counters + 4) : "memory");
    if (seen >= earlier_ctas) break;
    if ((++spins & 63u) == 0) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      if (now - t0 > kRendezvousLimitNs) {
        atomicOr(status, ERR_CALL_RENDEZVOUS_BIT);
        break;
      }
    }
    __nanosleep(64);
  }
  __threadfence();
  const uint32_t done = atomicAdd(&counters[3], 1u);
  if (done == gridDim.x - 1) {
    counters[0] = 0;
    counters[1] = 0;
    counters[2] = 0;
    counters[4] = 0;
    __threadfence();
    counters[3] = 0;
  }
}

// ---- device: block-wide exclusive scan of up to 1024 per-expert counts -----------------------
// counts are produced by `f(e)` for e in [0, n); results go to prefix[0..n] (prefix[n] = total).
// Must be called by all threads of a block whose size is a multiple of 32 and at most 1024.
template <class F>
__device__ __forceinline__ void block_exclusive_scan(int n, int* prefix, int* warp_sums /*[32]*/, F f) {
  const int tid = threadIdx.x;
  const int nthr = blockDim.x;
  const int per = (n + nthr - 1) / nthr;      // consecutive experts per thread
  const int lo = tid * per;
  int local = 0;
  for (int i = 0; i < per; ++i) {
    int e = lo + i;
    if (e < n) local += f(e);
  }
  // inclusive warp scan of `local`
  const int lane = tid & 31, warp = tid >> 5;
  int incl = local;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += t;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int nw = nthr >> 5;
    int v = lane < nw ? warp_sums[lane] : 0;
    int s = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, s, d);
      if (lane >= d) s += t;
    }
    warp_sums[lane] = s - v;   // exclusive
  }
  __syncthreads();
  int run = warp_sums[warp] + incl - local;
  for (int i = 0; i < per; ++i) {
    int e = lo + i;
    if (e < n) {
      prefix[e] = run;
      run += f(e);
    }
  }
  if (tid == nthr - 1) prefix[n] = run;   // last thread holds the grand total (threads past n add 0)
  __syncthreads();
}

// largest e in [0, n) with prefix[e] <= u  (prefix non-decreasing, prefix[0] = 0, u < prefix[n])
__device__ __forceinline__ int upper_bound_expert(const int* prefix, int n, int u) {
  int lo = 0, hi = n;   // invariant: prefix[lo] <= u < prefix[hi]
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (prefix[mid] <= u) lo = mid; else hi = mid;
  }
  return lo;
}

// ---- device: per-expert facts in shared memory ------------------------------------------------
// Every role of a grouped GEMM kernel needs the expert's row count, first row and first scale row for every work
// item.  Read from global memory that is a chain of dependent L2 round trips per item (~2000 cycles behind the binary
// search over the item prefix), which an MMA-issuing lane cannot hide when an item has only a few K steps.  The
// kernels therefore copy them once per CTA into the tail of the array that holds the item prefix: `table` has
// ES_B200_MAX_EXPERTS + 1 ints, the prefix takes n + 1 of them, the copies of as many experts as fit follow (all of
// them when n <= 256 with three tables); experts beyond that are read from global memory as before.
struct ExpertTable {
  const int* prefix;
  const int* rows;              // shared-memory copies for experts below `cached`
  const int* first_row;
  const int* scale_row0;
  int cached;
  const int* problem_sizes;     // global memory
  const int* expert_offsets;
  const int* blockscale_offsets;   // may be null (no third table)
  __device__ __forceinline__ int m(int e) const { return e < cached ? rows[e] : problem_sizes[e * 3]; }
  __device__ __forceinline__ int row0(int e) const { return e < cached ? first_row[e] : expert_offsets[e]; }
  __device__ __forceinline__ int scale0(int e) const { return e < cached ? scale_row0[e] : blockscale_offsets[e]; }
};
// Called by all threads after block_exclusive_scan has written table[0..n]; the caller synchronises the block before
// the table is read.
__device__ __forceinline__ ExpertTable fill_expert_table(int* table, int n, const int* problem_sizes,
                                                         const int* expert_offsets, const int* blockscale_offsets) {
  ExpertTable tab;
  const int tables = blockscale_offsets ? 3 : 2;
  const int room = (ES_B200_MAX_EXPERTS + 1 - (n + 1)) / tables;
  tab.cached = n < room ? n : room;
  int* rows = table + n + 1;
  int* first_row = rows + tab.cached;
  int* scale_row0 = first_row + tab.cached;
  for (int e = threadIdx.x; e < tab.cached; e += blockDim.x) {
    rows[e] = problem_sizes[e * 3];
    first_row[e] = expert_offsets[e];
    if (blockscale_offsets) scale_row0[e] = blockscale_offsets[e];
  }
  tab.prefix = table;
  tab.rows = rows;
  tab.first_row = first_row;
  tab.scale_row0 = scale_row0;
  tab.problem_sizes = problem_sizes;
  tab.expert_offsets = expert_offsets;
  tab.blockscale_offsets = blockscale_offsets;
  return tab;
}

}  // namespace es_b200
