// Routing tables of the expert-parallel exchange, computed on the device in three small launches:
//
//   es_b200_ep_route_count   per-segment histograms of this GPU's (token, j) pairs over the experts, their exclusive
//                            prefix over the segments, and this GPU's per-expert totals stored into every peer's
//                            copy of the count matrix counts_all [world, E]            (barrier between the two calls)
//   es_b200_ep_route_tables  from counts_all: rows / offsets of this GPU's experts, and for each of its own pairs the
//                            owner GPU, the row in the owner's receive buffer and the byte offset of the row's scale
//                            words (swizzled layout) — the inputs of es_b200_ep_dispatch_quant_push.
//
// Order on the owner: expert-major, inside an expert by source GPU, inside a source by pair index (token-major) — what
// a stable sort by expert followed by an all-to-all delivers.  A pair's rank among its GPU's pairs to the same expert
// is found without sorting: the pairs are cut into 256 contiguous segments, one warp walks one segment 32 pairs at a
// time (match_any gives the rank inside the step, a per-warp running count per expert the rank before it).
#include <mutex>

#include "common.cuh"
#include "mxfp8_quant_math.cuh"

namespace es_b200 {
namespace route {

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int BLOCKS = 32;
constexpr int SEGMENTS = BLOCKS * WARPS;       // 256
constexpr int MAX_WORLD = 16;
constexpr uint32_t ERR_CAPACITY = 0x80000u;    // more rows were routed to this GPU than its receive buffers hold

__device__ uint32_t g_status = 0;

struct PeerTable {
  void* ptr[MAX_WORLD];
};

__device__ __forceinline__ int load_id(const void* ids, int ids_int64, int i) {
  return ids_int64 ? (int)static_cast<const long long*>(ids)[i] : static_cast<const int*>(ids)[i];
}

__device__ __forceinline__ int segment_len(int pairs) {       // pairs per segment, a multiple of 32
  return ((pairs + SEGMENTS - 1) / SEGMENTS + 31) & ~31;
}

// seg_counts[seg][e] = number of pairs of segment seg routed to expert e (ids outside [0, E) are not counted)
__global__ void __launch_bounds__(THREADS)
count_kernel(const void* __restrict__ ids, int ids_int64, int pairs, int num_experts, int* __restrict__ seg_counts) {
  extern __shared__ int hist[];                 // [WARPS][E]
  pdl_wait_prior_grid();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int* mine = hist + warp * num_experts;
  for (int e = lane; e < num_experts; e += 32) mine[e] = 0;
  __syncwarp();
  const int seg = blockIdx.x * WARPS + warp;
  const int len = segment_len(pairs);
  const int begin = seg * len;
  const int end = min(begin + len, pairs);
  for (int i = begin + lane; i < end; i += 32) {
    const int e = load_id(ids, ids_int64, i);
    if (e >= 0 && e < num_experts) atomicAdd(&mine[e], 1);
  }
  __syncwarp();
  for (int e = lane; e < num_experts; e += 32) seg_counts[(int64_t)seg * num_experts + e] = mine[e];
}

// seg_base[seg][e] = pairs to expert e in segments before seg; this GPU's totals go to row my_rank of every peer's
// count matrix.  One block of 1024 threads: the segments are cut into 1024 / E groups (a power of two), thread
// (group, e) sums its group, a short scan over the groups gives its starting value, a second pass writes the prefixes.
__global__ void __launch_bounds__(1024)
publish_kernel(const int* __restrict__ seg_counts, int* __restrict__ seg_base, int num_experts,
               const __grid_constant__ PeerTable counts_all, int my_rank, int world) {
  __shared__ int group_sum[1024];
  pdl_wait_prior_grid();
  pdl_launch_dependents();
  int groups = 1;
  while (groups * 2 * num_experts <= 1024 && groups * 2 <= SEGMENTS) groups *= 2;
  const int per_group = SEGMENTS / groups;
  const int g = threadIdx.x / num_experts, e = threadIdx.x - g * num_experts;
  const bool active = g < groups;
  int total = 0;
  if (active) {
#pragma unroll 8
    for (int s = g * per_group; s < (g + 1) * per_group; ++s) total += seg_counts[(int64_t)s * num_experts + e];
    group_sum[g * num_experts + e] = total;
  }
  __syncthreads();
  if (active) {
    int running = 0;
    for (int h = 0; h < g; ++h) running += group_sum[h * num_experts + e];
#pragma unroll 8
    for (int s = g * per_group; s < (g + 1) * per_group; ++s) {
      const int c = seg_counts[(int64_t)s * num_experts + e];
      seg_base[(int64_t)s * num_experts + e] = running;
      running += c;
    }
    if (g == groups - 1)
      for (int p = 0; p < world; ++p) static_cast<int*>(counts_all.ptr[p])[my_rank * num_experts + e] = running;
  }
}

__global__ void __launch_bounds__(THREADS)
tables_kernel(const void* __restrict__ ids, int ids_int64, int pairs, int num_experts, const int* __restrict__ seg_base,
              const int* __restrict__ counts_all, int my_rank, int world, int k, int* __restrict__ dst_rank,
              int* __restrict__ dst_row, long long* __restrict__ dst_scale_offset, int* __restrict__ rows_out,
              int* __restrict__ eo_out, int* __restrict__ bo_out, int* __restrict__ total_rows_out,
              long long capacity_rows) {
  // shared: row_base[E] (row of the expert's first row from THIS GPU in the owner's buffer), sc_base[E] (scale-row
  // offset of the expert on its owner), in_expert[E] (rows of lower-ranked GPUs inside the expert), run[WARPS][E]
  extern __shared__ int sh[];
  int* eo_s = sh;
  int* bo_s = sh + num_experts;
  int* before_s = sh + 2 * num_experts;
  int* run = sh + 3 * num_experts;
  pdl_wait_prior_grid();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int e_local = num_experts / world;
  // per-expert totals; each owner's experts are then scanned serially by one thread (E / world entries: short)
  for (int e = threadIdx.x; e < num_experts; e += THREADS) {
    int m = 0, before = 0;
    for (int s = 0; s < world; ++s) {
      const int c = counts_all[s * num_experts + e];
      if (s < my_rank) before += c;
      m += c;
    }
    eo_s[e] = m;            // totals for now
    before_s[e] = before;
  }
  __syncthreads();
  if (threadIdx.x < world) {
    const int d = threadIdx.x;
    int rows = 0, srows = 0;
    for (int le = 0; le < e_local; ++le) {
      const int e = d * e_local + le;
      const int m = eo_s[e];
      eo_s[e] = rows;
      bo_s[e] = srows;
      if (d == my_rank && blockIdx.x == 0) {
        // Rows past the capacity of the receive buffers are dropped (the senders' stores to them are skipped by the
        // dispatch kernel's own range check): the expert that straddles the end is cut, later ones get no rows.
        long long room = capacity_rows - rows;
        if (room < 0) room = 0;
        const int kept = m < room ? m : (int)room;
        if (kept != m) atomicOr(&g_status, ERR_CAPACITY);
        rows_out[le] = kept;
        eo_out[le] = rows;
        bo_out[le] = srows;
      }
      rows += m;
      srows += (m + 127) & ~127;
    }
    if (d == my_rank && blockIdx.x == 0) *total_rows_out = rows < capacity_rows ? rows : (int)capacity_rows;
  }
  const int seg = blockIdx.x * WARPS + warp;
  int* my_run = run + warp * num_experts;
  for (int e = lane; e < num_experts; e += 32) my_run[e] = seg_base[(int64_t)seg * num_experts + e];
  __syncthreads();

  const int kt = k >> 7;
  const long long sf_row_bytes = k >> 5;
  const int len = segment_len(pairs);
  const int begin = seg * len;
  const int end = min(begin + len, pairs);
  for (int i0 = begin; i0 < end; i0 += 32) {
    const int i = i0 + lane;
    int e = i < end ? load_id(ids, ids_int64, i) : -1;
    if (e >= num_experts) e = -1;
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank_in_step = __popc(peers & ((1u << lane) - 1u));
    int pos = 0;
    if (e >= 0) pos = my_run[e] + rank_in_step;
    __syncwarp();
    if (e >= 0 && rank_in_step == 0) my_run[e] += __popc(peers);
    __syncwarp();
    if (i < end) {
      if (e >= 0) {
        const int r_local = before_s[e] + pos;                 // row inside the expert, on the owner
        dst_rank[i] = e / e_local;
        dst_row[i] = eo_s[e] + r_local;
        dst_scale_offset[i] = (long long)bo_s[e] * sf_row_bytes + scale_word_offset(r_local, kt);
      } else {
        dst_rank[i] = -1;                                       // reported and skipped by the dispatch kernel
        dst_row[i] = 0;
        dst_scale_offset[i] = 0;
      }
    }
  }
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

}  // namespace route
}  // namespace es_b200

extern "C" int es_b200_ep_route_count(const void* topk_ids, int ids_are_int64, int pairs, int num_experts,
                                      int32_t* segment_counts, int32_t* segment_base,
                                      const void* const* peer_counts_all, int my_rank, int world, void* stream) {
  using namespace es_b200;
  ES_REQUIRE(world >= 1 && world <= route::MAX_WORLD, "world size must be in [1, %d]", route::MAX_WORLD);
  ES_REQUIRE(my_rank >= 0 && my_rank < world, "rank out of range");
  ES_REQUIRE(num_experts >= 1 && num_experts <= ES_B200_MAX_EXPERTS && num_experts % world == 0,
             "num_experts must be a multiple of the world size and at most %d", ES_B200_MAX_EXPERTS);
  ES_REQUIRE(pairs >= 0, "pairs out of range");
  ES_REQUIRE(topk_ids && segment_counts && segment_base && peer_counts_all, "null pointer argument");
  route::PeerTable table;
  for (int i = 0; i < route::MAX_WORLD; ++i) table.ptr[i] = nullptr;
  for (int i = 0; i < world; ++i) {
    ES_REQUIRE(peer_counts_all[i] != nullptr, "peer pointer %d is null", i);
    table.ptr[i] = const_cast<void*>(peer_counts_all[i]);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)route::WARPS * num_experts * sizeof(int);
  route::count_kernel<<<route::BLOCKS, route::THREADS, smem, s>>>(topk_ids, ids_are_int64, pairs, num_experts,
                                                                  segment_counts);
  ES_CUDA_TRY(cudaGetLastError());
  route::publish_kernel<<<1, 1024, 0, s>>>(segment_counts, segment_base, num_experts, table, my_rank, world);
  ES_CUDA_TRY(cudaGetLastError());
  return ES_B200_OK;
}

extern "C" int es_b200_ep_route_tables(const void* topk_ids, int ids_are_int64, int pairs, int num_experts,
                                       const int32_t* segment_base, const int32_t* counts_all, int my_rank, int world,
                                       int k, int32_t* dst_rank, int32_t* dst_row, int64_t* dst_scale_offset,
                                       int32_t* rows, int32_t* expert_offsets, int32_t* blockscale_offsets,
                                       int32_t* total_rows, int64_t capacity_rows, void* stream) {
  using namespace es_b200;
  ES_REQUIRE(world >= 1 && world <= route::MAX_WORLD, "world size must be in [1, %d]", route::MAX_WORLD);
  ES_REQUIRE(my_rank >= 0 && my_rank < world, "rank out of range");
  ES_REQUIRE(num_experts >= 1 && num_experts <= ES_B200_MAX_EXPERTS && num_experts % world == 0,
             "num_experts must be a multiple of the world size and at most %d", ES_B200_MAX_EXPERTS);
  ES_REQUIRE(k > 0 && k % 128 == 0, "k must align to 128");
  ES_REQUIRE(pairs >= 0, "pairs out of range");
  ES_REQUIRE(capacity_rows > 0 && capacity_rows < (int64_t)1 << 31, "capacity_rows out of range");
  ES_REQUIRE(topk_ids && segment_base && counts_all && dst_rank && dst_row && dst_scale_offset && rows &&
                 expert_offsets && blockscale_offsets && total_rows,
             "null pointer argument");
  const size_t smem = (size_t)(3 + route::WARPS) * num_experts * sizeof(int);
  route::tables_kernel<<<route::BLOCKS, route::THREADS, smem, static_cast<cudaStream_t>(stream)>>>(
      topk_ids, ids_are_int64, pairs, num_experts, segment_base, counts_all, my_rank, world, k, dst_rank, dst_row,
      reinterpret_cast<long long*>(dst_scale_offset), rows, expert_offsets, blockscale_offsets, total_rows,
      capacity_rows);
  ES_CUDA_TRY(cudaGetLastError());
  return ES_B200_OK;
}

// ---------------------------------------------------------------------------------------------------------------------
// es_b200_ep_route_count for callers that cannot hand over scratch memory.
//
// The histogram step needs 256 x num_experts counters that are neither an input nor a result.  A serving process
// whose memory manager has claimed the whole GPU up front, or a host binding (cgo, JNI, a plugin ABI) that is given
// raw pointers by its caller and has no device allocator of its own, has nowhere to take them from on the request
// path.  For those callers the counters live in the library image: one array per GPU that loads the library, held
// until the process exits, sized for at most ES_B200_ROUTE_STATIC_MAX_EXPERTS experts (256 KB).
//
// `g_route_static_counts` is a device symbol: in host code its name is only a handle.  Its device address is looked
// up once per device (cudaGetSymbolAddress, with that device current) by the first call on that device and cached
// (under a lock); the cached address belongs to the device's primary context, so a process that destroys that context
// (cudaDeviceReset) must not call the library again afterwards.
// All calls on a device share the array: two calls that overlap on the GPU (different streams) would overwrite each
// other's counters.  Nothing has to be cleared between calls — the count kernel writes every counter it later reads.
static __device__ __align__(256) int32_t g_route_static_counts[es_b200::route::SEGMENTS * ES_B200_ROUTE_STATIC_MAX_EXPERTS];

extern "C" int es_b200_ep_route_count_static(const void* topk_ids, int ids_are_int64, int pairs, int num_experts,
                                             int32_t* segment_base, const void* const* peer_counts_all, int my_rank,
                                             int world, void* stream) {
  using namespace es_b200;
  ES_REQUIRE(num_experts >= 1 && num_experts <= ES_B200_ROUTE_STATIC_MAX_EXPERTS,
             "es_b200_ep_route_count_static holds counters for at most %d experts (got %d); use "
             "es_b200_ep_route_count with caller-provided scratch for more",
             ES_B200_ROUTE_STATIC_MAX_EXPERTS, num_experts);
  static int32_t* counters_of_device[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  ES_CUDA_TRY(cudaGetDevice(&dev));
  ES_REQUIRE(dev >= 0 && dev < 64, "device ordinal %d out of range", dev);
  int32_t* counters = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);       // first calls from several host threads
    if (counters_of_device[dev] == nullptr) {
      int32_t* p = nullptr;
      ES_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_route_static_counts));
      counters_of_device[dev] = p;
    }
    counters = counters_of_device[dev];
  }
  return es_b200_ep_route_count(topk_ids, ids_are_int64, pairs, num_experts, counters, segment_base, peer_counts_all,
                                my_rank, world, stream);
}
