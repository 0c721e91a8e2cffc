// Expert-parallel dispatch and combine over peer memory (NVLink / NVSwitch), fused with the work on either side of
// the exchange.  The reference has no distributed code; these kernels are what replaces an all-to-all + permutation
// + quantisation sequence when the experts of one MoE layer are spread over the GPUs of a node.
//
//   dispatch  es_b200_ep_dispatch_quant_push: every token row is quantised ONCE (MXFP8, same arithmetic as the grouped
//             quant kernel) and its codes plus one small side record (return address, position of its scales in the
//             owner's swizzled scale buffer, its k/32 scale bytes) are stored straight into the receive buffers of
//             the GPUs that own its top-k experts — 1.03 bytes per element cross NVLink instead of 2, and no bf16
//             copy of the routed rows ever exists.  The side record travels as one contiguous piece: sixteen
//             separate 4-byte scale stores per row cost a third of the dispatch time over NVLink (measured).
//   unpack    es_b200_ep_unpack_side (local, after the barrier): scale bytes of the received rows -> swizzled scale
//             buffer, return addresses -> the (GPU, slot) table the combine reads.
//   combine   es_b200_ep_combine_push: every expert-output row is stored into the (token, j) slot of the GPU the token
//             came from.
//   reduce    es_b200_ep_topk_weighted_sum: out[t] = sum_j w[t, j] * pairs[t, j], fp32 accumulation.
//
//   barrier   es_b200_ep_barrier: one small kernel per GPU; each GPU stores the next epoch number into its slot of every
//             peer's flag array and waits, for at most five seconds, until all of its own slots show that epoch.
//
// All remote accesses are plain stores through peer-mapped pointers (no multicast, no loads from peers); the three
// data kernels never wait on another GPU, ordering between GPUs is the barrier between the steps.  Every destination
// index is range-checked; a bad one is skipped, and a barrier that gives up returns: both are reported through
// es_b200_check_status.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "mxfp8_quant_math.cuh"

namespace es_b200 {
namespace ep {

constexpr int THREADS = 256;                 // 8 warps, one row per warp
constexpr int MAX_TOPK = 16;
constexpr int MAX_WORLD = 16;
constexpr uint32_t ERR_BAD_DESTINATION = 0x10000u, ERR_BARRIER_TIMEOUT = 0x20000u;
constexpr unsigned long long BARRIER_DEFAULT_LIMIT_NS = 5000000000ull;

__device__ uint32_t g_status = 0;

struct PeerTable {
  void* ptr[MAX_WORLD];
};

__device__ __forceinline__ void st_8B(void* p, uint2 v) {
  asm volatile("st.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

// Side record of a received row: { int32 source GPU, int32 pair index, int64 byte offset of the row's scale word for
// K tile 0 in the owner's swizzled scale buffer, k/32 scale bytes }, padded to a multiple of 16 bytes.
__host__ __device__ __forceinline__ int side_record_bytes(int k) { return 16 + (((k >> 5) + 15) & ~15); }

// One warp per token row.  Per pass a lane holds 4 x 8 elements (1024 elements per warp); the codes of the pass stay
// in registers while they are stored to each of the row's top-k destinations, the scale words collect in a per-warp
// shared-memory copy of the side record, which goes out once per destination after the last pass.
template <typename T>
__global__ void __launch_bounds__(THREADS)
dispatch_quant_push_kernel(const T* __restrict__ x, const int* __restrict__ dst_rank, const int* __restrict__ dst_row,
                           const long long* __restrict__ dst_sf_offset, const __grid_constant__ PeerTable codes,
                           const __grid_constant__ PeerTable side, int my_rank, int world, int tokens, int topk, int k,
                           long long capacity_rows, uint4* __restrict__ my_pairs, int pair_row_vec16) {
  // one side record per warp; dynamic, so that the kernel's footprint stays small enough to share an SM with a
  // grouped GEMM CTA of another stream
  extern __shared__ __align__(16) uint8_t side_s[];
  pdl_wait_prior_grid();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps_per_grid = gridDim.x * (THREADS / 32);
  const int side_bytes = side_record_bytes(k);
  uint8_t* rec = side_s + warp * side_bytes;
  for (int t = blockIdx.x * (THREADS / 32) + warp; t < tokens; t += warps_per_grid) {
    // lane j < topk holds destination j; bad destinations are dropped here, once
    int my_rank_j = -1, my_row_j = 0;
    long long my_sf_j = 0;
    if (lane < topk) {
      const int pair = t * topk + lane;
      my_rank_j = dst_rank[pair];
      my_row_j = dst_row[pair];
      my_sf_j = dst_sf_offset[pair];
      if (!(my_rank_j >= 0 && my_rank_j < world && my_row_j >= 0 && my_row_j < capacity_rows)) {
        atomicOr(&g_status, ERR_BAD_DESTINATION);
        my_rank_j = -1;
      }
    }
    // A dropped pair sends nothing, so nothing comes back into its (token, j) slot: clear the slot here, or the
    // weighted sum would add whatever an earlier step left there.  No peer writes this slot in this step, and stream
    // order puts the store after the previous step's weighted sum.
    if (my_pairs != nullptr) {
      for (int d = 0; d < topk; ++d) {
        if (__shfl_sync(0xffffffffu, my_rank_j, d) >= 0) continue;      // warp-uniform
        uint4* slot = my_pairs + ((int64_t)t * topk + d) * pair_row_vec16;
        for (int i = lane; i < pair_row_vec16; i += 32) slot[i] = make_uint4(0, 0, 0, 0);
      }
    }
    const T* in_row = x + (int64_t)t * k;
    for (int c0 = 0; c0 < k; c0 += 1024) {
      uint4 raw[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = c0 + j * 256 + lane * 8;
        raw[j] = col < k ? ld_stream_16B(in_row + col) : make_uint4(0, 0, 0, 0);
      }
      uint2 code[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t sf = quantize8<T>(raw[j], code[j]);
        // the four scale bytes of one K tile (lanes 0-15 / 16-31) as one 32-bit word in lanes 0 and 16
        uint32_t w = sf << (((lane >> 2) & 3) * 8);
        w |= __shfl_xor_sync(0xffffffffu, w, 4);
        w |= __shfl_xor_sync(0xffffffffu, w, 8);
        const int col = c0 + j * 256 + lane * 8;
        if ((lane & 15) == 0 && col < k) *reinterpret_cast<uint32_t*>(rec + 16 + (col >> 7) * 4) = w;
      }
      for (int d = 0; d < topk; ++d) {
        const int rank = __shfl_sync(0xffffffffu, my_rank_j, d);
        const int row = __shfl_sync(0xffffffffu, my_row_j, d);
        if (rank < 0) continue;                                   // warp-uniform
        uint8_t* out_row = reinterpret_cast<uint8_t*>(codes.ptr[rank]) + (int64_t)row * k;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int col = c0 + j * 256 + lane * 8;
          if (col < k) st_8B(out_row + col, code[j]);
        }
      }
    }
    __syncwarp();
    for (int d = 0; d < topk; ++d) {
      const int rank = __shfl_sync(0xffffffffu, my_rank_j, d);
      const int row = __shfl_sync(0xffffffffu, my_row_j, d);
      const long long sf_off = __shfl_sync(0xffffffffu, my_sf_j, d);
      if (rank < 0) continue;                                     // warp-uniform
      uint4* out = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(side.ptr[rank]) + (int64_t)row * side_bytes);
      for (int i = lane; i < side_bytes / 16; i += 32) {
        uint4 v;
        if (i == 0) {
          v = make_uint4((uint32_t)my_rank, (uint32_t)(t * topk + d), (uint32_t)(sf_off & 0xffffffffll),
                         (uint32_t)(sf_off >> 32));
        } else {
          v = *reinterpret_cast<const uint4*>(rec + i * 16);
        }
        out[i] = v;
      }
    }
    __syncwarp();                // the record is rewritten by the next row
  }
  // no fence here: the stores become visible to the peers with the completion of this kernel, and the barrier kernel
  // that follows on the stream orders them before its flag
}

// One warp per received row: the side record's scale bytes go to their swizzled position, its return address to the
// (GPU, slot) table.  Offsets are range-checked: a bad one is skipped and reported.
__global__ void __launch_bounds__(THREADS)
unpack_side_kernel(const uint8_t* __restrict__ side, const int* __restrict__ num_rows_dev, uint8_t* __restrict__ scales,
                   int2* __restrict__ meta, int k, long long capacity_rows, long long scale_bytes) {
  pdl_wait_prior_grid();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int warps_per_grid = gridDim.x * (THREADS / 32);
  const int side_bytes = side_record_bytes(k);
  const int kt = k >> 7;
  long long rows = *num_rows_dev;
  if (rows > capacity_rows) rows = capacity_rows;
  for (long long r = blockIdx.x * (THREADS / 32) + (threadIdx.x >> 5); r < rows; r += warps_per_grid) {
    const uint8_t* rec = side + r * side_bytes;
    const uint4 head = *reinterpret_cast<const uint4*>(rec);
    const long long sf_off = (long long)head.z | ((long long)head.w << 32);
    if (lane == 0) meta[r] = make_int2((int)head.x, (int)head.y);
    const bool ok = sf_off >= 0 && (sf_off & 3) == 0 && sf_off + (long long)(kt - 1) * 512 + 4 <= scale_bytes;
    if (!ok) {
      if (lane == 0) atomicOr(&g_status, ERR_BAD_DESTINATION);
      continue;
    }
    for (int q = lane; q < kt; q += 32)
      *reinterpret_cast<uint32_t*>(scales + sf_off + (long long)q * 512) = *reinterpret_cast<const uint32_t*>(rec + 16 + q * 4);
  }
}

// One warp per expert-output row: 16-byte loads of the local row, 16-byte stores into the owner's pair buffer.
__global__ void __launch_bounds__(THREADS)
combine_push_kernel(const uint4* __restrict__ y, const int2* __restrict__ meta, const int* __restrict__ num_rows_dev,
                    const __grid_constant__ PeerTable pairs, int world, long long capacity_rows,
                    long long pairs_per_rank, int row_vec16) {
  pdl_wait_prior_grid();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int warps_per_grid = gridDim.x * (THREADS / 32);
  long long rows = *num_rows_dev;
  if (rows > capacity_rows) rows = capacity_rows;
  for (long long r = blockIdx.x * (THREADS / 32) + (threadIdx.x >> 5); r < rows; r += warps_per_grid) {
    const int2 m = meta[r];
    if (m.x < 0 || m.x >= world || m.y < 0 || m.y >= pairs_per_rank) {
      if (lane == 0) atomicOr(&g_status, ERR_BAD_DESTINATION);
      continue;
    }
    const uint4* src = y + r * row_vec16;
    uint4* dst = reinterpret_cast<uint4*>(pairs.ptr[m.x]) + (long long)m.y * row_vec16;
    for (int c = lane; c < row_vec16; c += 128) {
      uint4 v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (c + j * 32 < row_vec16) v[j] = src[c + j * 32];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (c + j * 32 < row_vec16) dst[c + j * 32] = v[j];
    }
  }
}

template <typename T>
struct Pack2;
template <>
struct Pack2<__nv_bfloat16> {
  static __device__ __forceinline__ float2 unpack(uint32_t w) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w)); }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 r = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&r);
  }
};
template <>
struct Pack2<__half> {
  static __device__ __forceinline__ float2 unpack(uint32_t w) { return __half22float2(*reinterpret_cast<__half2*>(&w)); }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 r = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&r);
  }
};

// One warp per token; a lane accumulates 8 columns at a time in fp32 over the token's top-k rows, in order j = 0..topk-1.
template <typename T>
__global__ void __launch_bounds__(THREADS)
topk_weighted_sum_kernel(const uint4* __restrict__ pairs, const float* __restrict__ weights, uint4* __restrict__ out,
                         int tokens, int topk, int row_vec16) {
  pdl_wait_prior_grid();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int warps_per_grid = gridDim.x * (THREADS / 32);
  for (int t = blockIdx.x * (THREADS / 32) + (threadIdx.x >> 5); t < tokens; t += warps_per_grid) {
    const float w_lane = lane < topk ? weights[(int64_t)t * topk + lane] : 0.f;
    for (int c = lane; c < row_vec16; c += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < topk; ++j) {
        const float w = __shfl_sync(0xffffffffu, w_lane, j);
        const uint4 v = pairs[((int64_t)t * topk + j) * row_vec16 + c];
        const uint32_t vw[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = Pack2<T>::unpack(vw[i]);
          acc[2 * i] = fmaf(w, f.x, acc[2 * i]);
          acc[2 * i + 1] = fmaf(w, f.y, acc[2 * i + 1]);
        }
      }
      out[(int64_t)t * row_vec16 + c] = make_uint4(Pack2<T>::pack(acc[0], acc[1]), Pack2<T>::pack(acc[2], acc[3]),
                                                   Pack2<T>::pack(acc[4], acc[5]), Pack2<T>::pack(acc[6], acc[7]));
    }
  }
}

// flags layout (uint32, in every GPU's symmetric buffer): [0, MAX_WORLD) epoch last announced by each GPU,
// [MAX_WORLD] this GPU's own epoch counter (only ever touched by this GPU's barrier kernel).
__global__ void __launch_bounds__(32) barrier_kernel(const __grid_constant__ PeerTable flags, int my_rank, int world,
                                                      unsigned long long limit_ns) {
  const int lane = threadIdx.x;
  uint32_t* mine = reinterpret_cast<uint32_t*>(flags.ptr[my_rank]);
  uint32_t epoch = 0;
  if (lane == 0) {
    epoch = mine[MAX_WORLD] + 1;
    mine[MAX_WORLD] = epoch;
  }
  epoch = __shfl_sync(0xffffffffu, epoch, 0);
  __threadfence_system();       // everything this GPU stored to its peers before this launch is ordered before the flag
  if (lane < world) {
    uint32_t* theirs = reinterpret_cast<uint32_t*>(flags.ptr[lane]) + my_rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
    const unsigned long long t0 = [] { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }();
    uint32_t seen = 0;
    while (true) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine + lane) : "memory");
      if ((int32_t)(seen - epoch) >= 0) break;
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (now - t0 > limit_ns) {
        atomicOr(&g_status, ERR_BARRIER_TIMEOUT);
        break;
      }
      __nanosleep(100);
    }
  }
  __syncwarp();
  __threadfence_system();
}

static int fill_table(PeerTable* t, const void* const* host_ptrs, int world) {
  for (int i = 0; i < MAX_WORLD; ++i) t->ptr[i] = nullptr;
  for (int i = 0; i < world; ++i) {
    if (host_ptrs[i] == nullptr) return fail(ES_B200_ERR_INVALID_ARGUMENT, "peer pointer %d is null", i);
    if (!aligned16(host_ptrs[i])) return fail(ES_B200_ERR_INVALID_ARGUMENT, "peer pointer %d is not 16-byte aligned", i);
    t->ptr[i] = const_cast<void*>(host_ptrs[i]);
  }
  return ES_B200_OK;
}

static int grid_for(int64_t rows, int* grid) {
  DeviceInfo info;
  int rc = get_device_info(&info);
  if (rc != ES_B200_OK) return rc;
  const int64_t blocks = (rows + THREADS / 32 - 1) / (THREADS / 32);
  const int64_t resident = (int64_t)info.sm_count * 8;
  *grid = (int)(blocks < resident ? (blocks > 0 ? blocks : 1) : resident);
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

}  // namespace ep
}  // namespace es_b200

extern "C" int es_b200_ep_side_record_bytes(int k) { return es_b200::ep::side_record_bytes(k); }

extern "C" int es_b200_ep_dispatch_quant_push(const void* x, int x_dtype, const int32_t* dst_rank,
                                              const int32_t* dst_row, const int64_t* dst_scale_offset,
                                              const void* const* peer_codes, const void* const* peer_side, int my_rank,
                                              int world, int tokens, int topk, int k, int64_t capacity_rows,
                                              void* my_pairs, int pair_row_bytes, void* stream) {
  using namespace es_b200;
  ES_REQUIRE(my_pairs == nullptr || (aligned16(my_pairs) && pair_row_bytes > 0 && pair_row_bytes % 16 == 0),
             "my_pairs must be 16-byte aligned with rows of a multiple of 16 bytes");
  ES_REQUIRE(x_dtype == ES_B200_BF16 || x_dtype == ES_B200_FP16, "dtype must be kFloat16 or kBFloat16");
  ES_REQUIRE(k > 0 && k % 128 == 0 && k <= 16384, "k must align to 128 and be at most 16384");
  ES_REQUIRE(world >= 1 && world <= ep::MAX_WORLD, "world size must be in [1, %d]", ep::MAX_WORLD);
  ES_REQUIRE(my_rank >= 0 && my_rank < world, "rank out of range");
  ES_REQUIRE(topk >= 1 && topk <= ep::MAX_TOPK, "topk must be in [1, %d]", ep::MAX_TOPK);
  ES_REQUIRE(tokens >= 0 && (int64_t)tokens * topk < (int64_t)1 << 31, "tokens * topk out of range");
  ES_REQUIRE(capacity_rows > 0 && capacity_rows < (int64_t)1 << 31, "capacity_rows out of range");
  if (tokens == 0) return ES_B200_OK;
  ES_REQUIRE(x && dst_rank && dst_row && dst_scale_offset && peer_codes && peer_side, "null pointer argument");
  ES_REQUIRE(aligned16(x), "x must be 16-byte aligned");
  ep::PeerTable codes, side;
  int rc = ep::fill_table(&codes, peer_codes, world);
  if (rc == ES_B200_OK) rc = ep::fill_table(&side, peer_side, world);
  if (rc != ES_B200_OK) return rc;
  int grid = 1;
  rc = ep::grid_for(tokens, &grid);
  if (rc != ES_B200_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t side_smem = (size_t)(ep::THREADS / 32) * ep::side_record_bytes(k);
  if (x_dtype == ES_B200_BF16)
    ep::dispatch_quant_push_kernel<__nv_bfloat16><<<grid, ep::THREADS, side_smem, s>>>(
        static_cast<const __nv_bfloat16*>(x), dst_rank, dst_row, reinterpret_cast<const long long*>(dst_scale_offset),
        codes, side, my_rank, world, tokens, topk, k, capacity_rows, static_cast<uint4*>(my_pairs), pair_row_bytes / 16);
  else
    ep::dispatch_quant_push_kernel<__half><<<grid, ep::THREADS, side_smem, s>>>(
        static_cast<const __half*>(x), dst_rank, dst_row, reinterpret_cast<const long long*>(dst_scale_offset), codes,
        side, my_rank, world, tokens, topk, k, capacity_rows, static_cast<uint4*>(my_pairs), pair_row_bytes / 16);
  ES_CUDA_TRY(cudaGetLastError());
  return ES_B200_OK;
}

extern "C" int es_b200_ep_unpack_side(const void* side, const int32_t* num_rows_dev, uint8_t* scales, int32_t* meta,
                                      int k, int64_t capacity_rows, int64_t scale_bytes, void* stream) {
  using namespace es_b200;
  ES_REQUIRE(k > 0 && k % 128 == 0 && k <= 16384, "k must align to 128 and be at most 16384");
  ES_REQUIRE(capacity_rows > 0 && capacity_rows < (int64_t)1 << 31 && scale_bytes > 0, "buffer sizes out of range");
  ES_REQUIRE(side && num_rows_dev && scales && meta, "null pointer argument");
  ES_REQUIRE(aligned16(side) && (reinterpret_cast<uintptr_t>(scales) & 3u) == 0 &&
                 (reinterpret_cast<uintptr_t>(meta) & 7u) == 0,
             "side must be 16-byte, meta 8-byte and scales 4-byte aligned");
  int grid = 1;
  int rc = ep::grid_for(capacity_rows, &grid);
  if (rc != ES_B200_OK) return rc;
  ep::unpack_side_kernel<<<grid, ep::THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(side), num_rows_dev, scales, reinterpret_cast<int2*>(meta), k, capacity_rows,
      scale_bytes);
  ES_CUDA_TRY(cudaGetLastError());
  return ES_B200_OK;
}

extern "C" int es_b200_ep_combine_push(const void* y, const int32_t* meta, const int32_t* num_rows_dev,
                                       const void* const* peer_pairs, int world, int64_t capacity_rows,
                                       int64_t pairs_per_rank, int n, int elem_bytes, void* stream) {
  using namespace es_b200;
  ES_REQUIRE(world >= 1 && world <= ep::MAX_WORLD, "world size must be in [1, %d]", ep::MAX_WORLD);
  ES_REQUIRE(elem_bytes == 2, "rows must be bf16 or fp16");
  ES_REQUIRE(n > 0 && (n * elem_bytes) % 16 == 0, "row size must be a multiple of 16 bytes");
  ES_REQUIRE(capacity_rows > 0 && pairs_per_rank >= 0, "buffer sizes out of range");
  ES_REQUIRE(y && meta && num_rows_dev && peer_pairs, "null pointer argument");
  ES_REQUIRE(aligned16(y) && (reinterpret_cast<uintptr_t>(meta) & 7u) == 0, "y must be 16-byte and meta 8-byte aligned");
  ep::PeerTable pairs;
  int rc = ep::fill_table(&pairs, peer_pairs, world);
  if (rc != ES_B200_OK) return rc;
  int grid = 1;
  rc = ep::grid_for(capacity_rows, &grid);
  if (rc != ES_B200_OK) return rc;
  ep::combine_push_kernel<<<grid, ep::THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(y), reinterpret_cast<const int2*>(meta), num_rows_dev, pairs, world, capacity_rows,
      pairs_per_rank, n * elem_bytes / 16);
  ES_CUDA_TRY(cudaGetLastError());
  return ES_B200_OK;
}

extern "C" int es_b200_ep_topk_weighted_sum(const void* pairs, int dtype, const float* weights, void* out, int tokens,
                                            int topk, int n, void* stream) {
  using namespace es_b200;
  ES_REQUIRE(dtype == ES_B200_BF16 || dtype == ES_B200_FP16, "dtype must be kFloat16 or kBFloat16");
  ES_REQUIRE(topk >= 1 && topk <= 32, "topk must be in [1, 32]");
  ES_REQUIRE(n > 0 && n % 8 == 0, "n must be a multiple of 8");
  ES_REQUIRE(tokens >= 0, "tokens out of range");
  if (tokens == 0) return ES_B200_OK;
  ES_REQUIRE(pairs && weights && out, "null pointer argument");
  ES_REQUIRE(aligned16(pairs) && aligned16(out), "pairs and out must be 16-byte aligned");
  int grid = 1;
  int rc = ep::grid_for(tokens, &grid);
  if (rc != ES_B200_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == ES_B200_BF16)
    ep::topk_weighted_sum_kernel<__nv_bfloat16><<<grid, ep::THREADS, 0, s>>>(
        static_cast<const uint4*>(pairs), weights, static_cast<uint4*>(out), tokens, topk, n / 8);
  else
    ep::topk_weighted_sum_kernel<__half><<<grid, ep::THREADS, 0, s>>>(static_cast<const uint4*>(pairs), weights,
                                                                      static_cast<uint4*>(out), tokens, topk, n / 8);
  ES_CUDA_TRY(cudaGetLastError());
  return ES_B200_OK;
}

extern "C" int es_b200_ep_barrier_limit(const void* const* peer_flags, int my_rank, int world, int64_t limit_ns,
                                        void* stream) {
  using namespace es_b200;
  ES_REQUIRE(limit_ns > 0, "the wait limit must be positive");
  ES_REQUIRE(world >= 1 && world <= ep::MAX_WORLD, "world size must be in [1, %d]", ep::MAX_WORLD);
  ES_REQUIRE(my_rank >= 0 && my_rank < world, "rank out of range");
  ES_REQUIRE(peer_flags, "null pointer argument");
  ep::PeerTable flags;
  int rc = ep::fill_table(&flags, peer_flags, world);
  if (rc != ES_B200_OK) return rc;
  ep::barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flags, my_rank, world,
                                                                      (unsigned long long)limit_ns);
  ES_CUDA_TRY(cudaGetLastError());
  return ES_B200_OK;
}

extern "C" int es_b200_ep_barrier(const void* const* peer_flags, int my_rank, int world, void* stream) {
  return es_b200_ep_barrier_limit(peer_flags, my_rank, world, (int64_t)es_b200::ep::BARRIER_DEFAULT_LIMIT_NS, stream);
}
