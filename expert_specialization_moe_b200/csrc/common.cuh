// Shared host/device helpers of the es_b200 library (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

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

// ---- device: programmatic dependent launch ---------------------------------------------------
// Both are no-ops when the kernel was not launched with the programmatic-stream-serialization attribute.
__device__ __forceinline__ void pdl_wait_prior_grid() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

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

}  // namespace es_b200
