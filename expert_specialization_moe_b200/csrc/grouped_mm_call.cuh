// What the kernels of one MXFP8 grouped GEMM call share on the host: the call's arguments, and the launch functions of
// the CTA-pair kernel (mxfp8_grouped_mm_pair.cu) that the dispatcher in mxfp8_grouped_mm.cu chains behind the
// single-CTA kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "epilogue.cuh"

namespace es_b200 {
namespace mm {

struct CallArgs {
  const void* a;
  const void* b;
  const uint8_t* sfa;
  const uint8_t* sfb;
  void* d;
  const int32_t* ps;
  const int32_t* eo;
  const int32_t* bo;
  int num_experts;
  int64_t num_rows;
  int n, k;
  int64_t sfa_rows;
  const RowScatter* scatter;
  uint32_t* counters;      // work counters in the caller's scratch; null: tiles are dealt round-robin over each grid
  cudaStream_t stream;
};

}  // namespace mm

namespace mm2 {
// min_rows: experts with fewer rows belong to the other kernels; max_clusters: cap of the grid in CTA pairs (0 = as
// many as fit on the device); first / last: position of the launch in the call's chain of kernels; earlier_ctas: in/out,
// CTAs launched so far by the call (the last kernel waits for that many to report before it exits).
int launch_bf16(const mm::CallArgs& c, int min_rows, int max_clusters, bool first_of_call, bool last_of_call,
                uint32_t* earlier_ctas);
int launch_fp16(const mm::CallArgs& c, int min_rows, int max_clusters, bool first_of_call, bool last_of_call,
                uint32_t* earlier_ctas);
int read_and_clear_status(uint32_t* out);
}  // namespace mm2

}  // namespace es_b200
