// Row-count thresholds of the MXFP8 grouped GEMM's tile-shape buckets per weight shape (n, k).
//
// The reference picks its bucket rules per device and by arithmetic intensity
// (es_fp8_blockwise_functor.cuh:122-145,169-191,214-236: H20 and Hx00 use different filters).  Here the device is fixed
// (B200) and what moves the best threshold is the weight shape: how long a tile streams one [128 x k] slab (k) and
// how many CTAs one expert's tiles occupy (n).  Entries were measured (each threshold pair timed on the shape with
// Zipf(1.2) row counts, configurations interleaved, after the GPU had reached its power-capped steady state); shapes
// without an entry use the default.
#pragma once

namespace es_b200 {

struct BucketThresholds {
  int tiny_max_rows;    // experts with at most this many rows: 128 x <=32 streaming tiles (at most 32)
  int heavy_min_rows;   // experts with at least this many rows: CTA-pair tiles (at most 113: the larger streaming
                        // shape holds 112 token rows)
};

struct BucketTableEntry {
  int n, k;
  BucketThresholds t;
};

constexpr BucketThresholds kDefaultBuckets = {32, 113};
constexpr BucketTableEntry kBucketTable[] = {
    // n, k, {tiny_max, heavy_min}        measured (ms per call, Zipf(1.2) counts, power-capped steady state)
    {4096, 7168, {32, 65}},    // DeepSeek-V3 gate_up, 32768 rows: 1.81 (32/65) vs 1.90 (32/113), 1.98 (32/33)
    {7168, 2048, {32, 113}},   // DeepSeek-V3 down: 512 rows 0.272 (32/113) vs 0.277 (32/33); 16384 rows 0.84 either way
    {1536, 2048, {32, 113}},   // Qwen3-30B-A3B gate_up, 16384 rows: 0.125 (32/113) vs 0.139 (32/65)
    {2048, 768, {32, 113}},    // Qwen3-30B-A3B down, 16384 rows: 0.089 (32/113) vs 0.098 (32/65)
    {512, 7168, {32, 113}},    // DeepSeek-R1 gate_up TP8: with Zipf counts (8192 rows) 32/33 is 9 % faster than 32/113, with
                               // the reference benchmark's 70/15/10/5 % distribution 8 % slower: the default stays
};

inline BucketThresholds bucket_thresholds(int n, int k) {
  for (const BucketTableEntry& e : kBucketTable)
    if (e.n == n && e.k == k) return e.t;
  return kDefaultBuckets;
}

}  // namespace es_b200
