// Accumulator -> global memory for the swap-AB grouped GEMM kernels.
//
// In TMEM the accumulator's lane is the output COLUMN n and its column is the token ROW, so a thread that reads its
// lane with tcgen05.ld holds one n for many tokens — the transpose of what coalesced stores of d[token, n] want.
// Each epilogue warp therefore passes 32 tokens x 32 n at a time through a private 2 KB shared-memory tile: written
// as [token][n] with 2-byte stores (32 lanes = 64 contiguous bytes, conflict free), read back as 16-byte pieces of a
// token row, and stored to global memory as 128-bit stores, four lanes per 64-byte row segment.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "sm100_ptx.cuh"

namespace es_b200 {

constexpr int EPI_STAGE_BYTES_PER_WARP = 32 * 32 * 2;

// Optional destination map of the output rows (expert-parallel combine fused into the GEMM): output row r goes to row
// meta[r].y of the [slots, n] array base[meta[r].x] — another GPU's buffer mapped into this process, or a local one —
// instead of row r of d.  meta == nullptr: dense output.  Entries out of range are skipped and reported.
constexpr int SCATTER_MAX_GPUS = 16;
constexpr uint32_t ERR_SCATTER_DESTINATION = 0x40000u;
struct RowScatter {
  const int2* meta;
  void* base[SCATTER_MAX_GPUS];
  long long slots;
  int gpus;
};

template <typename OutT>
__device__ __forceinline__ OutT out_from_f32(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 out_from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half out_from_f32<__half>(float v) { return __float2half_rn(v); }

// Scatter destination of output row `row` as a pointer to the warp's first column in that row, or null (entry out of
// range: reported; row past the valid ones: silent).
template <typename OutT>
__device__ __forceinline__ OutT* scatter_row_ptr(const RowScatter& scatter, int64_t row, bool in_range, int64_t ld,
                                                 int col_off, uint32_t* status) {
  if (!in_range) return nullptr;
  const int2 m = scatter.meta[row];
  if (m.x >= 0 && m.x < scatter.gpus && m.y >= 0 && m.y < scatter.slots)
    return static_cast<OutT*>(scatter.base[m.x]) + (int64_t)m.y * ld + col_off;
  atomicOr(status, ERR_SCATTER_DESTINATION);
  return nullptr;
}

// One chunk of 32 accumulator columns (tokens c .. c+31, this warp's 32 n) from registers to global memory through the
// warp's shared-memory tile.  `dest_row` is the scatter destination of token c + lane (unused for a dense output).
template <typename OutT, int TOK>
__device__ __forceinline__ void store_chunk(const uint32_t (&v)[32], int c, int valid, OutT* stage_warp, OutT* dst,
                                            int64_t ld, int lane, const RowScatter& scatter, OutT* dest_row) {
  const int part = lane & 3;
#pragma unroll
  for (int p = 0; p < 32 / TOK; ++p) {
#pragma unroll
    for (int j = 0; j < TOK; ++j) stage_warp[j * 32 + lane] = out_from_f32<OutT>(__uint_as_float(v[p * TOK + j]));
    __syncwarp();
#pragma unroll
    for (int it = 0; it < TOK / 8; ++it) {
      const int tok = it * 8 + (lane >> 2);
      const uint4 val = *reinterpret_cast<const uint4*>(stage_warp + tok * 32 + part * 8);
      const int row = c + p * TOK + tok;
      if (scatter.meta == nullptr) {
        if (row < valid) *reinterpret_cast<uint4*>(dst + (int64_t)row * ld + part * 8) = val;
      } else {
        const unsigned long long bits = reinterpret_cast<unsigned long long>(dest_row);
        OutT* out = reinterpret_cast<OutT*>(__shfl_sync(0xffffffffu, bits, p * TOK + tok));
        if (out != nullptr) *reinterpret_cast<uint4*>(out + part * 8) = val;
      }
    }
    __syncwarp();
  }
}

// Drains `n_cols` accumulator columns (a multiple of 16) starting at TMEM address `taddr` (this warp's lane quadrant)
// and stores the first `valid` of them: column j goes to dst[j * ld + 0..31] (dst = &d[first token][first n of warp]).
// `release` is called once, right after the last TMEM read has completed (the accumulator may then be overwritten).
// TOK = tokens per pass through the shared-memory tile (32: 2 KB per warp; 16: 1 KB; 8: 512 bytes).
// With a scatter map, column j goes to the mapped row of output row `first_row + j`, at column offset `col_off`
// (`dst` is then unused); `status` is the kernel's error word.
template <typename OutT, int TOK = 32, class Release>
__device__ __forceinline__ void drain_accumulator(uint32_t taddr, int n_cols, int valid, OutT* stage_warp, OutT* dst,
                                                  int64_t ld, bool do_store, int lane, Release release,
                                                  const RowScatter& scatter, int64_t first_row, int col_off,
                                                  uint32_t* status) {
  // two register sets: the TMEM read of chunk c+1 is in flight while chunk c goes through shared memory
  uint32_t va[32], vb[32];
  ptx::tc_ld_32x32b_x32(taddr, va);
  for (int c0 = 0; c0 < n_cols; c0 += 64) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int c = c0 + h * 32;
      if (c >= n_cols) break;
      // scatter map: lane l fetches the destination of token c + l now, so that the load's latency hides behind the
      // TMEM read and the conversions; the store loop picks it up with a shuffle
      OutT* dest = nullptr;
      if (scatter.meta != nullptr && do_store)
        dest = scatter_row_ptr<OutT>(scatter, first_row + c + lane, c + lane < valid, ld, col_off, status);
      ptx::tc_wait_ld();                                    // chunk c is in registers (va if h == 0, vb otherwise)
      const bool more = c + 32 < n_cols;
      if (more) {
        if (h == 0) ptx::tc_ld_32x32b_x32(taddr + c + 32, vb); else ptx::tc_ld_32x32b_x32(taddr + c + 32, va);
      } else {
        release();
      }
      if (do_store) {
        if (h == 0) store_chunk<OutT, TOK>(va, c, valid, stage_warp, dst, ld, lane, scatter, dest);
        else store_chunk<OutT, TOK>(vb, c, valid, stage_warp, dst, ld, lane, scatter, dest);
      }
    }
  }
}

// Accumulator kept as PARTS partial sums (column blocks `part_stride` columns apart): several threads issue the MMAs
// of a tile, each into a block of its own, and the sum is taken here in fp32, in block order.  `parts_written` (1 ..
// PARTS) blocks hold data (a tile with fewer K steps than issuing threads leaves the others untouched).  Drains
// `n_cols` columns (a multiple of 16, at most 128) and stores the first `valid` of them like drain_accumulator;
// `release` is called once, after the last TMEM read.
template <typename OutT, int PARTS, class Release>
__device__ __forceinline__ void drain_partial_sums(uint32_t taddr, uint32_t part_stride, int parts_written, int n_cols,
                                                   int valid, OutT* stage_warp, OutT* dst, int64_t ld, int lane,
                                                   Release release, const RowScatter& scatter, int64_t first_row,
                                                   int col_off, uint32_t* status) {
  for (int c = 0; c < n_cols; c += 32) {
    OutT* dest = nullptr;
    if (scatter.meta != nullptr)
      dest = scatter_row_ptr<OutT>(scatter, first_row + c + lane, c + lane < valid, ld, col_off, status);
    uint32_t acc[32];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int c0 = c + h * 16;
      if (c0 < n_cols) {
        uint32_t v[PARTS][16];
#pragma unroll
        for (int p = 0; p < PARTS; ++p)
          if (p < parts_written) ptx::tc_ld_32x32b_x16(taddr + p * part_stride + c0, v[p]);   // warp-uniform
        ptx::tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float sum = __uint_as_float(v[0][i]);
#pragma unroll
          for (int p = 1; p < PARTS; ++p)
            if (p < parts_written) sum += __uint_as_float(v[p][i]);
          acc[h * 16 + i] = __float_as_uint(sum);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[h * 16 + i] = 0u;
      }
    }
    if (c + 32 >= n_cols) release();
    store_chunk<OutT, 32>(acc, c, valid, stage_warp, dst, ld, lane, scatter, dest);
  }
}

// The same for a warp that shares its lane quadrant with other warps: it takes the 32-column chunks first_chunk,
// first_chunk + chunk_stride, ... and keeps one register set — the warps of a quadrant hide each other's TMEM
// latency.  A warp without a chunk only calls `release`.
template <typename OutT, int TOK, class Release>
__device__ __forceinline__ void drain_accumulator_shared(uint32_t taddr, int n_cols, int valid, OutT* stage_warp,
                                                         OutT* dst, int64_t ld, bool do_store, int lane,
                                                         Release release, const RowScatter& scatter,
                                                         int64_t first_row, int col_off, uint32_t* status,
                                                         int first_chunk, int chunk_stride) {
  if (first_chunk >= n_cols) {
    release();
    return;
  }
  uint32_t v[32];
  for (int c = first_chunk; c < n_cols; c += chunk_stride) {
    OutT* dest = nullptr;
    if (scatter.meta != nullptr && do_store)
      dest = scatter_row_ptr<OutT>(scatter, first_row + c + lane, c + lane < valid, ld, col_off, status);
    ptx::tc_ld_32x32b_x32(taddr + c, v);
    ptx::tc_wait_ld();
    if (c + chunk_stride >= n_cols) release();
    if (do_store) store_chunk<OutT, TOK>(v, c, valid, stage_warp, dst, ld, lane, scatter, dest);
  }
}

}  // namespace es_b200
