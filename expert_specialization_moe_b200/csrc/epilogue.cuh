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

// Accumulator kept as PARTS partial sums (column blocks `part_stride` columns apart): several threads issue the MMAs
// of a tile, each into a block of its own, and the sum is taken here in fp32, in block order.  `parts_written` (1 ..
// PARTS) blocks hold data (a tile with fewer K steps than issuing threads leaves the others untouched).  Drains
// `n_cols` columns (a multiple of 16, at most 128) starting at TMEM address `taddr` (this warp's lane quadrant) and
// stores the first `valid` of them: column j goes to dst[j * ld + 0..31] (dst = &d[first token][first n of warp]); with
// a scatter map, to the mapped row of output row `first_row + j` at column offset `col_off` (`dst` is then unused).
// `release` is called once, after the last TMEM read (the accumulator may then be overwritten); `status` is the
// kernel's error word.
template <typename OutT, int PARTS, class Release>
__device__ __forceinline__ void drain_partial_sums(uint32_t taddr, uint32_t part_stride, int parts_written, int n_cols,
                                                   int valid, OutT* stage_warp, OutT* dst, int64_t ld, int lane,
                                                   Release release, const RowScatter& scatter, int64_t first_row,
                                                   int col_off, uint32_t* status, bool direct_stores,
                                                   int first_col = 0, int col_stride = 32) {
  // (a warp that shares its lane quadrant with another takes the 32-column chunks first_col, first_col + col_stride,
  // ...; one without a chunk in this tile only hands the accumulator back)
  if (first_col >= n_cols) {
    release();
    return;
  }
  for (int c = first_col; c < n_cols; c += col_stride) {
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
    if (c + col_stride >= n_cols) release();
    if (direct_stores && scatter.meta == nullptr) {
      // dense output without shared memory: a warp-wide 2-byte store writes the 64 contiguous bytes of one token row.
      // The caller asks for it when K is long (the output is a small part of the call's bytes): no store -> sync ->
      // load round trip behind the operand traffic in shared memory (reference distribution, k = 7168 and 4096: 3-4 %
      // per call).  With short K the output is a large part of the traffic and the staged 128-bit stores win
      // (k = 256, n = 7168: 0.194 vs 0.222 ms; k = 384: 0.080 vs 0.089).
      OutT* out = dst + (int64_t)c * ld + lane;
      const int rows = valid - c;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (j < rows) *out = out_from_f32<OutT>(__uint_as_float(acc[j]));
        out += ld;
      }
    } else {
      store_chunk<OutT, 32>(acc, c, valid, stage_warp, dst, ld, lane, scatter, dest);
    }
  }
}

template <typename OutT>
__device__ __forceinline__ uint32_t pack_pair_from_f32(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack_pair_from_f32<__nv_bfloat16>(float lo, float hi) {
  const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&p);
}
template <>
__device__ __forceinline__ uint32_t pack_pair_from_f32<__half>(float lo, float hi) {
  const __half2 p = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&p);
}

// ---- an epilogue that holds converted chunks in registers (the CTA-pair kernel) ---------------------------------
// A held chunk is 32 accumulator columns (tokens) of the warp's 32 lanes (n): register i = tokens (2i, 2i+1) as two
// 16-bit values.  The warp reads all its chunks of an accumulator into held registers, hands the accumulator back to
// the MMA lanes, and stores afterwards: the stores of an item take several thousand cycles while the K loop's operand
// traffic shares the memory system, and the next item's MMAs run meanwhile.

// TMEM -> held registers (the caller releases the accumulator after its last read_held_chunk)
template <typename OutT>
__device__ __forceinline__ void read_held_chunk(uint32_t taddr, uint32_t (&held)[16]) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint32_t v[16];
    ptx::tc_ld_32x32b_x16(taddr + h * 16, v);
    ptx::tc_wait_ld();
#pragma unroll
    for (int i = 0; i < 8; ++i)
      held[h * 8 + i] = pack_pair_from_f32<OutT>(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
  }
}

// Dense output without shared memory: a warp-wide 2-byte store writes the 64 contiguous bytes of one token row (two
// full sectors).  The CTA-pair kernel's K loop keeps the shared-memory pipe busy (operand reads of the MMAs plus the
// TMA fills come to ~120 of the 128 bytes per cycle) and every store -> sync -> load round trip of a staged epilogue
// queues behind that traffic (measured: ~2900 cycles per 32 x 32 chunk staged, ~2500 direct with 8x the stores;
// 16 x 8192-row experts at K = 768: 0.262 ms direct, 0.281 staged).
// `out` = &d[first token of the chunk][first n of the warp]; `rows` = token rows of the chunk that exist (may be
// <= 0 or > 32).
__device__ __forceinline__ void store_held_chunk_dense(const uint32_t (&held)[16], uint16_t* out, int64_t ld, int rows,
                                                       int lane) {
  out += lane;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    if (2 * i < rows) out[0] = (uint16_t)(held[i] & 0xFFFFu);
    if (2 * i + 1 < rows) out[ld] = (uint16_t)(held[i] >> 16);
    out += 2 * ld;
  }
}

// Scattered output: through the warp's 512-byte shared-memory tile, 8 tokens per pass, so that ONE shuffle per pass
// hands every lane the destination row it stores 16 bytes of; a shuffle per token row (what the direct form would
// need) costs more than the staging — shuffles share the pipe that the K loop keeps busy.  `dest_row`: lane l holds
// the destination of token l of the chunk (null = skip).
template <typename OutT>
__device__ __forceinline__ void store_held_chunk_scatter(const uint32_t (&held)[16], OutT* stage_warp, OutT* dest_row,
                                                         int lane) {
  const int part = lane & 3;
  const int tok = lane >> 2;
  uint16_t* stage16 = reinterpret_cast<uint16_t*>(stage_warp);
  const unsigned long long bits = reinterpret_cast<unsigned long long>(dest_row);
#pragma unroll
  for (int p = 0; p < 4; ++p) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      stage16[(2 * j) * 32 + lane] = (uint16_t)(held[p * 4 + j] & 0xFFFFu);
      stage16[(2 * j + 1) * 32 + lane] = (uint16_t)(held[p * 4 + j] >> 16);
    }
    __syncwarp();
    const uint4 val = *reinterpret_cast<const uint4*>(stage16 + tok * 32 + part * 8);
    OutT* out = reinterpret_cast<OutT*>(__shfl_sync(0xffffffffu, bits, p * 8 + tok));
    if (out != nullptr) *reinterpret_cast<uint4*>(out + part * 8) = val;
    __syncwarp();
  }
}

}  // namespace es_b200
