/*
 * es_b200 — C ABI of the B200 (sm_100a) MoE grouped-GEMM library.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle (passed as void* so that the
 * header needs no CUDA include), enqueues its work on that stream and returns without synchronising.  Nothing
 * is copied to the host and no host decision depends on device data, so every call can be captured in a CUDA
 * graph.  Return value: ES_B200_OK or an error code; es_b200_last_error() gives the message of the calling
 * thread's last failure.
 *
 * The three operators replace, one for one, the operators of the reference torch extension
 * (expert_specialization/csrc/expert_specialization.cpp:56-73).  The reference passes torch::Tensor objects;
 * here the same tensors arrive as (pointer, extent) pairs and the shape / stride checks that the reference does
 * with TORCH_CHECK are done by the caller-side shim (expert_specialization_moe_b200/ops.py) plus the argument
 * checks below.
 */
#ifndef ES_B200_H_
#define ES_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ES_B200_OK 0
#define ES_B200_ERR_INVALID_ARGUMENT 1 /* bad pointer / size / alignment; nothing was launched */
#define ES_B200_ERR_CUDA 2             /* a CUDA runtime or driver call failed */
#define ES_B200_ERR_UNSUPPORTED_DEVICE 3 /* current device is not compute capability 10.x */
#define ES_B200_ERR_SCRATCH_TOO_SMALL 4
#define ES_B200_ERR_DEVICE_TIMEOUT 5   /* a bounded device-side wait gave up (reported by es_b200_check_status) */

/* element types */
#define ES_B200_BF16 0
#define ES_B200_FP16 1

/* Most experts any call accepts (the reference launches one thread per expert in a single block:
 * es_sm100_mxfp8_blockscaled_launcher.cuh:53, es_fp8_blockwise_launcher.cuh:53). */
#define ES_B200_MAX_EXPERTS 1024

const char* es_b200_version(void);
const char* es_b200_strerror(int code);
const char* es_b200_last_error(void);

/*
 * MXFP8 grouped quantisation.
 * Replaces es_sm100_mxfp8_blockscaled_grouped_quant
 *   (expert_specialization/csrc/cuda/es_sm100_mxfp8_blockscaled_group_quant.cu:5-39, kernel in
 *    es_sm100_mxfp8_blockscaled_group_quant.cuh:261-355; Python: expert_specialization/ops.py:40-50).
 *
 *   input             [num_rows, k] bf16 or fp16, row-major, k % 128 == 0, 16-byte aligned
 *   problem_sizes     [num_experts, 3] int32 (m, n, k) per expert — only m is read, as in the reference
 *   expert_offsets    [num_experts] int32: first row of each expert in input / quant_output
 *   blockscale_offsets[num_experts] int32: first row of each expert in the scale tensor (cumulative
 *                     round-up-to-128 of m)
 *   quant_output      [num_rows, k] e4m3 codes; rows outside every expert's range are not written
 *   scale_factor      [sf_rows, k/32] UE8M0 bytes in the SM100 swizzled layout (512-byte atoms of 128 rows x 4
 *                     K-blocks), expert e starting at byte blockscale_offsets[e] * k/32.  sf_rows must be at least
 *                     sum(round_up(m_e, 128)).  Rows m_e..round_up(m_e,128)-1 of each expert are written as 0.
 * Codes and the scale bytes of valid rows are bit-identical to the reference kernel's.
 */
int es_b200_mxfp8_grouped_quant(const void* input, int input_dtype, const int32_t* problem_sizes,
                                const int32_t* expert_offsets, const int32_t* blockscale_offsets,
                                void* quant_output, uint8_t* scale_factor, int num_experts, int64_t num_rows, int k,
                                void* stream);

/*
 * Fused SiLU * mul + MXFP8 grouped quantisation (between the gate_up and the down GEMM of an MoE layer).
 * No counterpart in the reference, which has no fused ops; equivalent to computing
 *   act = round_to_input_type( silu(gate_up[:, :k]) * gate_up[:, k:2k] )   (fp32 arithmetic, x / (1 + exp(-x)))
 * and passing act to es_b200_mxfp8_grouped_quant — with the same result bits — but without writing and re-reading act.
 *   gate_up [num_rows, 2k] bf16 or fp16, row-major: gate in columns [0,k), up in [k,2k); all other arguments and
 *   the outputs (quant_output [num_rows, k], scale_factor) as for es_b200_mxfp8_grouped_quant.
 */
int es_b200_mxfp8_silu_mul_grouped_quant(const void* gate_up, int input_dtype, const int32_t* problem_sizes,
                                         const int32_t* expert_offsets, const int32_t* blockscale_offsets,
                                         void* quant_output, uint8_t* scale_factor, int num_experts, int64_t num_rows,
                                         int k, void* stream);

/*
 * Scratch requirement (bytes of device memory, 16-byte aligned) of the MXFP8 grouped GEMM entry points.  Stands where
 * the reference allocates per-call torch::empty scratch tensors and a CUTLASS workspace
 * (es_sm100_mxfp8_blockscaled_launcher.cuh:163-176,140-142).  The kernels build their work lists in shared memory;
 * the scratch only holds the work counters through which the kernels of one call share out their tiles.  Rules:
 *   - zero it once (cudaMemset) before the first call that uses it; every call leaves it zeroed, so the same buffer
 *     serves any number of calls on one stream, graph replays included;
 *   - calls that may overlap on the GPU (different streams) need different scratch buffers;
 *   - after es_b200_check_status has reported a device-side error, zero it again (a kernel that gave up may have
 *     left counters behind); es_b200_error_epoch() counts those reports, so an owner of scratch buffers can compare
 *     it with the value it saw when it last zeroed a buffer.
 * scratch may be NULL: the kernels then deal their tiles round-robin and a large call runs its row-count buckets one
 * after the other instead of side by side (slower, same results).
 */
size_t es_b200_grouped_mm_scratch_bytes(int num_experts, int64_t num_rows, int n, int k);
uint64_t es_b200_error_epoch(void);

/*
 * MXFP8 block-scaled grouped GEMM:  d[off_e + i, :] = sum_k a[off_e + i, k] 2^(sfa-127) * b[e, :, k] 2^(sfb-127)
 * Replaces es_sm100_mxfp8_blockscaled_grouped_mm
 *   (expert_specialization/csrc/cuda/es_sm100_mxfp8_blockscaled.cu:5-40, launcher
 *    es_sm100_mxfp8_blockscaled_launcher.cuh:16-212, addressing es_sm100_mxfp8_blockscaled_functor.cuh:61-75;
 *    Python: expert_specialization/ops.py:32-37).
 *
 *   a    [num_rows, k] e4m3, row-major                      b   [num_experts, n, k] e4m3 in memory (the reference's
 *   sfa  swizzled UE8M0, expert e at blockscale_offsets[e]*k/32     [E, k, n] view with stride(1) == 1)
 *   sfb  swizzled UE8M0, expert e at e*n*k/32                d   [num_rows, n] bf16 or fp16
 *   k % 128 == 0, n % 128 == 0; a, b, d 16-byte aligned; sfa, sfb 16-byte aligned; blockscale_offsets multiples of
 *   128 (they are cumulative round-ups of the row counts to 128, as the reference's callers build them).
 * fp32 accumulation on the tensor cores, round-to-nearest to the output type.  Rows outside every expert's range
 * are not written.
 */
int es_b200_mxfp8_grouped_mm(const void* a, const void* b, const uint8_t* sfa, const uint8_t* sfb, void* d,
                             int out_dtype, const int32_t* problem_sizes, const int32_t* expert_offsets,
                             const int32_t* blockscale_offsets, int num_experts, int64_t num_rows, int n, int k,
                             int64_t sfa_rows, void* scratch, size_t scratch_bytes, void* stream);

/*
 * FP8-blockwise grouped GEMM (fp32 scales: one per 1x128 of a, one per 128x128 of b).
 * Replaces es_fp8_blockwise_scaled_grouped_mm
 *   (expert_specialization/csrc/cuda/es_fp8_blockwise.cu:34-193, addressing es_fp8_blockwise_functor.cuh:57-74;
 *    Python: expert_specialization/ops.py:4-29).
 *
 *   a [num_rows, k] e4m3 row-major; b [num_experts, n, k] e4m3 in memory;
 *   scales_a [num_rows, k/128] f32 row-major; scales_b [num_experts, n/128, k/128] f32 in memory;
 *   d [num_rows, n] bf16 or fp16.  k % 128 == 0, n % 128 == 0.
 */
int es_b200_fp8_blockwise_grouped_mm(const void* a, const void* b, const float* scales_a, const float* scales_b,
                                     void* d, int out_dtype, const int32_t* problem_sizes,
                                     const int32_t* expert_offsets, int num_experts, int64_t num_rows, int n, int k,
                                     void* scratch, size_t scratch_bytes, void* stream);

/*
 * es_b200_mxfp8_grouped_mm with the expert-parallel combine fused into its epilogue: same operands and problem
 * description, but output row r is stored to row row_meta[2r+1] of the [slots_per_gpu, n] array
 * peer_out[row_meta[2r]] (HOST array of `world` device pointers: the GPUs' pair buffers mapped into this process)
 * instead of row r of a dense d — the (GPU, slot) pairs es_b200_ep_dispatch_quant_push delivered with the rows.
 * Entries out of range are skipped and reported by es_b200_check_status.  No counterpart in the reference.
 */
int es_b200_mxfp8_grouped_mm_scatter(const void* a, const void* b, const uint8_t* sfa, const uint8_t* sfb,
                                     int out_dtype, const int32_t* problem_sizes, const int32_t* expert_offsets,
                                     const int32_t* blockscale_offsets, int num_experts, int64_t num_rows, int n,
                                     int k, int64_t sfa_rows, const int32_t* row_meta, const void* const* peer_out,
                                     int world, int64_t slots_per_gpu, void* scratch, size_t scratch_bytes,
                                     void* stream);

/*
 * Expert-parallel exchange over peer memory (one process per GPU; the experts of a layer are spread over the GPUs of a
 * node).  No counterpart in the reference, which has no distributed code: these three calls replace what a caller
 * would otherwise build from an all-to-all, a permutation and es_sm100_mxfp8_blockscaled_grouped_quant
 * (ops.py:40-50) on the way in, and an all-to-all plus a weighted sum on the way out (the first four calls below;
 * es_b200_mxfp8_grouped_mm_scatter above fuses the way out into the GEMM).  The peer_* arrays are HOST
 * arrays of `world` device pointers, entry i being GPU i's buffer mapped into this process (peer access enabled;
 * entry my_rank is the local buffer).  The calls only enqueue plain stores to those buffers; the caller orders the
 * GPUs with a barrier after each step.  Destinations out of range are skipped and reported by es_b200_check_status.
 *
 * es_b200_ep_dispatch_quant_push: quantises each of the `tokens` rows of x [tokens, k] once (MXFP8, bit-identical to
 *   the grouped quant) and stores, for each of its topk destinations j (pair = token * topk + j): the codes to row
 *   dst_row[pair] of peer_codes[dst_rank[pair]] ([capacity_rows, k] bytes), and one side record to row dst_row[pair]
 *   of peer_side[dst_rank[pair]] ([capacity_rows, es_b200_ep_side_record_bytes(k)] bytes): { int32 my_rank, int32
 *   pair, int64 dst_scale_offset[pair], k/32 scale bytes }.  dst_scale_offset = byte offset of the row's scale word
 *   for K tile 0 in the owner's swizzled scale buffer (blockscale_offset * k/32 + the row's position inside its
 *   expert).  A pair whose destination is out of range (an expert id outside [0, E), or a row past the owner's
 *   capacity) is dropped and reported; if my_pairs is given (this GPU's [tokens * topk, pair_row_bytes] slot buffer
 *   that the expert outputs come back to, or NULL), the dropped pair's slot is cleared so that the weighted sum adds 0
 *   for it instead of a row left by an earlier step.
 * es_b200_ep_unpack_side (local, after the barrier): for rows r < *num_rows_dev of `side`, writes the scale bytes to
 *   `scales` (swizzled layout, scale_bytes long) and (source GPU, pair) to meta[r] ([capacity_rows, 2] int32).
 * es_b200_ep_combine_push: stores row r < *num_rows_dev of y [capacity_rows, n] (2-byte elements) to row meta[r][1]
 *   of peer_pairs[meta[r][0]] ([pairs_per_rank, n]).
 * es_b200_ep_topk_weighted_sum: out[t, :] = sum_j weights[t, j] * pairs[t * topk + j, :] (fp32 accumulation in j order).
 * es_b200_ep_barrier: every GPU calls it the same number of times; peer_flags[i] is GPU i's flag array (17 uint32,
 *   zeroed once before first use).  One 32-thread kernel announces this GPU's next epoch in every peer's array and
 *   waits until all peers have announced theirs (at most five seconds, then it sets a status bit and returns).  Work
 *   enqueued after it on `stream` sees everything the peers stored to this GPU before their matching call.
 */
int es_b200_ep_side_record_bytes(int k);
int es_b200_ep_dispatch_quant_push(const void* x, int x_dtype, const int32_t* dst_rank, const int32_t* dst_row,
                                   const int64_t* dst_scale_offset, const void* const* peer_codes,
                                   const void* const* peer_side, int my_rank, int world, int tokens, int topk, int k,
                                   int64_t capacity_rows, void* my_pairs, int pair_row_bytes, void* stream);
int es_b200_ep_unpack_side(const void* side, const int32_t* num_rows_dev, uint8_t* scales, int32_t* meta, int k,
                           int64_t capacity_rows, int64_t scale_bytes, void* stream);
int es_b200_ep_combine_push(const void* y, const int32_t* meta, const int32_t* num_rows_dev,
                            const void* const* peer_pairs, int world, int64_t capacity_rows, int64_t pairs_per_rank,
                            int n, int elem_bytes, void* stream);
int es_b200_ep_topk_weighted_sum(const void* pairs, int dtype, const float* weights, void* out, int tokens, int topk,
                                 int n, void* stream);
int es_b200_ep_barrier(const void* const* peer_flags, int my_rank, int world, void* stream);
/* the same with the wait limit given by the caller (nanoseconds) instead of five seconds */
int es_b200_ep_barrier_limit(const void* const* peer_flags, int my_rank, int world, int64_t limit_ns, void* stream);

/*
 * Routing tables of the exchange, on the device (no counterpart in the reference).  topk_ids holds this GPU's
 * `pairs` = tokens * topk expert ids (int32, or int64 when ids_are_int64), token-major.
 * es_b200_ep_route_count: histograms the ids (scratch: segment_counts and segment_base, 256 * num_experts int32 each)
 *   and stores this GPU's per-expert totals into row my_rank of every peer's count matrix peer_counts_all[i]
 *   ([world, num_experts] int32).  Then es_b200_ep_barrier, then
 * es_b200_ep_route_tables: reads the local count matrix and writes, for each pair, the owner GPU (expert / (E/world)),
 *   the row in the owner's receive buffer and the byte offset of the row's scale words (the three per-pair inputs of
 *   es_b200_ep_dispatch_quant_push; an id outside [0, E) gives owner -1, which that call reports and skips), and for
 *   this GPU's own experts: rows[e], expert_offsets[e], blockscale_offsets[e] (E/world entries each) and total_rows[0]
 *   — the problem description of the grouped GEMMs that follow.  On the owner, rows are ordered by expert, then
 *   source GPU, then pair index.  capacity_rows = rows this GPU's receive buffers hold: if more are routed to it, the
 *   surplus is dropped (rows[] is cut so that no operator downstream touches a row past the capacity) and
 *   es_b200_check_status reports it.
 */
int es_b200_ep_route_count(const void* topk_ids, int ids_are_int64, int pairs, int num_experts,
                           int32_t* segment_counts, int32_t* segment_base, const void* const* peer_counts_all,
                           int my_rank, int world, void* stream);
int es_b200_ep_route_tables(const void* topk_ids, int ids_are_int64, int pairs, int num_experts,
                            const int32_t* segment_base, const int32_t* counts_all, int my_rank, int world, int k,
                            int32_t* dst_rank, int32_t* dst_row, int64_t* dst_scale_offset, int32_t* rows,
                            int32_t* expert_offsets, int32_t* blockscale_offsets, int32_t* total_rows,
                            int64_t capacity_rows, void* stream);

/*
 * es_b200_ep_route_count without caller-provided scratch (no counterpart in the reference).  For callers that cannot
 * allocate device memory where they call this library — a server whose memory manager owns the whole GPU, a cgo / JNI /
 * plugin binding that only ever receives raw pointers — the 256 x num_experts histogram counters live in a static
 * device array inside the library (256 KB per GPU, held until the process exits) instead of `segment_counts`.
 * Limits and rules: num_experts <= ES_B200_ROUTE_STATIC_MAX_EXPERTS, otherwise ES_B200_ERR_INVALID_ARGUMENT and
 * nothing is launched; the call allocates and frees nothing; the first call on each device looks up the array's device
 * address (make that first call outside any stream capture; the address is cached for the life of the device's primary
 * context, so do not call the library after a cudaDeviceReset); all calls on one device share the array, so calls that
 * overlap on the GPU (different streams) race — serialise them.  Inputs, outputs and results are those of
 * es_b200_ep_route_count.
 */
#define ES_B200_ROUTE_STATIC_MAX_EXPERTS 256
int es_b200_ep_route_count_static(const void* topk_ids, int ids_are_int64, int pairs, int num_experts,
                                  int32_t* segment_base, const void* const* peer_counts_all, int my_rank, int world,
                                  void* stream);

/*
 * Tunables of the tile-shape dispatcher (no counterpart in the reference, whose bucket rules are compile-time
 * functors: es_fp8_blockwise_functor.cuh:122-256).  Process-wide; each also has an environment override read once,
 * ES_B200_<NAME IN CAPITALS>.  Names: "mm_heavy_min_rows" (experts with at least this many rows use CTA-pair tiles;
 * 0 = per-(n, k) table; at most 113), "mm_tiny_max_rows" (0 = table), "mm_pair_first_clusters",
 * "mm_split_min_rows", "mm_stream_max_ctas", "mm_pair_max_clusters" (grid shaping of a split call, 0 = no cap),
 * "mm_dynamic" (0: ignore the work counters), "mm_stream_lsu" (0: the streaming CTAs load by TMA only),
 * "mm_stream_mid_lead_ctas" (CTAs of the 112-token shape that start before the 32-token shape's; negative = built-in
 * default), "mm_item_k_steps" (K steps that a streaming work item should span: it takes that many weight tiles, at
 * most 8).  Unknown name: ES_B200_ERR_INVALID_ARGUMENT.
 */
int es_b200_set_tunable(const char* name, int value);

/*
 * Device-side status word of the grouped GEMMs.  Every wait inside the kernels is bounded; a wait that gives up
 * sets a bit in a library-owned device word and the kernel exits cleanly.  This call synchronises `stream`, copies
 * that word to the host, clears it, and returns ES_B200_OK or ES_B200_ERR_DEVICE_TIMEOUT.  Optional: intended for
 * tests and debugging, never needed on the hot path.  (No counterpart in the reference, which has no device-side
 * error reporting.)
 */
int es_b200_check_status(void* stream, uint32_t* raw_status);

#ifdef __cplusplus
}
#endif
#endif /* ES_B200_H_ */
