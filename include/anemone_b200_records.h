/*
 * anemone_b200_records.h: the by-value records the kernels of this library take, and the layout of every
 * array a record names. Compiles as C11 (host preparers, oracle, tests) and as CUDA C++ (kernel files).
 *
 * The universal kernel contract (reference: include/anemone/backend_seam.h:60-79,
 * include/anemone/linear_records.h:9-15): a kernel is
 *     extern "C" __global__ void name(struct <record> record, unsigned char *arena);
 * a record names memory only by byte offsets into the card's arena, never by address, so a prepared launch is
 * the same bytes on every card. Kernels validate nothing; the host preparer has checked every range.
 *
 * Every struct below whose comment names a reference header is ABI-identical to that header's struct (same
 * field order, sizes and offsets, asserted at the end of this file), so launch tables and job tables written
 * by reference-side code are read unchanged. Structs marked "B200 extension" have no reference counterpart.
 */
#ifndef ANEMONE_B200_RECORDS_H
#define ANEMONE_B200_RECORDS_H

#include <stdbool.h>
#include <stdint.h>

#ifdef __CUDACC__
#define AB_INLINE __host__ __device__ static inline
#else
#define AB_INLINE static inline
#endif

/* ------------------------------------------------------------------------------------------------------------
 * EXL3 "mul1" trellis format (reference: include/anemone/exl3_records.h:2-9, 45-119).
 *
 * A matrix of `inputs` x `outputs` weights is stored as
 *     codes  [inputs/16][outputs/16] tiles, each tile 16 x 16 weights = 128 * bits_x2 bits
 *            (little-endian uint32 words, bit stream MSB-first inside each word, cyclic),
 *     suh    FP16 [inputs]   (sign/scale applied to the input side before the 128-wide Hadamard transform),
 *     svh    FP16 [outputs]  (sign/scale applied to the output side after it).
 * bits_x2 is twice the bits per weight, so that half widths (2.5 bits) are whole numbers. The weight at stream
 * position p of a tile has the 16-bit state whose window ENDS at ring bit S(p) = floor((p + 1) * bits_x2 / 2);
 * its value is the codebook below. Stream position <-> (input, output) inside a tile follows the A-fragment
 * order of the m16n8k16 tensor-core instruction: see exl3_tile_position.
 * A "stored width" is K for whole K bits per weight and 16 K for a half width (K = 2.5 is stored as 40).
 * ---------------------------------------------------------------------------------------------------------- */
#define EXL3_TILE 16u
#define EXL3_TILE_VALUES 256u
#define EXL3_TRANSFORM 128u
#define EXL3_STATE_BITS 16u
#define EXL3_WORD_BITS 32u
#define EXL3_HALF_BYTES 2u
#define EXL3_K2 2u
#define EXL3_K2_5 40u
#define EXL3_K3 3u
#define EXL3_K4 4u
#define EXL3_BITS_X2_K2 4u
#define EXL3_BITS_X2_K2_5 5u
#define EXL3_BITS_X2_K3 6u
#define EXL3_BITS_X2_K4 8u
#define EXL3_MUL1_MULTIPLIER 0x83DCD12Du
#define EXL3_MUL1_BASE 0x6400u /* FP16 1024.0: adding a byte sum b < 1024 gives FP16 (1024 + b) exactly */
#define EXL3_MUL1_SCALE 0x1EEEu /* FP16 1774 / 2^18 */
#define EXL3_MUL1_BIAS 0xC931u /* FP16 -10.3828125 */
#define EXL3_NORMALIZATION 0.08838834764831845f /* 1 / sqrt(128), the Hadamard scale */
#define EXL3_PROJECTIONS 2u /* gate and up */
#define EXL3_EXPERT_LAUNCHES 5u
#define EXL3_KERNEL_FILE "kernel_exl3"
#define EXL3_RECONSTRUCT "exl3_reconstruct"
#define EXL3_ROW_SUM "exl3_row_sum"
/* B200 extension: a record's bits_per_weight that means "read each expert's stored width from the table at
 * widths_offset" (struct exl3_moe_record). No stored width has this value. */
#define EXL3_WIDTH_PER_EXPERT 0xFFFFu

/* bits_x2 of a stored width, 0 if the value is no width of the format (whole 1..8, half 1.5..7.5). */
AB_INLINE uint32_t exl3_bits_x2(uint32_t stored_width)
{
	if (stored_width >= 1u && stored_width <= 8u)
		return 2u * stored_width;
	if ((stored_width & 15u) == 8u && stored_width < 128u)
		return stored_width >> 3;
	return 0u;
}

/* The widths this library decodes: K2, K2.5, K3, K4 (the reference's EXL3_SUPPORTED_BITS_X2). */
AB_INLINE bool exl3_width_supported(uint32_t stored_width)
{
	const uint32_t b = exl3_bits_x2(stored_width);
	return b == EXL3_BITS_X2_K2 || b == EXL3_BITS_X2_K2_5 || b == EXL3_BITS_X2_K3 || b == EXL3_BITS_X2_K4;
}

/* S(p): the ring bit at which the 16-bit window of stream position p ends. */
AB_INLINE uint32_t exl3_window_end(uint32_t position, uint32_t bits_x2)
{
	return ((position + 1u) * bits_x2) >> 1;
}

/* Bytes of the codes of an inputs x outputs matrix (both whole tiles). Divides first: no 64-bit overflow. */
AB_INLINE uint64_t exl3_code_bytes(uint64_t inputs, uint64_t outputs, uint32_t bits_x2)
{
	return inputs * outputs / 16u * bits_x2;
}

/* Stored bytes of a matrix: codes, then suh[inputs], then svh[outputs]. */
AB_INLINE uint64_t exl3_matrix_bytes(uint64_t inputs, uint64_t outputs, uint32_t bits_x2)
{
	return exl3_code_bytes(inputs, outputs, bits_x2) + (inputs + outputs) * EXL3_HALF_BYTES;
}

/* Stream position of weight (input, output), both 0..15, inside its tile: lane l = 4 (output % 8) +
 * (input % 8) / 2 of a warp holds positions 8 l .. 8 l + 7, in the register order of the instruction's A operand. */
AB_INLINE uint32_t exl3_tile_position(uint32_t input, uint32_t output)
{
	const uint32_t lane = ((output & 7u) << 2) | ((input & 7u) >> 1);
	const uint32_t element = (input & 1u) | ((input >> 3) << 1) | ((output >> 3) << 2);
	return (lane << 3) | element;
}

/* kernel_exl3 / exl3_reconstruct (reference: include/anemone/exl3_records.h:123-130): decode a whole matrix to
 * FP16 [input][output], before either transform or scale. Bit-exact diagnostic. */
struct exl3_reconstruct_record {
	uint64_t matrix_offset;
	uint64_t output_offset;
	uint32_t input_size;
	uint32_t output_size;
	uint32_t bits_per_weight; /* stored width */
	uint32_t reserved_zero;
};

/* One expert layer's chain (reference: include/anemone/exl3_records.h:144-159).
 *   jobs      struct expert_job_record [job_count]
 *   input     bfloat16 [rows][input_size], rows = pair_count / pairs_per_row
 *   operands  FP16 [2][pair_count][input_size] for gate/up; reused as FP16 [pair_count][inner_size] for down
 *   products  FP32 [2][pair_count][inner_size] for gate/up; reused as FP32 [pair_count][input_size] for down
 *   hidden    bfloat16 [pair_count][inner_size] (side output of the activation)
 *   output    FP32 [pair_count][input_size]; equals products_offset (finish works in place) */
struct exl3_expert_record {
	uint64_t jobs_offset;
	uint64_t input_offset;
	uint64_t operands_offset;
	uint64_t products_offset;
	uint64_t hidden_offset;
	uint64_t output_offset;
	uint32_t input_size; /* hidden width H of the model */
	uint32_t inner_size; /* this rank's intermediate width */
	uint32_t pair_count;
	uint32_t pairs_per_row;
	uint32_t job_count;
	uint32_t bits_per_weight; /* stored width of every matrix of the launch */
	float activation_limit;
	uint32_t reserved_zero;
};

/* One routed expert with the rows routed to it (reference: include/anemone/linear_records.h:245-253). Written by
 * the router, read by every expert kernel. row_count 0 = empty job, nothing else of it is read. Column c < row_count
 * carries pair pair_index[c] = row * pairs_per_row + slot and that pair's route weight. */
#define LINEAR_MAXIMUM_ROWS 8u
#define LINEAR_OFFSET_ALIGNMENT_BYTES 16u
#define WEIGHT_FORMAT_MATRIX_ALIGNMENT_BYTES 64u
struct expert_job_record {
	uint64_t gate_offset;
	uint64_t up_offset;
	uint64_t down_offset;
	uint32_t row_count;
	uint32_t expert;
	uint32_t pair_index[LINEAR_MAXIMUM_ROWS];
	float route_weight[LINEAR_MAXIMUM_ROWS];
};

/* exl3_row_sum (reference: include/anemone/linear_records.h:209-216): row = sum of its pairs_per_row pair outputs,
 * from +0 in ascending slot order. FP32 [rows * pairs_per_row][width] -> FP32 [rows][width], rows = grid[1]. */
struct expert_row_sum_arguments {
	uint64_t pair_output_offset;
	uint64_t row_output_offset;
	uint32_t width;
	uint32_t pairs_per_row;
};

/* bb_exl3_activate_output_shard (reference: include/anemone/exl3_tp_records.h:17-23): the activation of a rank whose
 * gate/up are an output slice [down_input_begin, +base.inner_size) of the full intermediate and whose resident down
 * matrix has the stated full shape; it reads down's suh at down_input_begin. */
struct bb_exl3_shard_activation_record {
	struct exl3_expert_record base;
	uint32_t down_input_size;
	uint32_t down_output_size;
	uint32_t down_input_begin;
	uint32_t reserved_zero;
};

/* B200 extension, kernel file "kernel_exl3_b200": the whole routed-expert layer of one rank in four launches
 * (input transform; gate/up products fused with the SwiGLU activation and the down-side input transform; down
 * products fused with the output transform and route weight; ordered row sum), with a stored width per expert.
 * base is read as the five-pass chain reads it, except:
 *   - base.bits_per_weight may be EXL3_WIDTH_PER_EXPERT: expert e's three matrices then have stored width widths[e]
 *     (uint32 [expert_count] at widths_offset);
 *   - a product over K inputs is cut in S = exl3_moe_splits(K, outputs) runs (exl3_geometry.h of the kernel sources; the host
 *     preparer reports the sizes that follow through exl3_moe_sizes). products: FP32 partial sums
 *     [2][S(input_size)][pair_count][inner_size] for gate/up, then reused as [S(inner_size)][pair_count][input_size]
 *     for down; the pair outputs FP32 [pair_count][input_size] are run 0 of the latter (output_offset ==
 *     products_offset, as in the chain);
 *   - operands: FP16 [2][pair_count][input_size] for gate/up and, BEHIND them, FP16 [pair_count][inner_size] for
 *     down (the fused launch writes them while the gate/up operands are still being read);
 *   - counters: uint32 [job_count][inner_size / 128 + input_size / 128] at counters_offset, zero at load; every launch
 *     leaves them zero.
 * row_output: FP32 [rows][input_size]. */
#define EXL3_MOE_KERNEL_FILE "kernel_exl3_b200"
#define EXL3_MOE_LAUNCHES 4u
struct exl3_moe_record {
	struct exl3_expert_record base;
	uint64_t widths_offset;
	uint64_t row_output_offset;
	uint64_t counters_offset;
	uint32_t expert_count;
	uint32_t reserved_zero;
};

/* The block every step-dependent kernel reads on the device, so that one prepared launch (or one captured graph)
 * serves every step (reference: include/anemone/step_records.h:111-115). */
struct step_block {
	uint64_t sequence; /* of the step, from 1, strictly increasing */
	uint32_t row_count; /* live rows of this step */
	uint32_t flags;
};

/* ------------------------------------------------------------------------------------------------------------
 * B200 extension, kernel file "kernel_exl3_layer": one decode step (up to ROUTER_B200_MAXIMUM_ROWS rows) of a rank's
 * whole expert layer in FOUR launches, made for the step's latency on one to eight ranks:
 *   exl3_layer_route_input   grid (1 + T) x 256: every CTA chooses the live rows' experts itself (a warp a row, the
 *                            router's arithmetic, so all agree); CTA 0 writes picks, weights and the job table
 *                            (router_select_b200's bytes) and the live job count; the others transform the rows into
 *                            the FP16 operands of every (pair, gate or up): no launch and no trip through memory
 *                            stands between the router and the transform.
 *   exl3_layer_products      grid (job_count * items a job) x 128, a CTA an item of the step's list: first every
 *                            (job, gate or up, 128 outputs, run of the cut of K) in job order, then every (job, 128
 *                            outputs of down, run); a CTA takes the next item as it begins (a ticket), so the card
 *                            hands every freed place to the next item and its room is filled to the last one. The
 *                            CTA that completes a (job, 128 outputs) adds the runs' FP32 partial sums in ascending K
 *                            order from +0 and applies the epilogue (transform, SwiGLU and the down-side transform;
 *                            transform, scale and route weight). A down item waits (bounded) until the job's down
 *                            operands are all in place: a word a job counts the groups of inner channels done.
 *                            Every gate/up item has begun before any down item begins, so no wait is in vain.
 *   ordered_publish_reduce_flags  (kernel file "kernel_ordered_b200") adds each row's pairs in ascending slot order
 *                            from +0 straight into this rank's rows of the reduction slot, stores this rank's READY
 *                            word into EVERY rank's slot (plain peer stores), waits for the ranks' READY words in
 *                            its OWN memory (nobody polls across NVLink), pulls the ranks' rows by peer loads, adds
 *                            them in rank order from +0, rounds once to bfloat16, and stores its DONE word into
 *                            every rank's slot.
 * A slot of the reduction region in this form (two parity slots, parity_stride apart): 16 READY lines of 128 bytes
 * (line s: a 64-bit sequence written only by rank s), 16 DONE lines likewise, one local line (a block counter at
 * byte 64, the sequence of the slot's previous use at byte 72), then the FP32 rows at input_offset.
 * The cut of a product depends on the prepared shapes alone: the same inputs give the same bits on every run.
 * partial sums: FP32 [2][runs][pair_count][inner_size] for gate/up, then, in a range of their own, [runs][pair_count]
 * [input_size] for down (run 0 is also where the pair outputs go), both sized for EXL3_LAYER_MAXIMUM_RUNS runs; counters:
 * what struct exl3_moe_record asks for, then EXL3_LAYER_COUNTER_WORDS more uint32 (the live job count first), then a
 * word a job; zero at load.
 * ---------------------------------------------------------------------------------------------------------- */
#define EXL3_LAYER_KERNEL_FILE "kernel_exl3_layer"
#define EXL3_LAYER_LAUNCHES 3u
#define EXL3_LAYER_MAXIMUM_RUNS 16u /* runs of K of one product at most */
#define EXL3_LAYER_ROUTE_THREADS 1024u
#define EXL3_LAYER_COUNTER_WORDS 4u /* the live job count, the products' ticket and two reserved words */
#define EXL3_LAYER_READY_LINE 0u
#define EXL3_LAYER_DONE_LINE 16u
#define EXL3_LAYER_LOCAL_LINE 32u
#define EXL3_LAYER_SIGNAL_BYTES (33u * 128u)
struct exl3_layer_route_record {
	struct exl3_moe_record moe;
	uint64_t scores_offset; /* FP32 [row_capacity][routed_count] */
	uint64_t expert_table_offset; /* uint64 [routed_count + shared_count][3] */
	uint64_t picks_offset; /* written: uint32 [row_capacity][picks] */
	uint64_t weights_offset; /* written: FP32 [row_capacity][picks] */
	uint64_t bias_offset; /* FP32 [routed_count], 0: none */
	uint64_t step_offset;
	uint32_t routed_count;
	uint32_t shared_count;
	uint32_t picks;
	uint32_t row_capacity;
	uint32_t scoring;
	float route_scale;
};

/* the record of exl3_layer_products */
struct exl3_layer_products_record {
	struct exl3_moe_record moe;
	uint64_t down_products_offset; /* down's partial sums; run 0 of them the pair outputs */
	uint32_t gate_up_runs; /* the cut of K = input_size of gate and up */
	uint32_t down_runs; /* the cut of K = inner_size of down */
};

/* what exl3_layer_prepare is told about the reduction */
struct exl3_layer_publish_arguments {
	uint64_t peer_table_offset; /* struct ordered_collective_peer [rank_count] */
	uint64_t region_offset;
	uint64_t input_offset; /* of the FP32 rows inside a slot, at least EXL3_LAYER_SIGNAL_BYTES */
	uint64_t status_offset; /* the 16-byte status block of the reduction (arena offset) */
	uint64_t step_offset;
	uint64_t parity_stride;
	uint64_t deadline_cycles;
	uint32_t rank_count;
	uint32_t rank;
	uint32_t row_capacity;
	uint32_t reserved_zero;
};

/* ------------------------------------------------------------------------------------------------------------
 * Fixed-order reduction over ranks (reference: include/anemone/ordered_collective_records.h:45-98).
 *
 * Each rank owns a region of two parity slots (slot = sequence & 1) of parity_stride bytes. A slot begins with three
 * 128-byte signal lines (READY, REDUCED, DONE), each written only by its owner: a 32-bit commit generation at byte 0
 * and the 64-bit step sequence at byte 8; then the input, output and scratch arrays at the record's offsets (relative
 * to the slot). The peer table holds, per rank, the device address under which THIS card reaches that rank's arena
 * and that rank's region offset. Sum order: ((+0 + rank 0) + rank 1) + ..., one rounded FP32 add per rank.
 * ---------------------------------------------------------------------------------------------------------- */
#define KERNEL_FILE_ORDERED_COLLECTIVE "kernel_ordered_collective"
#define KERNEL_ORDERED_ALL_REDUCE "ordered_all_reduce"
#define KERNEL_ORDERED_TWO_SHOT "ordered_two_shot"
#define KERNEL_ORDERED_REDUCE_SCATTER "ordered_reduce_scatter"
#define KERNEL_ORDERED_GATHER "ordered_gather"
#define ORDERED_COLLECTIVE_MAXIMUM_RANKS 16u
#define ORDERED_COLLECTIVE_THREADS 256u
#define ORDERED_COLLECTIVE_LINE_BYTES 128ull
#define ORDERED_COLLECTIVE_PHASES 3u
#define ORDERED_COLLECTIVE_SIGNAL_BYTES (ORDERED_COLLECTIVE_PHASES * ORDERED_COLLECTIVE_LINE_BYTES)
#define ORDERED_COLLECTIVE_SLOTS 2u
#define ORDERED_COLLECTIVE_MAXIMUM_ELEMENTS 262144u
#define ORDERED_COLLECTIVE_SEQUENCE_OFFSET 8u
#define ORDERED_COLLECTIVE_DIRECT_ROUTE 0u
#define ORDERED_COLLECTIVE_HOST_ROUTE 1u /* PCIe host mirrors of the reference's cards: refused by this library */

enum ordered_collective_operation {
	ORDERED_ALL_REDUCE,
	ORDERED_TWO_SHOT,
	ORDERED_REDUCE_SCATTER,
	ORDERED_GATHER,
	ORDERED_COLLECTIVE_OPERATIONS
};

struct ordered_collective_peer {
	uint64_t arena_address;
	uint64_t region_offset;
	uint64_t host_address;
	uint32_t route;
	uint32_t reserved_zero;
};

struct ordered_collective_arguments {
	uint64_t peer_table_offset;
	uint64_t region_offset;
	uint64_t input_offset; /* the three arrays: offsets inside a parity slot, behind the signal lines */
	uint64_t output_offset;
	uint64_t scratch_offset;
	uint64_t step_offset; /* struct step_block in the arena */
	uint64_t parity_stride;
	uint64_t deadline_cycles; /* of the device clock; a wait that runs out sets the status word, never traps */
	uint32_t element_count;
	uint32_t rank_count;
	uint32_t rank;
	uint32_t reserved_zero;
};

/* B200 extension, kernel file "kernel_ordered_b200": the production reduction of expert partial sums. Many CTAs;
 * every rank pulls every rank's FP32 partial rows by peer loads over NVLink, adds them in rank order from +0 in FP32,
 * rounds ONCE to bfloat16 (to nearest even, a not-a-number to 0x7FC0: the arithmetic of the reference's
 * tp_exchange_owner_sum, source/kernel_tp_exchange.cu:190-247) and stores bfloat16 [rows][width] locally.
 * `collective` is read as the FP32 collective reads it, except: output_offset is an ARENA offset of the bfloat16
 * result (not inside the slot); scratch_offset is unused; element_count is the capacity rows * width and the live
 * element count is step.row_count * width. status_offset names a 16-byte status block in the arena:
 * {uint32 code (0 ok, 1 timed out, 2 bad sequence), uint32 phase, uint32 rank waited for, uint32 reserved},
 * written only on failure. */
#define KERNEL_FILE_ORDERED_B200 "kernel_ordered_b200"
#define KERNEL_ORDERED_REDUCE_BF16 "ordered_reduce_bf16"
#define KERNEL_ORDERED_ROW_SUM_PUBLISH "ordered_row_sum_publish"
#define ORDERED_B200_MAXIMUM_BLOCKS 64u
#define ORDERED_B200_STATUS_BYTES 16u
#define ORDERED_STATUS_OK 0u
#define ORDERED_STATUS_TIMED_OUT 1u
#define ORDERED_STATUS_BAD_SEQUENCE 2u
#define ORDERED_B200_MAXIMUM_ELEMENTS (1u << 28) /* of this reduction; the FP32 collectives keep the reference's limit */
#define ORDERED_B200_MAXIMUM_BLOCKS_LARGE 592u
#define ORDERED_B200_PUBLISH_ROW_BLOCKS 128u /* grid rows of ordered_row_sum_publish at most; a block strides over rows */
/* mode 0: every rank adds every element itself (no second hop: the lowest latency, the choice for decode steps).
 * mode 1: rank r adds the r-th of rank_count equal runs of four-element vectors (the first vectors % rank_count runs
 * one vector longer) and stores the bfloat16 values into EVERY rank's result by peer stores, publishes its REDUCED
 * line and waits for every rank's: each rank then reads 1 / rank_count of what mode 0 reads over NVLink, which is what
 * counts for many rows (prefill). Same arithmetic, same bits. In mode 1 the result of a step must be consumed in
 * stream order before the rank's next publish, as the graph of a layer does. */
#define ORDERED_REDUCE_EVERY_RANK 0u
#define ORDERED_REDUCE_OWNER_RUNS 1u
struct ordered_reduce_bf16_arguments {
	struct ordered_collective_arguments collective;
	uint64_t status_offset;
	uint32_t width; /* elements of a row */
	uint32_t mode;
};

/* B200 extension: row sums, READY, the rank-ordered sum, one rounding and DONE of a decode step in one launch
 * (ordered_publish_reduce_flags; the slot layout is the flags form's, see struct exl3_layer_route_record).
 * collective is read as struct ordered_reduce_bf16_arguments reads it. */
#define KERNEL_ORDERED_PUBLISH_REDUCE_FLAGS "ordered_publish_reduce_flags"
struct ordered_publish_reduce_arguments {
	struct ordered_collective_arguments collective;
	uint64_t status_offset;
	uint64_t pair_output_offset; /* FP32 [rows * pairs_per_row][width] */
	uint32_t width;
	uint32_t pairs_per_row;
};

/* B200 extension, entry "ordered_publish_reduce_flags_bf16": the same launch for pair outputs that are BFLOAT16
 * (the original-weights experts' expert_down outputs): a row's pairs added from +0 in ascending slot order as FP32,
 * then, where addend_offset is not 0, one FP32 addition of the bfloat16 row at addend_offset ([rows][width]: the
 * always-on expert's output); the sum is stored at row_output_offset where that is not 0 (FP32 [rows][width], for
 * readers of the rank's own rows) and enters the slot through one more addition onto +0: the operations of
 * expert_row_sum_entry, trunk_rows_add_entry and ordered_row_sum_publish with one "pair" a row, in their order. */
#define KERNEL_ORDERED_PUBLISH_REDUCE_FLAGS_BF16 "ordered_publish_reduce_flags_bf16"
struct ordered_publish_reduce_bf16_arguments {
	struct ordered_publish_reduce_arguments base; /* pair_output_offset: bfloat16 [rows * pairs_per_row][width] */
	uint64_t addend_offset;
	uint64_t row_output_offset;
};

/* B200 extension: the row sum of a rank written straight into its collective input slot of this step's parity
 * (FP32 [rows][width] at collective.input_offset of the slot), so that no copy stands between the experts and the
 * reduction. Rows at or beyond step.row_count are not written. grid (width / 512 rounded up, up to
 * ORDERED_B200_PUBLISH_ROW_BLOCKS row blocks). */
struct ordered_row_sum_publish_arguments {
	struct ordered_collective_arguments collective;
	uint64_t pair_output_offset; /* FP32 [rows * pairs_per_row][width] */
	uint32_t width;
	uint32_t pairs_per_row;
	uint64_t status_offset; /* the reduction's 16-byte status block: a wait for the slot that runs out is reported */
};

/* ------------------------------------------------------------------------------------------------------------
 * The output-axis exchanges of a tensor-parallel group (reference: include/anemone/exact_ring_records.h:43-56,
 * round_once_ring_records.h, compressed_ring_records.h): one record, three entries, packs of 16 bytes (eight
 * bfloat16 values, or any 16 bytes for the gather).
 *   ("kernel_exact_ring", "exact_ring")                      mode 0: a lossless gather of every owner's
 *       packs_per_owner packs (input owner-major, this rank's part read; output owner-major or, with vectors,
 *       [vector][all owners' channels]); modes 1, 2: the BF16 sum whose additions round to bfloat16 one after the
 *       other in the order the reference's ring visits the ranks: for owner o from rank o + 1 round to o; a +0 half
 *       that travels arrives as -0 (the reference's transport), so the owner keeps its sum and every other rank holds
 *       it without +0 halves;
 *   ("kernel_bf16_compressed_ring", "bf16_compressed_ring")  modes 1, 2: the same sum, every pack on the wire in the
 *       lossless exponent-delta code (anemone_b200_wire_codec.h): three words a lane where a warp's exponents allow;
 *   ("kernel_bf16_round_once_ring", "bf16_round_once_ring")  modes 1, 2 (the layout alone): FP32 sums of the ranks'
 *       bfloat16 values in rank order from +0, ONE rounding to bfloat16, the same bits on every rank.
 * Mode 1: owner o's part is the o-th run of packs_per_owner packs; mode 2 (column owners): input and output are
 * [vectors][row], owner o the o-th run of every row's packs. grid (at most EXACT_RING_BLOCKS) x EXACT_RING_THREADS;
 * packs_per_owner a positive multiple of 32; every rank the same counts and grid on one ordered stream. The bank:
 * EXACT_RING_METADATA_BYTES (a generation counter a block, a status word at EXACT_RING_STATUS_OFFSET), then the
 * exchange's own space (ring_exchange_bank_bytes of the host header); zero before the first call. Peers: the ordered
 * collective's table; a peer's bank lies at its region offset + peer_bank_delta. B200: 2, 4 or 8 ranks in
 * reserved_words[0] (0: the reference's 4); a deadline, an exhausted generation counter or a malformed record sets
 * the status word (1, 2, 3) and the kernel returns: nothing traps, and a bank with a status is not used again.
 * ---------------------------------------------------------------------------------------------------------- */
#define KERNEL_FILE_EXACT_RING "kernel_exact_ring"
#define KERNEL_EXACT_RING "exact_ring"
#define KERNEL_FILE_COMPRESSED_RING "kernel_bf16_compressed_ring"
#define KERNEL_COMPRESSED_RING "bf16_compressed_ring"
#define KERNEL_FILE_ROUND_ONCE_RING "kernel_bf16_round_once_ring"
#define KERNEL_ROUND_ONCE_RING "bf16_round_once_ring"
#define EXACT_RING_PACK_BYTES 16u
#define EXACT_RING_BLOCKS 16u
#define EXACT_RING_THREADS 256u
#define EXACT_RING_RANKS 4u
#define EXACT_RING_METADATA_BYTES 128u
#define EXACT_RING_STATUS_OFFSET 64u
#define EXACT_RING_STATUS_DEADLINE 1u
#define EXACT_RING_STATUS_GENERATION 2u
#define EXACT_RING_STATUS_ARGUMENTS 3u
#define EXACT_RING_GATHER 0u
#define EXACT_RING_BF16_SUM 1u
#define EXACT_RING_BF16_SUM_COLUMNS 2u
#define COMPRESSED_RING_PACKS 32u
#define COMPRESSED_RING_PACKET_WORDS 136u
#define COMPRESSED_RING_PACKET_BYTES 544u
#define COMPRESSED_RING_PAYLOAD_WORD 4u
#define COMPRESSED_RING_RAW_MASK_WORD 1u
#define COMPRESSED_RING_READY_WORD 132u
#define COMPRESSED_RING_ACK_WORD 133u
#define COMPRESSED_RING_COMPRESSED_WORDS 3u
struct exact_ring_arguments {
	uint64_t input_offset;
	uint64_t output_offset;
	uint64_t bank_offset;
	uint64_t peer_table_offset;
	uint64_t peer_bank_delta;
	uint64_t deadline_cycles;
	uint32_t packs_per_owner;
	uint32_t vectors;
	uint32_t rank;
	uint32_t mode;
	uint64_t reserved_words[2]; /* [0]: the rank count (0: four); [1]: zero */
};

/* ------------------------------------------------------------------------------------------------------------
 * One-shot push all-reduce and the tensor-parallel exchange built on it (reference:
 * include/anemone/ordered_push_records.h:8-33, include/anemone/tp_exchange_records.h:10-62).
 *
 * A slot begins with ORDERED_PUSH_PHASES * rank_count signal lines of 128 bytes: line (phase, source) of a rank's
 * slot is written only by rank `source` (by a peer store), so every wait polls local memory. Behind the lines, at
 * offsets relative to the slot: the FP32 input, the output, and rank_count inboxes inbox_rank_stride bytes apart.
 * A source stores its input (FP32, or rounded to bfloat16: payload_format) into inbox [source] of every rank, then
 * its READY line there; a rank adds its inboxes in ascending rank order from +0, one rounded FP32 add a rank; DONE
 * lines are an all-rank barrier before return, so an inbox may be refilled as soon as the launch has returned.
 * The launch runs groups x blocks CTAs (grid.x x grid.y, grid.x <= ORDERED_PUSH_GROUPS): group g moves and adds the
 * g-th part of the payload and owns the g-th 8-byte word of every line, which holds the sequence itself; the second
 * half of a rank's own READY and DONE lines holds the groups' arrival counters, touched by the rank's CTAs only.
 * ---------------------------------------------------------------------------------------------------------- */
#define KERNEL_FILE_ORDERED_PUSH "kernel_ordered_push"
#define KERNEL_ORDERED_PUSH "ordered_push"
#define ORDERED_PUSH_ARGUMENT_BYTES 96u
#define ORDERED_PUSH_FP32 0u
#define ORDERED_PUSH_BF16 1u
#define ORDERED_PUSH_PHASES 2u
#define ORDERED_PUSH_READY 0u
#define ORDERED_PUSH_DONE 1u
#define ORDERED_PUSH_GROUPS 8u /* grid.x at most: the flag words of a line */
#define ORDERED_PUSH_GROUP_BLOCKS 16u /* grid.y at most */
#define ORDERED_PUSH_BLOCK_VECTORS 1024u /* four-element vectors a CTA is given before another CTA is added */

struct ordered_push_arguments {
	uint64_t peer_table_offset; /* struct ordered_collective_peer [rank_count], indexed by destination */
	uint64_t region_offset;
	uint64_t input_offset; /* FP32 [element_count], inside a parity slot like the next two */
	uint64_t output_offset; /* FP32 [element_count]; bfloat16 [element_count] for the owner sums */
	uint64_t inbox_offset;
	uint64_t step_offset;
	uint64_t parity_stride;
	uint64_t deadline_cycles;
	uint64_t inbox_rank_stride;
	uint32_t element_count;
	uint32_t rank_count;
	uint32_t rank;
	uint32_t payload_format;
	uint32_t incoming_host_mask; /* the reference's PCIe host mirrors: must be 0 here */
	uint32_t reserved_zero;
};

/* B200 extension, kernel file "kernel_ordered_b200", entry "ordered_rows_push": the expert layer's reduction for a
 * decode step as ONE launch. Every rank adds its pair outputs to row sums (from +0, ascending slot), stores the FP32
 * rows of the step (step.row_count of them) into its inbox in every rank's slot, then adds its inboxes in rank order
 * from +0, rounds ONCE to bfloat16 (nearest even, a not-a-number to 0x7FC0) and keeps bfloat16 [rows][width] at the
 * ARENA offset push.output_offset. push.input_offset is unused (0); the wire is FP32. The DONE lines are published at
 * the end and looked at before the slot's next use, so no rank waits for another after its own adds. */
#define KERNEL_ORDERED_ROWS_PUSH "ordered_rows_push"
struct ordered_rows_push_arguments {
	struct ordered_push_arguments push;
	uint64_t pair_output_offset; /* FP32 [rows * pairs_per_row][width] */
	uint32_t width;
	uint32_t pairs_per_row;
};

/* The exchange of a tensor-parallel layer site: the push with the live rows of the step block and a sequence of its
 * own for every layer, 2 * (step sequence * layer_count + layer) + (step sequence & 1), so that the layers of a step
 * share one region and the step's parity still selects the slot. element_count is a whole number of rows of
 * row_width elements (the reference fixes the width at compile time to its model's 5120 and keeps 8 reserved bytes
 * where row_width is); step.row_count of them are exchanged.
 * Forms: the push (every rank gets the FP32 sums), and the owner sums: rank d owns rows [R d / ranks, R (d + 1) / ranks)
 * of the step's R, every rank stores only that shard into rank d's inbox, rank d adds it in rank order, rounds ONCE to
 * bfloat16 (nearest even, a not-a-number to 0x7FC0) and stores the bfloat16 values into every rank's output array. */
#define KERNEL_FILE_TP_EXCHANGE "kernel_tp_exchange"
#define KERNEL_TP_EXCHANGE "tp_exchange"
#define KERNEL_TP_EXCHANGE_OWNER "tp_exchange_owner"
#define KERNEL_TP_EXCHANGE_SETTLED "tp_exchange_settled"
#define TP_EXCHANGE_FORM_PUSH 0u
#define TP_EXCHANGE_FORM_OWNER_SUMS 1u
#define TP_EXCHANGE_FORM_OWNER_RING_SUMS 2u /* the reference's four-rank bfloat16 ring order: not offered */
#define TP_EXCHANGE_FORM_CE_OWNER_SUMS 3u /* its copy-engine forms: not offered */
#define TP_EXCHANGE_FORM_CE_OWNER_RING_SUMS 4u
#define TP_EXCHANGE_OWNER_ALIGNMENT 16u
#define TP_EXCHANGE_WIDE_LAUNCHES 4u
#define TP_EXCHANGE_MAXIMUM_PHASES 1024u /* layer_count at most (the reference: 8 phases a layer, 40 layers) */
#define TP_EXCHANGE_MAXIMUM_ELEMENTS (1u << 26) /* the reference: 5120 * 2 * 1024 */
#define TP_EXCHANGE_REFERENCE_ROW_WIDTH 5120u
#define TP_EXCHANGE_ARGUMENT_BYTES 112u

struct tp_exchange_arguments {
	struct ordered_push_arguments collective;
	uint32_t layer;
	uint32_t layer_count;
	uint32_t row_width;
	uint32_t reserved_zero;
};

/* ------------------------------------------------------------------------------------------------------------
 * Local completion around the exchange (reference: include/anemone/tp2_join_records.h:11-48): element-wise conversions,
 * the join of the always-on expert's bfloat16 rows with the routed FP32 sums, strided copies. Row strides count
 * elements, slot strides bytes; with a slot stride, source or output advance by (step.sequence & 1) strides.
 *   0 BFLOAT16_TO_FLOAT32        out f32 = [routed f32 +] value(bf16)          (one rounded FP32 add, routed first)
 *   1 FLOAT32_TO_BFLOAT16        out bf16 = round(f32): nearest even, a not-a-number to 0x7FC0
 *   2 BFLOAT16_COPY, 3 FLOAT32_COPY   raw words (negative zeros and not-a-number payloads kept)
 *   4 BFLOAT16_SUM_TO_BFLOAT16   out bf16 = round([routed f32 +] value(bf16)): 0 then 1 without the FP32 store
 *   5 RING_PACK, 6 RING_UNPACK   4 into, and bfloat16 rows back out of, the owner-major order of the reference's
 *                                four-rank ring: owner o holds quarter o of every slab of 8 rows, slab after slab
 * ---------------------------------------------------------------------------------------------------------- */
#define KERNEL_FILE_TP2_JOIN "kernel_tp2_join"
#define KERNEL_TP2_JOIN "tp2_join"
#define TP2_JOIN_ARGUMENT_BYTES 80u
#define TP2_JOIN_THREADS 256u
#define TP2_JOIN_BFLOAT16_TO_FLOAT32 0u
#define TP2_JOIN_FLOAT32_TO_BFLOAT16 1u
#define TP2_JOIN_BFLOAT16_COPY 2u
#define TP2_JOIN_FLOAT32_COPY 3u
#define TP2_JOIN_BFLOAT16_SUM_TO_BFLOAT16 4u
#define TP2_JOIN_RING_PACK 5u
#define TP2_JOIN_RING_UNPACK 6u
#define TP2_JOIN_RING_OWNERS 4u
#define TP2_JOIN_RING_SLAB_ROWS 8u
#define TP2_JOIN_OPERATION_COUNT 7u
#define TP2_JOIN_MAXIMUM_WIDTH 32768u /* the reference: its model's heads x head dimensions, the same number */
#define TP2_JOIN_MAXIMUM_ROWS 1024u

struct tp2_join_arguments {
	uint64_t source_offset;
	uint64_t routed_sums_offset;
	uint64_t output_offset;
	uint64_t step_offset;
	uint64_t source_slot_stride;
	uint64_t output_slot_stride;
	uint32_t width;
	uint32_t row_count;
	uint32_t source_row_stride;
	uint32_t routed_row_stride;
	uint32_t output_row_stride;
	uint32_t operation;
	uint32_t has_routed_sums;
	uint32_t reserved_zero;
};

/* ------------------------------------------------------------------------------------------------------------
 * Router (B200 extension of the reference's router_select_entry, include/anemone/router_records.h:7-52): scores
 * FP32 [rows][expert_count] -> for each live row the `picks` experts of largest score (a not-a-number above every
 * number, -0 below +0, the lower expert first among equals), slots in ascending expert order, affinity
 * a = 1 / (1 + exp(-s)) (scoring 0) or sqrt(softplus(s)) (scoring 1, the reference's), weights a / (t + 1e-20) *
 * route_scale with t the sum of the picked a from +0 in ascending expert order; then the whole job table: one job per
 * chosen expert in ascending expert order, split in jobs of at most 8 rows in ascending row order, then the
 * always-on experts (shared experts: ids expert_count .. expert_count + shared_count - 1, weight 1, pair slot
 * picks + s), then empty jobs to job_capacity. One block of 1024 threads. */
#define KERNEL_FILE_ROUTER_B200 "kernel_router_b200"
#define KERNEL_ROUTER_SELECT_B200 "router_select_b200"
#define ROUTER_B200_THREADS 1024u
#define ROUTER_B200_MAXIMUM_EXPERTS 512u
#define ROUTER_B200_MAXIMUM_PICKS 16u
#define ROUTER_B200_MAXIMUM_ROWS 64u
#define ROUTER_SCORING_SIGMOID 0u
#define ROUTER_SCORING_SQRT_SOFTPLUS 1u
struct router_select_b200_arguments {
	uint64_t scores_offset; /* FP32 [row_capacity][expert_count] */
	uint64_t expert_table_offset; /* uint64 [expert_count + shared_count][3]: gate, up, down matrix offsets */
	uint64_t picks_offset; /* written: uint32 [row_capacity][picks] experts by slot */
	uint64_t weights_offset; /* written: FP32 [row_capacity][picks] */
	uint64_t jobs_offset; /* written: struct expert_job_record [job_capacity] */
	uint64_t step_offset; /* struct step_block: row_count live rows */
	uint32_t expert_count;
	uint32_t shared_count;
	uint32_t picks;
	uint32_t row_capacity;
	uint32_t job_capacity;
	uint32_t scoring;
	float route_scale;
	uint32_t reserved_zero;
	uint64_t bias_offset; /* FP32 [expert_count] added to the affinities for the choice alone; 0: none */
};

/* ------------------------------------------------------------------------------------------------------------
 * B200 extension, kernel file "kernel_exl3_prefill": the routed-expert layer for many rows (prefill), where every
 * expert sees enough rows for a dense contraction. Rows are grouped per expert into tiles of 128; trellis tiles are
 * decoded once per row tile into shared memory as FP16 and multiplied on the fifth-generation tensor cores
 * (tcgen05.mma, FP32 accumulators in tensor memory). The reference's counterpart is its tensor-core prefill family
 * (source/kernel_exl3_tcp.cuh: route, operands, grouped GEMM, combine), fixed to its own model's shapes; this one takes
 * shapes, expert count, picks and a stored width per expert from the record, and a rank may hold any run of the routed
 * experts (expert parallelism) and its own slice of the always-on experts' columns. Arithmetic per value is the retained
 * chain's (FP16 operands from the FP32 Hadamard transform, exactly decoded FP16 weights, FP32 accumulation, FP32
 * transforms, SwiGLU, route weight last); only the association of the FP32 sums over K is the tensor cores'.
 * Seven launches, one record:
 *   exl3_prefill_picks     grid (ceil(rows / 32)) x 1024: each live row's picks and weights (router_select_b200's
 *                          conventions), from scores
 *   exl3_prefill_group     grid (local + shared) x 256: entries[local expert][...]: the pairs routed to the expert in
 *                          ascending row order, and their count
 *   exl3_prefill_tiles     grid 1 x 1024: the tile table: (expert, first entry, rows) per 128-row tile, tile count
 *   exl3_prefill_operands  grid (tile capacity, 4 ceil(H / 512), 2) x 128: FP16 gate and up operands of every tile row
 *   exl3_prefill_gate_up   grid (max(I, shared I) / 128, tile capacity) x 576: both products, SwiGLU, FP16 down operands
 *   exl3_prefill_down      grid (ceil(H / 256), tile capacity) x 576: down product, output transform: FP32 pair outputs
 *   exl3_prefill_row_sum   grid (ceil(H / 512), rows) x 128: FP32 row sums over the row's LOCAL pairs, ascending slots
 *                          from +0
 * Workspace at workspace_offset, parts in this order, each aligned to 1024 bytes (exl3_prefill_sizes gives them):
 *   counts uint32 [local + shared + 1] (the last: tile count) | tiles struct exl3_prefill_tile [tile capacity] |
 *   entries struct exl3_prefill_entry [local + shared][row_capacity] |
 *   gate/up operands FP16 [2][tile capacity][H / 64][128 x 64 block] |
 *   down operands FP16 [tile capacity][max(I, shared I) / 64][block]
 * where a 128 x 64 block is stored as the tensor cores read it without swizzling: the 16 bytes of row r, inputs
 * 8 c .. 8 c + 7 lie at byte 2048 c + 128 (r / 8) + 16 (r % 8).
 * tile capacity = ceil(row_capacity * (picks + shared) / 128) + local + shared; exl3_prefill_parts_of takes the local
 * expert count and the larger of the two intermediate widths.
 * Rows at or beyond step.row_count are not read and nothing is written for them; a pair output is written only for
 * live rows. expert_count <= 512, experts + shared <= 1024, picks <= 16, H and I multiples of 128. */
#define EXL3_PREFILL_KERNEL_FILE "kernel_exl3_prefill"
#define EXL3_PREFILL_LAUNCHES 7u
#define EXL3_PREFILL_TILE_ROWS 128u
#define EXL3_PREFILL_BLOCK_INPUTS 64u
#define EXL3_PREFILL_BLOCK_BYTES 16384u
struct exl3_prefill_tile {
	uint32_t expert; /* local numbering: the rank's routed experts, then its always-on experts */
	uint32_t first_entry; /* into the expert's entries */
	uint32_t row_count; /* 1 .. 128 */
	uint32_t reserved_zero;
};
struct exl3_prefill_entry {
	uint32_t pair; /* row * (picks + shared) + slot */
	float route_weight;
};
struct exl3_prefill_record {
	uint64_t scores_offset; /* FP32 [row_capacity][expert_count] */
	uint64_t input_offset; /* bfloat16 [row_capacity][input_size] */
	uint64_t expert_table_offset; /* uint64 [local_count + shared_count][3], by LOCAL expert */
	uint64_t widths_offset; /* uint32 [local_count + shared_count] stored widths, by local expert */
	uint64_t picks_offset; /* written: uint32 [row_capacity][picks], global expert numbers */
	uint64_t weights_offset; /* written: FP32 [row_capacity][picks] */
	uint64_t workspace_offset;
	uint64_t pair_output_offset; /* written: FP32 [row_capacity * (picks + shared)][input_size], local pairs only */
	uint64_t row_output_offset; /* written: FP32 [row_capacity][input_size] */
	uint64_t step_offset; /* struct step_block: row_count live rows */
	uint32_t input_size; /* H */
	uint32_t inner_size; /* intermediate width of the routed experts' matrices held here */
	uint32_t shared_inner_size; /* the same of the always-on experts' matrices (0 if shared_count is 0) */
	uint32_t expert_count; /* routed experts the router chooses among */
	uint32_t local_first; /* this rank holds the routed experts local_first .. local_first + local_count - 1 */
	uint32_t local_count; /* may be 0: a rank that only holds always-on experts */
	uint32_t shared_count; /* always-on experts held here (slot picks + s of every row, weight 1) */
	uint32_t picks;
	uint32_t row_capacity;
	uint32_t scoring;
	float route_scale;
	float activation_limit;
	uint64_t bias_offset; /* FP32 [expert_count] added to the affinities for the choice alone; 0: none */
};

/* Offsets of the workspace parts from workspace_offset, the workspace's bytes and the tile capacity. */
struct exl3_prefill_parts {
	uint64_t counts, tiles, entries, gate_up_operands, down_operands, total;
	uint32_t tile_capacity;
	uint32_t reserved_zero;
};

AB_INLINE uint64_t exl3_prefill_aligned(uint64_t bytes)
{
	return (bytes + 1023u) / 1024u * 1024u;
}

AB_INLINE struct exl3_prefill_parts exl3_prefill_parts_of(uint32_t row_capacity, uint32_t picks, uint32_t shared_count,
							    uint32_t local_count, uint32_t input_size, uint32_t inner_size)
{
	struct exl3_prefill_parts parts;
	const uint32_t experts = local_count + shared_count;
	const uint64_t pairs = (uint64_t)row_capacity * (picks + shared_count);
	parts.tile_capacity = (uint32_t)((pairs + EXL3_PREFILL_TILE_ROWS - 1u) / EXL3_PREFILL_TILE_ROWS) + experts;
	parts.reserved_zero = 0;
	parts.counts = 0;
	parts.tiles = exl3_prefill_aligned((uint64_t)(experts + 1u) * 4u);
	parts.entries = parts.tiles + exl3_prefill_aligned((uint64_t)parts.tile_capacity * 16u);
	parts.gate_up_operands = parts.entries + exl3_prefill_aligned((uint64_t)experts * row_capacity * 8u);
	parts.down_operands = parts.gate_up_operands + (uint64_t)EXL3_PROJECTIONS * parts.tile_capacity *
							       (input_size / EXL3_PREFILL_BLOCK_INPUTS) * EXL3_PREFILL_BLOCK_BYTES;
	parts.total = parts.down_operands +
		      (uint64_t)parts.tile_capacity * (inner_size / EXL3_PREFILL_BLOCK_INPUTS) * EXL3_PREFILL_BLOCK_BYTES;
	return parts;
}

/* B200 extension, kernel file "kernel_router_b200": the job table of MANY rows (up to the prefill's row capacity), for
 * expert launches that take jobs of at most eight rows (the original-weights experts' thin instances). Three launches:
 * the prefill's picks and grouping (exl3_prefill_picks, exl3_prefill_group with `routing`: every routed expert local,
 * no always-on expert, a workspace of exl3_prefill_parts_of(...).gate_up_operands bytes: counts, tiles, entries), then
 * router_wide_jobs (one block of ROUTER_B200_THREADS): expert e's rows, ascending, eight to a job, the experts'
 * jobs in ascending expert order: the table router_select_b200 writes for a step of few rows. pair = row * picks +
 * slot. Jobs from the live count on have a row count of zero. routing.expert_table_offset: uint64 [expert_count][3]. */
#define KERNEL_ROUTER_WIDE_JOBS "router_wide_jobs"
#define ROUTER_WIDE_LAUNCHES 3u
struct router_wide_arguments {
	struct exl3_prefill_record routing;
	uint64_t jobs_offset; /* written: struct expert_job_record [job_capacity] */
	uint32_t job_capacity; /* at least row_capacity * picks / 8 + expert_count */
	uint32_t reserved_zero;
};

/* ------------------------------------------------------------------------------------------------------------
 * Original-weights experts: MXFP4 (E2M1 weights, one E8M0 scale per 32 inputs) by E4M3 block-quantized activations
 * (reference: include/anemone/linear_records.h:36-99, 222-299; include/anemone/weight_format_seam.h:23-46).
 *
 * Arrays (a vector v is a row of the batch, or a pair):
 *   values     bfloat16 [v][width]
 *   codes      uint8 [v][width], E4M3 bytes in LANE ORDER: byte ((4 l + t) 4 + s) 4 + j of a vector is the code of its
 *              value 64 l + 16 s + 2 t + j / 2 + 8 (j % 2)
 *   exponents  uint8 [v][width / 32]: E8M0 code c of a block of 32 values; a value is its code's value times 2^(c-127)
 *   operands   uint16 [v][width] in OPERAND ORDER (half ((4 l + t) 4 + s) 4 + 2 r + h is the operand of value
 *              64 l + 16 s + 2 t + h + 8 r). On this library's arithmetic class the operand is the E4M3 code PLACED as
 *              an FP16 (sign to bit 15, the other seven bits to bits 7..13: the code's value times 2^-8, exact), which
 *              is what its products feed the tensor cores; the reference's class 80 stores a bfloat16 carry there.
 *   a matrix   WEIGHT_FORMAT_E2M1_SCALED: words uint32 [output / 16][input / 64][lane][step 0..3], the nibble at bit
 *              4 r + 16 h of a word is W[16 tile + g + 8 (r % 2)][64 load + 16 step + 2 t + 8 (r / 2) + h], lane =
 *              4 g + t; then scales uint32 [tile][load][g]: byte 2 q + r is the E8M0 scale of inputs 64 load + 32 q ..
 *              + 31 of output 16 tile + g + 8 r. output_size * input_size / 2 + output_size * input_size / 32 bytes.
 * Quantization: per block of 32 values, in FP32: m = max(largest magnitude, 1e-4f) * (1 / 448.0f); c - 127 is the
 * exponent of the smallest power of two not below m; each magnitude is divided by 2^(c-127), limited to 448 and
 * rounded to the nearest E4M3 number, a tie to the even code; the sign is kept, also of a zero.
 * A product: the L = input_size / 64 loads are cut in S slices (slice i: loads floor(i L / S) .. floor((i + 1) L / S)
 * - 1), a slice is one FP32 chain from +0: per block of 32 inputs ascending, chain = fma(p, 2^e, chain), p the tensor
 * cores' FP32 sum of the block's 32 products (two instructions of 16, the second accumulating on the first) and 2^e
 * the exact power of two that applies both scales and undoes the placements; the S chains are added from +0 in
 * ascending order and the sum is rounded once to bfloat16 (nearest even; a not-a-number to 0x7FC0).
 * Hidden step: gate and up rounded to bfloat16 first; g = min(gate, limit); u = up limited to -limit .. limit;
 * h = bfloat16(((g / (1 + exp(-g))) * u) * route weight).
 * ---------------------------------------------------------------------------------------------------------- */
#define KERNEL_FILE_ACTIVATION_QUANTIZE "kernel_activation_quantize"
#define KERNEL_FILE_EXPERT_LINEAR "kernel_expert_linear"
#define KERNEL_ACTIVATION_QUANTIZE "activation_quantize_entry"
#define KERNEL_EXPERT_GATE_UP_STEM "expert_gate_up_"
#define KERNEL_EXPERT_DOWN_STEM "expert_down_"
#define KERNEL_EXPERT_ROW_SUM "expert_row_sum_entry"
#define LINEAR_SLICE_INSTANCES 5u /* slice counts 1, 2, 4, 8, 16 */
#define LINEAR_VALUES_PER_LOAD 64u
#define LINEAR_OUTPUTS_PER_TILE 16u
#define LINEAR_VALUES_PER_BLOCK 32u
#define LINEAR_ELEMENT_THREADS 256u

/* The always-on (shared) expert's matrices, WEIGHT_FORMAT_E4M3_SCALED (reference: include/anemone/
 * weight_format_seam.h:36-42): bytes uint8 [tile = output / 16][group = input / 32][lane][16]: byte b of a lane is
 * W[16 tile + g + 8 (b % 2)][32 group + 8 (b / 4) + 2 t + (b / 2) % 2], an E4M3 byte; then scales uint8
 * [block = output / 32][group]: one E8M0 code per 32 outputs by 32 inputs (the last block may hold 16 outputs).
 * output_size * input_size + ((output_size + 31) / 32) * (input_size / 32) bytes. Its products
 * (trunk_linear_quantized_<S>, include/anemone/linear_records.h:308-330) are the routed experts' with a weight placed
 * as FP16 by its seven low bits to bits 7..13 (its value times 2^-8): chain = fma(p, 2^(weight code + activation code -
 * 111), chain) per block of 32 inputs, the same slices and roundings; rows 0 .. row_count - 1 (at most 8) stand in
 * the columns. trunk_hidden_entry is the hidden step with a route weight of 1 on bfloat16 gate and up. */
#define KERNEL_FILE_TRUNK_LINEAR "kernel_trunk_linear"
#define KERNEL_TRUNK_LINEAR_QUANTIZED_STEM "trunk_linear_quantized_"
#define KERNEL_TRUNK_HIDDEN_VALUE "trunk_hidden_entry"
#define KERNEL_TRUNK_ROWS_ADD "trunk_rows_add_entry"
#define LINEAR_MERGED_MATRICES 2u

/* trunk_linear_quantized_<S>: grid ((output_size[0] + output_size[1]) / 16), block 32 S; matrix m takes the tiles from
 * the first one's on (output_size[1] is 0 where there is one matrix); writes bfloat16 [row_count][output_size[m]] */
struct trunk_linear_quantized_arguments {
	uint64_t weights_offset[LINEAR_MERGED_MATRICES];
	uint64_t output_offset[LINEAR_MERGED_MATRICES];
	uint64_t codes_offset;
	uint64_t exponents_offset;
	uint64_t operands_offset;
	uint32_t output_size[LINEAR_MERGED_MATRICES];
	uint32_t input_size;
	uint32_t row_count;
};

/* trunk_hidden_entry: grid (ceil(width / 256), vectors), block 256: bfloat16 gate and up [v][width] -> hidden */
struct trunk_hidden_arguments {
	uint64_t gate_offset;
	uint64_t up_offset;
	uint64_t hidden_offset;
	uint32_t width;
	float activation_limit;
};

/* B200 extension, trunk_rows_add_entry: grid (ceil(width / 256), rows), block 256: FP32 sums [rows][width] +=
 * bfloat16 values [rows][width], one FP32 addition each: the always-on expert's rows joined to the routed experts'
 * row sums before the ranks' reduction (the reference joins them in its FFN join, outside this path). */
struct trunk_rows_add_arguments {
	uint64_t sums_offset;
	uint64_t values_offset;
	uint32_t width;
	uint32_t reserved_zero;
};

AB_INLINE uint64_t e4m3_scaled_byte_count(uint32_t output_size, uint32_t input_size)
{
	return (uint64_t)output_size * input_size + (uint64_t)((output_size + 31u) / 32u) * (input_size / 32u);
}

/* activation_quantize_entry: grid (width / 64, vectors), block 32 (a warp a load of 64 values) */
struct activation_quantize_arguments {
	uint64_t values_offset;
	uint64_t codes_offset;
	uint64_t exponents_offset;
	uint64_t operands_offset;
	uint32_t width;
	uint32_t reserved_zero;
};

/* B200 extension, kernel file "kernel_router_b200", entry "router_select_quantize": router_select_b200 and the
 * activation quantizer of the step's rows in ONE launch (neither reads what the other writes: a decode step of the
 * original-weights layer begins with both). Block 0 is router_select_b200's block; every warp of the blocks behind it
 * takes loads of 64 values of the rows (activation_quantize_entry's task). grid (1 + ceil(vector_count * width / 64 /
 * 32)), block ROUTER_B200_THREADS. */
#define KERNEL_ROUTER_SELECT_QUANTIZE "router_select_quantize"
struct router_select_quantize_arguments {
	struct router_select_b200_arguments router;
	struct activation_quantize_arguments quantize;
	uint32_t vector_count; /* rows the quantizer takes: the capacity, as the separate launch */
	uint32_t reserved_zero;
};


/* expert_gate_up_<S>: grid (output_size / 16, jobs), block 64 S; writes hidden bfloat16 [pair][output_size] */
struct expert_gate_up_arguments {
	uint64_t jobs_offset;
	uint64_t codes_offset;
	uint64_t exponents_offset;
	uint64_t operands_offset;
	uint64_t hidden_offset;
	uint32_t output_size;
	uint32_t input_size;
	uint32_t pair_count;
	uint32_t pairs_per_row;
	float activation_limit;
	uint32_t reserved_zero;
};

/* expert_down_<S>: grid (output_size / 16, jobs), block 32 S; writes bfloat16 [pair][output_size] */
struct expert_down_arguments {
	uint64_t jobs_offset;
	uint64_t codes_offset;
	uint64_t exponents_offset;
	uint64_t operands_offset;
	uint64_t output_offset;
	uint32_t output_size;
	uint32_t input_size;
	uint32_t pair_count;
	uint32_t reserved_zero;
};

/* B200 extension, kernel file "kernel_expert_linear", entries "expert_gate_up_many" and "expert_down_many": the
 * routed experts' products for MANY rows (the profile's prefill). A block takes LINEAR_MANY_JOBS consecutive jobs of
 * the table and several tiles of 16 outputs: a warp decodes its tile's words once a load of 64 inputs and multiplies
 * them with the columns of every job of the group that belongs to the same expert (a job table in expert order, as
 * router_wide_jobs writes it, has up to 32 rows of one expert in a group), and the warps of a block read the same
 * rows' operands: the bytes a product moves from L2 fall to a sixth of the thin instances'. Every value's arithmetic
 * is the thin instances' (a slice is one chain of fma(p, 2^e, chain), the `slice_count` chains added from +0 in
 * ascending order, one rounding), so the results are theirs bit for bit.
 *   expert_gate_up_many  grid (output_size / 64, ceil(job_count / 4)), block 256: warps 0..3 four tiles of gate, 4..7 of up
 *   expert_down_many     grid (output_size / 128, ceil(job_count / 4)), block 256: a warp a tile */
#define LINEAR_MANY_JOBS 2u
#define KERNEL_EXPERT_GATE_UP_MANY "expert_gate_up_many"
#define KERNEL_EXPERT_DOWN_MANY "expert_down_many"
struct expert_gate_up_many_arguments {
	struct expert_gate_up_arguments base;
	uint32_t slice_count; /* 1, 2, 4, 8 or 16 */
	uint32_t job_count;
};
struct expert_down_many_arguments {
	struct expert_down_arguments base;
	uint32_t slice_count;
	uint32_t job_count;
};

/* B200 extension, kernel file "kernel_router_b200", entry "step_input_select": the step driver's hand-over of one
 * step's inputs that already lie in device memory. A pool holds `pool_count` prepared step input areas of `byte_count`
 * bytes at `pool_stride` apart (each beginning with its struct step_block, sequences strictly increasing); the kernel
 * copies entry (cursor mod pool_count) to destination_offset and advances the 64-bit cursor at cursor_offset. One
 * block of 1024 threads; byte_count a multiple of 16. (The reference's step driver uploads each step block from the
 * host, source/step.c:1421-1497; this keeps a run of steps on the device, for captured graphs and for timing with
 * resident inputs.) */
#define KERNEL_STEP_INPUT_SELECT "step_input_select"
struct step_input_select_arguments {
	uint64_t pool_offset;
	uint64_t pool_stride;
	uint64_t destination_offset;
	uint64_t cursor_offset;
	uint32_t pool_count;
	uint32_t byte_count;
};

#ifdef __cplusplus
#define AB_RECORD_HAS(record, bytes) static_assert(sizeof(struct record) == (bytes), #record " ABI")
#else
#define AB_RECORD_HAS(record, bytes) _Static_assert(sizeof(struct record) == (bytes), #record " ABI")
#endif
AB_RECORD_HAS(exl3_reconstruct_record, 32);
AB_RECORD_HAS(exl3_expert_record, 80);
AB_RECORD_HAS(expert_job_record, 96);
AB_RECORD_HAS(expert_row_sum_arguments, 24);
AB_RECORD_HAS(bb_exl3_shard_activation_record, 96);
AB_RECORD_HAS(exl3_moe_record, 112);
AB_RECORD_HAS(step_block, 16);
AB_RECORD_HAS(ordered_collective_peer, 32);
AB_RECORD_HAS(ordered_collective_arguments, 80);
AB_RECORD_HAS(ordered_reduce_bf16_arguments, 96);
AB_RECORD_HAS(ordered_row_sum_publish_arguments, 104);
AB_RECORD_HAS(ordered_publish_reduce_arguments, 104);
AB_RECORD_HAS(ordered_publish_reduce_bf16_arguments, 120);
AB_RECORD_HAS(ordered_push_arguments, 96);
AB_RECORD_HAS(tp_exchange_arguments, 112);
AB_RECORD_HAS(ordered_rows_push_arguments, 112);
AB_RECORD_HAS(tp2_join_arguments, 80);
AB_RECORD_HAS(router_select_b200_arguments, 88);
AB_RECORD_HAS(step_input_select_arguments, 40);
AB_RECORD_HAS(exact_ring_arguments, 80);
AB_RECORD_HAS(exl3_layer_route_record, 184);
AB_RECORD_HAS(exl3_layer_products_record, 128);
AB_RECORD_HAS(exl3_layer_publish_arguments, 72);
AB_RECORD_HAS(exl3_prefill_tile, 16);
AB_RECORD_HAS(exl3_prefill_entry, 8);
AB_RECORD_HAS(exl3_prefill_record, 136);
AB_RECORD_HAS(router_wide_arguments, 152);
AB_RECORD_HAS(router_select_quantize_arguments, 136);
AB_RECORD_HAS(activation_quantize_arguments, 40);
AB_RECORD_HAS(expert_gate_up_arguments, 64);
AB_RECORD_HAS(expert_down_arguments, 56);
AB_RECORD_HAS(expert_gate_up_many_arguments, 72);
AB_RECORD_HAS(expert_down_many_arguments, 64);
AB_RECORD_HAS(trunk_linear_quantized_arguments, 72);
AB_RECORD_HAS(trunk_hidden_arguments, 32);
AB_RECORD_HAS(trunk_rows_add_arguments, 24);

#endif
