/*
 * anemone_b200_exl3_tc.h: the reference's DEFAULT entry points of the routed experts of one EXL3 layer, which its model
 * program calls at load (include/anemone/exl3_tc.h:22-59, called from source/model_v41_program.c:4311-4388): the
 * decode family (1 to 64 rows, the router's job table in) and the prefill family (65 to 2,048 rows, the router's
 * picks in). Same names, records, workspace sizes, argument meaning and refusals; the kernels behind them are this
 * library's (kernel file "kernel_exl3_tc": the fused products of the fixed cut with the retained chain's FP32
 * arithmetic, not the reference's FP64 transforms and hi/lo operand split: results agree within the cross-family
 * tolerance of the reference's own card test, tests/exl3_tc_card_test.c:40-41). The records carry no hidden size: as in
 * the reference these entry points serve its model's geometry alone, hidden 5120, six routes a row, 384 experts, a
 * rank's intermediate of 640 or 512 columns. Host C11; a refusal leaves the launch table (and the count) unchanged.
 */
#ifndef ANEMONE_B200_EXL3_TC_H
#define ANEMONE_B200_EXL3_TC_H

#include "anemone_b200_backend.h"
#include "anemone_b200_records.h"

#ifdef __cplusplus
extern "C" {
#endif

#define EXL3_TC_KERNEL_FILE "kernel_exl3_tc"
#define EXL3_TC_LAUNCHES 5u
#define EXL3_TC_HIDDEN 5120u
#define EXL3_TC_PAIRS_PER_ROW 6u
#define EXL3_TC_MOST_PAIRS 2688u
#define EXL3_TC_MOST_ROWS 64u
#define EXL3_TC_WIDE_INTERMEDIATE 640u
#define EXL3_TC_NARROW_INTERMEDIATE 512u
#define EXL3_TC_MOST_ROTATION 5u
#define EXL3_TCP_MOST_LAUNCHES 11u
#define EXL3_TCP_CHUNK_ROWS 2048u
#define EXL3_TCP_JOINT_ROWS 1024u
#define EXL3_TCP_EXPERTS 384u
#define EXL3_TCP_TILE_ROWS 64u

/* include/anemone/exl3_tc_records.h:40-58 */
struct exl3_tc_record {
	uint64_t jobs_offset; /* read: struct expert_job_record [job_capacity], ascending experts, empty ones last */
	uint64_t hidden_offset; /* read: bfloat16 [row_count][5120] */
	uint64_t workspace_offset; /* scratch: exl3_tc_workspace_bytes(6 row_count, intermediate) */
	uint64_t output_offset; /* written: FP32 [row_count][5120], each row's route-weighted expert sum */
	uint32_t row_count;
	uint32_t job_capacity;
	uint32_t intermediate; /* 640 or 512 */
	uint32_t bits_x2; /* 4, 5, 6 or 8 here (the reference: 6 or 4) */
	float activation_limit; /* the SwiGLU limit; 0: none */
	uint32_t pass; /* 0 in a caller's record */
	uint32_t rotation; /* the reference's mixed expert widths: refused here unless 0 */
	uint32_t shared_sum; /* 1: add each row's sum to the bfloat16 row at shared_offset and round once, in place */
	uint64_t shared_offset;
};

/* include/anemone/router_records.h:112-115 */
struct router_pick {
	uint32_t expert;
	float route_weight;
};

/* include/anemone/exl3_tc_records.h:244-264 */
struct exl3_tcp_record {
	uint64_t picks_offset; /* read: struct router_pick [row_count][6], a row's experts ascending */
	uint64_t expert_offsets_offset; /* read: uint64 [384][3] */
	uint64_t hidden_offset; /* read: bfloat16 [row_count][5120] */
	uint64_t workspace_offset; /* scratch: exl3_tcp_workspace_bytes(row_count, intermediate) */
	uint64_t output_offset; /* written: FP32 [row_count][5120] */
	uint32_t row_count; /* 1 to EXL3_TCP_CHUNK_ROWS */
	uint32_t intermediate;
	uint32_t bits_x2;
	uint32_t pass; /* 0 in a caller's record */
	float activation_limit;
	uint32_t rotation; /* refused here unless 0 */
	uint32_t half_rows; /* the reference's two-part overlap of one call: refused here unless 0 */
	uint32_t part; /* 0 in a caller's record */
	uint64_t step_offset;
	uint32_t cone_layer; /* rows a step leaves alone: refused here unless 0 */
	uint32_t two_blocks; /* 0 or 1: a choice among the reference's kernel forms, accepted and ignored */
};

/* The workspace sizes a caller reserves: the reference's formulas (include/anemone/exl3_tc_records.h:155-200,
 * 266-304), so that a caller's arena plan does not change. This library lays its own scratch out inside them. */
AB_INLINE uint64_t exl3_tc_aligned(uint64_t bytes)
{
	return (bytes + 255u) / 256u * 256u;
}

AB_INLINE uint64_t exl3_tc_workspace_bytes(uint64_t pair_count, uint64_t intermediate)
{
	/* FP32 gate, up (16 slices) and down (2 slices) partials; FP16 hi/lo operands of gate/up and of down; their
	 * scales; the job count; 16 bytes a pair: every part rounded up to 256 bytes */
	return 2u * exl3_tc_aligned(16u * pair_count * intermediate * 4u) +
	       exl3_tc_aligned(2u * pair_count * EXL3_TC_HIDDEN * 4u) +
	       exl3_tc_aligned(pair_count * 2u * 2u * EXL3_TC_HIDDEN * 2u) +
	       exl3_tc_aligned(pair_count * 2u * intermediate * 2u) + exl3_tc_aligned(pair_count * 2u * 16u * 4u) +
	       exl3_tc_aligned(pair_count * 2u * 4u) + exl3_tc_aligned(16u) + exl3_tc_aligned(pair_count * 16u);
}

AB_INLINE uint64_t exl3_tcp_tile_capacity(uint64_t pairs)
{
	const uint64_t halves = 2u * EXL3_TCP_EXPERTS;
	const uint64_t bound = pairs / EXL3_TCP_TILE_ROWS + (halves < pairs ? halves : pairs) + 1u;
	return bound < pairs ? bound : pairs;
}

AB_INLINE uint64_t exl3_tcp_sequence_words(uint64_t rows, uint64_t intermediate)
{
	const uint64_t pairs = rows * EXL3_TC_PAIRS_PER_ROW, projections = rows <= EXL3_TCP_JOINT_ROWS ? 2u : 1u;
	const uint64_t table = 4u + (pairs + 3u) / 4u * 4u + 4u * exl3_tcp_tile_capacity(pairs) + pairs;
	return pairs * projections * EXL3_TC_HIDDEN + pairs * 2u * intermediate + (pairs * projections + 3u) / 4u * 4u +
	       (table + 3u) / 4u * 4u;
}

AB_INLINE uint64_t exl3_tcp_workspace_bytes(uint64_t rows, uint64_t intermediate)
{
	const uint64_t joint = rows < EXL3_TCP_JOINT_ROWS ? rows : EXL3_TCP_JOINT_ROWS;
	const uint64_t first = exl3_tcp_sequence_words(rows, intermediate);
	const uint64_t second = exl3_tcp_sequence_words(joint, intermediate);
	return 4u * (first > second ? first : second);
}

/* The two workspace sizes as exports, for callers that cannot use the inline functions. */
uint64_t exl3_tc_workspace_byte_count(uint64_t pair_count, uint64_t intermediate);
uint64_t exl3_tcp_workspace_byte_count(uint64_t rows, uint64_t intermediate);

/* include/anemone/exl3_tc.h:22-39 (source/exl3_tc.c:120-268). Five launches: input transform (with the scratch's
 * counters set to zero), gate/up products with the activation, a launch that marks the pairs the job table holds,
 * down products with the output transform and route weight, the rows' sums in ascending slot order (a pair no job
 * holds adds nothing, as in the reference). The three entry points differ in the reference by the cut of its
 * products alone; here they prepare the same launches. Refusals as the reference's: STATUS_INVALID_ARGUMENT for a
 * null argument, no rows, an intermediate other than 640 or 512, no width of the format, no job capacity, a pass
 * other than 0, a negative or not-a-number limit, a rotation above 5 or without 640 columns, shared_sum above 1,
 * more than 2,688 pairs or more jobs than pairs, a range misaligned, outside the arena, empty or overlapping;
 * STATUS_UNSUPPORTED for a width these kernels do not decode and, here, for a rotation other than 0. */
MUST_CHECK result_status exl3_tc_prepare(const struct exl3_tc_record *record, uint64_t arena_byte_count,
					 const struct backend_operations *backend, struct device_card *card,
					 struct kernel_launch launches_out[EXL3_TC_LAUNCHES]);
MUST_CHECK result_status exl3_tc_prepare_short(const struct exl3_tc_record *record, uint64_t arena_byte_count,
					       const struct backend_operations *backend, struct device_card *card,
					       struct kernel_launch launches_out[EXL3_TC_LAUNCHES]);
MUST_CHECK result_status exl3_tc_prepare_paired(const struct exl3_tc_record *record, uint64_t arena_byte_count,
						const struct backend_operations *backend, struct device_card *card,
						struct kernel_launch launches_out[EXL3_TC_LAUNCHES]);

/* include/anemone/exl3_tc.h:41-59 (source/exl3_tc.c:304-513). The launches of one call of up to 2,048 rows from the
 * router's picks: a route launch that groups the pairs by expert into jobs of at most eight rows inside the
 * workspace, then the input transform, the two product launches and the rows' sums (every pair of a pick is routed,
 * so nothing is marked): five launches for up to 1,024 rows; a longer call is taken in two chunks of rows, one after
 * the other in the same workspace, ten launches. *launch_count_out receives their number. _base and _hybrid name
 * forms of the reference's GEMM for 640 columns; here all three prepare the same launches. Refusals as the reference's, and STATUS_UNSUPPORTED for rotation, half_rows or
 * cone_layer other than 0. */
MUST_CHECK result_status exl3_tcp_prepare(const struct exl3_tcp_record *record, uint64_t arena_byte_count,
					  const struct backend_operations *backend, struct device_card *card,
					  struct kernel_launch launches_out[EXL3_TCP_MOST_LAUNCHES],
					  uint32_t *launch_count_out);
MUST_CHECK result_status exl3_tcp_prepare_base(const struct exl3_tcp_record *record, uint64_t arena_byte_count,
					       const struct backend_operations *backend, struct device_card *card,
					       struct kernel_launch launches_out[EXL3_TCP_MOST_LAUNCHES],
					       uint32_t *launch_count_out);
MUST_CHECK result_status exl3_tcp_prepare_hybrid(const struct exl3_tcp_record *record, uint64_t arena_byte_count,
						 const struct backend_operations *backend, struct device_card *card,
						 struct kernel_launch launches_out[EXL3_TCP_MOST_LAUNCHES],
						 uint32_t *launch_count_out);

#ifdef __cplusplus
}
#endif
#endif
