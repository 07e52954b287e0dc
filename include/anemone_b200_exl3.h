/*
 * anemone_b200_exl3.h: load-time preparation of the EXL3 expert launches. Host C11, no allocation, no device call
 * except through backend->kernel_prepare. A refusal leaves every scalar output and the whole launch table unchanged.
 *
 * Each declaration names the reference declaration it replaces; argument order and meaning, refusals and the launch
 * records written are the reference's. Launch GEOMETRY is this library's own (its kernels are new): a caller must take
 * grids and blocks from the prepared launches, never assume them.
 */
#ifndef ANEMONE_B200_EXL3_H
#define ANEMONE_B200_EXL3_H

#include <stddef.h>

#include "anemone_b200_backend.h"
#include "anemone_b200_records.h"

#ifdef __cplusplus
extern "C" {
#endif

/* include/anemone/exl3.h:11: the format's table; stored_byte_count = codes + 2 (inputs + outputs) bytes. */
extern const struct weight_format_operations exl3_weight_operations;

/* include/anemone/exl3.h:14: "k2", "k2_5", "k3", "k4" of a bits_x2; NULL for a width without kernel entries. */
const char *exl3_width_name(uint32_t bits_x2);

/* include/anemone/exl3.h:16-18 (source/exl3.c:58-101). Matrix and FP16 [input][output] output 64-byte aligned,
 * inside the arena, disjoint. kernel: the handle of ("kernel_exl3", "exl3_reconstruct"). */
MUST_CHECK result_status exl3_reconstruct_prepare(const struct exl3_reconstruct_record *record,
						  uint64_t arena_byte_count, uint32_t kernel,
						  struct kernel_launch *launch_out);

/* include/anemone/exl3.h:31: operands + products scratch for pair_count pairs: 12 bytes per pair and input. */
uint64_t exl3_scratch_byte_count(uint32_t pair_count, uint32_t input_size);

/* include/anemone/exl3.h:35-39 (source/exl3.c:142-294): the five launches input, gate/up, activate, down, finish of
 * kernel file "kernel_exl3". arithmetic_class: ARITHMETIC_CLASS_SM_100 (the reference's three classes are
 * STATUS_UNSUPPORTED here: no build for them); any other value is STATUS_INVALID_ARGUMENT. */
MUST_CHECK result_status exl3_experts_prepare(const struct exl3_expert_record *record, uint64_t arena_byte_count,
					      const struct backend_operations *backend, struct device_card *card,
					      uint32_t arithmetic_class, struct kernel_launch *launches_out);

/* include/anemone/exl3.h:50-53: the reference's faster module for the same words. This library has one product
 * implementation, so this is exl3_experts_prepare under the reference's second name. */
MUST_CHECK result_status exl3_experts_fast_prepare(const struct exl3_expert_record *record,
						   uint64_t arena_byte_count,
						   const struct backend_operations *backend, struct device_card *card,
						   uint32_t arithmetic_class, struct kernel_launch *launches_out);

/* include/anemone/exl3.h:58-61: the eight-slice association of the reference's CMP cards. STATUS_UNSUPPORTED for
 * every class this library runs on, as the reference answers for every class but 80. */
MUST_CHECK result_status exl3_experts_relaxed_prepare(const struct exl3_expert_record *record,
						      uint64_t arena_byte_count,
						      const struct backend_operations *backend,
						      struct device_card *card, uint32_t arithmetic_class,
						      struct kernel_launch *launches_out);

/* B200 extension: bytes of the scratch ranges of struct exl3_moe_record, which depend on how the fused launches cut
 * their products (see the record). Zero sizes for shapes the chain refuses. */
struct exl3_moe_sizes {
	uint64_t operand_bytes; /* at base.operands_offset */
	uint64_t product_bytes; /* at base.products_offset */
	uint64_t counter_bytes; /* at counters_offset */
	uint32_t gate_up_splits;
	uint32_t down_splits;
};
void exl3_moe_sizes(uint32_t pair_count, uint32_t job_count, uint32_t input_size, uint32_t inner_size,
		    struct exl3_moe_sizes *sizes_out);

/* B200 extension (no reference counterpart): the four fused launches of kernel file "kernel_exl3_b200" for
 * struct exl3_moe_record: per-expert stored widths, row sums written to row_output_offset. launches_out has
 * EXL3_MOE_LAUNCHES entries. Validates what exl3_experts_prepare validates, plus the width table and the row output. */
MUST_CHECK result_status exl3_moe_prepare(const struct exl3_moe_record *record, uint64_t arena_byte_count,
					  const struct backend_operations *backend, struct device_card *card,
					  struct kernel_launch *launches_out);

/* B200 extension (the reference's counterpart: its tensor-core prefill family, include/anemone/exl3_tc.h:42-45): the seven
 * launches of kernel file "kernel_exl3_prefill" for struct exl3_prefill_record: router, grouping of rows per expert in
 * tiles of 128, operands, the grouped tensor-core products with their epilogues, row sums. launches_out has
 * EXL3_PREFILL_LAUNCHES entries. The workspace (exl3_prefill_parts_of(...).total bytes) begins on a multiple of 1024
 * bytes and needs no initial contents. */
MUST_CHECK result_status exl3_prefill_prepare(const struct exl3_prefill_record *record, uint64_t arena_byte_count,
					      const struct backend_operations *backend, struct device_card *card,
					      struct kernel_launch *launches_out);

/* B200 extension (no reference counterpart: its step is a router launch, five expert launches, a row sum and a
 * one-CTA exchange): ONE decode step of a rank's whole expert layer in the EXL3_LAYER_LAUNCHES launches of struct
 * exl3_layer_route_record (router with input transform; the products, one resident grid that walks the step's
 * items; row sums, READY and the reduction). Each launch is given its place on the card while the one before it still
 * runs (LAUNCH_OVERLAPS_PREVIOUS) and waits for that launch itself.
 * route.moe is read as exl3_moe_prepare reads it, with the scratch sizes of exl3_layer_sizes; publish names the
 * reduction's region (two parity slots of parity_stride bytes, the FP32 rows at input_offset inside a slot, behind
 * EXL3_LAYER_SIGNAL_BYTES of signal lines), the peer table (struct ordered_collective_peer [rank_count]), the status
 * block and the step block; result_offset: bfloat16 [row_capacity][input_size]. gate_up_runs, down_runs (powers of two
 * up to EXL3_LAYER_MAXIMUM_RUNS that divide the products' 128-input blocks): the cut of K of gate and up and of
 * down, 0 for this library's choice from the shapes. The region and the counters must be zero at load; after a
 * bounded wait has run out (backend_b200_waits_expired) the counters must be zeroed again before the next step. */
struct exl3_layer_description {
	struct exl3_layer_route_record route;
	struct exl3_layer_publish_arguments publish;
	uint64_t result_offset;
	uint64_t arena_byte_count;
	uint32_t gate_up_runs;
	uint32_t down_runs;
};
/* Scratch bytes of the layer form (see struct exl3_layer_route_record): operands as exl3_moe_sizes gives them;
 * products for EXL3_LAYER_MAXIMUM_RUNS runs; counters with the layer's own words. The two split counts are zero. */
void exl3_layer_sizes(uint32_t pair_count, uint32_t job_count, uint32_t input_size, uint32_t inner_size,
		      struct exl3_moe_sizes *sizes_out);
MUST_CHECK result_status exl3_layer_prepare(const struct exl3_layer_description *description,
					    const struct backend_operations *backend, struct device_card *card,
					    struct kernel_launch *launches_out);

/* The workspace layout of exl3_prefill_prepare for these shapes: exl3_prefill_parts_of as an export, for callers that
 * cannot use the inline function. */
void exl3_prefill_sizes(uint32_t row_capacity, uint32_t picks, uint32_t shared_count, uint32_t local_count,
			uint32_t input_size, uint32_t widest_inner_size, struct exl3_prefill_parts *parts_out);

/* ---- load-time slices for tensor parallelism (include/anemone/exl3_layout.h) ---- */

struct bb_exl3_matrix_slice {
	uint32_t input_size;
	uint32_t output_size;
	uint32_t input_begin;
	uint32_t input_count;
	uint32_t output_begin;
	uint32_t output_count;
	uint32_t bits_per_weight;
	uint32_t reserved_zero;
};

struct bb_exl3_slice_sizes {
	uint64_t source_bytes;
	uint64_t packed_bytes;
};

enum bb_exl3_product_order { BB_EXL3_REFERENCE_ORDER = 0, BB_EXL3_EIGHT_PART_ORDER = 1 };

struct bb_exl3_output_shard_plan {
	struct bb_exl3_matrix_slice gate_up;
	struct bb_exl3_matrix_slice down;
	uint32_t rank_count;
	uint32_t rank;
	uint32_t product_slices;
	enum bb_exl3_product_order order;
};

/* include/anemone/exl3_layout.h:38-40: sizes of a slice; every origin and count a multiple of 128. */
MUST_CHECK result_status bb_exl3_matrix_slice_prepare(const struct bb_exl3_matrix_slice *slice,
						      struct bb_exl3_slice_sizes *sizes_out);

/* include/anemone/exl3_layout.h:49-51: lossless host copy of a slice (tile rows of codes, then the two scale
 * sub-vectors); no decode, no floating point, no allocation. */
MUST_CHECK result_status bb_exl3_matrix_slice_copy(const struct bb_exl3_matrix_slice *slice, const void *source,
						   size_t source_bytes, void *destination,
						   size_t destination_bytes);

/* include/anemone/exl3_layout.h:98-101: the "exact output shards" plan: gate/up cut by output (inner) columns, down
 * cut by OUTPUT (outer) columns, both with their complete K. The reference takes 1 or 4 ranks; this library takes 1,
 * 2, 4 or 8. */
MUST_CHECK result_status bb_exl3_output_shard_prepare(uint32_t outer_size, uint32_t inner_size,
						      uint32_t bits_per_weight, uint32_t rank_count, uint32_t rank,
						      enum bb_exl3_product_order order,
						      struct bb_exl3_output_shard_plan *plan_out);

/* B200 extension: the "inner" tensor-parallel plan the expert-layer reduction is built on (the split the reference's
 * model program uses for its routed experts, source/model_v41_program.c:2618-2770): rank r owns intermediate columns
 * [blocks r / R, blocks (r + 1) / R) x 128; gate/up are cut by OUTPUT columns (complete K), down by INPUT rows
 * (complete outputs), so each rank's down product is an FP32 partial of every output and the ranks' partials are
 * summed in rank order. Same plan struct: .gate_up as above, .down = { inner, outer, inner_begin, count, 0, outer }. */
MUST_CHECK result_status bb_exl3_inner_shard_prepare(uint32_t outer_size, uint32_t inner_size,
						     uint32_t bits_per_weight, uint32_t rank_count, uint32_t rank,
						     struct bb_exl3_output_shard_plan *plan_out);

/* ---- single passes on local shard shapes (include/anemone/exl3_tp.h) ---- */

enum bb_exl3_pass {
	BB_EXL3_INPUT_PASS = 0,
	BB_EXL3_GATE_UP_PASS = 1,
	BB_EXL3_ACTIVATE_PASS = 2,
	BB_EXL3_DOWN_PASS = 3,
	BB_EXL3_FINISH_PASS = 4,
	BB_EXL3_PASSES = 5
};

struct bb_exl3_pass_description {
	const struct bb_exl3_output_shard_plan *plan;
	struct exl3_expert_record record;
	uint64_t arena_bytes;
	uint64_t weight_offset;
	uint64_t weight_bytes;
	enum bb_exl3_pass pass;
	uint32_t product_tiles; /* the reference's choice among identical-word product modules: accepted (0, 1, 2, 4, 8)
				   and ignored, this library having one */
};

/* include/anemone/exl3_tp.h:65-68 (source/exl3_tp.c:53-248): one launch of one pass for a rank of an output-shard
 * plan: INPUT/GATE_UP/ACTIVATE on (full outer, local inner), DOWN/FINISH on (local outer, full inner); the activation
 * is "bb_exl3_activate_output_shard" with its 96-byte record. */
MUST_CHECK result_status bb_exl3_pass_prepare(const struct bb_exl3_pass_description *description,
					      const struct backend_operations *backend, struct device_card *card,
					      struct kernel_launch *launch_out);

/* include/anemone/exl3_tp.h:77-80 (source/exl3_tp.c:250-292): exl3_row_sum over `rows` rows. */
MUST_CHECK result_status bb_exl3_row_sum_prepare(const struct expert_row_sum_arguments *record, uint32_t rows,
						 uint64_t arena_bytes, const struct backend_operations *backend,
						 struct device_card *card, struct kernel_launch *launch_out);

#ifdef __cplusplus
}
#endif
#endif
