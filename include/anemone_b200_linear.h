/*
 * anemone_b200_linear.h: load-time preparation of the original-weights experts (MXFP4 weights by E4M3 block-quantized
 * activations). Host C11. A refusal leaves every output unchanged. Replaces, for the routed experts of the path, the
 * part of the reference's include/anemone/linear.h named at each declaration, and for its always-on (shared) expert
 * the thin trunk product of E4M3 matrices (at most 8 rows). The reference's other trunk products (bfloat16 rows, wide
 * and interleaved instances: the attention side) are not part of this library: their handles are BACKEND_NO_KERNEL.
 */
#ifndef ANEMONE_B200_LINEAR_H
#define ANEMONE_B200_LINEAR_H

#include "anemone_b200_backend.h"
#include "anemone_b200_records.h"

#ifdef __cplusplus
extern "C" {
#endif

/* include/anemone/linear.h:193-196 */
struct linear_range {
	uint64_t byte_offset;
	uint64_t byte_count;
};

/* include/anemone/linear.h:97-108, member for member. Product kernels: one handle per slice count 1, 2, 4, 8, 16. */
struct linear_kernels_record {
	uint32_t activation_quantize;
	uint32_t expert_gate_up[LINEAR_SLICE_INSTANCES];
	uint32_t expert_down[LINEAR_SLICE_INSTANCES];
	uint32_t expert_row_sum;
	uint32_t trunk_linear_quantized[LINEAR_SLICE_INSTANCES];
	uint32_t trunk_linear_bfloat16[LINEAR_SLICE_INSTANCES];
	uint32_t trunk_hidden;
	uint32_t trunk_linear_quantized_wide[LINEAR_SLICE_INSTANCES];
	uint32_t trunk_linear_bfloat16_wide[LINEAR_SLICE_INSTANCES];
	uint32_t trunk_linear_quantized_interleaved;
};

/* include/anemone/linear.h:117-119: prepares activation_quantize_entry, expert_gate_up_<S>, expert_down_<S> and
 * trunk_linear_quantized_<S> for every S, expert_row_sum_entry, trunk_hidden_entry; every other trunk member is
 * BACKEND_NO_KERNEL. arithmetic_class: ARITHMETIC_CLASS_SM_100; the
 * reference's classes are STATUS_UNSUPPORTED, any other value STATUS_INVALID_ARGUMENT. */
MUST_CHECK result_status linear_kernels_prepare(const struct backend_operations *backend, struct device_card *card,
						uint32_t arithmetic_class, struct linear_kernels_record *kernels_out);

/* include/anemone/linear.h:214-226: one launch of activation_quantize_entry: grid (width / 64, row_count), block 32.
 * width a multiple of 64; every range 16-byte aligned, inside the arena, large enough, disjoint. */
struct linear_quantize_description {
	struct linear_range values;
	struct linear_range codes;
	struct linear_range exponents;
	struct linear_range operands;
	uint32_t width;
	uint32_t row_count;
};
MUST_CHECK result_status linear_quantize_prepare(const struct linear_quantize_description *description,
						 uint64_t arena_byte_count, const struct linear_kernels_record *kernels,
						 struct kernel_launch *launch_out);

/* include/anemone/linear.h:264-310: the routed experts of a layer from the rows' codes to the FP32 row sums: four
 * launches (gate/up with the hidden step; quantization of every pair's hidden vector; down; row sum). */
enum linear_routed_experts_launch {
	LINEAR_ROUTED_EXPERTS_GATE_UP = 0,
	LINEAR_ROUTED_EXPERTS_QUANTIZE = 1,
	LINEAR_ROUTED_EXPERTS_DOWN = 2,
	LINEAR_ROUTED_EXPERTS_ROW_SUM = 3,
	LINEAR_ROUTED_EXPERTS_LAUNCH_COUNT = 4
};
struct linear_routed_experts_description {
	struct linear_range jobs;
	struct linear_range expert_weights;
	struct linear_range codes;
	struct linear_range exponents;
	struct linear_range operands;
	struct linear_range hidden;
	struct linear_range hidden_codes;
	struct linear_range hidden_exponents;
	struct linear_range hidden_operands;
	struct linear_range pair_output;
	struct linear_range row_output;
	struct matrix_shape_record gate_up_shape;
	struct matrix_shape_record down_shape;
	enum weight_format_code weight_format; /* WEIGHT_FORMAT_E2M1_SCALED */
	uint32_t job_count;
	uint32_t row_count;
	uint32_t pairs_per_row;
	uint32_t gate_up_slice_count; /* 1, 2, 4, 8 or 16, at most the loads (input_size / 64) of the product */
	uint32_t down_slice_count;
	float activation_limit;
	uint32_t reserved_zero;
};
MUST_CHECK result_status linear_routed_experts_prepare(const struct linear_routed_experts_description *description,
						       uint64_t arena_byte_count,
						       const struct linear_kernels_record *kernels,
						       struct kernel_launch *launches_out);

/* B200 extension: the routed experts for a job table of MANY rows (the original-weights profile's prefill): the same
 * description and the same four launches with the two product launches given to "expert_gate_up_many" and
 * "expert_down_many" (struct expert_gate_up_many_arguments: a block a group of LINEAR_MANY_JOBS consecutive jobs and
 * several tiles, the words of a tile placed once for the group's jobs of one expert), prepared here. The results are
 * linear_routed_experts_prepare's bit for bit. gate_up_shape.output_size a multiple of 64, input_size of 128. */
MUST_CHECK result_status linear_routed_experts_wide_prepare(const struct linear_routed_experts_description *description,
							    uint64_t arena_byte_count,
							    const struct linear_kernels_record *kernels,
							    const struct backend_operations *backend,
							    struct device_card *card, struct kernel_launch *launches_out);

/* include/anemone/linear.h:200-208: a matrix where it lies in the arena and the slices its products are cut into.
 * wide_form: 0 (this library has the thin instances only). */
struct linear_matrix {
	struct linear_range stored; /* exactly the bytes its format stores for its shape */
	struct matrix_shape_record shape;
	enum weight_format_code weight_format;
	uint32_t slice_count;
	uint32_t wide_form;
	uint32_t reserved_zero;
};

/* include/anemone/linear.h:323-367: the always-on (shared) expert of a layer on at most 8 rows that are already
 * quantized (the routed experts read the same arrays): four launches: trunk_linear_quantized_<S> for gate and up (one
 * launch of two matrices), trunk_hidden_entry, activation_quantize_entry on the hidden vectors,
 * trunk_linear_quantized_<S> for down. The three matrices are WEIGHT_FORMAT_E4M3_SCALED, gate and up of one shape and
 * slice count, input sizes multiples of 64. */
enum linear_shared_expert_launch {
	LINEAR_SHARED_EXPERT_GATE_UP = 0,
	LINEAR_SHARED_EXPERT_HIDDEN = 1,
	LINEAR_SHARED_EXPERT_QUANTIZE = 2,
	LINEAR_SHARED_EXPERT_DOWN = 3,
	LINEAR_SHARED_EXPERT_LAUNCH_COUNT = 4
};
struct linear_shared_expert_description {
	struct linear_matrix gate;
	struct linear_matrix up;
	struct linear_matrix down;
	struct linear_range codes; /* read: codes [row_count][gate.shape.input_size] */
	struct linear_range exponents;
	struct linear_range operands;
	struct linear_range gate_output; /* scratch: values [row_count][gate.shape.output_size] */
	struct linear_range up_output;
	struct linear_range hidden;
	struct linear_range hidden_codes;
	struct linear_range hidden_exponents;
	struct linear_range hidden_operands;
	struct linear_range output; /* written: values [row_count][down.shape.output_size] */
	uint32_t row_count;
	float activation_limit;
};
MUST_CHECK result_status linear_shared_expert_prepare(const struct linear_shared_expert_description *description,
						      uint64_t arena_byte_count,
						      const struct linear_kernels_record *kernels,
						      struct kernel_launch *launches_out);

/* B200 extension (no counterpart in the reference, whose E4M3 format is one E8M0 code per 32 by 32 weights): the
 * always-on expert with WEIGHT_FORMAT_E4M3_BLOCK128 matrices: stored bytes = the E4M3 bytes in
 * WEIGHT_FORMAT_E4M3_SCALED's lane order, then FP32 scales [ceil(output_size / 128)][input_size / 128]; input sizes
 * multiples of 128. Everything else as linear_shared_expert_prepare (same description, same four launches, the hidden
 * step and the quantization shared); the kernels are "trunk_linear_block128_<S>", prepared here. */
MUST_CHECK result_status linear_shared_expert_block128_prepare(const struct linear_shared_expert_description *description,
							       uint64_t arena_byte_count,
							       const struct linear_kernels_record *kernels,
							       const struct backend_operations *backend,
							       struct device_card *card, struct kernel_launch *launches_out);

/* B200 extension: the always-on expert for ANY number of rows (up to 65535), in either E4M3 format (the description's
 * gate.weight_format decides): the same four launches with a block column per eight rows in the two product launches
 * (grid[1]); everything else as the two entries above. For calls of many rows (the original-weights profile's
 * prefill), whose rows the reference's thin launches would take eight at a time. */
MUST_CHECK result_status linear_shared_expert_wide_prepare(const struct linear_shared_expert_description *description,
							   uint64_t arena_byte_count,
							   const struct linear_kernels_record *kernels,
							   const struct backend_operations *backend,
							   struct device_card *card, struct kernel_launch *launches_out);
extern const struct weight_format_operations e4m3_block128_weight_operations;

/* B200 extension (the reference joins the two in its FFN join, outside this path): one launch of
 * trunk_rows_add_entry: FP32 sums [row_count][width] += bfloat16 values [row_count][width]. */
MUST_CHECK result_status linear_rows_add_prepare(const struct linear_range *sums, const struct linear_range *values,
						 uint32_t width, uint32_t row_count, uint64_t arena_byte_count,
						 const struct backend_operations *backend, struct device_card *card,
						 struct kernel_launch *launch_out);

/* include/anemone/linear.h:401-411: the bytes of the arrays of linear_records.h */
uint64_t linear_values_byte_count(uint64_t vector_count, uint32_t width);
uint64_t linear_codes_byte_count(uint64_t vector_count, uint32_t width);
uint64_t linear_exponents_byte_count(uint64_t vector_count, uint32_t width);
uint64_t linear_sums_byte_count(uint64_t row_count, uint32_t width);
uint64_t linear_jobs_byte_count(uint64_t job_count);

/* include/anemone/weight_format_seam.h (weight_format_operations_of for WEIGHT_FORMAT_E2M1_SCALED): stored bytes of an
 * output_size x input_size matrix: output_size * input_size / 2 + output_size * input_size / 32. */
extern const struct weight_format_operations e2m1_scaled_weight_operations;
/* the same for WEIGHT_FORMAT_E4M3_SCALED: output_size * input_size + ((output_size + 31) / 32) * (input_size / 32) */
extern const struct weight_format_operations e4m3_scaled_weight_operations;

#ifdef __cplusplus
}
#endif
#endif
