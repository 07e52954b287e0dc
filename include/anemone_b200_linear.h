/*
 * anemone_b200_linear.h: load-time preparation of the original-weights experts (MXFP4 weights by E4M3 block-quantized
 * activations). Host C11. A refusal leaves every output unchanged. Replaces, for the routed experts of the path, the
 * part of the reference's include/anemone/linear.h named at each declaration; the reference's trunk products (FP8
 * matrices of the shared expert and the attention side) are not part of this library: their handles are
 * BACKEND_NO_KERNEL.
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

/* include/anemone/linear.h:117-119: prepares activation_quantize_entry, expert_gate_up_<S>, expert_down_<S> for every
 * S, expert_row_sum_entry; every trunk member is BACKEND_NO_KERNEL. arithmetic_class: ARITHMETIC_CLASS_SM_100; the
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

/* include/anemone/linear.h:401-411: the bytes of the arrays of linear_records.h */
uint64_t linear_values_byte_count(uint64_t vector_count, uint32_t width);
uint64_t linear_codes_byte_count(uint64_t vector_count, uint32_t width);
uint64_t linear_exponents_byte_count(uint64_t vector_count, uint32_t width);
uint64_t linear_sums_byte_count(uint64_t row_count, uint32_t width);
uint64_t linear_jobs_byte_count(uint64_t job_count);

/* include/anemone/weight_format_seam.h (weight_format_operations_of for WEIGHT_FORMAT_E2M1_SCALED): stored bytes of an
 * output_size x input_size matrix: output_size * input_size / 2 + output_size * input_size / 32. */
extern const struct weight_format_operations e2m1_scaled_weight_operations;

#ifdef __cplusplus
}
#endif
#endif
