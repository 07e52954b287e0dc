/*
 * exl3_tp.c: single passes of the expert chain on a rank's local shard shapes, and the row sum.
 * Takes the place of the reference's source/exl3_tp.c (bb_exl3_pass_prepare :53-248, bb_exl3_row_sum_prepare
 * :250-292): same descriptions, validation and records; the launch shapes are this library's.
 */
#include "anemone_b200_exl3.h"

#include <math.h>
#include <stdio.h>
#include <string.h>

#include "../kernels/exl3_geometry.h"
#include "prepare_common.h"

#define MAXIMUM_GRID_ROWS 65535u

result_status bb_exl3_pass_prepare(const struct bb_exl3_pass_description *description,
				   const struct backend_operations *backend, struct device_card *card,
				   struct kernel_launch *launch_out)
{
	if (description == NULL || description->plan == NULL || backend == NULL || backend->kernel_prepare == NULL ||
	    card == NULL || launch_out == NULL || (uint32_t)description->pass >= BB_EXL3_PASSES)
		return STATUS_INVALID_ARGUMENT;
	const struct bb_exl3_output_shard_plan plan = *description->plan;
	struct bb_exl3_output_shard_plan canonical;
	memset(&canonical, 0, sizeof(canonical));
	if (bb_exl3_output_shard_prepare(plan.gate_up.input_size, plan.down.input_size, plan.gate_up.bits_per_weight,
					 plan.rank_count, plan.rank, plan.order, &canonical) != STATUS_OK ||
	    memcmp(&plan, &canonical, sizeof(plan)) != 0)
		return STATUS_INVALID_ARGUMENT;
	const uint32_t tiles = description->product_tiles;
	if ((tiles != 0 && tiles != 1 && tiles != 2 && tiles != 4 && tiles != 8) ||
	    plan.order == BB_EXL3_EIGHT_PART_ORDER)
		return STATUS_UNSUPPORTED; /* the eight-part order is the relaxed association: no build here */
	const struct exl3_expert_record record = description->record;
	const enum bb_exl3_pass pass = description->pass;
	const bool down_shape = pass >= BB_EXL3_DOWN_PASS;
	if (record.reserved_zero != 0 || record.pair_count == 0 || record.pairs_per_row == 0 ||
	    record.pair_count % record.pairs_per_row != 0 || record.job_count == 0 ||
	    record.job_count > MAXIMUM_GRID_ROWS ||
	    description->weight_offset % WEIGHT_FORMAT_MATRIX_ALIGNMENT_BYTES != 0 ||
	    record.bits_per_weight != plan.gate_up.bits_per_weight ||
	    record.input_size != (down_shape ? plan.down.output_count : plan.gate_up.input_count) ||
	    record.inner_size != (down_shape ? plan.down.input_count : plan.gate_up.output_count) ||
	    !isfinite(record.activation_limit) || record.activation_limit <= 0 ||
	    (pass == BB_EXL3_FINISH_PASS && record.output_offset != record.products_offset))
		return STATUS_INVALID_ARGUMENT;
	const uint64_t outer_values = (uint64_t)record.pair_count * record.input_size;
	const uint64_t inner_values = (uint64_t)record.pair_count * record.inner_size;
	struct checked_range ranges[6] = { { "weights", description->weight_offset, description->weight_bytes },
					   { "jobs", record.jobs_offset,
					     (uint64_t)record.job_count * sizeof(struct expert_job_record) } };
	uint32_t count = 2;
	if (pass == BB_EXL3_INPUT_PASS)
		ranges[count++] = (struct checked_range){ "input", record.input_offset,
							  outer_values / record.pairs_per_row * EXL3_HALF_BYTES };
	if (pass <= BB_EXL3_DOWN_PASS)
		ranges[count++] = (struct checked_range){
			"operands", record.operands_offset,
			(pass <= BB_EXL3_GATE_UP_PASS ? outer_values * EXL3_PROJECTIONS : inner_values) * EXL3_HALF_BYTES
		};
	if (pass >= BB_EXL3_GATE_UP_PASS)
		ranges[count++] = (struct checked_range){
			"products", record.products_offset,
			(pass <= BB_EXL3_ACTIVATE_PASS ? inner_values * EXL3_PROJECTIONS : outer_values) * 4u
		};
	if (pass == BB_EXL3_ACTIVATE_PASS)
		ranges[count++] = (struct checked_range){ "hidden", record.hidden_offset, inner_values * EXL3_HALF_BYTES };
	if (!prepare_ranges_are_valid("EXL3 pass", ranges, count, description->arena_bytes))
		return STATUS_INVALID_ARGUMENT;
	const uint32_t bits_x2 = exl3_bits_x2(record.bits_per_weight);
	const char *const width = exl3_width_name(bits_x2);
	char gate_up[64], down[64];
	if (width == NULL || snprintf(gate_up, sizeof(gate_up), "exl3_gate_up_%s", width) <= 0 ||
	    snprintf(down, sizeof(down), "exl3_down_%s", width) <= 0)
		return STATUS_INVALID_ARGUMENT;
	const char *const names[BB_EXL3_PASSES] = { "exl3_input", gate_up, "bb_exl3_activate_output_shard", down,
						    "exl3_finish" };
	const bool activation = pass == BB_EXL3_ACTIVATE_PASS;
	const bool product = pass == BB_EXL3_GATE_UP_PASS || pass == BB_EXL3_DOWN_PASS;
	const uint32_t argument_bytes =
		activation ? (uint32_t)sizeof(struct bb_exl3_shard_activation_record) : (uint32_t)sizeof(record);
	uint32_t kernel = BACKEND_NO_KERNEL;
	const result_status status = backend->kernel_prepare(card, EXL3_KERNEL_FILE, names[pass], argument_bytes, &kernel);
	if (status != STATUS_OK)
		return status;
	if (kernel == BACKEND_NO_KERNEL)
		return STATUS_UNSUPPORTED;
	const uint32_t width_of_pass = pass == BB_EXL3_GATE_UP_PASS || activation ? record.inner_size : record.input_size;
	const uint32_t grid_x = product ? width_of_pass / EXL3_TRANSFORM :
					  (width_of_pass / EXL3_TRANSFORM + EXL3_TRANSFORM_WARPS - 1u) / EXL3_TRANSFORM_WARPS;
	const uint32_t grid_z = pass <= BB_EXL3_GATE_UP_PASS ? EXL3_PROJECTIONS : 1u;
	if (activation) {
		const struct bb_exl3_shard_activation_record arguments = { .base = record,
									   .down_input_size = plan.down.input_count,
									   .down_output_size = plan.down.output_count,
									   .down_input_begin = plan.gate_up.output_begin };
		prepare_launch_fill(launch_out, kernel, grid_x, record.job_count, grid_z, EXL3_TRANSFORM_THREADS, 0,
				    &arguments, sizeof(arguments));
	} else {
		prepare_launch_fill(launch_out, kernel, grid_x, record.job_count, grid_z,
				    product ? EXL3_PRODUCT_THREADS : EXL3_TRANSFORM_THREADS,
				    product ? exl3_product_dynamic_bytes(bits_x2) : 0u, &record, sizeof(record));
	}
	return STATUS_OK;
}

result_status bb_exl3_row_sum_prepare(const struct expert_row_sum_arguments *record, uint32_t rows,
				      uint64_t arena_bytes, const struct backend_operations *backend,
				      struct device_card *card, struct kernel_launch *launch_out)
{
	if (record == NULL || backend == NULL || backend->kernel_prepare == NULL || card == NULL || launch_out == NULL ||
	    rows == 0 || rows > MAXIMUM_GRID_ROWS || record->width == 0 || record->pairs_per_row == 0 ||
	    record->width % 4u != 0)
		return STATUS_INVALID_ARGUMENT;
	const uint64_t row_values = (uint64_t)rows * record->width;
	if (row_values > UINT64_MAX / 4u / record->pairs_per_row)
		return STATUS_INVALID_ARGUMENT;
	const struct checked_range ranges[2] = { { "pair outputs", record->pair_output_offset,
						   row_values * record->pairs_per_row * 4u },
						 { "row sums", record->row_output_offset, row_values * 4u } };
	if (!prepare_ranges_are_valid("EXL3 row sum", ranges, 2, arena_bytes))
		return STATUS_INVALID_ARGUMENT;
	uint32_t kernel = BACKEND_NO_KERNEL;
	const result_status status =
		backend->kernel_prepare(card, EXL3_KERNEL_FILE, EXL3_ROW_SUM, sizeof(*record), &kernel);
	if (status != STATUS_OK)
		return status;
	if (kernel == BACKEND_NO_KERNEL)
		return STATUS_UNSUPPORTED;
	prepare_launch_fill(launch_out, kernel, (record->width + EXL3_ROW_SUM_THREADS - 1u) / EXL3_ROW_SUM_THREADS, rows,
			    1, EXL3_ROW_SUM_THREADS, 0, record, sizeof(*record));
	return STATUS_OK;
}
