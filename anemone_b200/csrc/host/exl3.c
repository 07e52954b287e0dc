/*
 * exl3.c: EXL3 format sizes and the load-time preparation of the expert launches (anemone_b200_exl3.h).
 * Takes the place of the reference's source/exl3.c: same entry points, same validation and refusals, same records;
 * the kernels behind the names and therefore the launch shapes are this library's.
 */
#include "anemone_b200_exl3.h"

#include <math.h>
#include <stdio.h>
#include <string.h>

#include "../kernels/exl3_geometry.h"
#include "prepare_common.h"

#define EXL3_MAXIMUM_GRID_ROWS 65535u
#define EXL3_OPERAND_BYTES_PER_INPUT 4u /* FP16, gate and up */
#define EXL3_PRODUCT_BYTES_PER_INPUT 8u /* FP32, gate and up (inner <= input) */

static result_status exl3_stored_byte_count(const struct matrix_shape_record *shape, uint64_t *byte_count_out)
{
	if (shape == NULL || byte_count_out == NULL || shape->reserved_must_be_zero != 0 || shape->input_size == 0 ||
	    shape->output_size == 0 || shape->input_size % EXL3_TRANSFORM != 0 ||
	    shape->output_size % EXL3_TRANSFORM != 0 || exl3_bits_x2(shape->bits_per_weight) == 0)
		return STATUS_INVALID_ARGUMENT;
	if (!exl3_width_supported(shape->bits_per_weight))
		return STATUS_UNSUPPORTED;
	*byte_count_out = exl3_matrix_bytes(shape->input_size, shape->output_size, exl3_bits_x2(shape->bits_per_weight));
	return STATUS_OK;
}

const struct weight_format_operations exl3_weight_operations = { .name = "exl3_mul1",
								  .stored_byte_count = exl3_stored_byte_count };

const char *exl3_width_name(uint32_t bits_x2)
{
	switch (bits_x2) {
	case EXL3_BITS_X2_K2:
		return "k2";
	case EXL3_BITS_X2_K2_5:
		return "k2_5";
	case EXL3_BITS_X2_K3:
		return "k3";
	case EXL3_BITS_X2_K4:
		return "k4";
	default:
		return NULL;
	}
}

static bool range_inside(uint64_t offset, uint64_t bytes, uint64_t capacity)
{
	return offset <= capacity && bytes <= capacity - offset;
}

result_status exl3_reconstruct_prepare(const struct exl3_reconstruct_record *record, uint64_t arena_byte_count,
				       uint32_t kernel, struct kernel_launch *launch_out)
{
	if (record == NULL || launch_out == NULL || kernel == BACKEND_NO_KERNEL || record->reserved_zero != 0)
		return STATUS_INVALID_ARGUMENT;
	const struct matrix_shape_record shape = { record->output_size, record->input_size, record->bits_per_weight, 0 };
	uint64_t matrix_bytes = 0;
	if (exl3_stored_byte_count(&shape, &matrix_bytes) != STATUS_OK)
		return STATUS_INVALID_ARGUMENT;
	const uint64_t values = (uint64_t)record->input_size * record->output_size;
	const uint64_t output_bytes = values * EXL3_HALF_BYTES;
	if (record->matrix_offset % WEIGHT_FORMAT_MATRIX_ALIGNMENT_BYTES != 0 ||
	    record->output_offset % WEIGHT_FORMAT_MATRIX_ALIGNMENT_BYTES != 0 ||
	    !range_inside(record->matrix_offset, matrix_bytes, arena_byte_count) ||
	    !range_inside(record->output_offset, output_bytes, arena_byte_count) ||
	    (record->matrix_offset < record->output_offset + output_bytes &&
	     record->output_offset < record->matrix_offset + matrix_bytes) ||
	    values / EXL3_RECONSTRUCT_THREADS > UINT32_MAX)
		return STATUS_INVALID_ARGUMENT;
	prepare_launch_fill(launch_out, kernel,
			    (uint32_t)((values + EXL3_RECONSTRUCT_THREADS - 1u) / EXL3_RECONSTRUCT_THREADS), 1, 1,
			    EXL3_RECONSTRUCT_THREADS, 0, record, sizeof(*record));
	return STATUS_OK;
}

uint64_t exl3_scratch_byte_count(uint32_t pair_count, uint32_t input_size)
{
	const uint64_t values = (uint64_t)pair_count * input_size;
	const uint64_t per_input = EXL3_OPERAND_BYTES_PER_INPUT + EXL3_PRODUCT_BYTES_PER_INPUT;
	return values > UINT64_MAX / per_input ? UINT64_MAX : values * per_input;
}

/* What every chain shares: the record's own consistency and its five ranges. width_known: the record carries one
 * stored width (else widths come from a table and the widest supported shape is assumed for nothing: matrices are
 * placed by the router's table, which this function does not see). */
static result_status chain_validate(const char *what, const struct exl3_expert_record *record,
				    uint64_t arena_byte_count, bool width_known, const struct checked_range *extra,
				    uint32_t extra_count)
{
	if (record->reserved_zero != 0 || record->pair_count == 0 || record->pairs_per_row == 0 ||
	    record->pair_count % record->pairs_per_row != 0 || record->output_offset != record->products_offset ||
	    record->job_count == 0 || record->job_count > EXL3_MAXIMUM_GRID_ROWS ||
	    record->inner_size > record->input_size || !isfinite(record->activation_limit) ||
	    record->activation_limit <= 0)
		return STATUS_INVALID_ARGUMENT;
	const struct matrix_shape_record shape = { record->inner_size, record->input_size,
						   width_known ? record->bits_per_weight : EXL3_K4, 0 };
	uint64_t bytes = 0;
	if (exl3_stored_byte_count(&shape, &bytes) != STATUS_OK)
		return STATUS_INVALID_ARGUMENT;
	const uint64_t inputs = (uint64_t)record->pair_count * record->input_size;
	if (inputs > UINT64_MAX / (EXL3_OPERAND_BYTES_PER_INPUT + EXL3_PRODUCT_BYTES_PER_INPUT))
		return STATUS_INVALID_ARGUMENT;
	struct checked_range ranges[16] = {
		{ "jobs", record->jobs_offset, (uint64_t)record->job_count * sizeof(struct expert_job_record) },
		{ "input", record->input_offset, inputs / record->pairs_per_row * EXL3_HALF_BYTES },
		{ "operands", record->operands_offset, inputs * EXL3_OPERAND_BYTES_PER_INPUT },
		{ "products", record->products_offset, inputs * EXL3_PRODUCT_BYTES_PER_INPUT },
		{ "hidden", record->hidden_offset, (uint64_t)record->pair_count * record->inner_size * EXL3_HALF_BYTES }
	};
	uint32_t count = 5;
	for (uint32_t index = 0; index < extra_count; index++)
		ranges[count++] = extra[index];
	return prepare_ranges_are_valid(what, ranges, count, arena_byte_count) ? STATUS_OK : STATUS_INVALID_ARGUMENT;
}

static uint32_t transform_grid(uint32_t width)
{
	return (width / EXL3_TRANSFORM + EXL3_TRANSFORM_WARPS - 1u) / EXL3_TRANSFORM_WARPS;
}

static result_status class_check(uint32_t arithmetic_class)
{
	if (arithmetic_class == ARITHMETIC_CLASS_SM_100)
		return STATUS_OK;
	if (arithmetic_class == ARITHMETIC_CLASS_SM_80 || arithmetic_class == ARITHMETIC_CLASS_SM_120 ||
	    arithmetic_class == ARITHMETIC_CLASS_SM_120_NATIVE)
		return STATUS_UNSUPPORTED; /* the reference's classes: this library has no build for them */
	return STATUS_INVALID_ARGUMENT;
}

result_status exl3_experts_prepare(const struct exl3_expert_record *record, uint64_t arena_byte_count,
				   const struct backend_operations *backend, struct device_card *card,
				   uint32_t arithmetic_class, struct kernel_launch *launches_out)
{
	if (record == NULL || backend == NULL || card == NULL || launches_out == NULL ||
	    backend->kernel_prepare == NULL)
		return STATUS_INVALID_ARGUMENT;
	result_status status = class_check(arithmetic_class);
	if (status == STATUS_INVALID_ARGUMENT)
		return status;
	const result_status valid = chain_validate("EXL3 experts", record, arena_byte_count, true, NULL, 0);
	if (valid != STATUS_OK)
		return valid;
	if (status != STATUS_OK)
		return status;
	const uint32_t bits_x2 = exl3_bits_x2(record->bits_per_weight);
	const char *const width = exl3_width_name(bits_x2);
	char gate_up[64], down[64];
	if (width == NULL || snprintf(gate_up, sizeof(gate_up), "exl3_gate_up_%s", width) <= 0 ||
	    snprintf(down, sizeof(down), "exl3_down_%s", width) <= 0)
		return STATUS_INVALID_ARGUMENT;
	const char *const names[EXL3_EXPERT_LAUNCHES] = { "exl3_input", gate_up, "exl3_activate", down, "exl3_finish" };
	const uint32_t H = record->input_size, I = record->inner_size, jobs = record->job_count;
	const uint32_t shared = exl3_product_dynamic_bytes(bits_x2);
	const struct {
		uint32_t x, z, threads, shared;
	} shapes[EXL3_EXPERT_LAUNCHES] = { { transform_grid(H), EXL3_PROJECTIONS, EXL3_TRANSFORM_THREADS, 0 },
					   { I / EXL3_TRANSFORM, EXL3_PROJECTIONS, EXL3_PRODUCT_THREADS, shared },
					   { transform_grid(I), 1, EXL3_TRANSFORM_THREADS, 0 },
					   { H / EXL3_TRANSFORM, 1, EXL3_PRODUCT_THREADS, shared },
					   { transform_grid(H), 1, EXL3_TRANSFORM_THREADS, 0 } };
	struct kernel_launch launches[EXL3_EXPERT_LAUNCHES];
	for (uint32_t index = 0; index < EXL3_EXPERT_LAUNCHES; index++) {
		uint32_t kernel = BACKEND_NO_KERNEL;
		status = backend->kernel_prepare(card, EXL3_KERNEL_FILE, names[index], sizeof(*record), &kernel);
		if (status != STATUS_OK)
			return status;
		if (kernel == BACKEND_NO_KERNEL)
			return STATUS_UNSUPPORTED;
		prepare_launch_fill(&launches[index], kernel, shapes[index].x, jobs, shapes[index].z,
				    shapes[index].threads, shapes[index].shared, record, sizeof(*record));
	}
	memcpy(launches_out, launches, sizeof(launches));
	return STATUS_OK;
}

result_status exl3_experts_fast_prepare(const struct exl3_expert_record *record, uint64_t arena_byte_count,
					const struct backend_operations *backend, struct device_card *card,
					uint32_t arithmetic_class, struct kernel_launch *launches_out)
{
	return exl3_experts_prepare(record, arena_byte_count, backend, card, arithmetic_class, launches_out);
}

result_status exl3_experts_relaxed_prepare(const struct exl3_expert_record *record, uint64_t arena_byte_count,
					   const struct backend_operations *backend, struct device_card *card,
					   uint32_t arithmetic_class, struct kernel_launch *launches_out)
{
	if (record == NULL || backend == NULL || card == NULL || launches_out == NULL ||
	    backend->kernel_prepare == NULL || class_check(arithmetic_class) == STATUS_INVALID_ARGUMENT)
		return STATUS_INVALID_ARGUMENT;
	const result_status valid = chain_validate("EXL3 experts", record, arena_byte_count, true, NULL, 0);
	return valid != STATUS_OK ? valid : STATUS_UNSUPPORTED;
}

void exl3_moe_sizes(uint32_t pair_count, uint32_t job_count, uint32_t input_size, uint32_t inner_size,
		    struct exl3_moe_sizes *sizes_out)
{
	struct exl3_moe_sizes sizes = { 0, 0, 0, 0, 0 };
	if (sizes_out == NULL)
		return;
	if (input_size != 0 && inner_size != 0 && input_size % EXL3_TRANSFORM == 0 && inner_size % EXL3_TRANSFORM == 0) {
		sizes.gate_up_splits = exl3_moe_splits(input_size, inner_size);
		sizes.down_splits = exl3_moe_splits(inner_size, input_size);
		const uint64_t gate_up = (uint64_t)EXL3_PROJECTIONS * sizes.gate_up_splits * pair_count * inner_size * 4u;
		const uint64_t down = (uint64_t)sizes.down_splits * pair_count * input_size * 4u;
		sizes.product_bytes = gate_up > down ? gate_up : down;
		sizes.operand_bytes = (uint64_t)pair_count * input_size * EXL3_OPERAND_BYTES_PER_INPUT +
				      (uint64_t)pair_count * inner_size * EXL3_HALF_BYTES;
		sizes.counter_bytes = (uint64_t)job_count * (inner_size / EXL3_TRANSFORM + input_size / EXL3_TRANSFORM) * 4u;
	}
	*sizes_out = sizes;
}

result_status exl3_moe_prepare(const struct exl3_moe_record *record, uint64_t arena_byte_count,
			       const struct backend_operations *backend, struct device_card *card,
			       struct kernel_launch *launches_out)
{
	if (record == NULL || backend == NULL || card == NULL || launches_out == NULL ||
	    backend->kernel_prepare == NULL || record->reserved_zero != 0 || record->expert_count == 0)
		return STATUS_INVALID_ARGUMENT;
	const struct exl3_expert_record *const base = &record->base;
	const bool per_expert = base->bits_per_weight == EXL3_WIDTH_PER_EXPERT;
	const uint64_t rows = base->pairs_per_row == 0 ? 0 : base->pair_count / base->pairs_per_row;
	struct exl3_moe_sizes sizes;
	exl3_moe_sizes(base->pair_count, base->job_count, base->input_size, base->inner_size, &sizes);
	if (sizes.gate_up_splits == 0 || base->pair_count == 0 || base->input_size == 0)
		return STATUS_INVALID_ARGUMENT;
	/* the chain's own checks cover 4 pair_count input_size bytes of operands and 8 pair_count input_size bytes of
	 * products from the same offsets; what the fused launches use beyond that is checked as further ranges */
	const uint64_t chain_operands = (uint64_t)base->pair_count * base->input_size * EXL3_OPERAND_BYTES_PER_INPUT;
	const uint64_t chain_products = (uint64_t)base->pair_count * base->input_size * EXL3_PRODUCT_BYTES_PER_INPUT;
	if (base->operands_offset > UINT64_MAX - chain_operands || base->products_offset > UINT64_MAX - chain_products)
		return STATUS_INVALID_ARGUMENT;
	const struct checked_range extra[5] = {
		{ "row output", record->row_output_offset, rows * base->input_size * 4u },
		{ "width table", record->widths_offset, per_expert ? (uint64_t)record->expert_count * 4u : 0u },
		{ "down operands", base->operands_offset + chain_operands, sizes.operand_bytes - chain_operands },
		{ "split products", base->products_offset + chain_products,
		  sizes.product_bytes > chain_products ? sizes.product_bytes - chain_products : 0u },
		{ "counters", record->counters_offset, sizes.counter_bytes }
	};
	const result_status valid = chain_validate("EXL3 MoE", base, arena_byte_count, !per_expert, extra, 5);
	if (valid != STATUS_OK)
		return valid;
	static const char *const names[EXL3_MOE_LAUNCHES] = { "exl3_moe_input", "exl3_moe_gate_up", "exl3_moe_down",
							      "exl3_moe_row_sum" };
	const uint32_t H = base->input_size, I = base->inner_size, jobs = base->job_count;
	const uint32_t shared =
		exl3_product_dynamic_bytes(per_expert ? EXL3_BITS_X2_K4 : exl3_bits_x2(base->bits_per_weight));
	const struct {
		uint32_t x, y, z, threads, shared;
	} shapes[EXL3_MOE_LAUNCHES] = { { transform_grid(H), jobs, EXL3_PROJECTIONS, EXL3_TRANSFORM_THREADS, 0 },
					{ I / EXL3_TRANSFORM * sizes.gate_up_splits, jobs, EXL3_PROJECTIONS,
					  EXL3_PRODUCT_THREADS, shared },
					{ H / EXL3_TRANSFORM * sizes.down_splits, jobs, 1, EXL3_PRODUCT_THREADS, shared },
					{ (H + EXL3_ROW_SUM_THREADS - 1u) / EXL3_ROW_SUM_THREADS, (uint32_t)rows, 1,
					  EXL3_ROW_SUM_THREADS, 0 } };
	struct kernel_launch launches[EXL3_MOE_LAUNCHES];
	for (uint32_t index = 0; index < EXL3_MOE_LAUNCHES; index++) {
		uint32_t kernel = BACKEND_NO_KERNEL;
		const result_status status =
			backend->kernel_prepare(card, EXL3_MOE_KERNEL_FILE, names[index], sizeof(*record), &kernel);
		if (status != STATUS_OK)
			return status;
		if (kernel == BACKEND_NO_KERNEL)
			return STATUS_UNSUPPORTED;
		prepare_launch_fill(&launches[index], kernel, shapes[index].x, shapes[index].y, shapes[index].z,
				    shapes[index].threads, shapes[index].shared, record, sizeof(*record));
	}
	memcpy(launches_out, launches, sizeof(launches));
	return STATUS_OK;
}

void exl3_layer_sizes(uint32_t pair_count, uint32_t job_count, uint32_t input_size, uint32_t inner_size,
		      struct exl3_moe_sizes *sizes_out)
{
	struct exl3_moe_sizes sizes = { 0, 0, 0, 0, 0 };
	if (sizes_out == NULL)
		return;
	if (input_size != 0 && inner_size != 0 && input_size % EXL3_TRANSFORM == 0 && inner_size % EXL3_TRANSFORM == 0) {
		/* down's partial sums in a range of their own: the down launch may write while gate/up's are still read */
		const uint64_t gate_up = exl3_layer_gate_up_product_bytes(pair_count, inner_size);
		const uint64_t down = (uint64_t)EXL3_LAYER_MAXIMUM_RUNS * pair_count * input_size * 4u;
		sizes.product_bytes = gate_up + down;
		sizes.operand_bytes = (uint64_t)pair_count * input_size * EXL3_OPERAND_BYTES_PER_INPUT +
				      (uint64_t)pair_count * inner_size * EXL3_HALF_BYTES;
		sizes.counter_bytes = exl3_layer_counter_bytes(job_count, input_size, inner_size);
	}
	*sizes_out = sizes;
}

static bool layer_runs_are_valid(uint32_t runs, uint32_t blocks)
{
	return runs != 0 && runs <= EXL3_LAYER_MAXIMUM_RUNS && (runs & (runs - 1u)) == 0 && blocks % runs == 0;
}

result_status exl3_layer_prepare(const struct exl3_layer_description *description,
				 const struct backend_operations *backend, struct device_card *card,
				 struct kernel_launch *launches_out)
{
	if (description == NULL || backend == NULL || card == NULL || launches_out == NULL ||
	    backend->kernel_prepare == NULL)
		return STATUS_INVALID_ARGUMENT;
	const struct exl3_layer_route_record *const route = &description->route;
	const struct exl3_layer_publish_arguments *const publish = &description->publish;
	const struct exl3_moe_record *const moe = &route->moe;
	const struct exl3_expert_record *const base = &moe->base;
	const bool per_expert = base->bits_per_weight == EXL3_WIDTH_PER_EXPERT;
	const uint64_t capacity = description->arena_byte_count;
	const uint32_t H = base->input_size, I = base->inner_size, rows = route->row_capacity;
	const uint32_t slots = route->picks + route->shared_count;
	if (moe->reserved_zero != 0 || publish->reserved_zero != 0 || route->routed_count == 0 ||
	    route->routed_count + route->shared_count > ROUTER_B200_MAXIMUM_EXPERTS ||
	    route->routed_count + route->shared_count < route->routed_count || route->picks == 0 ||
	    route->picks > ROUTER_B200_MAXIMUM_PICKS || route->picks > route->routed_count || rows == 0 ||
	    rows > ROUTER_B200_MAXIMUM_ROWS || route->scoring > ROUTER_SCORING_SQRT_SOFTPLUS ||
	    !isfinite(route->route_scale) || route->route_scale <= 0 || base->pairs_per_row != slots ||
	    base->pair_count != rows * slots || moe->expert_count != route->routed_count + route->shared_count ||
	    base->job_count < rows * route->picks + route->shared_count * ((rows + LINEAR_MAXIMUM_ROWS - 1u) / LINEAR_MAXIMUM_ROWS) ||
	    publish->rank_count == 0 || publish->rank_count > ORDERED_COLLECTIVE_MAXIMUM_RANKS ||
	    publish->rank >= publish->rank_count || publish->row_capacity != rows || publish->deadline_cycles == 0 ||
	    publish->step_offset != route->step_offset || publish->input_offset < EXL3_LAYER_SIGNAL_BYTES ||
	    publish->input_offset % 16u != 0 || publish->parity_stride % ORDERED_COLLECTIVE_LINE_BYTES != 0 ||
	    publish->region_offset % ORDERED_COLLECTIVE_LINE_BYTES != 0 || H == 0 ||
	    publish->parity_stride < publish->input_offset + (uint64_t)rows * H * 4u || H % EXL3_TRANSFORM != 0 ||
	    I == 0 || I % EXL3_TRANSFORM != 0)
		return STATUS_INVALID_ARGUMENT;
	/* the cut of the products: the caller's, or the measured default of exl3_geometry.h */
	const uint32_t gate_up_runs =
		description->gate_up_runs != 0 ? description->gate_up_runs : exl3_layer_gate_up_runs(H, I);
	const uint32_t down_runs = description->down_runs != 0 ? description->down_runs : 1u;
	if (!layer_runs_are_valid(gate_up_runs, H / EXL3_TRANSFORM) || !layer_runs_are_valid(down_runs, I / EXL3_TRANSFORM))
		return STATUS_INVALID_ARGUMENT;
	struct exl3_moe_sizes sizes;
	exl3_layer_sizes(base->pair_count, base->job_count, H, I, &sizes);
	if (sizes.operand_bytes == 0)
		return STATUS_INVALID_ARGUMENT;
	const uint64_t chain_operands = (uint64_t)base->pair_count * H * EXL3_OPERAND_BYTES_PER_INPUT;
	const uint64_t chain_products = (uint64_t)base->pair_count * H * EXL3_PRODUCT_BYTES_PER_INPUT;
	if (base->operands_offset > UINT64_MAX - chain_operands || base->products_offset > UINT64_MAX - chain_products)
		return STATUS_INVALID_ARGUMENT;
	const struct checked_range extra[11] = {
		{ "width table", moe->widths_offset, per_expert ? (uint64_t)moe->expert_count * 4u : 0u },
		{ "down operands", base->operands_offset + chain_operands, sizes.operand_bytes - chain_operands },
		{ "run products", base->products_offset + chain_products,
		  sizes.product_bytes > chain_products ? sizes.product_bytes - chain_products : 0u },
		{ "counters", moe->counters_offset, sizes.counter_bytes },
		{ "scores", route->scores_offset, (uint64_t)rows * route->routed_count * 4u },
		{ "expert table", route->expert_table_offset, (uint64_t)moe->expert_count * 24u },
		{ "picks", route->picks_offset, (uint64_t)rows * route->picks * 4u },
		{ "weights", route->weights_offset, (uint64_t)rows * route->picks * 4u },
		{ "bias", route->bias_offset, route->bias_offset != 0 ? (uint64_t)route->routed_count * 4u : 0u },
		{ "step block", route->step_offset, sizeof(struct step_block) },
		{ "result", description->result_offset, (uint64_t)rows * H * 2u }
	};
	const result_status valid = chain_validate("EXL3 layer", base, capacity, !per_expert, extra, 11);
	if (valid != STATUS_OK)
		return valid;
	const struct checked_range reduction[3] = {
		{ "region", publish->region_offset, publish->parity_stride * ORDERED_COLLECTIVE_SLOTS },
		{ "status", publish->status_offset, ORDERED_B200_STATUS_BYTES },
		{ "peer table", publish->peer_table_offset,
		  (uint64_t)publish->rank_count * sizeof(struct ordered_collective_peer) }
	};
	if (!prepare_ranges_are_valid("EXL3 layer", reduction, 3, capacity))
		return STATUS_INVALID_ARGUMENT;
	const struct ordered_publish_reduce_arguments reduce = {
		.collective = { .peer_table_offset = publish->peer_table_offset,
				.region_offset = publish->region_offset,
				.input_offset = publish->input_offset,
				.output_offset = description->result_offset,
				.scratch_offset = 0,
				.step_offset = publish->step_offset,
				.parity_stride = publish->parity_stride,
				.deadline_cycles = publish->deadline_cycles,
				.element_count = rows * H,
				.rank_count = publish->rank_count,
				.rank = publish->rank,
				.reserved_zero = 0 },
		.status_offset = publish->status_offset,
		.pair_output_offset = base->output_offset + exl3_layer_gate_up_product_bytes(base->pair_count, I),
		.width = H,
		.pairs_per_row = slots
	};
	/* the products' record: down's partial sums and the pair outputs (run 0 of them) behind gate/up's */
	const struct exl3_layer_products_record products = {
		.moe = *moe,
		.down_products_offset = base->products_offset + exl3_layer_gate_up_product_bytes(base->pair_count, I),
		.gate_up_runs = gate_up_runs,
		.down_runs = down_runs
	};
	/* the transform's warp tasks: (pair, gate or up, 128 inputs); eight warps a CTA, a few tasks a warp */
	const uint64_t tasks = (uint64_t)rows * slots * EXL3_PROJECTIONS * (H / EXL3_TRANSFORM);
	/* a task is a chain of dependent loads (pick, table, scale, row): one a warp where the card holds that many
	 * CTAs, so that the launch lasts one such chain and not several */
	uint64_t transform_ctas = (tasks + EXL3_LAYER_ROUTE_THREADS / EXL3_WARP - 1u) / (EXL3_LAYER_ROUTE_THREADS / EXL3_WARP);
	if (transform_ctas > 2u * EXL3_LAYER_DEFAULT_SMS - 1u)
		transform_ctas = 2u * EXL3_LAYER_DEFAULT_SMS - 1u;
	uint32_t reduce_blocks = (rows * H / 4u + ORDERED_COLLECTIVE_THREADS - 1u) / ORDERED_COLLECTIVE_THREADS;
	if (reduce_blocks > ORDERED_B200_MAXIMUM_BLOCKS)
		reduce_blocks = ORDERED_B200_MAXIMUM_BLOCKS;
	const uint32_t shared = exl3_product_dynamic_bytes(EXL3_BITS_X2_K4);
	const struct {
		const char *file, *name;
		const void *record;
		uint32_t record_bytes, x, y, z, threads, shared;
	} shapes[EXL3_LAYER_LAUNCHES] = {
		{ EXL3_LAYER_KERNEL_FILE, "exl3_layer_route_input", route, sizeof(*route), 1u + (uint32_t)transform_ctas, 1, 1,
		  EXL3_LAYER_ROUTE_THREADS, 0 },
		{ EXL3_LAYER_KERNEL_FILE, "exl3_layer_products", &products, sizeof(products),
		  base->job_count * (EXL3_PROJECTIONS * (I / EXL3_TRANSFORM) * gate_up_runs + H / EXL3_TRANSFORM * down_runs), 1,
		  1, EXL3_PRODUCT_THREADS, shared },
		{ KERNEL_FILE_ORDERED_B200, KERNEL_ORDERED_PUBLISH_REDUCE_FLAGS, &reduce, sizeof(reduce), reduce_blocks, 1, 1,
		  ORDERED_COLLECTIVE_THREADS, 0 }
	};
	struct kernel_launch launches[EXL3_LAYER_LAUNCHES];
	for (uint32_t index = 0; index < EXL3_LAYER_LAUNCHES; index++) {
		uint32_t kernel = BACKEND_NO_KERNEL;
		const result_status status = backend->kernel_prepare(card, shapes[index].file, shapes[index].name,
								     shapes[index].record_bytes, &kernel);
		if (status != STATUS_OK)
			return status;
		if (kernel == BACKEND_NO_KERNEL)
			return STATUS_UNSUPPORTED;
		prepare_launch_fill(&launches[index], kernel, shapes[index].x, shapes[index].y, shapes[index].z,
				    shapes[index].threads, shapes[index].shared, shapes[index].record,
				    shapes[index].record_bytes);
	}
	/* Each launch may be given its place on the card while the one before it still runs: the products and the
	 * reduction wait for the whole launch before them as their first act. */
	for (uint32_t index = 1; index < EXL3_LAYER_LAUNCHES; index++)
		launches[index].branch = LAUNCH_CHAIN | LAUNCH_OVERLAPS_PREVIOUS;
	memcpy(launches_out, launches, sizeof(launches));
	return STATUS_OK;
}

result_status exl3_prefill_prepare(const struct exl3_prefill_record *record, uint64_t arena_byte_count,
				   const struct backend_operations *backend, struct device_card *card,
				   struct kernel_launch *launches_out)
{
	if (record == NULL || backend == NULL || card == NULL || launches_out == NULL ||
	    backend->kernel_prepare == NULL)
		return STATUS_INVALID_ARGUMENT;
	const uint32_t H = record->input_size, I = record->inner_size, shared_I = record->shared_inner_size;
	const uint32_t experts = record->local_count + record->shared_count;
	if (record->expert_count == 0 || record->expert_count > ROUTER_B200_MAXIMUM_EXPERTS ||
	    record->local_first > record->expert_count || record->local_count > record->expert_count - record->local_first ||
	    experts == 0 || record->shared_count > ROUTER_B200_THREADS - ROUTER_B200_MAXIMUM_EXPERTS ||
	    record->picks == 0 || record->picks > ROUTER_B200_MAXIMUM_PICKS || record->picks > record->expert_count ||
	    record->row_capacity == 0 || record->row_capacity > EXL3_MAXIMUM_GRID_ROWS || H == 0 ||
	    H % EXL3_TRANSFORM != 0 || I % EXL3_TRANSFORM != 0 || shared_I % EXL3_TRANSFORM != 0 ||
	    (record->local_count != 0) != (I != 0) || (record->shared_count != 0) != (shared_I != 0) ||
	    record->scoring > ROUTER_SCORING_SQRT_SOFTPLUS || !isfinite(record->route_scale) ||
	    !isfinite(record->activation_limit) || record->activation_limit <= 0)
		return STATUS_INVALID_ARGUMENT;
	const uint32_t widest = I > shared_I ? I : shared_I;
	const struct exl3_prefill_parts parts = exl3_prefill_parts_of(record->row_capacity, record->picks,
								      record->shared_count, record->local_count, H, widest);
	if (parts.tile_capacity > EXL3_MAXIMUM_GRID_ROWS)
		return STATUS_INVALID_ARGUMENT;
	const uint64_t rows = record->row_capacity, slots = record->picks + record->shared_count;
	const struct checked_range ranges[11] = {
		{ "bias", record->bias_offset, record->bias_offset != 0 ? (uint64_t)record->expert_count * 4u : 0u },
		{ "scores", record->scores_offset, rows * record->expert_count * 4u },
		{ "input", record->input_offset, rows * H * EXL3_HALF_BYTES },
		{ "expert table", record->expert_table_offset, (uint64_t)experts * 24u },
		{ "width table", record->widths_offset, (uint64_t)experts * 4u },
		{ "picks", record->picks_offset, rows * record->picks * 4u },
		{ "weights", record->weights_offset, rows * record->picks * 4u },
		{ "workspace", record->workspace_offset, parts.total },
		{ "pair outputs", record->pair_output_offset, rows * slots * H * 4u },
		{ "row outputs", record->row_output_offset, rows * H * 4u },
		{ "step", record->step_offset, sizeof(struct step_block) }
	};
	if (record->workspace_offset % 1024u != 0 ||
	    !prepare_ranges_are_valid("EXL3 prefill", ranges, 11, arena_byte_count))
		return STATUS_INVALID_ARGUMENT;
	static const char *const names[EXL3_PREFILL_LAUNCHES] = { "exl3_prefill_picks",	   "exl3_prefill_group",
								  "exl3_prefill_tiles",	   "exl3_prefill_operands",
								  "exl3_prefill_gate_up",  "exl3_prefill_down",
								  "exl3_prefill_row_sum" };
	const uint32_t row_warps = ROUTER_B200_THREADS / EXL3_WARP;
	const struct {
		uint32_t x, y, z, threads, shared;
	} shapes[EXL3_PREFILL_LAUNCHES] = {
		{ (record->row_capacity + row_warps - 1u) / row_warps, 1, 1, ROUTER_B200_THREADS, 0 },
		{ experts, 1, 1, 256u, 0 },
		{ 1, 1, 1, ROUTER_B200_THREADS, 0 },
		{ parts.tile_capacity, transform_grid(H) * EXL3_PREFILL_OPERAND_PARTS, EXL3_PROJECTIONS,
		  EXL3_TRANSFORM_THREADS, 0 },
		{ widest / EXL3_TRANSFORM, parts.tile_capacity, 1, EXL3_PREFILL_GEMM_THREADS, EXL3_PREFILL_DYNAMIC_BYTES },
		{ (H / EXL3_TRANSFORM + 1u) / 2u, parts.tile_capacity, 1, EXL3_PREFILL_GEMM_THREADS,
		  EXL3_PREFILL_DYNAMIC_BYTES },
		{ (H / 4u + EXL3_ROW_SUM_THREADS - 1u) / EXL3_ROW_SUM_THREADS, record->row_capacity, 1, EXL3_ROW_SUM_THREADS,
		  0 }
	};
	struct kernel_launch launches[EXL3_PREFILL_LAUNCHES];
	for (uint32_t index = 0; index < EXL3_PREFILL_LAUNCHES; index++) {
		uint32_t kernel = BACKEND_NO_KERNEL;
		const result_status status =
			backend->kernel_prepare(card, EXL3_PREFILL_KERNEL_FILE, names[index], sizeof(*record), &kernel);
		if (status != STATUS_OK)
			return status;
		if (kernel == BACKEND_NO_KERNEL)
			return STATUS_UNSUPPORTED;
		prepare_launch_fill(&launches[index], kernel, shapes[index].x, shapes[index].y, shapes[index].z,
				    shapes[index].threads, shapes[index].shared, record, sizeof(*record));
	}
	memcpy(launches_out, launches, sizeof(launches));
	return STATUS_OK;
}

void exl3_prefill_sizes(uint32_t row_capacity, uint32_t picks, uint32_t shared_count, uint32_t local_count,
			uint32_t input_size, uint32_t widest_inner_size, struct exl3_prefill_parts *parts_out)
{
	if (parts_out != NULL)
		*parts_out = exl3_prefill_parts_of(row_capacity, picks, shared_count, local_count, input_size,
						   widest_inner_size);
}
