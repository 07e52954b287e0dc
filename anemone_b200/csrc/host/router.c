/* router.c: preparation of router_select_b200 (anemone_b200_router.h). */
#include "anemone_b200_router.h"

#include <math.h>
#include <stddef.h>

#include "prepare_common.h"

uint32_t router_b200_job_capacity(uint32_t rows, uint32_t picks, uint32_t shared_count)
{
	return rows * picks + shared_count * ((rows + LINEAR_MAXIMUM_ROWS - 1u) / LINEAR_MAXIMUM_ROWS);
}

result_status router_select_b200_prepare(const struct router_select_b200_arguments *arguments,
					 uint64_t arena_byte_count, const struct backend_operations *backend,
					 struct device_card *card, struct kernel_launch *launch_out)
{
	if (arguments == NULL || backend == NULL || backend->kernel_prepare == NULL || card == NULL ||
	    launch_out == NULL || arguments->reserved_zero != 0 || arguments->expert_count == 0 ||
	    arguments->expert_count + arguments->shared_count > ROUTER_B200_MAXIMUM_EXPERTS ||
	    arguments->expert_count + arguments->shared_count < arguments->expert_count || arguments->picks == 0 ||
	    arguments->picks > ROUTER_B200_MAXIMUM_PICKS || arguments->picks > arguments->expert_count ||
	    arguments->row_capacity == 0 || arguments->row_capacity > ROUTER_B200_MAXIMUM_ROWS ||
	    arguments->scoring > ROUTER_SCORING_SQRT_SOFTPLUS || !isfinite(arguments->route_scale) ||
	    arguments->route_scale <= 0 ||
	    arguments->job_capacity <
		    router_b200_job_capacity(arguments->row_capacity, arguments->picks, arguments->shared_count))
		return STATUS_INVALID_ARGUMENT;
	const uint64_t rows = arguments->row_capacity;
	const struct checked_range ranges[7] = {
		{ "bias", arguments->bias_offset, arguments->bias_offset != 0 ? (uint64_t)arguments->expert_count * 4u : 0u },
		{ "scores", arguments->scores_offset, rows * arguments->expert_count * 4u },
		{ "expert table", arguments->expert_table_offset,
		  (uint64_t)(arguments->expert_count + arguments->shared_count) * 24u },
		{ "picks", arguments->picks_offset, rows * arguments->picks * 4u },
		{ "weights", arguments->weights_offset, rows * arguments->picks * 4u },
		{ "jobs", arguments->jobs_offset, (uint64_t)arguments->job_capacity * sizeof(struct expert_job_record) },
		{ "step block", arguments->step_offset, sizeof(struct step_block) }
	};
	if (!prepare_ranges_are_valid("router select", ranges, 7, arena_byte_count))
		return STATUS_INVALID_ARGUMENT;
	uint32_t kernel = BACKEND_NO_KERNEL;
	const result_status status = backend->kernel_prepare(card, KERNEL_FILE_ROUTER_B200, KERNEL_ROUTER_SELECT_B200,
							     sizeof(*arguments), &kernel);
	if (status != STATUS_OK)
		return status;
	prepare_launch_fill(launch_out, kernel, 1, 1, 1, ROUTER_B200_THREADS, 0, arguments, sizeof(*arguments));
	return STATUS_OK;
}

/* router_select_b200 and the quantizer of the step's rows in one launch: both records as their own preparers accept
 * them (the quantizer's as linear_quantize_prepare writes it, handed over with that launch). */
result_status router_select_quantize_prepare(const struct router_select_b200_arguments *router,
					     const struct kernel_launch *quantize_launch, uint64_t arena_byte_count,
					     const struct backend_operations *backend, struct device_card *card,
					     struct kernel_launch *launch_out)
{
	struct kernel_launch checked;
	if (quantize_launch == NULL || quantize_launch->argument_byte_count != sizeof(struct activation_quantize_arguments) ||
	    quantize_launch->block[0] != 32u || quantize_launch->grid[0] == 0 || quantize_launch->grid[1] == 0)
		return STATUS_INVALID_ARGUMENT;
	const result_status valid = router_select_b200_prepare(router, arena_byte_count, backend, card, &checked);
	if (valid != STATUS_OK)
		return valid;
	struct router_select_quantize_arguments arguments = { .router = *router,
							       .vector_count = quantize_launch->grid[1],
							       .reserved_zero = 0 };
	memcpy(&arguments.quantize, quantize_launch->argument, sizeof(arguments.quantize));
	if (arguments.quantize.width == 0 || arguments.quantize.width % 64u != 0 ||
	    arguments.quantize.width / 64u != quantize_launch->grid[0] || arguments.quantize.reserved_zero != 0)
		return STATUS_INVALID_ARGUMENT;
	uint32_t kernel = BACKEND_NO_KERNEL;
	const result_status status = backend->kernel_prepare(card, KERNEL_FILE_ROUTER_B200, KERNEL_ROUTER_SELECT_QUANTIZE,
							     sizeof(arguments), &kernel);
	if (status != STATUS_OK)
		return status;
	if (kernel == BACKEND_NO_KERNEL)
		return STATUS_UNSUPPORTED;
	const uint64_t tasks = (uint64_t)arguments.vector_count * (arguments.quantize.width / 64u);
	const uint64_t warps = ROUTER_B200_THREADS / 32u;
	uint64_t blocks = (tasks + warps - 1u) / warps;
	if (blocks > 1024u)
		blocks = 1024u; /* the warps walk the rest */
	prepare_launch_fill(launch_out, kernel, 1u + (uint32_t)blocks, 1, 1, ROUTER_B200_THREADS, 0, &arguments,
			    sizeof(arguments));
	return STATUS_OK;
}

result_status router_wide_prepare(const struct router_wide_arguments *arguments, uint64_t arena_byte_count,
				  const struct backend_operations *backend, struct device_card *card,
				  struct kernel_launch *launches_out)
{
	if (arguments == NULL || backend == NULL || backend->kernel_prepare == NULL || card == NULL || launches_out == NULL)
		return STATUS_INVALID_ARGUMENT;
	const struct exl3_prefill_record *const routing = &arguments->routing;
	const uint64_t rows = routing->row_capacity;
	if (arguments->reserved_zero != 0 || routing->expert_count == 0 ||
	    routing->expert_count > ROUTER_B200_MAXIMUM_EXPERTS || routing->local_first != 0 ||
	    routing->local_count != routing->expert_count || routing->shared_count != 0 || routing->picks == 0 ||
	    routing->picks > ROUTER_B200_MAXIMUM_PICKS || routing->picks > routing->expert_count || rows == 0 ||
	    rows > 65535u || routing->scoring > ROUTER_SCORING_SQRT_SOFTPLUS || !isfinite(routing->route_scale) ||
	    routing->route_scale <= 0 || routing->workspace_offset % 1024u != 0 ||
	    arguments->job_capacity < rows * routing->picks / LINEAR_MAXIMUM_ROWS + routing->expert_count)
		return STATUS_INVALID_ARGUMENT;
	const struct exl3_prefill_parts parts = exl3_prefill_parts_of(routing->row_capacity, routing->picks, 0,
								      routing->expert_count, routing->input_size,
								      routing->inner_size);
	const struct checked_range ranges[8] = {
		{ "bias", routing->bias_offset, routing->bias_offset != 0 ? (uint64_t)routing->expert_count * 4u : 0u },
		{ "scores", routing->scores_offset, rows * routing->expert_count * 4u },
		{ "expert table", routing->expert_table_offset, (uint64_t)routing->expert_count * 24u },
		{ "picks", routing->picks_offset, rows * routing->picks * 4u },
		{ "weights", routing->weights_offset, rows * routing->picks * 4u },
		{ "workspace", routing->workspace_offset, parts.gate_up_operands },
		{ "jobs", arguments->jobs_offset, (uint64_t)arguments->job_capacity * sizeof(struct expert_job_record) },
		{ "step block", routing->step_offset, sizeof(struct step_block) }
	};
	if (!prepare_ranges_are_valid("router wide", ranges, 8, arena_byte_count))
		return STATUS_INVALID_ARGUMENT;
	const uint32_t row_warps = ROUTER_B200_THREADS / 32u;
	const struct {
		const char *file, *name;
		const void *record;
		uint32_t bytes, blocks, threads;
	} shapes[ROUTER_WIDE_LAUNCHES] = {
		{ EXL3_PREFILL_KERNEL_FILE, "exl3_prefill_picks", routing, sizeof(*routing),
		  (routing->row_capacity + row_warps - 1u) / row_warps, ROUTER_B200_THREADS },
		{ EXL3_PREFILL_KERNEL_FILE, "exl3_prefill_group", routing, sizeof(*routing), routing->expert_count, 256u },
		{ KERNEL_FILE_ROUTER_B200, KERNEL_ROUTER_WIDE_JOBS, arguments, sizeof(*arguments), 1u, ROUTER_B200_THREADS }
	};
	struct kernel_launch launches[ROUTER_WIDE_LAUNCHES];
	for (uint32_t index = 0; index < ROUTER_WIDE_LAUNCHES; index++) {
		uint32_t kernel = BACKEND_NO_KERNEL;
		const result_status status =
			backend->kernel_prepare(card, shapes[index].file, shapes[index].name, shapes[index].bytes, &kernel);
		if (status != STATUS_OK)
			return status;
		if (kernel == BACKEND_NO_KERNEL)
			return STATUS_UNSUPPORTED;
		prepare_launch_fill(&launches[index], kernel, shapes[index].blocks, 1, 1, shapes[index].threads, 0,
				    shapes[index].record, shapes[index].bytes);
	}
	memcpy(launches_out, launches, sizeof(launches));
	return STATUS_OK;
}

result_status step_input_select_prepare(const struct step_input_select_arguments *arguments, uint64_t arena_byte_count,
					const struct backend_operations *backend, struct device_card *card,
					struct kernel_launch *launch_out)
{
	if (arguments == NULL || backend == NULL || backend->kernel_prepare == NULL || card == NULL ||
	    launch_out == NULL || arguments->pool_count == 0 || arguments->byte_count == 0 ||
	    arguments->byte_count % 16u != 0 || arguments->byte_count > arguments->pool_stride ||
	    arguments->pool_stride % 16u != 0 || arguments->pool_stride > UINT64_MAX / arguments->pool_count)
		return STATUS_INVALID_ARGUMENT;
	const struct checked_range ranges[3] = {
		{ "step pool", arguments->pool_offset, arguments->pool_stride * arguments->pool_count },
		{ "step input area", arguments->destination_offset, arguments->byte_count },
		{ "cursor", arguments->cursor_offset, 16u }
	};
	if (!prepare_ranges_are_valid("step input select", ranges, 3, arena_byte_count))
		return STATUS_INVALID_ARGUMENT;
	uint32_t kernel = BACKEND_NO_KERNEL;
	const result_status status = backend->kernel_prepare(card, KERNEL_FILE_ROUTER_B200, KERNEL_STEP_INPUT_SELECT,
							     sizeof(*arguments), &kernel);
	if (status != STATUS_OK)
		return status;
	prepare_launch_fill(launch_out, kernel, 1, 1, 1, ROUTER_B200_THREADS, 0, arguments, sizeof(*arguments));
	return STATUS_OK;
}
