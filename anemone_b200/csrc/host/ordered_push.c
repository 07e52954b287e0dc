/*
 * ordered_push.c: preparation of the one-shot push all-reduce and of the tensor-parallel exchange built on it
 * (anemone_b200_collective.h). Takes the place of the reference's source/ordered_push.c and source/tp_exchange.c:
 * the same records, checks and refusals; the launch geometry is this library's.
 */
#include "anemone_b200_collective.h"

#include <stddef.h>
#include <string.h>

#include "prepare_common.h"

#define VALUE_BYTES 4u
#define WIRE_BF16_BYTES 2u
#define ADDRESS_BYTES 8u
#define STEP_BLOCK_BYTES 16u

static bool push_fits(uint64_t offset, uint64_t bytes, uint64_t capacity)
{
	return offset <= capacity && bytes <= capacity - offset;
}

static bool push_overlaps(uint64_t first, uint64_t first_bytes, uint64_t second, uint64_t second_bytes)
{
	return first < second + second_bytes && second < first + first_bytes;
}

result_status ordered_push_routes_prepare(const struct ordered_collective_route_description *description,
					  uint32_t *host_writer_masks_out)
{
	if (description == NULL || description->operation != ORDERED_ALL_REDUCE || description->paired_scatter_gather)
		return STATUS_INVALID_ARGUMENT;
	return ordered_collective_routes_prepare(description, host_writer_masks_out);
}

result_status ordered_push_kernel_prepare(const struct backend_operations *backend, struct device_card *card,
					  uint32_t *kernel_out)
{
	if (backend == NULL || backend->kernel_prepare == NULL || card == NULL || kernel_out == NULL)
		return STATUS_INVALID_ARGUMENT;
	return backend->kernel_prepare(card, KERNEL_FILE_ORDERED_PUSH, KERNEL_ORDERED_PUSH, ORDERED_PUSH_ARGUMENT_BYTES,
				       kernel_out);
}

/* what source/ordered_push.c:63-146 checks, in its order of concerns: scalars, region and tables, the arrays of a
 * slot behind the signal lines and disjoint (the inbox last; `slot_arrays` of input, output, inbox are in the slot),
 * region against table and step block */
static result_status push_is_valid(const struct ordered_push_description *description, uint32_t kernel,
				   uint32_t maximum_elements, uint32_t slot_arrays)
{
	if (description == NULL || kernel == BACKEND_NO_KERNEL || maximum_elements == 0)
		return STATUS_INVALID_ARGUMENT;
	const struct ordered_push_arguments *const a = &description->arguments;
	if (a->rank_count == 0 || a->rank_count > ORDERED_COLLECTIVE_MAXIMUM_RANKS || a->rank >= a->rank_count ||
	    a->element_count == 0 || a->element_count > maximum_elements || a->payload_format > ORDERED_PUSH_BF16 ||
	    a->reserved_zero != 0 || a->deadline_cycles == 0 ||
	    (a->incoming_host_mask & ~((1u << a->rank_count) - 1u)) != 0 || (a->incoming_host_mask & (1u << a->rank)) != 0)
		return STATUS_INVALID_ARGUMENT;
	const uint64_t capacity = description->arena_byte_count;
	const uint64_t signal_bytes = (uint64_t)ORDERED_PUSH_PHASES * a->rank_count * ORDERED_COLLECTIVE_LINE_BYTES;
	const uint64_t value_bytes = (uint64_t)a->element_count * VALUE_BYTES;
	const uint64_t wire_bytes =
		(uint64_t)a->element_count * (a->payload_format == ORDERED_PUSH_FP32 ? VALUE_BYTES : WIRE_BF16_BYTES);
	const uint64_t table_bytes = (uint64_t)a->rank_count * sizeof(struct ordered_collective_peer);
	if (a->region_offset % ORDERED_COLLECTIVE_LINE_BYTES != 0 || a->parity_stride % ORDERED_COLLECTIVE_LINE_BYTES != 0 ||
	    a->parity_stride > UINT64_MAX / ORDERED_COLLECTIVE_SLOTS ||
	    !push_fits(a->region_offset, a->parity_stride * ORDERED_COLLECTIVE_SLOTS, capacity) ||
	    a->peer_table_offset % ADDRESS_BYTES != 0 || a->step_offset % ADDRESS_BYTES != 0 ||
	    !push_fits(a->peer_table_offset, table_bytes, capacity) ||
	    !push_fits(a->step_offset, STEP_BLOCK_BYTES, capacity) || a->inbox_rank_stride < wire_bytes ||
	    a->inbox_rank_stride % VALUE_BYTES != 0 || a->inbox_rank_stride > UINT64_MAX / a->rank_count)
		return STATUS_INVALID_ARGUMENT;
	const uint64_t offsets[3] = { a->input_offset, a->output_offset, a->inbox_offset };
	const uint64_t sizes[3] = { value_bytes, value_bytes, a->inbox_rank_stride * a->rank_count };
	for (uint32_t array = 3u - slot_arrays; array < 3; array++) {
		if (offsets[array] < signal_bytes || offsets[array] % VALUE_BYTES != 0 ||
		    !push_fits(offsets[array], sizes[array], a->parity_stride))
			return STATUS_INVALID_ARGUMENT;
		for (uint32_t earlier = 3u - slot_arrays; earlier < array; earlier++)
			if (push_overlaps(offsets[array], sizes[array], offsets[earlier], sizes[earlier]))
				return STATUS_INVALID_ARGUMENT;
	}
	const uint64_t region_bytes = a->parity_stride * ORDERED_COLLECTIVE_SLOTS;
	if (push_overlaps(a->peer_table_offset, table_bytes, a->region_offset, region_bytes) ||
	    push_overlaps(a->step_offset, STEP_BLOCK_BYTES, a->region_offset, region_bytes) ||
	    push_overlaps(a->step_offset, STEP_BLOCK_BYTES, a->peer_table_offset, table_bytes))
		return STATUS_INVALID_ARGUMENT;
	/* a well-formed record that asks for a host mirror: the reference's PCIe cards have them, NVLink ranks do not */
	if (a->incoming_host_mask != 0)
		return STATUS_UNSUPPORTED;
	return STATUS_OK;
}

/* groups x blocks CTAs for a payload of this many elements: a CTA for every ORDERED_PUSH_BLOCK_VECTORS vectors,
 * spread over up to ORDERED_PUSH_GROUPS groups first */
static void push_grid(uint32_t element_count, uint32_t *groups_out, uint32_t *blocks_out)
{
	const uint32_t vectors = element_count / 4u + 1u;
	uint32_t total = (vectors + ORDERED_PUSH_BLOCK_VECTORS - 1u) / ORDERED_PUSH_BLOCK_VECTORS;
	if (total > ORDERED_PUSH_GROUPS * ORDERED_PUSH_GROUP_BLOCKS)
		total = ORDERED_PUSH_GROUPS * ORDERED_PUSH_GROUP_BLOCKS;
	*groups_out = total < ORDERED_PUSH_GROUPS ? total : ORDERED_PUSH_GROUPS;
	*blocks_out = (total + *groups_out - 1u) / *groups_out;
}

result_status ordered_push_prepare(const struct ordered_push_description *description, uint32_t kernel,
				   struct kernel_launch *launch_out)
{
	if (launch_out == NULL)
		return STATUS_INVALID_ARGUMENT;
	const result_status status = push_is_valid(description, kernel, ORDERED_COLLECTIVE_MAXIMUM_ELEMENTS, 3);
	if (status != STATUS_OK)
		return status;
	uint32_t groups, blocks;
	push_grid(description->arguments.element_count, &groups, &blocks);
	prepare_launch_fill(launch_out, kernel, groups, blocks, 1, ORDERED_COLLECTIVE_THREADS, 0, &description->arguments,
			    sizeof(description->arguments));
	return STATUS_OK;
}

/* ---- the exchange of a tensor-parallel layer site ---- */

result_status tp_exchange_kernel_prepare(const struct backend_operations *backend, struct device_card *card,
					 uint32_t *kernel_out)
{
	if (backend == NULL || backend->kernel_prepare == NULL || card == NULL || kernel_out == NULL)
		return STATUS_INVALID_ARGUMENT;
	return backend->kernel_prepare(card, KERNEL_FILE_TP_EXCHANGE, KERNEL_TP_EXCHANGE, TP_EXCHANGE_ARGUMENT_BYTES,
				       kernel_out);
}

result_status tp_exchange_rows_prepare(const struct ordered_push_description *description, uint32_t row_width,
				       uint32_t layer, uint32_t layer_count, uint32_t kernel,
				       struct kernel_launch *launch_out)
{
	if (description == NULL || launch_out == NULL || layer_count == 0 || layer_count > TP_EXCHANGE_MAXIMUM_PHASES ||
	    layer >= layer_count || row_width == 0 || row_width % 4u != 0 ||
	    description->arguments.element_count % row_width != 0)
		return STATUS_INVALID_ARGUMENT;
	const result_status status = push_is_valid(description, kernel, TP_EXCHANGE_MAXIMUM_ELEMENTS, 3);
	if (status != STATUS_OK)
		return status;
	const struct tp_exchange_arguments arguments = { description->arguments, layer, layer_count, row_width, 0 };
	uint32_t groups, blocks;
	push_grid(description->arguments.element_count, &groups, &blocks);
	prepare_launch_fill(launch_out, kernel, groups, blocks, 1, ORDERED_COLLECTIVE_THREADS, 0, &arguments,
			    sizeof(arguments));
	return STATUS_OK;
}

result_status tp_exchange_prepare(const struct ordered_push_description *description, uint32_t layer,
				  uint32_t layer_count, uint32_t kernel, struct kernel_launch *launch_out)
{
	return tp_exchange_rows_prepare(description, TP_EXCHANGE_REFERENCE_ROW_WIDTH, layer, layer_count, kernel,
					launch_out);
}

result_status tp_exchange_wide_kernels_prepare(const struct backend_operations *backend, struct device_card *card,
					       uint32_t form, uint32_t kernels_out[TP_EXCHANGE_WIDE_LAUNCHES])
{
	if (backend == NULL || backend->kernel_prepare == NULL || card == NULL || kernels_out == NULL ||
	    form > TP_EXCHANGE_FORM_CE_OWNER_RING_SUMS)
		return STATUS_INVALID_ARGUMENT;
	if (form > TP_EXCHANGE_FORM_OWNER_SUMS)
		return STATUS_UNSUPPORTED;
	const char *const names[TP_EXCHANGE_WIDE_LAUNCHES] = { form == TP_EXCHANGE_FORM_PUSH ? KERNEL_TP_EXCHANGE :
											       KERNEL_TP_EXCHANGE_OWNER,
							       KERNEL_TP_EXCHANGE_SETTLED, KERNEL_TP_EXCHANGE_SETTLED,
							       KERNEL_TP_EXCHANGE_SETTLED };
	uint32_t kernels[TP_EXCHANGE_WIDE_LAUNCHES];
	for (uint32_t index = 0; index < TP_EXCHANGE_WIDE_LAUNCHES; index++) {
		const result_status status = backend->kernel_prepare(card, KERNEL_FILE_TP_EXCHANGE, names[index],
								     TP_EXCHANGE_ARGUMENT_BYTES, &kernels[index]);
		if (status != STATUS_OK)
			return status;
	}
	memcpy(kernels_out, kernels, sizeof(kernels));
	return STATUS_OK;
}

result_status tp_exchange_wide_rows_prepare(const struct ordered_push_description *description, uint32_t row_width,
					    uint32_t layer, uint32_t layer_count,
					    const uint32_t kernels[TP_EXCHANGE_WIDE_LAUNCHES], uint32_t form,
					    struct kernel_launch launches_out[TP_EXCHANGE_WIDE_LAUNCHES])
{
	if (kernels == NULL || launches_out == NULL || description == NULL || form > TP_EXCHANGE_FORM_CE_OWNER_RING_SUMS)
		return STATUS_INVALID_ARGUMENT;
	const struct ordered_push_arguments *const a = &description->arguments;
	/* the reference's conditions on its forms (source/tp_exchange.c:101-120), before this library's answer that it
	 * runs only the first two */
	if ((form == TP_EXCHANGE_FORM_CE_OWNER_SUMS &&
	     (a->payload_format != ORDERED_PUSH_BF16 || a->rank_count == 0 || row_width == 0 ||
	      a->element_count % (a->rank_count * row_width) != 0)) ||
	    ((form == TP_EXCHANGE_FORM_OWNER_RING_SUMS || form == TP_EXCHANGE_FORM_CE_OWNER_RING_SUMS) &&
	     (a->rank_count != 4u || a->payload_format != ORDERED_PUSH_BF16)) ||
	    (form != TP_EXCHANGE_FORM_PUSH &&
	     (a->incoming_host_mask != 0 || (a->region_offset | a->input_offset | a->output_offset | a->inbox_offset |
					     a->inbox_rank_stride | a->parity_stride) %
						    TP_EXCHANGE_OWNER_ALIGNMENT !=
					    0)))
		return STATUS_INVALID_ARGUMENT;
	struct kernel_launch launches[TP_EXCHANGE_WIDE_LAUNCHES];
	for (uint32_t index = 0; index < TP_EXCHANGE_WIDE_LAUNCHES; index++) {
		const result_status status =
			tp_exchange_rows_prepare(description, row_width, layer, layer_count, kernels[index], &launches[index]);
		if (status != STATUS_OK)
			return status;
		if (index != 0) /* the settled launches: one small CTA each */
			launches[index].grid[0] = launches[index].grid[1] = 1, launches[index].block[0] = 32;
	}
	if (form > TP_EXCHANGE_FORM_OWNER_SUMS)
		return STATUS_UNSUPPORTED;
	memcpy(launches_out, launches, sizeof(launches));
	return STATUS_OK;
}

result_status tp_exchange_wide_prepare(const struct ordered_push_description *description, uint32_t layer,
				       uint32_t layer_count, const uint32_t kernels[TP_EXCHANGE_WIDE_LAUNCHES],
				       uint32_t form, struct kernel_launch launches_out[TP_EXCHANGE_WIDE_LAUNCHES])
{
	return tp_exchange_wide_rows_prepare(description, TP_EXCHANGE_REFERENCE_ROW_WIDTH, layer, layer_count, kernels,
					     form, launches_out);
}

/* ---- the expert layer's form: row sums pushed to every rank, added in rank order, one rounding to bfloat16 ---- */

result_status ordered_rows_push_prepare(const struct ordered_rows_push_description *description,
					const struct backend_operations *backend, struct device_card *card,
					struct kernel_launch *launch_out)
{
	if (description == NULL || backend == NULL || backend->kernel_prepare == NULL || card == NULL || launch_out == NULL)
		return STATUS_INVALID_ARGUMENT;
	const struct ordered_rows_push_arguments *const rows = &description->arguments;
	const struct ordered_push_arguments *const a = &rows->push;
	if (rows->width == 0 || rows->width % 4u != 0 || rows->pairs_per_row == 0 || a->element_count % rows->width != 0 ||
	    a->payload_format != ORDERED_PUSH_FP32 || a->input_offset != 0 ||
	    (a->output_offset | a->inbox_offset | a->inbox_rank_stride | rows->pair_output_offset) % 16u != 0)
		return STATUS_INVALID_ARGUMENT;
	const struct ordered_push_description push = { *a, description->arena_byte_count };
	result_status status = push_is_valid(&push, 0, ORDERED_B200_MAXIMUM_ELEMENTS, 1);
	if (status != STATUS_OK)
		return status;
	const uint64_t value_bytes = (uint64_t)a->element_count * VALUE_BYTES;
	if (value_bytes > UINT64_MAX / rows->pairs_per_row)
		return STATUS_INVALID_ARGUMENT;
	const struct checked_range ranges[4] = {
		{ "result", a->output_offset, (uint64_t)a->element_count * 2u },
		{ "pair outputs", rows->pair_output_offset, value_bytes * rows->pairs_per_row },
		{ "region", a->region_offset, a->parity_stride * ORDERED_COLLECTIVE_SLOTS },
		{ "peer table", a->peer_table_offset & ~(uint64_t)15u,
		  (uint64_t)a->rank_count * sizeof(struct ordered_collective_peer) + 16u }
	};
	if (!prepare_ranges_are_valid("ordered rows push", ranges, 4, description->arena_byte_count))
		return STATUS_INVALID_ARGUMENT;
	uint32_t kernel = BACKEND_NO_KERNEL;
	status = backend->kernel_prepare(card, KERNEL_FILE_ORDERED_B200, KERNEL_ORDERED_ROWS_PUSH, sizeof(*rows), &kernel);
	if (status != STATUS_OK)
		return status;
	uint32_t groups, blocks;
	push_grid(a->element_count, &groups, &blocks);
	prepare_launch_fill(launch_out, kernel, groups, blocks, 1, ORDERED_COLLECTIVE_THREADS, 0, rows, sizeof(*rows));
	return STATUS_OK;
}
