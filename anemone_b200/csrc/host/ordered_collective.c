/*
 * ordered_collective.c: preparation of the fixed-order reductions (anemone_b200_collective.h) and their host twin.
 * Takes the place of the reference's source/ordered_collective.c.
 */
#include "anemone_b200_collective.h"

#include <fenv.h>
#include <stddef.h>
#include <string.h>

#include "prepare_common.h"

#define VALUE_BYTES 4u
#define ADDRESS_BYTES 8u
#define STEP_BLOCK_BYTES 16u

static bool range_fits(uint64_t offset, uint64_t bytes, uint64_t capacity)
{
	return offset <= capacity && bytes <= capacity - offset;
}

static bool ranges_overlap(uint64_t first, uint64_t first_bytes, uint64_t second, uint64_t second_bytes)
{
	return first < second + second_bytes && second < first + first_bytes;
}

result_status ordered_collective_routes_prepare(const struct ordered_collective_route_description *description,
						uint32_t *host_reader_masks_out)
{
	if (description == NULL || host_reader_masks_out == NULL || description->direct_reader_masks == NULL ||
	    description->rank_count == 0 || description->rank_count > ORDERED_COLLECTIVE_MAXIMUM_RANKS ||
	    description->element_count == 0 || description->element_count > ORDERED_COLLECTIVE_MAXIMUM_ELEMENTS ||
	    (uint32_t)description->operation >= ORDERED_COLLECTIVE_OPERATIONS ||
	    (description->paired_scatter_gather && description->operation != ORDERED_REDUCE_SCATTER &&
	     description->operation != ORDERED_GATHER))
		return STATUS_INVALID_ARGUMENT;
	const uint32_t group = description->rank_count == 32u ? UINT32_MAX : (1u << description->rank_count) - 1u;
	uint32_t masks[ORDERED_COLLECTIVE_MAXIMUM_RANKS];
	for (uint32_t source = 0; source < description->rank_count; source++) {
		const uint32_t direct = description->direct_reader_masks[source];
		if ((direct & ~group) != 0 || (direct & (1u << source)) == 0)
			return STATUS_INVALID_ARGUMENT;
		masks[source] = group & ~direct;
	}
	memcpy(host_reader_masks_out, masks, description->rank_count * sizeof(masks[0]));
	return STATUS_OK;
}

result_status ordered_collective_kernels_prepare(const struct backend_operations *backend, struct device_card *card,
						 struct ordered_collective_kernels *kernels_out)
{
	static const char *const names[ORDERED_COLLECTIVE_OPERATIONS] = { KERNEL_ORDERED_ALL_REDUCE,
									 KERNEL_ORDERED_TWO_SHOT,
									 KERNEL_ORDERED_REDUCE_SCATTER,
									 KERNEL_ORDERED_GATHER };
	if (backend == NULL || backend->kernel_prepare == NULL || card == NULL || kernels_out == NULL)
		return STATUS_INVALID_ARGUMENT;
	struct ordered_collective_kernels prepared;
	for (uint32_t operation = 0; operation < ORDERED_COLLECTIVE_OPERATIONS; operation++) {
		const result_status status =
			backend->kernel_prepare(card, KERNEL_FILE_ORDERED_COLLECTIVE, names[operation],
						sizeof(struct ordered_collective_arguments), &prepared.handles[operation]);
		if (status != STATUS_OK)
			return status;
	}
	*kernels_out = prepared;
	return STATUS_OK;
}

result_status ordered_collective_host(const float *const *inputs, float *const *outputs, uint32_t rank_count,
				      uint32_t element_count, enum ordered_collective_operation operation)
{
	if (inputs == NULL || outputs == NULL || rank_count == 0 || rank_count > ORDERED_COLLECTIVE_MAXIMUM_RANKS ||
	    element_count == 0 || element_count > ORDERED_COLLECTIVE_MAXIMUM_ELEMENTS ||
	    (uint32_t)operation >= ORDERED_COLLECTIVE_OPERATIONS || fegetround() != FE_TONEAREST)
		return STATUS_INVALID_ARGUMENT;
	const uint64_t bytes = (uint64_t)element_count * VALUE_BYTES;
	for (uint32_t rank = 0; rank < rank_count; rank++) {
		const uint64_t in = (uint64_t)(uintptr_t)inputs[rank], out = (uint64_t)(uintptr_t)outputs[rank];
		if (inputs[rank] == NULL || outputs[rank] == NULL || in % VALUE_BYTES != 0 || out % VALUE_BYTES != 0 ||
		    in > UINT64_MAX - bytes || out > UINT64_MAX - bytes)
			return STATUS_INVALID_ARGUMENT;
	}
	for (uint32_t rank = 0; rank < rank_count; rank++)
		for (uint32_t other = 0; other < rank_count; other++)
			if (ranges_overlap((uint64_t)(uintptr_t)outputs[rank], bytes, (uint64_t)(uintptr_t)inputs[other],
					   bytes) ||
			    (other != rank && ranges_overlap((uint64_t)(uintptr_t)outputs[rank], bytes,
							     (uint64_t)(uintptr_t)outputs[other], bytes)))
				return STATUS_INVALID_ARGUMENT;
	const uint32_t slice = (element_count + rank_count - 1u) / rank_count;
	for (uint32_t element = 0; element < element_count; element++) {
		volatile float sum = 0.0f; /* one rounding per add, whatever the compiler's contraction settings */
		if (operation == ORDERED_GATHER)
			sum = inputs[element / slice][element];
		else
			for (uint32_t rank = 0; rank < rank_count; rank++)
				sum = sum + inputs[rank][element];
		if (operation == ORDERED_REDUCE_SCATTER)
			outputs[element / slice][element] = sum;
		else
			for (uint32_t rank = 0; rank < rank_count; rank++)
				outputs[rank][element] = sum;
	}
	return STATUS_OK;
}

/* The checks the FP32 collectives and the bfloat16 reduction share: ranks, region and slots, peer table, step block.
 * arrays: the offsets inside a parity slot (each `bytes` long), pairwise disjoint, behind the signal lines. */
static bool collective_is_valid(const struct ordered_collective_arguments *arguments, uint64_t capacity,
				const uint64_t *arrays, uint32_t array_count, uint64_t bytes, uint32_t maximum_elements)
{
	const uint64_t table_bytes = (uint64_t)arguments->rank_count * sizeof(struct ordered_collective_peer);
	if (arguments->element_count == 0 || arguments->element_count > maximum_elements ||
	    arguments->rank_count == 0 || arguments->rank_count > ORDERED_COLLECTIVE_MAXIMUM_RANKS ||
	    arguments->rank >= arguments->rank_count || arguments->reserved_zero != 0 ||
	    arguments->deadline_cycles == 0 || arguments->region_offset % ORDERED_COLLECTIVE_LINE_BYTES != 0 ||
	    arguments->parity_stride % ORDERED_COLLECTIVE_LINE_BYTES != 0 ||
	    arguments->parity_stride > UINT64_MAX / ORDERED_COLLECTIVE_SLOTS ||
	    !range_fits(arguments->region_offset, arguments->parity_stride * ORDERED_COLLECTIVE_SLOTS, capacity) ||
	    arguments->peer_table_offset % ADDRESS_BYTES != 0 || arguments->step_offset % ADDRESS_BYTES != 0 ||
	    !range_fits(arguments->peer_table_offset, table_bytes, capacity) ||
	    !range_fits(arguments->step_offset, STEP_BLOCK_BYTES, capacity))
		return false;
	for (uint32_t array = 0; array < array_count; array++) {
		if (arrays[array] < ORDERED_COLLECTIVE_SIGNAL_BYTES || arrays[array] % VALUE_BYTES != 0 ||
		    !range_fits(arrays[array], bytes, arguments->parity_stride))
			return false;
		for (uint32_t earlier = 0; earlier < array; earlier++)
			if (ranges_overlap(arrays[array], bytes, arrays[earlier], bytes))
				return false;
	}
	const uint64_t region_bytes = arguments->parity_stride * ORDERED_COLLECTIVE_SLOTS;
	return !ranges_overlap(arguments->peer_table_offset, table_bytes, arguments->region_offset, region_bytes) &&
	       !ranges_overlap(arguments->step_offset, STEP_BLOCK_BYTES, arguments->region_offset, region_bytes) &&
	       !ranges_overlap(arguments->step_offset, STEP_BLOCK_BYTES, arguments->peer_table_offset, table_bytes);
}

result_status ordered_collective_prepare(const struct ordered_collective_description *description,
					 const struct ordered_collective_kernels *kernels,
					 struct kernel_launch *launch_out)
{
	if (description == NULL || kernels == NULL || launch_out == NULL ||
	    (uint32_t)description->operation >= ORDERED_COLLECTIVE_OPERATIONS)
		return STATUS_INVALID_ARGUMENT;
	const struct ordered_collective_arguments *const arguments = &description->arguments;
	const uint64_t arrays[3] = { arguments->input_offset, arguments->output_offset, arguments->scratch_offset };
	if (!collective_is_valid(arguments, description->arena_byte_count, arrays, 3,
				 (uint64_t)arguments->element_count * VALUE_BYTES, ORDERED_COLLECTIVE_MAXIMUM_ELEMENTS))
		return STATUS_INVALID_ARGUMENT;
	prepare_launch_fill(launch_out, kernels->handles[description->operation], 1, 1, 1, ORDERED_COLLECTIVE_THREADS, 0,
			    arguments, sizeof(*arguments));
	return STATUS_OK;
}

result_status ordered_reduce_bf16_prepare(const struct ordered_reduce_bf16_description *description,
					  const struct backend_operations *backend, struct device_card *card,
					  struct kernel_launch *launches_out)
{
	if (description == NULL || backend == NULL || backend->kernel_prepare == NULL || card == NULL ||
	    launches_out == NULL)
		return STATUS_INVALID_ARGUMENT;
	const struct ordered_reduce_bf16_arguments *const reduce = &description->reduce;
	const struct ordered_collective_arguments *const collective = &reduce->collective;
	const uint64_t capacity = description->arena_byte_count;
	if (reduce->mode > ORDERED_REDUCE_OWNER_RUNS || reduce->width == 0 || reduce->width % 4u != 0 ||
	    description->row_capacity == 0 || description->row_capacity > 65535u || description->pairs_per_row == 0 ||
	    (uint64_t)description->row_capacity * reduce->width != collective->element_count)
		return STATUS_INVALID_ARGUMENT;
	const uint64_t input_bytes = (uint64_t)collective->element_count * VALUE_BYTES;
	if (!collective_is_valid(collective, capacity, &collective->input_offset, 1, input_bytes,
				 ORDERED_B200_MAXIMUM_ELEMENTS))
		return STATUS_INVALID_ARGUMENT;
	const uint64_t region_bytes = collective->parity_stride * ORDERED_COLLECTIVE_SLOTS;
	const struct checked_range ranges[5] = {
		{ "result", collective->output_offset, (uint64_t)collective->element_count * 2u },
		{ "status", reduce->status_offset, ORDERED_B200_STATUS_BYTES },
		{ "pair outputs", description->pair_output_offset, input_bytes * description->pairs_per_row },
		{ "region", collective->region_offset, region_bytes },
		{ "peer table", collective->peer_table_offset & ~(uint64_t)15u,
		  (uint64_t)collective->rank_count * sizeof(struct ordered_collective_peer) + 16u }
	};
	if (input_bytes > UINT64_MAX / description->pairs_per_row ||
	    !prepare_ranges_are_valid("ordered reduce", ranges, 5, capacity))
		return STATUS_INVALID_ARGUMENT;
	uint32_t publish = BACKEND_NO_KERNEL, sum = BACKEND_NO_KERNEL;
	result_status status = backend->kernel_prepare(card, KERNEL_FILE_ORDERED_B200, KERNEL_ORDERED_ROW_SUM_PUBLISH,
						       sizeof(struct ordered_row_sum_publish_arguments), &publish);
	if (status == STATUS_OK)
		status = backend->kernel_prepare(card, KERNEL_FILE_ORDERED_B200, KERNEL_ORDERED_REDUCE_BF16,
						 sizeof(*reduce), &sum);
	if (status != STATUS_OK)
		return status;
	const struct ordered_row_sum_publish_arguments publish_arguments = { .collective = *collective,
									      .pair_output_offset =
										      description->pair_output_offset,
									      .width = reduce->width,
									      .pairs_per_row = description->pairs_per_row,
									      .status_offset = reduce->status_offset };
	const uint32_t vectors = reduce->width / 4u;
	uint32_t blocks = (collective->element_count / 4u + ORDERED_COLLECTIVE_THREADS - 1u) / ORDERED_COLLECTIVE_THREADS;
	/* few rows: a small grid, whose last block is found quickly; many rows: enough blocks to fill the card */
	const uint32_t most = collective->element_count > ORDERED_COLLECTIVE_MAXIMUM_ELEMENTS ?
				      ORDERED_B200_MAXIMUM_BLOCKS_LARGE :
				      ORDERED_B200_MAXIMUM_BLOCKS;
	if (blocks > most)
		blocks = most;
	struct kernel_launch launches[ORDERED_REDUCE_BF16_LAUNCHES];
	prepare_launch_fill(&launches[0], publish, (vectors + 127u) / 128u,
			    description->row_capacity < ORDERED_B200_PUBLISH_ROW_BLOCKS ? description->row_capacity :
											  ORDERED_B200_PUBLISH_ROW_BLOCKS,
			    1, 128, 0, &publish_arguments, sizeof(publish_arguments));
	prepare_launch_fill(&launches[1], sum, blocks, 1, 1, ORDERED_COLLECTIVE_THREADS, 0, reduce, sizeof(*reduce));
	memcpy(launches_out, launches, sizeof(launches));
	return STATUS_OK;
}
