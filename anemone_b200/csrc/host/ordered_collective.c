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

static bool policy_row_is_well_formed(const struct ordered_collective_route_policy *row)
{
	if (row->rank_count == 0 || row->rank_count > ORDERED_COLLECTIVE_MAXIMUM_RANKS || row->element_count == 0 ||
	    row->element_count > ORDERED_COLLECTIVE_MAXIMUM_ELEMENTS ||
	    (uint32_t)row->operation >= ORDERED_COLLECTIVE_OPERATIONS ||
	    (row->paired_scatter_gather && row->operation != ORDERED_REDUCE_SCATTER && row->operation != ORDERED_GATHER))
		return false;
	const uint32_t group = (1u << row->rank_count) - 1u;
	for (uint32_t source = 0; source < row->rank_count; source++) {
		const uint32_t direct = row->expected_direct_reader_masks[source], host = row->host_reader_masks[source];
		const uint32_t self = 1u << source;
		/* inside the group; a source reads itself directly and never through a mirror; whoever is denied direct
		 * access has a mirror */
		if (((direct | host) & ~group) != 0 || (direct & self) == 0 || (host & self) != 0 ||
		    (group & ~direct & ~host) != 0)
			return false;
	}
	return true;
}

static bool policy_rows_bind_alike(const struct ordered_collective_route_policy *first,
				   const struct ordered_collective_route_policy *second)
{
	for (uint32_t source = 0; source < first->rank_count; source++)
		if (first->host_reader_masks[source] != second->host_reader_masks[source] ||
		    first->expected_direct_reader_masks[source] != second->expected_direct_reader_masks[source] ||
		    first->arithmetic_classes[source] != second->arithmetic_classes[source] ||
		    first->link_generations[source] != second->link_generations[source] ||
		    first->link_lane_counts[source] != second->link_lane_counts[source])
			return false;
	return true;
}

result_status ordered_collective_routes_prepare_measured(const struct ordered_collective_route_description *description,
							 const struct ordered_collective_route_policy *rows,
							 uint32_t row_count, uint32_t *host_reader_masks_out)
{
	if (description == NULL || host_reader_masks_out == NULL || row_count > ORDERED_ROUTE_POLICY_MAXIMUM_ROWS ||
	    (row_count != 0 && rows == NULL))
		return STATUS_INVALID_ARGUMENT;
	/* what holds without a table: direct where qualified, a host mirror where denied */
	uint32_t masks[ORDERED_COLLECTIVE_MAXIMUM_RANKS];
	struct ordered_collective_route_description plain = *description;
	plain.common_numa_root = false;
	const result_status status = ordered_collective_routes_prepare(&plain, masks);
	if (status != STATUS_OK)
		return status;
	const struct ordered_collective_route_policy *match = NULL;
	for (uint32_t index = 0; index < row_count; index++) {
		const struct ordered_collective_route_policy *const row = &rows[index];
		if (!policy_row_is_well_formed(row))
			return STATUS_INVALID_ARGUMENT;
		for (uint32_t earlier = 0; earlier < index; earlier++) {
			const struct ordered_collective_route_policy *const other = &rows[earlier];
			if (other->rank_count != row->rank_count || other->element_count != row->element_count)
				continue;
			if (other->operation == row->operation && other->paired_scatter_gather == row->paired_scatter_gather)
				return STATUS_INVALID_ARGUMENT; /* one key twice */
			if (other->paired_scatter_gather && row->paired_scatter_gather && !policy_rows_bind_alike(other, row))
				return STATUS_INVALID_ARGUMENT; /* the two rows of a pair must be one plan */
		}
		if (row->rank_count == description->rank_count && row->element_count == description->element_count &&
		    row->operation == description->operation &&
		    row->paired_scatter_gather == description->paired_scatter_gather)
			match = row;
	}
	if (match != NULL)
		for (uint32_t source = 0; source < description->rank_count; source++) {
			const struct card_description_record *const card = &description->cards[source];
			if (match->expected_direct_reader_masks[source] != description->direct_reader_masks[source] ||
			    match->arithmetic_classes[source] != (uint32_t)card->arithmetic_class ||
			    match->link_generations[source] != card->link_generation ||
			    match->link_lane_counts[source] != card->link_lane_count)
				return STATUS_UNSUPPORTED; /* measured under another access pattern or on other cards */
			masks[source] = match->host_reader_masks[source];
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

/* One launch: ordered_publish_reduce_flags_bf16 (row sums of bfloat16 pair outputs, the optional bfloat16 addend, READY
 * and the reduction, with flags that arrive in the reader's own memory: the slot layout of the EXL3 layer's step). */
result_status ordered_publish_reduce_bf16_prepare(const struct ordered_reduce_bf16_description *description,
						  uint64_t addend_offset, uint64_t row_output_offset,
						  const struct backend_operations *backend, struct device_card *card,
						  struct kernel_launch *launch_out)
{
	if (description == NULL || backend == NULL || backend->kernel_prepare == NULL || card == NULL || launch_out == NULL)
		return STATUS_INVALID_ARGUMENT;
	const struct ordered_reduce_bf16_arguments *const reduce = &description->reduce;
	const struct ordered_collective_arguments *const collective = &reduce->collective;
	const uint64_t capacity = description->arena_byte_count;
	if (reduce->mode != ORDERED_REDUCE_EVERY_RANK || reduce->width == 0 || reduce->width % 4u != 0 ||
	    description->row_capacity == 0 || description->row_capacity > ORDERED_COLLECTIVE_MAXIMUM_ELEMENTS / 4u ||
	    description->pairs_per_row == 0 ||
	    (uint64_t)description->row_capacity * reduce->width != collective->element_count ||
	    collective->element_count > ORDERED_COLLECTIVE_MAXIMUM_ELEMENTS || collective->rank_count == 0 ||
	    collective->rank_count > ORDERED_COLLECTIVE_MAXIMUM_RANKS || collective->rank >= collective->rank_count ||
	    collective->reserved_zero != 0 || collective->scratch_offset != 0 || collective->deadline_cycles == 0 ||
	    collective->input_offset < EXL3_LAYER_SIGNAL_BYTES || collective->input_offset % 16u != 0 ||
	    collective->parity_stride % ORDERED_COLLECTIVE_LINE_BYTES != 0 ||
	    collective->region_offset % ORDERED_COLLECTIVE_LINE_BYTES != 0 ||
	    collective->parity_stride < collective->input_offset + (uint64_t)collective->element_count * VALUE_BYTES ||
	    collective->peer_table_offset % ADDRESS_BYTES != 0 || collective->step_offset % ADDRESS_BYTES != 0 ||
	    addend_offset % 16u != 0 || row_output_offset % 16u != 0 || description->pair_output_offset % 16u != 0)
		return STATUS_INVALID_ARGUMENT;
	const uint64_t elements = collective->element_count;
	const struct checked_range ranges[8] = {
		{ "result", collective->output_offset, elements * 2u },
		{ "status", reduce->status_offset, ORDERED_B200_STATUS_BYTES },
		{ "pair outputs", description->pair_output_offset, elements * 2u * description->pairs_per_row },
		{ "region", collective->region_offset, collective->parity_stride * ORDERED_COLLECTIVE_SLOTS },
		{ "peer table", collective->peer_table_offset,
		  (uint64_t)collective->rank_count * sizeof(struct ordered_collective_peer) },
		{ "step block", collective->step_offset, STEP_BLOCK_BYTES },
		{ "addend", addend_offset, addend_offset != 0 ? elements * 2u : 0u },
		{ "row output", row_output_offset, row_output_offset != 0 ? elements * 4u : 0u }
	};
	if (!prepare_ranges_are_valid("ordered publish and reduce", ranges, 8, capacity))
		return STATUS_INVALID_ARGUMENT;
	uint32_t kernel = BACKEND_NO_KERNEL;
	const result_status status = backend->kernel_prepare(card, KERNEL_FILE_ORDERED_B200,
							     KERNEL_ORDERED_PUBLISH_REDUCE_FLAGS_BF16,
							     sizeof(struct ordered_publish_reduce_bf16_arguments), &kernel);
	if (status != STATUS_OK)
		return status;
	if (kernel == BACKEND_NO_KERNEL)
		return STATUS_UNSUPPORTED;
	const struct ordered_publish_reduce_bf16_arguments arguments = {
		.base = { .collective = *collective,
			  .status_offset = reduce->status_offset,
			  .pair_output_offset = description->pair_output_offset,
			  .width = reduce->width,
			  .pairs_per_row = description->pairs_per_row },
		.addend_offset = addend_offset,
		.row_output_offset = row_output_offset
	};
	uint32_t blocks = ((uint32_t)(elements / 4u) + ORDERED_COLLECTIVE_THREADS - 1u) / ORDERED_COLLECTIVE_THREADS;
	if (blocks > ORDERED_B200_MAXIMUM_BLOCKS) /* the blocks wait for a word their own grid's last block stores */
		blocks = ORDERED_B200_MAXIMUM_BLOCKS;
	prepare_launch_fill(launch_out, kernel, blocks, 1, 1, ORDERED_COLLECTIVE_THREADS, 0, &arguments, sizeof(arguments));
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
