/*
 * exl3_layout.c: load-time EXL3 slices for tensor parallelism: sizes, the lossless host copy, and the two shard plans.
 * Takes the place of the reference's source/exl3_layout.c; rank counts 1, 2, 4 and 8 instead of 1 and 4.
 */
#include "anemone_b200_exl3.h"

#include <string.h>

static bool whole_blocks(uint32_t value)
{
	return value % EXL3_TRANSFORM == 0;
}

result_status bb_exl3_matrix_slice_prepare(const struct bb_exl3_matrix_slice *slice,
					   struct bb_exl3_slice_sizes *sizes_out)
{
	if (slice == NULL || sizes_out == NULL || slice->reserved_zero != 0 || slice->input_count == 0 ||
	    slice->output_count == 0 || !whole_blocks(slice->input_size) || !whole_blocks(slice->output_size) ||
	    !whole_blocks(slice->input_begin) || !whole_blocks(slice->input_count) ||
	    !whole_blocks(slice->output_begin) || !whole_blocks(slice->output_count) ||
	    slice->input_begin > slice->input_size || slice->input_count > slice->input_size - slice->input_begin ||
	    slice->output_begin > slice->output_size ||
	    slice->output_count > slice->output_size - slice->output_begin ||
	    !exl3_width_supported(slice->bits_per_weight))
		return STATUS_INVALID_ARGUMENT;
	const uint32_t bits_x2 = exl3_bits_x2(slice->bits_per_weight);
	sizes_out->source_bytes = exl3_matrix_bytes(slice->input_size, slice->output_size, bits_x2);
	sizes_out->packed_bytes = exl3_matrix_bytes(slice->input_count, slice->output_count, bits_x2);
	return STATUS_OK;
}

result_status bb_exl3_matrix_slice_copy(const struct bb_exl3_matrix_slice *slice, const void *source,
					size_t source_bytes, void *destination, size_t destination_bytes)
{
	if (slice == NULL)
		return STATUS_INVALID_ARGUMENT;
	const struct bb_exl3_matrix_slice kept = *slice; /* the destination may hold the description */
	struct bb_exl3_slice_sizes sizes;
	if (source == NULL || destination == NULL || bb_exl3_matrix_slice_prepare(&kept, &sizes) != STATUS_OK ||
	    sizes.source_bytes > source_bytes || sizes.packed_bytes > destination_bytes)
		return STATUS_INVALID_ARGUMENT;
	const uintptr_t from = (uintptr_t)source, to = (uintptr_t)destination;
	if (source_bytes > UINTPTR_MAX - from || destination_bytes > UINTPTR_MAX - to ||
	    (from < to + destination_bytes && to < from + source_bytes))
		return STATUS_INVALID_ARGUMENT;
	const uint32_t bits_x2 = exl3_bits_x2(kept.bits_per_weight);
	const unsigned char *const bytes = source;
	unsigned char *cursor = destination;
	/* codes: of each kept tile row, the kept tiles are contiguous */
	const uint64_t row_bytes = exl3_code_bytes(EXL3_TILE, kept.output_size, bits_x2);
	const uint64_t kept_bytes = exl3_code_bytes(EXL3_TILE, kept.output_count, bits_x2);
	const unsigned char *row = bytes + (uint64_t)(kept.input_begin / EXL3_TILE) * row_bytes +
				   exl3_code_bytes(EXL3_TILE, kept.output_begin, bits_x2);
	for (uint32_t index = 0; index < kept.input_count / EXL3_TILE; index++, row += row_bytes, cursor += kept_bytes)
		memcpy(cursor, row, (size_t)kept_bytes);
	/* then the matching parts of suh and svh */
	const unsigned char *const scales = bytes + exl3_code_bytes(kept.input_size, kept.output_size, bits_x2);
	memcpy(cursor, scales + (uint64_t)kept.input_begin * EXL3_HALF_BYTES, (size_t)kept.input_count * EXL3_HALF_BYTES);
	cursor += (size_t)kept.input_count * EXL3_HALF_BYTES;
	memcpy(cursor, scales + ((uint64_t)kept.input_size + kept.output_begin) * EXL3_HALF_BYTES,
	       (size_t)kept.output_count * EXL3_HALF_BYTES);
	return STATUS_OK;
}

static bool ranks_taken(uint32_t rank_count)
{
	return rank_count == 1 || rank_count == 2 || rank_count == 4 || rank_count == 8;
}

/* blocks [blocks r / R, blocks (r + 1) / R) of 128 */
static void rank_blocks(uint32_t size, uint32_t rank_count, uint32_t rank, uint32_t *begin_out, uint32_t *count_out)
{
	const uint32_t blocks = size / EXL3_TRANSFORM;
	*begin_out = blocks * rank / rank_count * EXL3_TRANSFORM;
	*count_out = blocks * (rank + 1u) / rank_count * EXL3_TRANSFORM - *begin_out;
}

static result_status plan_finish(const struct bb_exl3_output_shard_plan *plan,
				 struct bb_exl3_output_shard_plan *plan_out)
{
	struct bb_exl3_slice_sizes sizes;
	result_status status = bb_exl3_matrix_slice_prepare(&plan->gate_up, &sizes);
	if (status == STATUS_OK)
		status = bb_exl3_matrix_slice_prepare(&plan->down, &sizes);
	if (status == STATUS_OK)
		*plan_out = *plan;
	return status;
}

result_status bb_exl3_output_shard_prepare(uint32_t outer_size, uint32_t inner_size, uint32_t bits_per_weight,
					   uint32_t rank_count, uint32_t rank, enum bb_exl3_product_order order,
					   struct bb_exl3_output_shard_plan *plan_out)
{
	if (plan_out == NULL || !ranks_taken(rank_count) || rank >= rank_count ||
	    (order != BB_EXL3_REFERENCE_ORDER && order != BB_EXL3_EIGHT_PART_ORDER) || !whole_blocks(outer_size) ||
	    !whole_blocks(inner_size) || outer_size / EXL3_TRANSFORM < rank_count ||
	    inner_size / EXL3_TRANSFORM < rank_count)
		return STATUS_INVALID_ARGUMENT;
	uint32_t outer_begin, outer_count, inner_begin, inner_count;
	rank_blocks(outer_size, rank_count, rank, &outer_begin, &outer_count);
	rank_blocks(inner_size, rank_count, rank, &inner_begin, &inner_count);
	const struct bb_exl3_output_shard_plan plan = {
		.gate_up = { outer_size, inner_size, 0, outer_size, inner_begin, inner_count, bits_per_weight, 0 },
		.down = { inner_size, outer_size, 0, inner_size, outer_begin, outer_count, bits_per_weight, 0 },
		.rank_count = rank_count,
		.rank = rank,
		.product_slices = order == BB_EXL3_REFERENCE_ORDER ? 4u : 8u,
		.order = order
	};
	return plan_finish(&plan, plan_out);
}

result_status bb_exl3_inner_shard_prepare(uint32_t outer_size, uint32_t inner_size, uint32_t bits_per_weight,
					  uint32_t rank_count, uint32_t rank,
					  struct bb_exl3_output_shard_plan *plan_out)
{
	if (plan_out == NULL || !ranks_taken(rank_count) || rank >= rank_count || !whole_blocks(outer_size) ||
	    !whole_blocks(inner_size) || inner_size / EXL3_TRANSFORM < rank_count || outer_size == 0)
		return STATUS_INVALID_ARGUMENT;
	uint32_t inner_begin, inner_count;
	rank_blocks(inner_size, rank_count, rank, &inner_begin, &inner_count);
	const struct bb_exl3_output_shard_plan plan = {
		.gate_up = { outer_size, inner_size, 0, outer_size, inner_begin, inner_count, bits_per_weight, 0 },
		.down = { inner_size, outer_size, inner_begin, inner_count, 0, outer_size, bits_per_weight, 0 },
		.rank_count = rank_count,
		.rank = rank,
		.product_slices = 4u,
		.order = BB_EXL3_REFERENCE_ORDER
	};
	return plan_finish(&plan, plan_out);
}
