/*
 * tp2_join.c: preparation of the local completion launch (anemone_b200_collective.h). Takes the place of the
 * reference's source/tp2_join.c: the same description, checks, refusals and record.
 */
#include "anemone_b200_collective.h"

#include <stddef.h>

#include "prepare_common.h"

#define STEP_BLOCK_BYTES 16u
#define JOIN_RANGES_MOST 6u

result_status tp2_join_kernel_prepare(const struct backend_operations *backend, struct device_card *card,
				      uint32_t *kernel_out)
{
	if (backend == NULL || backend->kernel_prepare == NULL || card == NULL || kernel_out == NULL)
		return STATUS_INVALID_ARGUMENT;
	uint32_t kernel = BACKEND_NO_KERNEL;
	const result_status status =
		backend->kernel_prepare(card, KERNEL_FILE_TP2_JOIN, KERNEL_TP2_JOIN, TP2_JOIN_ARGUMENT_BYTES, &kernel);
	if (status == STATUS_OK)
		*kernel_out = kernel;
	return status;
}

/* bytes from a strided array's first element to the end of its last row */
static uint64_t join_span(uint32_t rows, uint32_t width, uint32_t stride, uint32_t element_bytes)
{
	return ((uint64_t)(rows - 1u) * stride + width) * element_bytes;
}

/* the planner's range holds what is touched, in the second parity slot too */
static bool join_range_holds(const struct tp2_join_range *range, uint64_t touched, uint64_t slot_stride, uint64_t arena)
{
	return range->byte_offset % LINEAR_OFFSET_ALIGNMENT_BYTES == 0 && slot_stride % LINEAR_OFFSET_ALIGNMENT_BYTES == 0 &&
	       range->byte_offset <= arena && range->byte_count <= arena - range->byte_offset &&
	       touched <= range->byte_count &&
	       (slot_stride == 0 || (slot_stride >= touched && slot_stride <= range->byte_count - touched));
}

result_status tp2_join_prepare(const struct tp2_join_description *description, uint64_t arena_byte_count,
			       uint32_t kernel, struct kernel_launch *launch_out)
{
	if (description == NULL || launch_out == NULL)
		return STATUS_INVALID_ARGUMENT;
	const struct tp2_join_description *const d = description;
	const uint32_t width = d->width, rows = d->row_count, operation = d->operation;
	const bool routed = d->routed_sums.byte_count != 0;
	const bool stepped = d->source_slot_stride != 0 || d->output_slot_stride != 0;
	const bool adds = operation == TP2_JOIN_BFLOAT16_TO_FLOAT32 || operation == TP2_JOIN_BFLOAT16_SUM_TO_BFLOAT16 ||
			  operation == TP2_JOIN_RING_PACK;
	const bool ring = operation == TP2_JOIN_RING_PACK || operation == TP2_JOIN_RING_UNPACK;
	if (width == 0 || width > TP2_JOIN_MAXIMUM_WIDTH || rows == 0 || rows > TP2_JOIN_MAXIMUM_ROWS ||
	    operation >= TP2_JOIN_OPERATION_COUNT || d->source_row_stride < width || d->output_row_stride < width ||
	    (routed && (!adds || d->routed_row_stride < width)) ||
	    (ring && (width % TP2_JOIN_RING_OWNERS != 0 ||
		      (operation == TP2_JOIN_RING_PACK ? d->output_row_stride : d->source_row_stride) != width)) ||
	    (!routed && (d->routed_sums.byte_offset != 0 || d->routed_row_stride != 0)) ||
	    (!stepped && (d->step.byte_offset != 0 || d->step.byte_count != 0)) || d->reserved_zero != 0 ||
	    kernel == BACKEND_NO_KERNEL)
		return STATUS_INVALID_ARGUMENT;
	const uint32_t in_bytes = operation == TP2_JOIN_FLOAT32_TO_BFLOAT16 || operation == TP2_JOIN_FLOAT32_COPY ? 4u : 2u;
	const uint32_t out_bytes = operation == TP2_JOIN_BFLOAT16_TO_FLOAT32 || operation == TP2_JOIN_FLOAT32_COPY ? 4u : 2u;
	const uint64_t source_bytes = join_span(rows, width, d->source_row_stride, in_bytes);
	const uint64_t output_bytes = join_span(rows, width, d->output_row_stride, out_bytes);
	const uint64_t routed_bytes = join_span(rows, width, d->routed_row_stride, 4u);
	if (!join_range_holds(&d->source, source_bytes, d->source_slot_stride, arena_byte_count) ||
	    !join_range_holds(&d->output, output_bytes, d->output_slot_stride, arena_byte_count) ||
	    (routed && !join_range_holds(&d->routed_sums, routed_bytes, 0, arena_byte_count)) ||
	    (stepped && !join_range_holds(&d->step, STEP_BLOCK_BYTES, 0, arena_byte_count)))
		return STATUS_INVALID_ARGUMENT;
	struct checked_range ranges[JOIN_RANGES_MOST];
	uint32_t count = 0;
	ranges[count++] = (struct checked_range){ "the source", d->source.byte_offset, source_bytes };
	ranges[count++] = (struct checked_range){ "the output", d->output.byte_offset, output_bytes };
	if (d->source_slot_stride != 0)
		ranges[count++] = (struct checked_range){ "the second source slot",
							  d->source.byte_offset + d->source_slot_stride, source_bytes };
	if (d->output_slot_stride != 0)
		ranges[count++] = (struct checked_range){ "the second output slot",
							  d->output.byte_offset + d->output_slot_stride, output_bytes };
	if (routed)
		ranges[count++] = (struct checked_range){ "the routed sums", d->routed_sums.byte_offset, routed_bytes };
	if (stepped)
		ranges[count++] = (struct checked_range){ "the step block", d->step.byte_offset, STEP_BLOCK_BYTES };
	if (!prepare_ranges_are_valid("the local completion", ranges, count, arena_byte_count))
		return STATUS_INVALID_ARGUMENT;
	const struct tp2_join_arguments arguments = { .source_offset = d->source.byte_offset,
						      .routed_sums_offset = d->routed_sums.byte_offset,
						      .output_offset = d->output.byte_offset,
						      .step_offset = d->step.byte_offset,
						      .source_slot_stride = d->source_slot_stride,
						      .output_slot_stride = d->output_slot_stride,
						      .width = width,
						      .row_count = rows,
						      .source_row_stride = d->source_row_stride,
						      .routed_row_stride = d->routed_row_stride,
						      .output_row_stride = d->output_row_stride,
						      .operation = operation,
						      .has_routed_sums = routed ? 1u : 0u,
						      .reserved_zero = 0 };
	prepare_launch_fill(launch_out, kernel, (width + TP2_JOIN_THREADS - 1u) / TP2_JOIN_THREADS, rows, 1,
			    TP2_JOIN_THREADS, 0, &arguments, sizeof(arguments));
	return STATUS_OK;
}
