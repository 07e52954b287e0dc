/*
 * exl3_tc.c: load-time preparation behind the reference's default entry points of the routed experts
 * (anemone_b200_exl3_tc.h). Takes the place of the reference's source/exl3_tc.c: same entry points, records,
 * validation and refusals; the launches are this library's (kernel file "kernel_exl3_tc").
 */
#include "anemone_b200_exl3_tc.h"

#include <string.h>

#include "../kernels/exl3_tc_layout.h"
#include "anemone_b200_exl3.h"
#include "prepare_common.h"

uint64_t exl3_tc_workspace_byte_count(uint64_t pair_count, uint64_t intermediate)
{
	return exl3_tc_workspace_bytes(pair_count, intermediate);
}

uint64_t exl3_tcp_workspace_byte_count(uint64_t rows, uint64_t intermediate)
{
	return exl3_tcp_workspace_bytes(rows, intermediate);
}

struct tc_range {
	uint64_t offset, bytes;
};

/* the reference's rule for these records (source/exl3_tc.c:45-62): 16-byte aligned, inside the arena, not empty, no
 * two sharing a byte */
static bool tc_ranges_are_valid(const struct tc_range *ranges, uint32_t count, uint64_t arena_bytes)
{
	for (uint32_t index = 0; index < count; index++) {
		const struct tc_range *const range = &ranges[index];
		if (range->offset % LINEAR_OFFSET_ALIGNMENT_BYTES != 0 || range->offset > arena_bytes || range->bytes == 0 ||
		    range->bytes > arena_bytes - range->offset)
			return false;
		for (uint32_t earlier = 0; earlier < index; earlier++)
			if (range->offset < ranges[earlier].offset + ranges[earlier].bytes &&
			    ranges[earlier].offset < range->offset + range->bytes)
				return false;
	}
	return true;
}

struct tc_shape {
	const char *name;
	uint32_t x, y, z, threads, shared;
};

static result_status tc_launches_fill(const struct tc_shape *shapes, uint32_t count, const void *const *records,
				      uint32_t record_bytes, const struct backend_operations *backend,
				      struct device_card *card, struct kernel_launch *launches)
{
	for (uint32_t index = 0; index < count; index++) {
		uint32_t kernel = BACKEND_NO_KERNEL;
		const result_status status =
			backend->kernel_prepare(card, EXL3_TC_KERNEL_FILE, shapes[index].name, record_bytes, &kernel);
		if (status != STATUS_OK)
			return status;
		if (kernel == BACKEND_NO_KERNEL)
			return STATUS_UNSUPPORTED;
		prepare_launch_fill(&launches[index], kernel, shapes[index].x, shapes[index].y, shapes[index].z,
				    shapes[index].threads, shapes[index].shared, records[index], record_bytes);
	}
	return STATUS_OK;
}

static uint32_t transform_blocks(uint32_t width)
{
	return (width / EXL3_TRANSFORM + EXL3_TRANSFORM_WARPS - 1u) / EXL3_TRANSFORM_WARPS;
}

static result_status tc_prepare(const struct exl3_tc_record *record, uint64_t arena_byte_count,
				const struct backend_operations *backend, struct device_card *card,
				struct kernel_launch *launches_out)
{
	if (record == NULL || backend == NULL || backend->kernel_prepare == NULL || card == NULL || launches_out == NULL ||
	    record->row_count == 0 ||
	    (record->intermediate != EXL3_TC_WIDE_INTERMEDIATE && record->intermediate != EXL3_TC_NARROW_INTERMEDIATE) ||
	    exl3_width_name(record->bits_x2) == NULL || record->job_capacity == 0 || record->pass != 0 ||
	    !(record->activation_limit >= 0.0f) || record->rotation > EXL3_TC_MOST_ROTATION ||
	    (record->rotation != 0 && record->intermediate != EXL3_TC_WIDE_INTERMEDIATE) || record->shared_sum > 1u)
		return STATUS_INVALID_ARGUMENT;
	const uint64_t pairs = (uint64_t)record->row_count * EXL3_TC_PAIRS_PER_ROW;
	if (pairs > EXL3_TC_MOST_PAIRS || record->job_capacity > pairs)
		return STATUS_INVALID_ARGUMENT;
	const uint64_t workspace = exl3_tc_workspace_bytes(pairs, record->intermediate);
	const struct tc_range ranges[5] = {
		{ record->jobs_offset, (uint64_t)record->job_capacity * sizeof(struct expert_job_record) },
		{ record->hidden_offset, (uint64_t)record->row_count * EXL3_TC_HIDDEN * 2u },
		{ record->workspace_offset, workspace },
		{ record->output_offset, (uint64_t)record->row_count * EXL3_TC_HIDDEN * 4u },
		{ record->shared_offset, (uint64_t)record->row_count * EXL3_TC_HIDDEN * 2u }
	};
	if (!tc_ranges_are_valid(ranges, record->shared_sum != 0 ? 5u : 4u, arena_byte_count))
		return STATUS_INVALID_ARGUMENT;
	if (record->rotation != 0)
		return STATUS_UNSUPPORTED; /* the reference's mixed expert widths of one record: not built */
	const struct exl3_tc_layout layout = exl3_tc_layout_of(pairs, record->job_capacity, record->intermediate, 0u, workspace);
	if (layout.total > workspace)
		return STATUS_UNSUPPORTED;
	struct exl3_tc_record down = *record;
	down.pass = 1u; /* as the reference marks its down products launch */
	const uint32_t jobs = record->job_capacity, I = record->intermediate;
	const uint32_t shared = exl3_product_dynamic_bytes(record->bits_x2);
	const struct tc_shape shapes[EXL3_TC_LAUNCHES] = {
		{ "exl3_tc_operands", transform_blocks(EXL3_TC_HIDDEN), jobs, EXL3_PROJECTIONS, EXL3_TRANSFORM_THREADS, 0 },
		{ "exl3_tc_gate_up", I / EXL3_TRANSFORM * layout.gate_up_runs, jobs, EXL3_PROJECTIONS, EXL3_PRODUCT_THREADS,
		  shared },
		{ "exl3_tc_mark", (jobs + 127u) / 128u, 1, 1, 128u, 0 },
		{ "exl3_tc_down", EXL3_TC_HIDDEN / EXL3_TRANSFORM * layout.down_runs, jobs, 1, EXL3_PRODUCT_THREADS, shared },
		{ "exl3_tc_combine", EXL3_TC_HIDDEN / 512u, record->row_count, 1, 128u, 0 }
	};
	const void *const records[EXL3_TC_LAUNCHES] = { record, record, record, &down, record };
	struct kernel_launch launches[EXL3_TC_LAUNCHES];
	const result_status status =
		tc_launches_fill(shapes, EXL3_TC_LAUNCHES, records, sizeof(*record), backend, card, launches);
	if (status == STATUS_OK)
		memcpy(launches_out, launches, sizeof(launches));
	return status;
}

result_status exl3_tc_prepare(const struct exl3_tc_record *record, uint64_t arena_byte_count,
			      const struct backend_operations *backend, struct device_card *card,
			      struct kernel_launch launches_out[EXL3_TC_LAUNCHES])
{
	return tc_prepare(record, arena_byte_count, backend, card, launches_out);
}

result_status exl3_tc_prepare_short(const struct exl3_tc_record *record, uint64_t arena_byte_count,
				    const struct backend_operations *backend, struct device_card *card,
				    struct kernel_launch launches_out[EXL3_TC_LAUNCHES])
{
	return tc_prepare(record, arena_byte_count, backend, card, launches_out);
}

result_status exl3_tc_prepare_paired(const struct exl3_tc_record *record, uint64_t arena_byte_count,
				     const struct backend_operations *backend, struct device_card *card,
				     struct kernel_launch launches_out[EXL3_TC_LAUNCHES])
{
	return tc_prepare(record, arena_byte_count, backend, card, launches_out);
}

#define TCP_LAUNCHES 5u /* of one chunk */
#define TCP_CHUNKS 2u /* EXL3_TCP_CHUNK_ROWS / EXL3_TCP_JOINT_ROWS */
/* the reference's bounds of cone_layer (its model's decoder layers, include/anemone/model_layout.h): checked only to
 * refuse what it refuses */
#define TCP_CONE_FIRST_LAYER 1u
#define TCP_CONE_LAYERS 62u

static result_status tcp_prepare(const struct exl3_tcp_record *record, uint64_t arena_byte_count,
				 const struct backend_operations *backend, struct device_card *card,
				 struct kernel_launch *launches_out, uint32_t *launch_count_out)
{
	if (record == NULL || backend == NULL || backend->kernel_prepare == NULL || card == NULL || launches_out == NULL ||
	    launch_count_out == NULL || record->row_count == 0 || record->row_count > EXL3_TCP_CHUNK_ROWS ||
	    (record->intermediate != EXL3_TC_WIDE_INTERMEDIATE && record->intermediate != EXL3_TC_NARROW_INTERMEDIATE) ||
	    exl3_width_name(record->bits_x2) == NULL || record->pass != 0 || record->rotation > EXL3_TC_MOST_ROTATION ||
	    (record->rotation != 0 && record->intermediate != EXL3_TC_WIDE_INTERMEDIATE) ||
	    !(record->activation_limit >= 0.0f) || record->half_rows >= record->row_count || record->part != 0 ||
	    record->two_blocks > 1u ||
	    (record->cone_layer != 0 &&
	     (record->cone_layer < TCP_CONE_FIRST_LAYER || record->cone_layer >= TCP_CONE_LAYERS)))
		return STATUS_INVALID_ARGUMENT;
	const uint64_t pairs = (uint64_t)record->row_count * EXL3_TC_PAIRS_PER_ROW;
	const uint64_t workspace = exl3_tcp_workspace_bytes(record->row_count, record->intermediate);
	const struct tc_range ranges[5] = {
		{ record->picks_offset, pairs * sizeof(struct router_pick) },
		{ record->expert_offsets_offset, (uint64_t)EXL3_TCP_EXPERTS * 3u * sizeof(uint64_t) },
		{ record->hidden_offset, (uint64_t)record->row_count * EXL3_TC_HIDDEN * 2u },
		{ record->workspace_offset, workspace },
		{ record->output_offset, (uint64_t)record->row_count * EXL3_TC_HIDDEN * 4u }
	};
	if (!tc_ranges_are_valid(ranges, 5, arena_byte_count))
		return STATUS_INVALID_ARGUMENT;
	if (record->rotation != 0 || record->half_rows != 0 || record->cone_layer != 0)
		return STATUS_UNSUPPORTED; /* mixed widths, the two-part overlap of one call, rows a step leaves alone */
	/* chunks of at most EXL3_TCP_JOINT_ROWS rows, one after the other in the same workspace */
	const uint32_t chunks = (record->row_count + EXL3_TCP_JOINT_ROWS - 1u) / EXL3_TCP_JOINT_ROWS;
	const uint32_t I = record->intermediate, shared = exl3_product_dynamic_bytes(record->bits_x2);
	struct kernel_launch launches[TCP_CHUNKS * TCP_LAUNCHES];
	struct exl3_tcp_record of_chunk[TCP_CHUNKS], down[TCP_CHUNKS];
	for (uint32_t chunk = 0; chunk < chunks; chunk++) {
		const uint32_t rows = record->row_count - chunk * EXL3_TCP_JOINT_ROWS < EXL3_TCP_JOINT_ROWS ?
					      record->row_count - chunk * EXL3_TCP_JOINT_ROWS :
					      EXL3_TCP_JOINT_ROWS;
		const uint64_t chunk_pairs = (uint64_t)rows * EXL3_TC_PAIRS_PER_ROW;
		const uint32_t jobs = exl3_tcp_job_capacity(chunk_pairs);
		/* cut as the chunk's own workspace size allows (it is never more than the call's) */
		const uint64_t chunk_workspace = exl3_tcp_workspace_bytes(rows, I);
		const struct exl3_tc_layout layout = exl3_tc_layout_of(chunk_pairs, 0u, I, jobs, chunk_workspace);
		if (layout.total > chunk_workspace || chunk_workspace > workspace)
			return STATUS_UNSUPPORTED;
		const struct tc_shape shapes[TCP_LAUNCHES] = {
			{ "exl3_tcp_route", 1, 1, 1, 1024u, 0 },
			{ "exl3_tcp_operands", transform_blocks(EXL3_TC_HIDDEN), jobs, EXL3_PROJECTIONS, EXL3_TRANSFORM_THREADS, 0 },
			{ "exl3_tcp_gate_up", I / EXL3_TRANSFORM * layout.gate_up_runs, jobs, EXL3_PROJECTIONS,
			  EXL3_PRODUCT_THREADS, shared },
			{ "exl3_tcp_down", EXL3_TC_HIDDEN / EXL3_TRANSFORM * layout.down_runs, jobs, 1, EXL3_PRODUCT_THREADS,
			  shared },
			{ "exl3_tcp_combine", EXL3_TC_HIDDEN / 512u, rows, 1, 128u, 0 }
		};
		of_chunk[chunk] = *record;
		of_chunk[chunk].part = chunk;
		down[chunk] = of_chunk[chunk];
		down[chunk].pass = 3u; /* the reference's EXL3_TCP_DOWN */
		const void *const records[TCP_LAUNCHES] = { &of_chunk[chunk], &of_chunk[chunk], &of_chunk[chunk], &down[chunk],
							    &of_chunk[chunk] };
		const result_status status = tc_launches_fill(shapes, TCP_LAUNCHES, records, sizeof(*record), backend, card,
							      &launches[chunk * TCP_LAUNCHES]);
		if (status != STATUS_OK)
			return status;
	}
	memcpy(launches_out, launches, (size_t)chunks * TCP_LAUNCHES * sizeof(launches[0]));
	*launch_count_out = chunks * TCP_LAUNCHES;
	return STATUS_OK;
}

result_status exl3_tcp_prepare(const struct exl3_tcp_record *record, uint64_t arena_byte_count,
			       const struct backend_operations *backend, struct device_card *card,
			       struct kernel_launch launches_out[EXL3_TCP_MOST_LAUNCHES], uint32_t *launch_count_out)
{
	return tcp_prepare(record, arena_byte_count, backend, card, launches_out, launch_count_out);
}

result_status exl3_tcp_prepare_base(const struct exl3_tcp_record *record, uint64_t arena_byte_count,
				    const struct backend_operations *backend, struct device_card *card,
				    struct kernel_launch launches_out[EXL3_TCP_MOST_LAUNCHES], uint32_t *launch_count_out)
{
	return tcp_prepare(record, arena_byte_count, backend, card, launches_out, launch_count_out);
}

result_status exl3_tcp_prepare_hybrid(const struct exl3_tcp_record *record, uint64_t arena_byte_count,
				      const struct backend_operations *backend, struct device_card *card,
				      struct kernel_launch launches_out[EXL3_TCP_MOST_LAUNCHES],
				      uint32_t *launch_count_out)
{
	return tcp_prepare(record, arena_byte_count, backend, card, launches_out, launch_count_out);
}
