/* prepare_common.c: range checks and launch filling shared by the preparers. */
#include "prepare_common.h"

#include <inttypes.h>
#include <stdio.h>
#include <string.h>

#include "anemone_b200_records.h"

bool prepare_ranges_are_valid(const char *what, const struct checked_range *ranges, uint32_t range_count,
			      uint64_t arena_byte_count)
{
	for (uint32_t index = 0; index < range_count; index++) {
		const struct checked_range *const range = &ranges[index];
		if (range->offset % LINEAR_OFFSET_ALIGNMENT_BYTES != 0 || range->byte_count == UINT64_MAX ||
		    range->offset > arena_byte_count || range->byte_count > arena_byte_count - range->offset) {
			(void)fprintf(stderr,
				      "%s: %s (offset %" PRIu64 ", %" PRIu64 " bytes) is misaligned or outside the arena of %" PRIu64
				      " bytes\n",
				      what, range->name, range->offset, range->byte_count, arena_byte_count);
			return false;
		}
		for (uint32_t earlier = 0; earlier < index; earlier++) {
			const struct checked_range *const other = &ranges[earlier];
			if (range->byte_count != 0 && other->byte_count != 0 &&
			    range->offset < other->offset + other->byte_count &&
			    other->offset < range->offset + range->byte_count) {
				(void)fprintf(stderr, "%s: %s overlaps %s\n", what, range->name, other->name);
				return false;
			}
		}
	}
	return true;
}

void prepare_launch_fill(struct kernel_launch *launch, uint32_t kernel, uint32_t grid_x, uint32_t grid_y,
			 uint32_t grid_z, uint32_t block_threads, uint32_t dynamic_shared_byte_count,
			 const void *record, uint32_t record_byte_count)
{
	memset(launch, 0, sizeof(*launch));
	launch->kernel = kernel;
	launch->grid[0] = grid_x;
	launch->grid[1] = grid_y;
	launch->grid[2] = grid_z;
	launch->block[0] = block_threads;
	launch->block[1] = launch->block[2] = 1;
	launch->dynamic_shared_byte_count = dynamic_shared_byte_count;
	launch->argument_byte_count = record_byte_count;
	launch->branch = LAUNCH_CHAIN;
	memcpy(launch->argument, record, record_byte_count);
}
