/*
 * prepare_common.h: the checks every preparer makes and the one way it fills a launch. Private to csrc/host.
 * Same rules as the reference's source/prepare_common.h:33-44: a range begins on a 16-byte multiple, lies inside the
 * arena (64-bit, no wrap), and no two ranges of one description share a byte.
 */
#ifndef AB_PREPARE_COMMON_H
#define AB_PREPARE_COMMON_H

#include <stdbool.h>
#include <stdint.h>

#include "anemone_b200_backend.h"

struct checked_range {
	const char *name;
	uint64_t offset;
	uint64_t byte_count;
};

/* true, or false behind one error line that begins with `what` */
bool prepare_ranges_are_valid(const char *what, const struct checked_range *ranges, uint32_t range_count,
			      uint64_t arena_byte_count);
/* writes every byte of the launch: a grid of x by y by z blocks of block_threads threads, the record, zero behind */
void prepare_launch_fill(struct kernel_launch *launch, uint32_t kernel, uint32_t grid_x, uint32_t grid_y,
			 uint32_t grid_z, uint32_t block_threads, uint32_t dynamic_shared_byte_count,
			 const void *record, uint32_t record_byte_count);

#endif
