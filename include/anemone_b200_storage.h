/*
 * anemone_b200_storage.h: where the bytes of an EXL3 pack come from at load time: the read-only virtual pack
 * (".exl3map") and its way into a card's arena.
 *
 * Replaces the reference's include/anemone/storage_seam.h:49-74 (struct storage_description, struct
 * storage_operations_record) and include/anemone/storage_exl3.h:17-46 (the map's limits, storage_exl3,
 * storage_exl3_read_mode, storage_for_path, storage_device_path); the map's file format is that of
 * source/storage_exl3_linux.c:27-40: a header of 64 bytes ("ANEXL3\0\0", the pack's logical byte count, the counts of
 * sources and segments, 40 zero bytes), a table of source paths of 512 bytes each (source 0, the map file itself, is
 * the empty path; every other one absolute), then segments of 32 bytes (logical offset, byte count, offset in the
 * source, source index, a zero word), sorted by logical offset and disjoint. Logical bytes no segment holds read as
 * zero.
 *
 * Contract of the table, as the reference states it: reader_open opens everything or nothing and leaves reader_out
 * untouched when it refuses; a read is synchronous, holds no cursor (any number of threads may read through one
 * reader), delivers every byte or fails, and wants offset, count and destination address on multiples of the block
 * alignment (EXL3_MAP_BLOCK_BYTES); reader_close accepts NULL.
 * Differences, all deliberate: one copy only (the reference's flat replica copies 1.. go through its direct-read
 * storage, which this library does not have: a copy_count above 1 is STATUS_UNSUPPORTED); no drive read-bound policy
 * (every source is accepted as the reference accepts a drive that states no bound); a direct read that the file
 * system refuses is done again through the page cache instead of failing.
 */
#ifndef ANEMONE_B200_STORAGE_H
#define ANEMONE_B200_STORAGE_H

#include <stdint.h>

#include "anemone_b200_backend.h"
#include "anemone_b200_status.h"

#ifdef __cplusplus
extern "C" {
#endif

#define STORAGE_MAXIMUM_COPIES 8
#define EXL3_MAP_PATH_BYTES 512u
#define EXL3_MAP_MAXIMUM_SOURCES 128u
#define EXL3_MAP_MAXIMUM_SEGMENTS 262144u
#define EXL3_MAP_HEADER_BYTES 64u
#define EXL3_MAP_SEGMENT_BYTES 32u
#define EXL3_MAP_BLOCK_BYTES 4096u

struct storage_description {
	uint64_t byte_count;
	uint32_t copy_count;
	uint32_t block_alignment_bytes;
	uint64_t first_device, first_inode; /* copy 0 as it was opened */
};

struct storage_reader;

struct storage_operations_record {
	const char *name;
	MUST_CHECK result_status (*reader_open)(const char *const *copy_paths, uint32_t copy_count,
						struct storage_reader **reader_out);
	void (*reader_close)(struct storage_reader *reader);
	MUST_CHECK result_status (*reader_describe)(const struct storage_reader *reader,
						    struct storage_description *description_out);
	MUST_CHECK result_status (*reader_read)(const struct storage_reader *reader, uint32_t copy_index,
						uint64_t byte_offset, void *destination, uint64_t byte_count);
};

extern const struct storage_operations_record storage_exl3;

/* How a map reads its sources (process-wide, read at every read): through the page cache; the same with the pages
 * dropped behind the read; directly (O_DIRECT) where offset, size and address allow; or direct where aligned and
 * dropped for the rest. Without a call: direct. */
enum exl3_read_mode {
	EXL3_READS_BUFFERED,
	EXL3_READS_DROPPED,
	EXL3_READS_DIRECT,
	EXL3_READS_DIRECT_DROPPED,
	EXL3_READ_MODES
};
void storage_exl3_read_mode(enum exl3_read_mode mode);

/* &storage_exl3 for a path that ends in ".exl3map", else NULL (the reference answers its direct-read storage there,
 * which this library does not have). */
const struct storage_operations_record *storage_for_path(const char *path);

/* The file whose device holds most of a map's logical bytes, copied into output; path itself for any other path, for
 * a map that does not open, or when the map file itself holds the most. */
const char *storage_device_path(const char *path, char output[EXL3_MAP_PATH_BYTES]);

/* New with this library: a run of a pack's logical bytes into a card's arena, read through `storage` in pieces into
 * page-locked memory the caller got from backend->staging_allocate and uploaded piece by piece, the read of a piece
 * overlapping the upload of the one before (the staging is used as two halves). pack_offset, byte_count (the tail is
 * read in whole blocks; only byte_count bytes are uploaded) and staging_byte_count (at least two blocks) are multiples
 * of EXL3_MAP_BLOCK_BYTES except byte_count, which is any positive count inside the pack when rounded up. On return
 * every byte is in the arena (the uploads have been waited for, each within wait_limit_nanoseconds). */
MUST_CHECK result_status exl3_map_upload(const struct storage_operations_record *storage,
					 const struct storage_reader *reader, uint64_t pack_offset, uint64_t byte_count,
					 const struct backend_operations *backend, struct device_card *card,
					 uint64_t arena_byte_offset, void *staging, uint64_t staging_byte_count,
					 uint64_t wait_limit_nanoseconds);

#ifdef __cplusplus
}
#endif
#endif
