/*
 * storage_exl3.c: the read-only EXL3 virtual pack (anemone_b200_storage.h) and its upload into an arena. Linux, C11.
 * The file format and every refusal are the reference's (source/storage_exl3_linux.c:147-300); the reader itself is
 * written for this library: the whole manifest is read and checked in one piece, a read looks up its first segment
 * by bisection and fills the holes between segments as it walks.
 */
#define _GNU_SOURCE
#include "anemone_b200_storage.h"

#include <errno.h>
#include <fcntl.h>
#include <stdbool.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>

#define PIECE_BYTES (8ull << 20u) /* one positioned read */

struct manifest_header {
	unsigned char magic[8];
	uint64_t byte_count;
	uint32_t source_count;
	uint32_t segment_count;
	unsigned char reserved[40];
};
struct manifest_segment {
	uint64_t byte_offset;
	uint64_t byte_count;
	uint64_t source_offset;
	uint32_t source_index;
	uint32_t reserved_zero;
};
_Static_assert(sizeof(struct manifest_header) == EXL3_MAP_HEADER_BYTES, "the map's header");
_Static_assert(sizeof(struct manifest_segment) == EXL3_MAP_SEGMENT_BYTES, "a segment of the map");

struct storage_reader {
	uint64_t byte_count;
	uint32_t source_count, segment_count;
	struct manifest_segment *segments;
	int buffered[EXL3_MAP_MAXIMUM_SOURCES], direct[EXL3_MAP_MAXIMUM_SOURCES];
	char (*paths)[EXL3_MAP_PATH_BYTES];
	uint64_t device, inode;
};

static enum exl3_read_mode read_mode = EXL3_READS_DIRECT;

void storage_exl3_read_mode(enum exl3_read_mode mode)
{
	read_mode = (unsigned)mode < EXL3_READ_MODES ? mode : EXL3_READS_BUFFERED;
}

/* every byte, or false (a short file counts as a failure) */
static bool read_all(int descriptor, uint64_t offset, unsigned char *destination, uint64_t count)
{
	while (count != 0) {
		const ssize_t got = pread(descriptor, destination, count > PIECE_BYTES ? PIECE_BYTES : (size_t)count,
					  (off_t)offset);
		if (got < 0 && errno == EINTR)
			continue;
		if (got <= 0)
			return false;
		offset += (uint64_t)got, destination += got, count -= (uint64_t)got;
	}
	return true;
}

static void reader_close(struct storage_reader *reader)
{
	if (reader == NULL)
		return;
	for (uint32_t source = 0; source < EXL3_MAP_MAXIMUM_SOURCES; source++) {
		if (reader->buffered[source] >= 0)
			(void)close(reader->buffered[source]);
		if (reader->direct[source] >= 0)
			(void)close(reader->direct[source]);
	}
	free(reader->segments);
	free(reader->paths);
	free(reader);
}

/* a source's size if it is a regular file with bytes, else 0 */
static uint64_t regular_size(int descriptor, struct stat *metadata)
{
	return descriptor >= 0 && fstat(descriptor, metadata) == 0 && S_ISREG(metadata->st_mode) && metadata->st_size > 0 ?
		       (uint64_t)metadata->st_size :
		       0u;
}

static result_status reader_open(const char *const *copy_paths, uint32_t copy_count, struct storage_reader **reader_out)
{
	if (copy_paths == NULL || copy_count == 0 || copy_count > STORAGE_MAXIMUM_COPIES || copy_paths[0] == NULL ||
	    reader_out == NULL)
		return STATUS_INVALID_ARGUMENT;
	if (copy_count > 1)
		return STATUS_UNSUPPORTED; /* flat replica copies: not offered */
	struct storage_reader *const reader = calloc(1, sizeof(*reader));
	if (reader == NULL)
		return STATUS_OUT_OF_MEMORY;
	for (uint32_t source = 0; source < EXL3_MAP_MAXIMUM_SOURCES; source++)
		reader->buffered[source] = reader->direct[source] = -1;
	result_status status = STATUS_INPUT_OUTPUT_ERROR;
	struct manifest_header header;
	struct stat metadata;
	uint64_t sizes[EXL3_MAP_MAXIMUM_SOURCES] = { 0 };
	reader->buffered[0] = open(copy_paths[0], O_RDONLY | O_CLOEXEC | O_NONBLOCK);
	if (reader->buffered[0] < 0 || fstat(reader->buffered[0], &metadata) != 0 ||
	    !read_all(reader->buffered[0], 0, (unsigned char *)&header, sizeof(header)))
		goto refused;
	reader->device = metadata.st_dev, reader->inode = metadata.st_ino;
	status = STATUS_CORRUPT_PACK;
	static const unsigned char zeros[sizeof(header.reserved)] = { 0 };
	if (memcmp(header.magic, "ANEXL3\0", 8) != 0 || header.byte_count == 0 || header.byte_count > INT64_MAX ||
	    header.byte_count % EXL3_MAP_BLOCK_BYTES != 0 || header.source_count == 0 ||
	    header.source_count > EXL3_MAP_MAXIMUM_SOURCES || header.segment_count == 0 ||
	    header.segment_count > EXL3_MAP_MAXIMUM_SEGMENTS || memcmp(header.reserved, zeros, sizeof(zeros)) != 0)
		goto refused;
	reader->byte_count = header.byte_count;
	reader->source_count = header.source_count, reader->segment_count = header.segment_count;
	const uint64_t path_bytes = (uint64_t)header.source_count * EXL3_MAP_PATH_BYTES;
	const uint64_t segment_bytes = (uint64_t)header.segment_count * sizeof(struct manifest_segment);
	const uint64_t manifest_end = sizeof(header) + path_bytes + segment_bytes;
	reader->paths = malloc(path_bytes);
	reader->segments = malloc(segment_bytes);
	if (reader->paths == NULL || reader->segments == NULL) {
		status = STATUS_OUT_OF_MEMORY;
		goto refused;
	}
	if (!read_all(reader->buffered[0], sizeof(header), (unsigned char *)reader->paths, path_bytes) ||
	    !read_all(reader->buffered[0], sizeof(header) + path_bytes, (unsigned char *)reader->segments, segment_bytes))
		goto refused;
	for (uint32_t source = 0; source < header.source_count; source++) {
		const char *const path = reader->paths[source];
		if (memchr(path, 0, EXL3_MAP_PATH_BYTES) == NULL || (source == 0 ? path[0] != 0 : path[0] != '/'))
			goto refused;
		if (source != 0)
			reader->buffered[source] = open(path, O_RDONLY | O_CLOEXEC | O_NONBLOCK);
		sizes[source] = regular_size(reader->buffered[source], &metadata);
		if (sizes[source] == 0) {
			status = STATUS_INPUT_OUTPUT_ERROR;
			goto refused;
		}
		/* once more for direct reads; it must be the same file, else the buffered descriptor serves alone */
		struct stat again;
		reader->direct[source] = open(source == 0 ? copy_paths[0] : path, O_RDONLY | O_DIRECT | O_CLOEXEC | O_NONBLOCK);
		if (reader->direct[source] >= 0 && (fstat(reader->direct[source], &again) != 0 ||
						    again.st_dev != metadata.st_dev || again.st_ino != metadata.st_ino)) {
			(void)close(reader->direct[source]);
			reader->direct[source] = -1;
		}
	}
	uint64_t covered_to = 0;
	for (uint32_t index = 0; index < header.segment_count; index++) {
		const struct manifest_segment *const segment = &reader->segments[index];
		if (segment->reserved_zero != 0 || segment->source_index >= header.source_count ||
		    segment->byte_count == 0 || segment->byte_offset < covered_to ||
		    segment->byte_offset > header.byte_count ||
		    segment->byte_count > header.byte_count - segment->byte_offset ||
		    segment->source_offset > sizes[segment->source_index] ||
		    segment->byte_count > sizes[segment->source_index] - segment->source_offset ||
		    (segment->source_index == 0 && segment->source_offset < manifest_end)) /* never the manifest itself */
			goto refused;
		covered_to = segment->byte_offset + segment->byte_count;
	}
	*reader_out = reader;
	return STATUS_OK;
refused:
	reader_close(reader);
	return status;
}

static result_status reader_describe(const struct storage_reader *reader, struct storage_description *description_out)
{
	if (reader == NULL || description_out == NULL)
		return STATUS_INVALID_ARGUMENT;
	*description_out =
		(struct storage_description){ reader->byte_count, 1u, EXL3_MAP_BLOCK_BYTES, reader->device, reader->inode };
	return STATUS_OK;
}

/* the first segment that ends behind `offset` */
static uint32_t first_segment_behind(const struct storage_reader *reader, uint64_t offset)
{
	uint32_t low = 0, high = reader->segment_count;
	while (low < high) {
		const uint32_t middle = low + (high - low) / 2u;
		if (reader->segments[middle].byte_offset + reader->segments[middle].byte_count <= offset)
			low = middle + 1u;
		else
			high = middle;
	}
	return low;
}

static bool source_read(const struct storage_reader *reader, uint32_t source, uint64_t source_offset,
			unsigned char *destination, uint64_t count)
{
	const enum exl3_read_mode mode = read_mode;
	const bool wants_direct = mode == EXL3_READS_DIRECT || mode == EXL3_READS_DIRECT_DROPPED;
	if (wants_direct && reader->direct[source] >= 0 &&
	    (source_offset | count | (uint64_t)(uintptr_t)destination) % EXL3_MAP_BLOCK_BYTES == 0 &&
	    read_all(reader->direct[source], source_offset, destination, count))
		return true; /* past the page cache */
	if (!read_all(reader->buffered[source], source_offset, destination, count))
		return false;
	if (mode == EXL3_READS_DROPPED || mode == EXL3_READS_DIRECT_DROPPED)
		(void)posix_fadvise(reader->buffered[source], (off_t)source_offset, (off_t)count, POSIX_FADV_DONTNEED);
	return true;
}

static result_status reader_read(const struct storage_reader *reader, uint32_t copy_index, uint64_t byte_offset,
				 void *destination, uint64_t byte_count)
{
	if (reader == NULL || destination == NULL || copy_index != 0 || byte_count == 0 ||
	    byte_offset > reader->byte_count || byte_count > reader->byte_count - byte_offset ||
	    (byte_offset | byte_count | (uint64_t)(uintptr_t)destination) % EXL3_MAP_BLOCK_BYTES != 0 ||
	    byte_count > SIZE_MAX)
		return STATUS_INVALID_ARGUMENT;
	unsigned char *const bytes = destination;
	const uint64_t end = byte_offset + byte_count;
	uint64_t filled_to = byte_offset; /* every byte below it has been written, once */
	for (uint32_t index = first_segment_behind(reader, byte_offset);
	     index < reader->segment_count && reader->segments[index].byte_offset < end; index++) {
		const struct manifest_segment *const segment = &reader->segments[index];
		const uint64_t from = segment->byte_offset > byte_offset ? segment->byte_offset : byte_offset;
		const uint64_t segment_end = segment->byte_offset + segment->byte_count;
		const uint64_t to = segment_end < end ? segment_end : end;
		memset(bytes + (filled_to - byte_offset), 0, (size_t)(from - filled_to)); /* the hole in front of it */
		if (!source_read(reader, segment->source_index, segment->source_offset + (from - segment->byte_offset),
				 bytes + (from - byte_offset), to - from))
			return STATUS_INPUT_OUTPUT_ERROR;
		filled_to = to;
	}
	memset(bytes + (filled_to - byte_offset), 0, (size_t)(end - filled_to));
	return STATUS_OK;
}

const struct storage_operations_record storage_exl3 = { .name = "exl3_map",
							.reader_open = reader_open,
							.reader_close = reader_close,
							.reader_describe = reader_describe,
							.reader_read = reader_read };

const struct storage_operations_record *storage_for_path(const char *path)
{
	static const char suffix[] = ".exl3map";
	const size_t length = path == NULL ? 0u : strlen(path), tail = sizeof(suffix) - 1u;
	return length >= tail && strcmp(path + length - tail, suffix) == 0 ? &storage_exl3 : NULL;
}

const char *storage_device_path(const char *path, char output[EXL3_MAP_PATH_BYTES])
{
	struct storage_reader *reader = NULL;
	if (output == NULL || storage_for_path(path) == NULL || reader_open(&path, 1, &reader) != STATUS_OK)
		return path;
	uint64_t held[EXL3_MAP_MAXIMUM_SOURCES] = { 0 };
	for (uint32_t index = 0; index < reader->segment_count; index++)
		held[reader->segments[index].source_index] += reader->segments[index].byte_count;
	uint32_t most = 0;
	for (uint32_t source = 1; source < reader->source_count; source++)
		if (held[source] > held[most])
			most = source; /* ties: the lowest source */
	if (most != 0)
		memcpy(output, reader->paths[most], EXL3_MAP_PATH_BYTES);
	reader_close(reader);
	return most != 0 ? output : path;
}

result_status exl3_map_upload(const struct storage_operations_record *storage, const struct storage_reader *reader,
			      uint64_t pack_offset, uint64_t byte_count, const struct backend_operations *backend,
			      struct device_card *card, uint64_t arena_byte_offset, void *staging,
			      uint64_t staging_byte_count, uint64_t wait_limit_nanoseconds)
{
	if (storage == NULL || storage->reader_read == NULL || storage->reader_describe == NULL || reader == NULL ||
	    backend == NULL || backend->upload_begin == NULL || backend->upload_wait == NULL || card == NULL ||
	    staging == NULL || byte_count == 0 || pack_offset % EXL3_MAP_BLOCK_BYTES != 0 ||
	    staging_byte_count % EXL3_MAP_BLOCK_BYTES != 0 || staging_byte_count < 2u * EXL3_MAP_BLOCK_BYTES ||
	    (uint64_t)(uintptr_t)staging % EXL3_MAP_BLOCK_BYTES != 0)
		return STATUS_INVALID_ARGUMENT;
	struct storage_description description;
	result_status status = storage->reader_describe(reader, &description);
	if (status != STATUS_OK)
		return status;
	const uint64_t rounded = (byte_count + EXL3_MAP_BLOCK_BYTES - 1u) / EXL3_MAP_BLOCK_BYTES * EXL3_MAP_BLOCK_BYTES;
	if (rounded < byte_count || pack_offset > description.byte_count || rounded > description.byte_count - pack_offset)
		return STATUS_INVALID_ARGUMENT;
	/* two halves: while one is on its way to the card the other is filled from the drives */
	const uint64_t half = staging_byte_count / 2u / EXL3_MAP_BLOCK_BYTES * EXL3_MAP_BLOCK_BYTES;
	uint64_t tickets[2] = { 0, 0 };
	bool in_flight[2] = { false, false };
	uint64_t done = 0;
	for (uint32_t turn = 0; done < byte_count && status == STATUS_OK; turn ^= 1u) {
		unsigned char *const buffer = (unsigned char *)staging + turn * half;
		if (in_flight[turn]) { /* the upload that last used this half */
			status = backend->upload_wait(card, tickets[turn], wait_limit_nanoseconds);
			in_flight[turn] = false;
			if (status != STATUS_OK)
				break;
		}
		const uint64_t left = byte_count - done, piece = left < half ? left : half;
		const uint64_t read_bytes = (piece + EXL3_MAP_BLOCK_BYTES - 1u) / EXL3_MAP_BLOCK_BYTES * EXL3_MAP_BLOCK_BYTES;
		status = storage->reader_read(reader, 0, pack_offset + done, buffer, read_bytes);
		if (status != STATUS_OK)
			break;
		status = backend->upload_begin(card, arena_byte_offset + done, buffer, piece, &tickets[turn]);
		in_flight[turn] = status == STATUS_OK;
		done += piece;
	}
	for (uint32_t turn = 0; turn < 2; turn++)
		if (in_flight[turn]) { /* nothing of the staging is in use when this returns, whatever the outcome */
			const result_status waited = backend->upload_wait(card, tickets[turn], wait_limit_nanoseconds);
			status = status == STATUS_OK ? waited : status;
		}
	return status;
}
