/*
 * backend_cuda.c: the card table (anemone_b200_backend.h) over the CUDA driver API, for B200 (sm_100a).
 *
 * Takes the place of the reference's source/backend_cuda.c and source/backend_cuda_launch.c for the subset the
 * expert-layer path uses: cards and arenas, staging memory, uploads and downloads with tickets, the embedded kernel
 * images and kernel_prepare, launch_run / launch_wait, graphs by stream capture, marks, peer_connect and device
 * timing. One stream and one mutex a card; any thread may call; the card's context is pushed for the call.
 * A card that reported a driver error once is failed: it begins no new work and answers STATUS_DEVICE_ERROR.
 */
#include "anemone_b200_backend.h"

#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "driver_api.h"
#include "kernel_images.h"

#define CARD_MODULES_MOST 24u
#define NANOSECONDS_PER_SECOND 1000000000ull
#define POLL_NANOSECONDS 20000l
#define SMALL_WRITE_SLOTS 64u

struct prepared_kernel {
	const struct ab_kernel_image *image;
	char function[96];
	CUfunction handle;
	uint32_t argument_byte_count;
};

struct transfer_ticket {
	CUevent done;
	uint64_t ticket; /* 0: slot free */
};

/* An address word of the arena as the host remembers it: copy launches name memory by such words. */
#define PEER_WORDS_MOST 256u
struct peer_word {
	uint64_t word_offset;
	CUdeviceptr address;
	uint64_t byte_count; /* from the address to the end of the owner's arena */
};

struct ipc_mapping {
	unsigned char handle[BACKEND_B200_IPC_HANDLE_BYTES];
	CUdeviceptr base;
};

struct device_card {
	uint32_t index;
	CUdevice device;
	CUcontext context;
	CUstream stream;
	CUdeviceptr arena;
	uint64_t arena_byte_count;
	pthread_mutex_t mutex;
	bool failed;
	int shared_memory_most; /* opt-in bytes per block */
	int threads_most;
	CUmodule modules[CARD_MODULES_MOST]; /* by image index, loaded at first kernel_prepare of the file */
	struct prepared_kernel kernels[BACKEND_MAXIMUM_KERNELS];
	uint32_t kernel_count;
	CUgraphExec graphs[BACKEND_MAXIMUM_GRAPHS];
	uint32_t graph_kernel_nodes[BACKEND_MAXIMUM_GRAPHS];
	uint32_t graph_count;
	CUevent marks[BACKEND_MAXIMUM_MARKS];
	bool mark_set[BACKEND_MAXIMUM_MARKS];
	struct transfer_ticket transfers[BACKEND_MAXIMUM_UPLOADS_IN_FLIGHT];
	uint64_t next_ticket, finished_ticket, failed_ticket;
	CUevent measure_begin_event, measure_end_event;
	int measure_state; /* 0 idle, 1 begun, 2 ended */
	struct ipc_mapping mappings[BACKEND_MAXIMUM_CARDS];
	uint32_t mapping_count;
	struct peer_word peer_words[PEER_WORDS_MOST]; /* what peer_connect wrote where: a copy launch's places */
	uint32_t peer_word_count;
	uint64_t *small_words; /* page-locked: address words written at load */
	uint32_t small_word_next;
	uint64_t launches_queued;
};

struct staging_block {
	void *memory;
	uint64_t byte_count;
};

static pthread_mutex_t global_mutex = PTHREAD_MUTEX_INITIALIZER;
static struct device_card *open_cards[BACKEND_MAXIMUM_CARDS];
static struct staging_block staging_blocks[BACKEND_MAXIMUM_STAGING_BLOCKS];

static uint64_t now_nanoseconds(void)
{
	struct timespec now;
	(void)clock_gettime(CLOCK_MONOTONIC, &now);
	return (uint64_t)now.tv_sec * NANOSECONDS_PER_SECOND + (uint64_t)now.tv_nsec;
}

static void pause_briefly(void)
{
	const struct timespec pause = { 0, POLL_NANOSECONDS };
	(void)nanosleep(&pause, NULL);
}

/* One error line for a driver failure; the card, if any, becomes failed. */
static result_status driver_failure(struct device_card *card, const char *what, CUresult result)
{
	const struct ab_driver *const cu = ab_driver();
	const char *text = NULL;
	if (cu != NULL)
		(void)cu->cuGetErrorString(result, &text);
	(void)fprintf(stderr, "anemone_b200: card %d: %s failed: %s (%d)\n", card != NULL ? (int)card->index : -1, what,
		      text != NULL ? text : "unknown error", (int)result);
	if (card != NULL)
		card->failed = true;
	return result == CUDA_ERROR_OUT_OF_MEMORY ? STATUS_OUT_OF_MEMORY : STATUS_DEVICE_ERROR;
}

#define DRIVER(card, call)                                               \
	do {                                                             \
		const CUresult driver_result_ = cu->call;                \
		if (driver_result_ != CUDA_SUCCESS) {                    \
			status = driver_failure(card, #call, driver_result_); \
			goto done;                                       \
		}                                                        \
	} while (0)

/* Every entry: lock the card, push its context; leave through `done`. */
#define CARD_ENTER(card)                                                   \
	const struct ab_driver *const cu = ab_driver();                    \
	result_status status = STATUS_OK;                                  \
	if (cu == NULL)                                                    \
		return STATUS_UNSUPPORTED;                                 \
	(void)pthread_mutex_lock(&(card)->mutex);                          \
	if (cu->cuCtxPushCurrent((card)->context) != CUDA_SUCCESS) {       \
		(card)->failed = true;                                     \
		(void)pthread_mutex_unlock(&(card)->mutex);                \
		return STATUS_DEVICE_ERROR;                                \
	}
#define CARD_LEAVE(card)                                  \
	do {                                              \
		CUcontext popped_;                        \
		(void)cu->cuCtxPopCurrent(&popped_);      \
		(void)pthread_mutex_unlock(&(card)->mutex); \
		return status;                            \
	} while (0)

static bool range_inside(uint64_t offset, uint64_t bytes, uint64_t capacity)
{
	return offset <= capacity && bytes <= capacity - offset;
}

/* ------------------------------------------------------------------ cards */

static result_status cuda_card_count(uint32_t *card_count_out)
{
	if (card_count_out == NULL)
		return STATUS_INVALID_ARGUMENT;
	const struct ab_driver *const cu = ab_driver();
	int count = 0;
	if (cu != NULL && cu->cuDeviceGetCount(&count) != CUDA_SUCCESS)
		return STATUS_DEVICE_ERROR;
	if (count > BACKEND_MAXIMUM_CARDS)
		return STATUS_UNSUPPORTED;
	*card_count_out = (uint32_t)count;
	return STATUS_OK;
}

static uint32_t arithmetic_class_of(const struct ab_driver *cu, CUdevice device)
{
	int major = 0;
	if (cu->cuDeviceGetAttribute(&major, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR, device) != CUDA_SUCCESS)
		return 0;
	return major == 10 ? ARITHMETIC_CLASS_SM_100 : 0u;
}

static result_status cuda_card_describe(uint32_t card_index, struct card_description_record *description_out)
{
	uint32_t count = 0;
	if (description_out == NULL || cuda_card_count(&count) != STATUS_OK || card_index >= count)
		return STATUS_INVALID_ARGUMENT;
	const struct ab_driver *const cu = ab_driver();
	struct card_description_record description;
	memset(&description, 0, sizeof(description));
	CUdevice device;
	size_t total = 0;
	if (cu->cuDeviceGet(&device, (int)card_index) != CUDA_SUCCESS ||
	    cu->cuDeviceGetName(description.name, CARD_NAME_CAPACITY - 1, device) != CUDA_SUCCESS ||
	    cu->cuDeviceTotalMem(&total, device) != CUDA_SUCCESS)
		return STATUS_DEVICE_ERROR;
	(void)cu->cuDeviceGetPCIBusId(description.bus_address, CARD_BUS_ADDRESS_CAPACITY - 1, device);
	description.arithmetic_class = arithmetic_class_of(cu, device);
	description.memory_total_bytes = total;
	description.memory_free_bytes = total; /* refined below where a context can be had */
	description.memory_reserved_bytes = BACKEND_CUDA_MEMORY_RESERVED_BYTES;
	CUcontext context;
	if (cu->cuDevicePrimaryCtxRetain(&context, device) == CUDA_SUCCESS) {
		if (cu->cuCtxPushCurrent(context) == CUDA_SUCCESS) {
			size_t free_bytes = 0, total_bytes = 0;
			if (cu->cuMemGetInfo(&free_bytes, &total_bytes) == CUDA_SUCCESS)
				description.memory_free_bytes = free_bytes;
			CUcontext popped;
			(void)cu->cuCtxPopCurrent(&popped);
		}
		(void)cu->cuDevicePrimaryCtxRelease(device);
	}
	*description_out = description;
	return STATUS_OK;
}

static void card_release(const struct ab_driver *cu, struct device_card *card)
{
	if (card->context != NULL && cu->cuCtxPushCurrent(card->context) == CUDA_SUCCESS) {
		for (uint32_t graph = 0; graph < card->graph_count; graph++)
			(void)cu->cuGraphExecDestroy(card->graphs[graph]);
		for (uint32_t mark = 0; mark < BACKEND_MAXIMUM_MARKS; mark++)
			if (card->marks[mark] != NULL)
				(void)cu->cuEventDestroy(card->marks[mark]);
		for (uint32_t slot = 0; slot < BACKEND_MAXIMUM_UPLOADS_IN_FLIGHT; slot++)
			if (card->transfers[slot].done != NULL)
				(void)cu->cuEventDestroy(card->transfers[slot].done);
		if (card->measure_begin_event != NULL)
			(void)cu->cuEventDestroy(card->measure_begin_event);
		if (card->measure_end_event != NULL)
			(void)cu->cuEventDestroy(card->measure_end_event);
		for (uint32_t mapping = 0; mapping < card->mapping_count; mapping++)
			(void)cu->cuIpcCloseMemHandle(card->mappings[mapping].base);
		for (uint32_t module = 0; module < CARD_MODULES_MOST; module++)
			if (card->modules[module] != NULL)
				(void)cu->cuModuleUnload(card->modules[module]);
		if (card->small_words != NULL)
			(void)cu->cuMemFreeHost(card->small_words);
		if (card->arena != 0)
			(void)cu->cuMemFree(card->arena);
		if (card->stream != NULL)
			(void)cu->cuStreamDestroy(card->stream);
		CUcontext popped;
		(void)cu->cuCtxPopCurrent(&popped);
	}
	if (card->context != NULL)
		(void)cu->cuDevicePrimaryCtxRelease(card->device);
	(void)pthread_mutex_destroy(&card->mutex);
	free(card);
}

static result_status cuda_card_open(uint32_t card_index, uint64_t arena_byte_count, struct device_card **card_out)
{
	uint32_t count = 0;
	if (card_out == NULL || arena_byte_count == 0 || cuda_card_count(&count) != STATUS_OK || card_index >= count)
		return STATUS_INVALID_ARGUMENT;
	const struct ab_driver *const cu = ab_driver();
	result_status status = STATUS_OK;
	(void)pthread_mutex_lock(&global_mutex);
	struct device_card *card = NULL;
	if (open_cards[card_index] != NULL) {
		status = STATUS_INVALID_ARGUMENT; /* opened once */
		goto unlock;
	}
	card = calloc(1, sizeof(*card));
	if (card == NULL) {
		status = STATUS_OUT_OF_MEMORY;
		goto unlock;
	}
	card->index = card_index;
	(void)pthread_mutex_init(&card->mutex, NULL);
	bool pushed = false;
	if (cu->cuDeviceGet(&card->device, (int)card_index) != CUDA_SUCCESS ||
	    cu->cuDevicePrimaryCtxRetain(&card->context, card->device) != CUDA_SUCCESS) {
		card->context = NULL;
		status = STATUS_DEVICE_ERROR;
		goto fail;
	}
	if (cu->cuCtxPushCurrent(card->context) != CUDA_SUCCESS) {
		status = STATUS_DEVICE_ERROR;
		goto fail;
	}
	pushed = true;
	(void)cu->cuDeviceGetAttribute(&card->shared_memory_most,
				       CU_DEVICE_ATTRIBUTE_MAX_SHARED_MEMORY_PER_BLOCK_OPTIN, card->device);
	(void)cu->cuDeviceGetAttribute(&card->threads_most, CU_DEVICE_ATTRIBUTE_MAX_THREADS_PER_BLOCK, card->device);
	CUresult result = cu->cuStreamCreate(&card->stream, CU_STREAM_NON_BLOCKING);
	if (result == CUDA_SUCCESS)
		result = cu->cuMemAlloc(&card->arena, arena_byte_count);
	if (result == CUDA_SUCCESS)
		result = cu->cuMemHostAlloc((void **)&card->small_words, SMALL_WRITE_SLOTS * sizeof(uint64_t),
					    CU_MEMHOSTALLOC_PORTABLE);
	if (result != CUDA_SUCCESS) {
		status = driver_failure(card, "opening the card", result);
		goto fail;
	}
	card->arena_byte_count = arena_byte_count;
	card->next_ticket = 1;
	{
		CUcontext popped;
		(void)cu->cuCtxPopCurrent(&popped);
	}
	open_cards[card_index] = card;
	*card_out = card;
	goto unlock;
fail:
	if (pushed) {
		CUcontext popped;
		(void)cu->cuCtxPopCurrent(&popped);
	}
	card_release(cu, card);
unlock:
	(void)pthread_mutex_unlock(&global_mutex);
	return status;
}

static void cuda_card_close(struct device_card *card, uint64_t wait_limit_nanoseconds)
{
	const struct ab_driver *const cu = ab_driver();
	if (card == NULL || cu == NULL)
		return;
	(void)pthread_mutex_lock(&card->mutex);
	if (cu->cuCtxPushCurrent(card->context) == CUDA_SUCCESS) {
		const uint64_t deadline = now_nanoseconds() + wait_limit_nanoseconds;
		CUresult state;
		while ((state = cu->cuStreamQuery(card->stream)) == CUDA_ERROR_NOT_READY && now_nanoseconds() < deadline)
			pause_briefly();
		if (state == CUDA_ERROR_NOT_READY) {
			(void)fprintf(stderr, "anemone_b200: card %u: work still queued at close; draining\n", card->index);
			state = cu->cuStreamSynchronize(card->stream);
		}
		CUcontext popped;
		(void)cu->cuCtxPopCurrent(&popped);
		if (state != CUDA_SUCCESS) {
			/* a failed drain retains the failed card and what its copies may still read */
			(void)driver_failure(card, "draining at close", state);
			(void)pthread_mutex_unlock(&card->mutex);
			return;
		}
	}
	(void)pthread_mutex_unlock(&card->mutex);
	(void)pthread_mutex_lock(&global_mutex);
	open_cards[card->index] = NULL;
	(void)pthread_mutex_unlock(&global_mutex);
	card_release(cu, card);
}

/* ------------------------------------------------------------------ staging, uploads, downloads */

static result_status cuda_staging_allocate(uint64_t byte_count, void **page_locked_memory_out)
{
	const struct ab_driver *const cu = ab_driver();
	if (page_locked_memory_out == NULL || byte_count == 0)
		return STATUS_INVALID_ARGUMENT;
	if (cu == NULL)
		return STATUS_UNSUPPORTED;
	result_status status = STATUS_BUSY_VALUE;
	(void)pthread_mutex_lock(&global_mutex);
	for (uint32_t slot = 0; slot < BACKEND_MAXIMUM_STAGING_BLOCKS; slot++) {
		if (staging_blocks[slot].memory != NULL)
			continue;
		/* page-locked for every context; a device must exist for the allocation to have a context */
		CUcontext context = NULL;
		CUdevice device;
		void *memory = NULL;
		if (cu->cuDeviceGet(&device, 0) != CUDA_SUCCESS ||
		    cu->cuDevicePrimaryCtxRetain(&context, device) != CUDA_SUCCESS) {
			status = STATUS_DEVICE_ERROR;
			break;
		}
		CUresult result = cu->cuCtxPushCurrent(context);
		if (result == CUDA_SUCCESS) {
			result = cu->cuMemHostAlloc(&memory, byte_count, CU_MEMHOSTALLOC_PORTABLE);
			CUcontext popped;
			(void)cu->cuCtxPopCurrent(&popped);
		}
		/* the retained context stays retained while the block lives: its memory belongs to it */
		if (result != CUDA_SUCCESS) {
			(void)cu->cuDevicePrimaryCtxRelease(device);
			status = result == CUDA_ERROR_OUT_OF_MEMORY ? STATUS_OUT_OF_MEMORY : STATUS_DEVICE_ERROR;
			break;
		}
		staging_blocks[slot].memory = memory;
		staging_blocks[slot].byte_count = byte_count;
		*page_locked_memory_out = memory;
		status = STATUS_OK;
		break;
	}
	(void)pthread_mutex_unlock(&global_mutex);
	return status;
}

static void cuda_staging_free(void *page_locked_memory)
{
	const struct ab_driver *const cu = ab_driver();
	if (page_locked_memory == NULL || cu == NULL)
		return;
	(void)pthread_mutex_lock(&global_mutex);
	bool found = false;
	for (uint32_t slot = 0; slot < BACKEND_MAXIMUM_STAGING_BLOCKS && !found; slot++) {
		if (staging_blocks[slot].memory != page_locked_memory)
			continue;
		found = true;
		staging_blocks[slot].memory = NULL;
		CUdevice device;
		CUcontext context;
		if (cu->cuDeviceGet(&device, 0) == CUDA_SUCCESS &&
		    cu->cuDevicePrimaryCtxRetain(&context, device) == CUDA_SUCCESS) {
			if (cu->cuCtxPushCurrent(context) == CUDA_SUCCESS) {
				(void)cu->cuMemFreeHost(page_locked_memory);
				CUcontext popped;
				(void)cu->cuCtxPopCurrent(&popped);
			}
			(void)cu->cuDevicePrimaryCtxRelease(device); /* this call's */
			(void)cu->cuDevicePrimaryCtxRelease(device); /* the allocation's */
		}
	}
	(void)pthread_mutex_unlock(&global_mutex);
	if (!found)
		(void)fprintf(stderr, "anemone_b200: staging_free of an address that is no block's start\n");
}

static bool inside_one_staging_block(const void *memory, uint64_t byte_count)
{
	bool inside = false;
	(void)pthread_mutex_lock(&global_mutex);
	for (uint32_t slot = 0; slot < BACKEND_MAXIMUM_STAGING_BLOCKS && !inside; slot++) {
		const unsigned char *const begin = staging_blocks[slot].memory;
		inside = begin != NULL && (const unsigned char *)memory >= begin &&
			 range_inside((uint64_t)((const unsigned char *)memory - begin), byte_count,
				      staging_blocks[slot].byte_count);
	}
	(void)pthread_mutex_unlock(&global_mutex);
	return inside;
}

/* Retire finished transfers in ticket order; with the card's mutex held and its context current. */
static void transfers_poll(const struct ab_driver *cu, struct device_card *card)
{
	for (;;) {
		struct transfer_ticket *oldest = NULL;
		for (uint32_t slot = 0; slot < BACKEND_MAXIMUM_UPLOADS_IN_FLIGHT; slot++) {
			struct transfer_ticket *const transfer = &card->transfers[slot];
			if (transfer->ticket != 0 && (oldest == NULL || transfer->ticket < oldest->ticket))
				oldest = transfer;
		}
		if (oldest == NULL)
			return;
		const CUresult state = cu->cuEventQuery(oldest->done);
		if (state == CUDA_ERROR_NOT_READY)
			return;
		if (state != CUDA_SUCCESS) {
			if (card->failed_ticket == 0)
				card->failed_ticket = oldest->ticket;
			(void)driver_failure(card, "a transfer", state);
			return;
		}
		card->finished_ticket = oldest->ticket;
		oldest->ticket = 0;
	}
}

static result_status transfer_begin(struct device_card *card, uint64_t arena_byte_offset, void *host,
				    uint64_t byte_count, uint64_t *ticket_out, bool upload)
{
	if (card == NULL || host == NULL || ticket_out == NULL || byte_count == 0 ||
	    !range_inside(arena_byte_offset, byte_count, card->arena_byte_count) ||
	    !inside_one_staging_block(host, byte_count))
		return STATUS_INVALID_ARGUMENT;
	CARD_ENTER(card);
	if (card->failed) {
		status = STATUS_DEVICE_ERROR;
		goto done;
	}
	transfers_poll(cu, card);
	struct transfer_ticket *transfer = NULL;
	for (uint32_t slot = 0; slot < BACKEND_MAXIMUM_UPLOADS_IN_FLIGHT && transfer == NULL; slot++)
		if (card->transfers[slot].ticket == 0)
			transfer = &card->transfers[slot];
	if (transfer == NULL) {
		status = STATUS_BUSY_VALUE;
		goto done;
	}
	if (transfer->done == NULL)
		DRIVER(card, cuEventCreate(&transfer->done, CU_EVENT_DISABLE_TIMING));
	if (upload)
		DRIVER(card, cuMemcpyHtoDAsync(card->arena + arena_byte_offset, host, byte_count, card->stream));
	else
		DRIVER(card, cuMemcpyDtoHAsync(host, card->arena + arena_byte_offset, byte_count, card->stream));
	DRIVER(card, cuEventRecord(transfer->done, card->stream));
	transfer->ticket = card->next_ticket++;
	*ticket_out = transfer->ticket;
done:
	CARD_LEAVE(card);
}

static result_status cuda_upload_begin(struct device_card *card, uint64_t arena_byte_offset,
				       const void *page_locked_source, uint64_t byte_count, uint64_t *upload_ticket_out)
{
	return transfer_begin(card, arena_byte_offset, (void *)(uintptr_t)page_locked_source, byte_count,
			      upload_ticket_out, true);
}

static result_status cuda_download_begin(struct device_card *card, uint64_t arena_byte_offset,
					 void *page_locked_destination, uint64_t byte_count,
					 uint64_t *download_ticket_out)
{
	return transfer_begin(card, arena_byte_offset, page_locked_destination, byte_count, download_ticket_out, false);
}

static result_status cuda_upload_wait(struct device_card *card, uint64_t upload_ticket,
				      uint64_t wait_limit_nanoseconds)
{
	if (card == NULL || upload_ticket == 0)
		return STATUS_INVALID_ARGUMENT;
	const uint64_t deadline = now_nanoseconds() + wait_limit_nanoseconds;
	for (;;) {
		CARD_ENTER(card);
		if (upload_ticket >= card->next_ticket) {
			status = STATUS_INVALID_ARGUMENT;
		} else {
			transfers_poll(cu, card);
			if (card->failed_ticket != 0 && upload_ticket >= card->failed_ticket)
				status = STATUS_DEVICE_ERROR;
			else if (upload_ticket <= card->finished_ticket)
				status = STATUS_OK;
			else
				status = card->failed ? STATUS_DEVICE_ERROR : STATUS_TIMED_OUT;
		}
		if (status != STATUS_TIMED_OUT || now_nanoseconds() >= deadline)
			CARD_LEAVE(card);
		{
			CUcontext popped;
			(void)cu->cuCtxPopCurrent(&popped);
			(void)pthread_mutex_unlock(&card->mutex);
		}
		pause_briefly();
	}
}

/* ------------------------------------------------------------------ kernels */

/* kernel images a caller registered at run time (backend_b200_image_register), behind the embedded ones */
#define REGISTERED_IMAGES_MOST 4u
static struct ab_kernel_image registered_images[REGISTERED_IMAGES_MOST];
static char registered_names[REGISTERED_IMAGES_MOST][64];
static uint32_t registered_image_count;

static const struct ab_kernel_image *image_of(const char *kernel_file_name, uint32_t *index_out)
{
	for (uint32_t index = 0; index < ab_kernel_image_count; index++)
		if (strcmp(ab_kernel_images[index].file_name, kernel_file_name) == 0) {
			*index_out = index;
			return &ab_kernel_images[index];
		}
	const struct ab_kernel_image *found = NULL;
	(void)pthread_mutex_lock(&global_mutex);
	for (uint32_t index = 0; index < registered_image_count; index++)
		if (strcmp(registered_images[index].file_name, kernel_file_name) == 0) {
			*index_out = ab_kernel_image_count + index;
			found = &registered_images[index];
		}
	(void)pthread_mutex_unlock(&global_mutex);
	return found;
}

result_status backend_b200_image_register(const char *kernel_file_name, const void *image, uint64_t image_byte_count)
{
	if (kernel_file_name == NULL || image == NULL || image_byte_count == 0 || kernel_file_name[0] == 0 ||
	    strlen(kernel_file_name) >= sizeof(registered_names[0]))
		return STATUS_INVALID_ARGUMENT;
	uint32_t taken = 0;
	if (image_of(kernel_file_name, &taken) != NULL)
		return STATUS_INVALID_ARGUMENT; /* a name is never given twice: no embedded file is shadowed */
	unsigned char *const copy = malloc(image_byte_count + 1u);
	if (copy == NULL)
		return STATUS_OUT_OF_MEMORY;
	memcpy(copy, image, image_byte_count);
	copy[image_byte_count] = 0;
	result_status status = STATUS_OK;
	(void)pthread_mutex_lock(&global_mutex);
	if (registered_image_count == REGISTERED_IMAGES_MOST ||
	    ab_kernel_image_count + registered_image_count >= CARD_MODULES_MOST) {
		status = STATUS_BUSY_VALUE;
	} else {
		const uint32_t slot = registered_image_count;
		(void)snprintf(registered_names[slot], sizeof(registered_names[slot]), "%s", kernel_file_name);
		registered_images[slot].file_name = registered_names[slot];
		registered_images[slot].begin = copy;
		registered_images[slot].end = copy + image_byte_count;
		registered_image_count = slot + 1u;
	}
	(void)pthread_mutex_unlock(&global_mutex);
	if (status != STATUS_OK)
		free(copy);
	return status;
}

static result_status cuda_kernel_prepare(struct device_card *card, const char *kernel_file_name,
					 const char *function_name, uint32_t argument_byte_count,
					 uint32_t *kernel_out)
{
	if (card == NULL || kernel_file_name == NULL || function_name == NULL || kernel_out == NULL ||
	    argument_byte_count == 0 || argument_byte_count > LAUNCH_ARGUMENT_BYTES ||
	    strlen(function_name) >= sizeof(card->kernels[0].function))
		return STATUS_INVALID_ARGUMENT;
	uint32_t image_index = 0;
	const struct ab_kernel_image *const image = image_of(kernel_file_name, &image_index);
	if (image == NULL || image_index >= CARD_MODULES_MOST) {
		(void)fprintf(stderr, "anemone_b200: no sm_100a build of kernel file %s\n", kernel_file_name);
		return STATUS_UNSUPPORTED;
	}
	CARD_ENTER(card);
	if (card->failed) {
		status = STATUS_DEVICE_ERROR;
		goto done;
	}
	if (arithmetic_class_of(cu, card->device) != ARITHMETIC_CLASS_SM_100) {
		(void)fprintf(stderr, "anemone_b200: card %u is not compute capability 10.x: no kernel build runs on it\n",
			      card->index);
		status = STATUS_UNSUPPORTED;
		goto done;
	}
	for (uint32_t kernel = 0; kernel < card->kernel_count; kernel++) {
		if (card->kernels[kernel].image == image && strcmp(card->kernels[kernel].function, function_name) == 0) {
			if (card->kernels[kernel].argument_byte_count != argument_byte_count) {
				status = STATUS_INVALID_ARGUMENT;
				goto done;
			}
			*kernel_out = kernel;
			goto done;
		}
	}
	if (card->kernel_count == BACKEND_MAXIMUM_KERNELS) {
		status = STATUS_BUSY_VALUE;
		goto done;
	}
	if (card->modules[image_index] == NULL)
		DRIVER(card, cuModuleLoadData(&card->modules[image_index], image->begin));
	CUfunction function;
	if (cu->cuModuleGetFunction(&function, card->modules[image_index], function_name) != CUDA_SUCCESS) {
		(void)fprintf(stderr, "anemone_b200: kernel file %s has no function %s\n", kernel_file_name, function_name);
		status = STATUS_INVALID_ARGUMENT;
		goto done;
	}
	/* exactly (record of argument_byte_count bytes, address): a third parameter must not exist */
	size_t offset = 0, size = 0;
	if (cu->cuFuncGetParamInfo(function, 0, &offset, &size) != CUDA_SUCCESS || size != argument_byte_count ||
	    cu->cuFuncGetParamInfo(function, 1, &offset, &size) != CUDA_SUCCESS || size != sizeof(CUdeviceptr) ||
	    cu->cuFuncGetParamInfo(function, 2, &offset, &size) == CUDA_SUCCESS) {
		(void)fprintf(stderr, "anemone_b200: %s/%s does not take (record of %u bytes, arena address)\n",
			      kernel_file_name, function_name, argument_byte_count);
		status = STATUS_INVALID_ARGUMENT;
		goto done;
	}
	int static_shared = 0;
	DRIVER(card, cuFuncGetAttribute(&static_shared, CU_FUNC_ATTRIBUTE_SHARED_SIZE_BYTES, function));
	DRIVER(card, cuFuncSetAttribute(function, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES,
					card->shared_memory_most - static_shared));
	struct prepared_kernel *const prepared = &card->kernels[card->kernel_count];
	prepared->image = image;
	prepared->handle = function;
	prepared->argument_byte_count = argument_byte_count;
	(void)snprintf(prepared->function, sizeof(prepared->function), "%s", function_name);
	*kernel_out = card->kernel_count++;
done:
	CARD_LEAVE(card);
}

/* A copy's place: the card's own arena, or the memory behind an address word a connect call wrote. */
static bool copy_place_resolve(const struct device_card *card, struct exchange_place place, uint64_t byte_count,
			       CUdeviceptr *address_out)
{
	CUdeviceptr base = card->arena;
	uint64_t limit = card->arena_byte_count;
	if (place.address_word_offset != EXCHANGE_OWN_ARENA) {
		const struct peer_word *found = NULL;
		for (uint32_t entry = 0; entry < card->peer_word_count; entry++)
			if (card->peer_words[entry].word_offset == place.address_word_offset)
				found = &card->peer_words[entry];
		if (found == NULL)
			return false;
		base = found->address;
		limit = found->byte_count;
	}
	if (!range_inside(place.offset, byte_count, limit))
		return false;
	*address_out = base + place.offset;
	return true;
}

static bool copy_is_valid(const struct device_card *card, const struct kernel_launch *launch, CUdeviceptr *source_out,
			  CUdeviceptr *destination_out)
{
	struct exchange_copy_arguments copy;
	if (launch->argument_byte_count != sizeof(copy) || launch->dynamic_shared_byte_count != 0 ||
	    launch->branch > LAUNCH_SIDE_MORE)
		return false;
	for (uint32_t byte = sizeof(copy); byte < LAUNCH_ARGUMENT_BYTES; byte++)
		if (launch->argument[byte] != 0)
			return false;
	memcpy(&copy, launch->argument, sizeof(copy));
	return copy.byte_count != 0 && copy_place_resolve(card, copy.source, copy.byte_count, source_out) &&
	       copy_place_resolve(card, copy.destination, copy.byte_count, destination_out);
}

static void peer_word_remember(struct device_card *card, uint64_t word_offset, CUdeviceptr address, uint64_t byte_count)
{
	uint32_t entry = 0;
	while (entry < card->peer_word_count && card->peer_words[entry].word_offset != word_offset)
		entry++;
	if (entry == PEER_WORDS_MOST)
		return; /* the word is written all the same: kernels read it; only copy launches cannot name it */
	card->peer_words[entry] = (struct peer_word){ word_offset, address, byte_count };
	if (entry == card->peer_word_count)
		card->peer_word_count++;
}

static bool launch_is_valid(const struct device_card *card, const struct kernel_launch *launch)
{
	if (launch->kernel == BACKEND_COPY) {
		CUdeviceptr source, destination;
		return copy_is_valid(card, launch, &source, &destination);
	}
	if (launch->kernel >= card->kernel_count ||
	    launch->argument_byte_count != card->kernels[launch->kernel].argument_byte_count ||
	    launch->dynamic_shared_byte_count > (uint32_t)card->shared_memory_most ||
	    (launch->branch > LAUNCH_SIDE_MORE && launch->branch != (LAUNCH_CHAIN | LAUNCH_OVERLAPS_PREVIOUS)))
		return false;
	uint64_t threads = 1;
	for (uint32_t axis = 0; axis < LAUNCH_DIMENSIONS; axis++) {
		if (launch->grid[axis] == 0 || launch->block[axis] == 0)
			return false;
		threads *= launch->block[axis];
	}
	if (threads > (uint64_t)card->threads_most)
		return false;
	for (uint32_t byte = launch->argument_byte_count; byte < LAUNCH_ARGUMENT_BYTES; byte++)
		if (launch->argument[byte] != 0)
			return false;
	return true;
}

/* Queue the table on the card's stream (which may be capturing). Context current, mutex held. */
static result_status launches_queue(const struct ab_driver *cu, struct device_card *card,
				    const struct kernel_launch *launches, uint32_t launch_count)
{
	result_status status = STATUS_OK;
	for (uint32_t index = 0; index < launch_count; index++) {
		const struct kernel_launch *const launch = &launches[index];
		if (launch->kernel == BACKEND_COPY) {
			CUdeviceptr source = 0, destination = 0;
			struct exchange_copy_arguments copy;
			memcpy(&copy, launch->argument, sizeof(copy));
			if (!copy_is_valid(card, launch, &source, &destination))
				return STATUS_INVALID_ARGUMENT;
			DRIVER(card, cuMemcpyDtoDAsync(destination, source, copy.byte_count, card->stream));
			continue;
		}
		unsigned char record[LAUNCH_ARGUMENT_BYTES];
		memcpy(record, launch->argument, launch->argument_byte_count);
		CUdeviceptr arena = card->arena;
		void *parameters[] = { record, &arena };
		if ((launch->branch & LAUNCH_OVERLAPS_PREVIOUS) != 0 && index != 0) {
			/* behind the launch before it by a programmatic edge: it may start once that launch lets it */
			CUlaunchAttribute attribute;
			memset(&attribute, 0, sizeof(attribute));
			attribute.id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
			attribute.value.programmaticStreamSerializationAllowed = 1;
			CUlaunchConfig config;
			memset(&config, 0, sizeof(config));
			config.gridDimX = launch->grid[0], config.gridDimY = launch->grid[1], config.gridDimZ = launch->grid[2];
			config.blockDimX = launch->block[0], config.blockDimY = launch->block[1];
			config.blockDimZ = launch->block[2];
			config.sharedMemBytes = launch->dynamic_shared_byte_count;
			config.hStream = card->stream;
			config.attrs = &attribute;
			config.numAttrs = 1;
			DRIVER(card, cuLaunchKernelEx(&config, card->kernels[launch->kernel].handle, parameters, NULL));
			continue;
		}
		DRIVER(card, cuLaunchKernel(card->kernels[launch->kernel].handle, launch->grid[0], launch->grid[1],
					    launch->grid[2], launch->block[0], launch->block[1], launch->block[2],
					    launch->dynamic_shared_byte_count, card->stream, parameters, NULL));
	}
done:
	return status;
}

static result_status table_check(const struct device_card *card, const struct kernel_launch *launches,
				 uint32_t launch_count)
{
	if (card == NULL || launches == NULL || launch_count == 0)
		return STATUS_INVALID_ARGUMENT;
	for (uint32_t index = 0; index < launch_count; index++)
		if (!launch_is_valid(card, &launches[index]))
			return STATUS_INVALID_ARGUMENT;
	return STATUS_OK;
}

static uint32_t kernel_launches_of(const struct kernel_launch *launches, uint32_t launch_count)
{
	uint32_t kernels = 0;
	for (uint32_t index = 0; index < launch_count; index++)
		kernels += launches[index].kernel != BACKEND_COPY;
	return kernels;
}

result_status backend_b200_launch_order(const struct kernel_launch *launches, uint32_t launch_count,
					struct launch_order *order_out)
{
	if (launches == NULL || order_out == NULL || launch_count == 0)
		return STATUS_INVALID_ARGUMENT;
	/* two passes: the grammar first, so that a refusal leaves order_out as it was */
	for (uint32_t pass = 0; pass < 2; pass++) {
		const uint32_t none = UINT32_MAX;
		uint32_t fork = none, run_last[LAUNCH_MOST_SIDE_RUNS], runs = 0;
		for (uint32_t index = 0; index < launch_count; index++) {
			const uint32_t overlap = (uint32_t)LAUNCH_OVERLAPS_PREVIOUS;
			const uint32_t branch = launches[index].branch == (LAUNCH_CHAIN | overlap) ? LAUNCH_CHAIN :
												  launches[index].branch;
			const uint32_t previous = index == 0 ? none : index - 1u;
			const uint32_t before = index == 0 ? LAUNCH_CHAIN : launches[index - 1u].branch & ~overlap;
			const bool in_side = before == LAUNCH_SIDE || before == LAUNCH_SIDE_MORE;
			uint32_t wanted[1u + LAUNCH_MOST_SIDE_RUNS], wanted_count = 0;
			switch (branch) {
			case LAUNCH_CHAIN:
				wanted[wanted_count++] = previous;
				break;
			case LAUNCH_SIDE:
				if (before == LAUNCH_SIDE_MORE)
					return STATUS_INVALID_ARGUMENT;
				if (before == LAUNCH_SIDE) { /* the run goes on */
					wanted[wanted_count++] = previous;
					run_last[runs - 1u] = index;
				} else { /* a fork: the launch before the run */
					fork = previous;
					wanted[wanted_count++] = fork;
					runs = 1;
					run_last[0] = index;
				}
				break;
			case LAUNCH_SIDE_MORE:
				if (!in_side || runs == LAUNCH_MOST_SIDE_RUNS)
					return STATUS_INVALID_ARGUMENT;
				wanted[wanted_count++] = fork;
				run_last[runs++] = index;
				break;
			case LAUNCH_RESUME:
				if (!in_side)
					return STATUS_INVALID_ARGUMENT;
				wanted[wanted_count++] = fork;
				break;
			case LAUNCH_JOIN:
				if (runs == 0)
					return STATUS_INVALID_ARGUMENT;
				for (uint32_t run = 0; run < runs; run++)
					if (run_last[run] != previous)
						wanted[wanted_count++] = run_last[run];
				wanted[wanted_count++] = previous; /* the largest index: the list stays ascending */
				runs = 0;
				break;
			default:
				return STATUS_INVALID_ARGUMENT;
			}
			if (pass == 0)
				continue;
			struct launch_order *const order = &order_out[index];
			memset(order, 0, sizeof(*order));
			for (uint32_t entry = 0; entry < wanted_count; entry++)
				if (wanted[entry] != none)
					order->behind[order->behind_count++] = wanted[entry];
		}
	}
	return STATUS_OK;
}

static bool table_is_a_plain_chain(const struct kernel_launch *launches, uint32_t launch_count)
{
	for (uint32_t index = 0; index < launch_count; index++)
		if (launches[index].kernel == BACKEND_COPY ||
		    (launches[index].branch & ~(uint32_t)LAUNCH_OVERLAPS_PREVIOUS) != LAUNCH_CHAIN)
			return false;
	return true;
}

/* The table as a graph built node by node, every node behind the nodes its launch's order names. Context current,
 * mutex held; the table has passed table_check and backend_b200_launch_order. */
static result_status graph_build(const struct ab_driver *cu, struct device_card *card,
				 const struct kernel_launch *launches, const struct launch_order *order,
				 uint32_t launch_count, CUgraphNode *nodes, CUgraph graph)
{
	result_status status = STATUS_OK;
	for (uint32_t index = 0; index < launch_count; index++) {
		const struct kernel_launch *const launch = &launches[index];
		CUgraphNode behind[1u + LAUNCH_MOST_SIDE_RUNS];
		for (uint32_t entry = 0; entry < order[index].behind_count; entry++)
			behind[entry] = nodes[order[index].behind[entry]];
		const CUgraphNode *const depends = order[index].behind_count == 0 ? NULL : behind;
		if (launch->kernel == BACKEND_COPY) {
			CUdeviceptr source = 0, destination = 0;
			struct exchange_copy_arguments copy;
			memcpy(&copy, launch->argument, sizeof(copy));
			if (!copy_is_valid(card, launch, &source, &destination))
				return STATUS_INVALID_ARGUMENT;
			CUDA_MEMCPY3D parameters;
			memset(&parameters, 0, sizeof(parameters));
			parameters.srcMemoryType = parameters.dstMemoryType = CU_MEMORYTYPE_DEVICE;
			parameters.srcDevice = source;
			parameters.dstDevice = destination;
			parameters.srcPitch = parameters.dstPitch = parameters.WidthInBytes = copy.byte_count;
			parameters.Height = parameters.Depth = 1;
			DRIVER(card, cuGraphAddMemcpyNode(&nodes[index], graph, depends, order[index].behind_count,
							  &parameters, card->context));
			continue;
		}
		unsigned char record[LAUNCH_ARGUMENT_BYTES];
		memcpy(record, launch->argument, launch->argument_byte_count);
		CUdeviceptr arena = card->arena;
		void *kernel_parameters[] = { record, &arena };
		CUDA_KERNEL_NODE_PARAMS parameters;
		memset(&parameters, 0, sizeof(parameters));
		parameters.func = card->kernels[launch->kernel].handle;
		parameters.gridDimX = launch->grid[0], parameters.gridDimY = launch->grid[1];
		parameters.gridDimZ = launch->grid[2];
		parameters.blockDimX = launch->block[0], parameters.blockDimY = launch->block[1];
		parameters.blockDimZ = launch->block[2];
		parameters.sharedMemBytes = launch->dynamic_shared_byte_count;
		parameters.kernelParams = kernel_parameters; /* copied into the node by the call */
		DRIVER(card, cuGraphAddKernelNode(&nodes[index], graph, depends, order[index].behind_count, &parameters));
	}
done:
	return status;
}

static result_status cuda_launch_run(struct device_card *card, const struct kernel_launch *launches,
				     uint32_t launch_count)
{
	if (card == NULL)
		return STATUS_INVALID_ARGUMENT;
	CARD_ENTER(card);
	status = card->failed ? STATUS_DEVICE_ERROR : table_check(card, launches, launch_count);
	if (status == STATUS_OK) {
		/* the eager form runs the table in its serial order, whatever its branches */
		status = launches_queue(cu, card, launches, launch_count);
		if (status == STATUS_OK)
			card->launches_queued += kernel_launches_of(launches, launch_count);
	}
	CARD_LEAVE(card);
}

static result_status cuda_launch_wait(struct device_card *card, uint64_t wait_limit_nanoseconds)
{
	if (card == NULL)
		return STATUS_INVALID_ARGUMENT;
	const uint64_t deadline = now_nanoseconds() + wait_limit_nanoseconds;
	for (;;) {
		CARD_ENTER(card);
		if (card->failed) {
			status = STATUS_DEVICE_ERROR;
		} else {
			const CUresult state = cu->cuStreamQuery(card->stream);
			status = state == CUDA_SUCCESS	       ? STATUS_OK :
				 state == CUDA_ERROR_NOT_READY ? STATUS_TIMED_OUT :
								 driver_failure(card, "the card's queued work", state);
		}
		if (status != STATUS_TIMED_OUT || now_nanoseconds() >= deadline)
			CARD_LEAVE(card);
		{
			CUcontext popped;
			(void)cu->cuCtxPopCurrent(&popped);
			(void)pthread_mutex_unlock(&card->mutex);
		}
		pause_briefly();
	}
}

static bool cuda_format_supported(uint32_t card_index, enum weight_format_code format)
{
	uint32_t count = 0;
	const struct ab_driver *const cu = ab_driver();
	CUdevice device;
	if (cu == NULL || cuda_card_count(&count) != STATUS_OK || card_index >= count ||
	    cu->cuDeviceGet(&device, (int)card_index) != CUDA_SUCCESS ||
	    arithmetic_class_of(cu, device) != ARITHMETIC_CLASS_SM_100)
		return false;
	return format == WEIGHT_FORMAT_EXL3;
}

/* ------------------------------------------------------------------ graphs, marks, peers, timing */

static result_status cuda_graph_capture(struct device_card *card, const struct kernel_launch *launches,
					uint32_t launch_count, uint32_t *graph_out)
{
	if (card == NULL || graph_out == NULL)
		return STATUS_INVALID_ARGUMENT;
	CARD_ENTER(card);
	CUgraph graph = NULL;
	struct launch_order *order = NULL;
	CUgraphNode *nodes = NULL;
	status = card->failed ? STATUS_DEVICE_ERROR : table_check(card, launches, launch_count);
	if (status != STATUS_OK)
		goto done;
	order = calloc(launch_count, sizeof(*order));
	nodes = calloc(launch_count, sizeof(*nodes));
	if (order == NULL || nodes == NULL) {
		status = STATUS_OUT_OF_MEMORY;
		goto done;
	}
	status = backend_b200_launch_order(launches, launch_count, order);
	if (status != STATUS_OK)
		goto done;
	if (card->graph_count == BACKEND_MAXIMUM_GRAPHS) {
		status = STATUS_BUSY_VALUE;
		goto done;
	}
	if (table_is_a_plain_chain(launches, launch_count)) {
		DRIVER(card, cuStreamBeginCapture(card->stream, CU_STREAM_CAPTURE_MODE_THREAD_LOCAL));
		status = launches_queue(cu, card, launches, launch_count);
		const CUresult ended = cu->cuStreamEndCapture(card->stream, &graph);
		if (status == STATUS_OK && ended != CUDA_SUCCESS)
			status = driver_failure(card, "ending the capture", ended);
	} else {
		DRIVER(card, cuGraphCreate(&graph, 0));
		status = graph_build(cu, card, launches, order, launch_count, nodes, graph);
	}
	if (status != STATUS_OK)
		goto done;
	DRIVER(card, cuGraphInstantiateWithFlags(&card->graphs[card->graph_count], graph, 0));
	card->graph_kernel_nodes[card->graph_count] = kernel_launches_of(launches, launch_count);
	*graph_out = card->graph_count++;
done:
	if (graph != NULL)
		(void)cu->cuGraphDestroy(graph);
	free(order);
	free(nodes);
	CARD_LEAVE(card);
}

static result_status cuda_graph_run(struct device_card *card, uint32_t graph)
{
	if (card == NULL)
		return STATUS_INVALID_ARGUMENT;
	CARD_ENTER(card);
	if (card->failed) {
		status = STATUS_DEVICE_ERROR;
	} else if (graph >= card->graph_count) {
		status = STATUS_INVALID_ARGUMENT;
	} else {
		DRIVER(card, cuGraphLaunch(card->graphs[graph], card->stream));
		card->launches_queued += card->graph_kernel_nodes[graph];
	}
done:
	CARD_LEAVE(card);
}

static result_status cuda_mark_record(struct device_card *card, uint32_t mark)
{
	if (card == NULL || mark >= BACKEND_MAXIMUM_MARKS)
		return STATUS_INVALID_ARGUMENT;
	CARD_ENTER(card);
	if (card->failed) {
		status = STATUS_DEVICE_ERROR;
		goto done;
	}
	if (card->marks[mark] == NULL)
		DRIVER(card, cuEventCreate(&card->marks[mark], CU_EVENT_DISABLE_TIMING));
	DRIVER(card, cuEventRecord(card->marks[mark], card->stream));
	card->mark_set[mark] = true;
done:
	CARD_LEAVE(card);
}

static result_status cuda_mark_follow(struct device_card *card, struct device_card *owner, uint32_t mark)
{
	if (card == NULL || owner == NULL || mark >= BACKEND_MAXIMUM_MARKS)
		return STATUS_INVALID_ARGUMENT;
	/* the owner's event is read without its mutex: events are created once and never destroyed before close */
	CARD_ENTER(card);
	if (card->failed || owner->failed)
		status = STATUS_DEVICE_ERROR;
	else if (owner->mark_set[mark])
		DRIVER(card, cuStreamWaitEvent(card->stream, owner->marks[mark], 0));
done:
	CARD_LEAVE(card);
}

/* Write one 64-bit word into the arena at load time (synchronous: the word is in place when the call returns). */
static result_status address_word_write(const struct ab_driver *cu, struct device_card *card, uint64_t word,
					uint64_t address_word_offset)
{
	result_status status = STATUS_OK;
	uint64_t *const slot = &card->small_words[card->small_word_next++ % SMALL_WRITE_SLOTS];
	*slot = word;
	DRIVER(card, cuMemcpyHtoD(card->arena + address_word_offset, slot, sizeof(word)));
done:
	return status;
}

static bool address_word_is_valid(const struct device_card *card, uint64_t address_word_offset)
{
	return address_word_offset % BACKEND_ADDRESS_WORD_BYTES == 0 &&
	       range_inside(address_word_offset, BACKEND_ADDRESS_WORD_BYTES, card->arena_byte_count);
}

static result_status cuda_peer_connect(struct device_card *accessor, struct device_card *owner,
				       uint64_t owner_offset, uint64_t address_word_offset)
{
	if (accessor == NULL || owner == NULL || owner_offset >= owner->arena_byte_count ||
	    !address_word_is_valid(accessor, address_word_offset))
		return STATUS_INVALID_ARGUMENT;
	CARD_ENTER(accessor);
	if (accessor->failed || owner->failed) {
		status = STATUS_DEVICE_ERROR;
		goto done;
	}
	if (accessor != owner) {
		int reachable = 0;
		DRIVER(accessor, cuDeviceCanAccessPeer(&reachable, accessor->device, owner->device));
		if (reachable == 0) {
			status = STATUS_UNSUPPORTED; /* no word is written */
			goto done;
		}
		const CUresult enabled = cu->cuCtxEnablePeerAccess(owner->context, 0);
		if (enabled != CUDA_SUCCESS && enabled != CUDA_ERROR_PEER_ACCESS_ALREADY_ENABLED) {
			status = driver_failure(accessor, "enabling peer access", enabled);
			goto done;
		}
	}
	status = address_word_write(cu, accessor, (uint64_t)owner->arena + owner_offset, address_word_offset);
	if (status == STATUS_OK)
		peer_word_remember(accessor, address_word_offset, owner->arena + owner_offset,
				   owner->arena_byte_count - owner_offset);
done:
	CARD_LEAVE(accessor);
}

static result_status cuda_measure_begin(struct device_card *card)
{
	if (card == NULL)
		return STATUS_INVALID_ARGUMENT;
	CARD_ENTER(card);
	if (card->failed) {
		status = STATUS_DEVICE_ERROR;
		goto done;
	}
	if (card->measure_state != 0) {
		status = STATUS_BUSY_VALUE;
		goto done;
	}
	if (card->measure_begin_event == NULL) {
		DRIVER(card, cuEventCreate(&card->measure_begin_event, CU_EVENT_DEFAULT));
		DRIVER(card, cuEventCreate(&card->measure_end_event, CU_EVENT_DEFAULT));
	}
	DRIVER(card, cuEventRecord(card->measure_begin_event, card->stream));
	card->measure_state = 1;
done:
	CARD_LEAVE(card);
}

static result_status cuda_measure_end(struct device_card *card)
{
	if (card == NULL)
		return STATUS_INVALID_ARGUMENT;
	CARD_ENTER(card);
	if (card->failed) {
		status = STATUS_DEVICE_ERROR;
		goto done;
	}
	if (card->measure_state != 1) {
		status = STATUS_INVALID_ARGUMENT;
		goto done;
	}
	DRIVER(card, cuEventRecord(card->measure_end_event, card->stream));
	card->measure_state = 2;
done:
	CARD_LEAVE(card);
}

static result_status cuda_measure_elapsed_us(struct device_card *card, uint64_t wait_limit_nanoseconds,
					     double *microseconds_out)
{
	if (card == NULL || microseconds_out == NULL)
		return STATUS_INVALID_ARGUMENT;
	const uint64_t deadline = now_nanoseconds() + wait_limit_nanoseconds;
	for (;;) {
		CARD_ENTER(card);
		if (card->failed) {
			status = STATUS_DEVICE_ERROR;
		} else if (card->measure_state != 2) {
			status = STATUS_INVALID_ARGUMENT;
		} else {
			const CUresult state = cu->cuEventQuery(card->measure_end_event);
			if (state == CUDA_ERROR_NOT_READY) {
				status = STATUS_TIMED_OUT;
			} else if (state != CUDA_SUCCESS) {
				status = driver_failure(card, "the timed work", state);
			} else {
				float milliseconds = 0;
				const CUresult elapsed = cu->cuEventElapsedTime(&milliseconds, card->measure_begin_event,
										card->measure_end_event);
				if (elapsed != CUDA_SUCCESS) {
					status = driver_failure(card, "reading the interval", elapsed);
				} else {
					*microseconds_out = (double)milliseconds * 1000.0;
					card->measure_state = 0;
				}
			}
		}
		if (status != STATUS_TIMED_OUT || now_nanoseconds() >= deadline)
			CARD_LEAVE(card);
		{
			CUcontext popped;
			(void)cu->cuCtxPopCurrent(&popped);
			(void)pthread_mutex_unlock(&card->mutex);
		}
		pause_briefly();
	}
}

/* ------------------------------------------------------------------ B200 extensions */

result_status backend_b200_ipc_export(struct device_card *card, unsigned char handle_out[BACKEND_B200_IPC_HANDLE_BYTES])
{
	_Static_assert(sizeof(CUipcMemHandle) == BACKEND_B200_IPC_HANDLE_BYTES, "inter-process handle size");
	if (card == NULL || handle_out == NULL)
		return STATUS_INVALID_ARGUMENT;
	CARD_ENTER(card);
	CUipcMemHandle handle;
	DRIVER(card, cuIpcGetMemHandle(&handle, card->arena));
	memcpy(handle_out, &handle, sizeof(handle));
done:
	CARD_LEAVE(card);
}

result_status backend_b200_ipc_connect(struct device_card *accessor,
				       const unsigned char handle[BACKEND_B200_IPC_HANDLE_BYTES], uint64_t owner_offset,
				       uint64_t address_word_offset)
{
	if (accessor == NULL || handle == NULL || !address_word_is_valid(accessor, address_word_offset))
		return STATUS_INVALID_ARGUMENT;
	CARD_ENTER(accessor);
	if (accessor->failed) {
		status = STATUS_DEVICE_ERROR;
		goto done;
	}
	CUdeviceptr base = 0;
	for (uint32_t mapping = 0; mapping < accessor->mapping_count; mapping++)
		if (memcmp(accessor->mappings[mapping].handle, handle, BACKEND_B200_IPC_HANDLE_BYTES) == 0)
			base = accessor->mappings[mapping].base;
	if (base == 0) {
		if (accessor->mapping_count == BACKEND_MAXIMUM_CARDS) {
			status = STATUS_BUSY_VALUE;
			goto done;
		}
		CUipcMemHandle opened;
		memcpy(&opened, handle, sizeof(opened));
		DRIVER(accessor, cuIpcOpenMemHandle(&base, opened, CU_IPC_MEM_LAZY_ENABLE_PEER_ACCESS));
		memcpy(accessor->mappings[accessor->mapping_count].handle, handle, BACKEND_B200_IPC_HANDLE_BYTES);
		accessor->mappings[accessor->mapping_count++].base = base;
	}
	status = address_word_write(cu, accessor, (uint64_t)base + owner_offset, address_word_offset);
	if (status == STATUS_OK) {
		/* how much of the owner's allocation lies behind the word: what a copy launch may name through it */
		CUdeviceptr range_base = 0;
		size_t range_bytes = 0;
		if (cu->cuMemGetAddressRange(&range_base, &range_bytes, base) == CUDA_SUCCESS &&
		    owner_offset < range_bytes - (size_t)(base - range_base))
			peer_word_remember(accessor, address_word_offset, base + owner_offset,
					   range_bytes - (size_t)(base - range_base) - owner_offset);
	}
done:
	CARD_LEAVE(accessor);
}

result_status backend_b200_fill(struct device_card *card, uint64_t arena_byte_offset, unsigned char value,
				uint64_t byte_count)
{
	if (card == NULL || byte_count == 0 || !range_inside(arena_byte_offset, byte_count, card->arena_byte_count))
		return STATUS_INVALID_ARGUMENT;
	CARD_ENTER(card);
	if (card->failed)
		status = STATUS_DEVICE_ERROR;
	else
		DRIVER(card, cuMemsetD8Async(card->arena + arena_byte_offset, value, byte_count, card->stream));
done:
	CARD_LEAVE(card);
}

result_status backend_b200_waits_expired(struct device_card *card, uint32_t *expired_out)
{
	if (card == NULL || expired_out == NULL)
		return STATUS_INVALID_ARGUMENT;
	uint32_t expired = 0;
	CARD_ENTER(card);
	if (card->failed) {
		status = STATUS_DEVICE_ERROR;
		goto done;
	}
	DRIVER(card, cuStreamSynchronize(card->stream));
	for (uint32_t module = 0; module < CARD_MODULES_MOST; module++) {
		CUdeviceptr address = 0;
		size_t bytes = 0;
		uint32_t word = 0;
		if (card->modules[module] == NULL ||
		    cu->cuModuleGetGlobal(&address, &bytes, card->modules[module], "exl3_wait_expired") != CUDA_SUCCESS ||
		    bytes != sizeof(word))
			continue; /* a kernel file without bounded barrier waits */
		DRIVER(card, cuMemcpyDtoH(&word, address, sizeof(word)));
		expired |= word;
	}
	*expired_out = expired;
done:
	CARD_LEAVE(card);
}

result_status backend_b200_step_run(struct device_card *card, uint32_t graph, uint64_t input_arena_offset,
				    const void *page_locked_input, uint64_t input_byte_count,
				    uint64_t output_arena_offset, void *page_locked_output, uint64_t output_byte_count)
{
	if (card == NULL ||
	    (input_byte_count != 0 &&
	     (page_locked_input == NULL || !range_inside(input_arena_offset, input_byte_count, card->arena_byte_count) ||
	      !inside_one_staging_block(page_locked_input, input_byte_count))) ||
	    (output_byte_count != 0 &&
	     (page_locked_output == NULL || !range_inside(output_arena_offset, output_byte_count, card->arena_byte_count) ||
	      !inside_one_staging_block(page_locked_output, output_byte_count))))
		return STATUS_INVALID_ARGUMENT;
	CARD_ENTER(card);
	if (card->failed) {
		status = STATUS_DEVICE_ERROR;
		goto done;
	}
	if (graph >= card->graph_count) {
		status = STATUS_INVALID_ARGUMENT;
		goto done;
	}
	if (input_byte_count != 0)
		DRIVER(card, cuMemcpyHtoDAsync(card->arena + input_arena_offset, page_locked_input, input_byte_count,
					       card->stream));
	DRIVER(card, cuGraphLaunch(card->graphs[graph], card->stream));
	card->launches_queued += card->graph_kernel_nodes[graph];
	if (output_byte_count != 0)
		DRIVER(card, cuMemcpyDtoHAsync(page_locked_output, card->arena + output_arena_offset, output_byte_count,
					       card->stream));
	DRIVER(card, cuStreamSynchronize(card->stream));
done:
	CARD_LEAVE(card);
}

result_status backend_b200_step_capture(struct device_card *card, const struct kernel_launch *launches,
					uint32_t launch_count, uint64_t input_arena_offset, const void *page_locked_input,
					uint64_t input_byte_count, uint64_t output_arena_offset, void *page_locked_output,
					uint64_t output_byte_count, uint32_t *graph_out)
{
	if (card == NULL || graph_out == NULL ||
	    (input_byte_count != 0 &&
	     (page_locked_input == NULL || !range_inside(input_arena_offset, input_byte_count, card->arena_byte_count) ||
	      !inside_one_staging_block(page_locked_input, input_byte_count))) ||
	    (output_byte_count != 0 &&
	     (page_locked_output == NULL || !range_inside(output_arena_offset, output_byte_count, card->arena_byte_count) ||
	      !inside_one_staging_block(page_locked_output, output_byte_count))))
		return STATUS_INVALID_ARGUMENT;
	CARD_ENTER(card);
	CUgraph graph = NULL;
	status = card->failed ? STATUS_DEVICE_ERROR : table_check(card, launches, launch_count);
	if (status != STATUS_OK)
		goto done;
	if (!table_is_a_plain_chain(launches, launch_count)) {
		status = STATUS_UNSUPPORTED; /* side runs and copy launches: graph_capture and backend_b200_step_run */
		goto done;
	}
	if (card->graph_count == BACKEND_MAXIMUM_GRAPHS) {
		status = STATUS_BUSY_VALUE;
		goto done;
	}
	DRIVER(card, cuStreamBeginCapture(card->stream, CU_STREAM_CAPTURE_MODE_THREAD_LOCAL));
	{
		CUresult copied = CUDA_SUCCESS;
		if (input_byte_count != 0)
			copied = cu->cuMemcpyHtoDAsync(card->arena + input_arena_offset, page_locked_input, input_byte_count,
						       card->stream);
		status = copied == CUDA_SUCCESS ? launches_queue(cu, card, launches, launch_count) :
						  driver_failure(card, "capturing the copy in", copied);
		if (status == STATUS_OK && output_byte_count != 0) {
			copied = cu->cuMemcpyDtoHAsync(page_locked_output, card->arena + output_arena_offset, output_byte_count,
						       card->stream);
			if (copied != CUDA_SUCCESS)
				status = driver_failure(card, "capturing the copy out", copied);
		}
		const CUresult ended = cu->cuStreamEndCapture(card->stream, &graph);
		if (status == STATUS_OK && ended != CUDA_SUCCESS)
			status = driver_failure(card, "ending the capture", ended);
	}
	if (status != STATUS_OK)
		goto done;
	DRIVER(card, cuGraphInstantiateWithFlags(&card->graphs[card->graph_count], graph, 0));
	card->graph_kernel_nodes[card->graph_count] = kernel_launches_of(launches, launch_count);
	*graph_out = card->graph_count++;
done:
	if (graph != NULL)
		(void)cu->cuGraphDestroy(graph);
	CARD_LEAVE(card);
}

result_status backend_b200_graph_run_wait(struct device_card *card, uint32_t graph)
{
	if (card == NULL)
		return STATUS_INVALID_ARGUMENT;
	CARD_ENTER(card);
	if (card->failed) {
		status = STATUS_DEVICE_ERROR;
		goto done;
	}
	if (graph >= card->graph_count) {
		status = STATUS_INVALID_ARGUMENT;
		goto done;
	}
	DRIVER(card, cuGraphLaunch(card->graphs[graph], card->stream));
	card->launches_queued += card->graph_kernel_nodes[graph];
	DRIVER(card, cuStreamSynchronize(card->stream));
done:
	CARD_LEAVE(card);
}

uint64_t backend_b200_launch_count(const struct device_card *card)
{
	return card != NULL ? card->launches_queued : 0;
}

uint64_t backend_b200_arena_address(const struct device_card *card)
{
	return card != NULL ? (uint64_t)card->arena : 0;
}

const struct backend_operations backend_cuda_value = {
	.name = "cuda-sm_100a",
	.card_count = cuda_card_count,
	.card_describe = cuda_card_describe,
	.card_open = cuda_card_open,
	.card_close = cuda_card_close,
	.staging_allocate = cuda_staging_allocate,
	.staging_free = cuda_staging_free,
	.upload_begin = cuda_upload_begin,
	.upload_wait = cuda_upload_wait,
	.digest = NULL,
	.download_begin = cuda_download_begin,
	.kernel_prepare = cuda_kernel_prepare,
	.launch_run = cuda_launch_run,
	.launch_wait = cuda_launch_wait,
	.format_supported = cuda_format_supported,
	.exchange_allocate = NULL,
	.exchange_free = NULL,
	.exchange_attach = NULL,
	.peer_attach = NULL,
	.graph_capture = cuda_graph_capture,
	.graph_run = cuda_graph_run,
	.mark_record = cuda_mark_record,
	.mark_follow = cuda_mark_follow,
	.staging_retire = NULL,
	.peer_connect = cuda_peer_connect,
	.measure_begin = cuda_measure_begin,
	.measure_end = cuda_measure_end,
	.measure_elapsed_us = cuda_measure_elapsed_us,
};

const struct backend_operations *backend_b200_operations(void)
{
	return &backend_cuda_value;
}
