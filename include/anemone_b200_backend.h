/*
 * anemone_b200_backend.h: the card boundary. Everything that touches a GPU goes through the table below.
 *
 * Replaces the reference's include/anemone/backend_seam.h:143-310 (struct kernel_launch, struct
 * card_description_record, struct backend_operations, backend_cuda_value) and the part of
 * include/anemone/weight_format_seam.h:56-86 its preparers use. Struct layouts, the order of the table's members,
 * constants and the meaning of every call are kept, so the reference's preparers, step driver and card tests bind to
 * this table unchanged. The implementation (csrc/host/backend_cuda.c) is C11 over the CUDA driver API, which it
 * resolves from libcuda.so.1 at first use: the library loads on a machine without a driver, and every call that needs
 * a card then answers STATUS_UNSUPPORTED or a card count of zero. There is no CPU execution path.
 *
 * Differences from the reference backend, all deliberate:
 *   - one kernel build, for sm_100a; a card of compute capability 10.x is ARITHMETIC_CLASS_SM_100, any other card
 *     has arithmetic class 0 and kernel_prepare answers STATUS_UNSUPPORTED for it;
 *   - kernel parameters are verified with cuFuncGetParamInfo (the reference's cuFuncGetParamCount,
 *     source/backend_cuda_launch.c:170, does not exist in CUDA 12.9);
 *   - the card uses the device's primary context, so that runtime-API code of the same process shares its memory;
 *   - peer_connect needs no gate record: on NVLink/NVSwitch every ordered pair is direct;
 *   - exchange memory, peer_attach (the gated form), digest and staging_retire are not offered (NULL members /
 *     STATUS_UNSUPPORTED), as the table's contract allows for an entry a backend does not have;
 *   - a table whose branches do not follow the grammar of LAUNCH_* is refused with STATUS_INVALID_ARGUMENT before the
 *     driver is asked for anything (the reference finds out while it builds the graph: STATUS_DEVICE_ERROR);
 *   - a table of LAUNCH_CHAIN kernel launches alone becomes a graph by stream capture; any other table (side runs,
 *     BACKEND_COPY launches) is built node by node with the dependencies backend_b200_launch_order states.
 */
#ifndef ANEMONE_B200_BACKEND_H
#define ANEMONE_B200_BACKEND_H

#include <stdbool.h>
#include <stdint.h>

#include "anemone_b200_status.h"

#ifdef __cplusplus
extern "C" {
#endif

#define BACKEND_MAXIMUM_CARDS 16
#define BACKEND_MAXIMUM_KERNELS 256
#define BACKEND_NO_KERNEL UINT32_MAX
#define BACKEND_COPY (UINT32_MAX - 1u)
#define BACKEND_ADDRESS_WORD_BYTES 8
#define BACKEND_MAXIMUM_GRAPHS 512
#define BACKEND_MAXIMUM_MARKS 256
#define LAUNCH_DIMENSIONS 3
#define LAUNCH_ARGUMENT_BYTES 192
#define BACKEND_MAXIMUM_UPLOADS_IN_FLIGHT 16
#define BACKEND_STAGING_ALIGNMENT_BYTES 4096
#define BACKEND_MAXIMUM_STAGING_BLOCKS 256
#define CARD_NAME_CAPACITY 96
#define CARD_BUS_ADDRESS_CAPACITY 32
#define ARITHMETIC_CLASS_SM_80 80u
#define ARITHMETIC_CLASS_SM_120 120u
#define ARITHMETIC_CLASS_SM_120_NATIVE 1200u
#define ARITHMETIC_CLASS_SM_100 100u /* new: compute capability 10.x, the only class this library has kernels for */
#define BACKEND_CUDA_MEMORY_RESERVED_BYTES (256ull << 20u)

/* include/anemone/weight_format_seam.h:58-86 */
enum weight_format_code {
	WEIGHT_FORMAT_NONE = 0,
	WEIGHT_FORMAT_FLOAT16 = 1,
	WEIGHT_FORMAT_EXL3 = 2,
	WEIGHT_FORMAT_E2M1_SCALED = 3,
	WEIGHT_FORMAT_INT4_SCALED = 4,
	WEIGHT_FORMAT_E4M3_SCALED = 5,
	WEIGHT_FORMAT_COUNT = 6,
	/* B200 extension, behind the reference's codes: E4M3 bytes in WEIGHT_FORMAT_E4M3_SCALED's order with one FP32 scale
	 * per 128 outputs by 128 inputs (the block-scaled FP8 of the original-weights checkpoints) */
	WEIGHT_FORMAT_E4M3_BLOCK128 = 6
};

struct matrix_shape_record {
	uint32_t output_size;
	uint32_t input_size;
	uint32_t bits_per_weight;
	uint32_t reserved_must_be_zero;
};

struct weight_format_operations {
	const char *name;
	MUST_CHECK result_status (*stored_byte_count)(const struct matrix_shape_record *shape,
						      uint64_t *byte_count_out);
};

/* include/anemone/backend_seam.h:164-181 */
struct card_description_record {
	char name[CARD_NAME_CAPACITY];
	char bus_address[CARD_BUS_ADDRESS_CAPACITY];
	uint32_t arithmetic_class;
	uint32_t link_generation;
	uint32_t link_lane_count;
	uint32_t reserved_zero;
	uint64_t memory_total_bytes;
	uint64_t memory_free_bytes;
	uint64_t memory_reserved_bytes;
};

struct device_card; /* opaque to every caller */

/* include/anemone/backend_seam.h:183-204. One prepared launch: plain bytes, no address. */
#define LAUNCH_CHAIN 0u
#define LAUNCH_SIDE 1u
#define LAUNCH_RESUME 2u
#define LAUNCH_JOIN 3u
#define LAUNCH_SIDE_MORE 4u
#define LAUNCH_MOST_SIDE_RUNS 4u
/* New with this library, OR-ed into a LAUNCH_CHAIN branch: the launch may begin while the launch before it still runs
 * (programmatic dependent launch). Only for a kernel that orders itself behind what it reads of that launch (with
 * griddepcontrol.wait, or flags that launch sets); launch_run and a captured chain honour it, a graph built node by
 * node runs the launch behind the whole of the launch before it. The bit is set only in launches this library's own layer preparers write; the
 * reference's backend would refuse it as a branch it does not know. */
#define LAUNCH_OVERLAPS_PREVIOUS 0x100u
struct kernel_launch {
	uint32_t kernel;
	uint32_t grid[LAUNCH_DIMENSIONS];
	uint32_t block[LAUNCH_DIMENSIONS];
	uint32_t dynamic_shared_byte_count;
	uint32_t argument_byte_count;
	uint32_t branch;
	unsigned char argument[LAUNCH_ARGUMENT_BYTES];
};

/* A launch whose kernel is BACKEND_COPY is a copy between device memories, run by a copy engine (a memcpy node of a
 * graph, an asynchronous copy of launch_run); its record (include/anemone/exchange_records.h:81-84, 128-133): */
#define EXCHANGE_OWN_ARENA UINT64_MAX /* in place of an address word: the card's own arena */
#define EXCHANGE_COPY_ARGUMENT_BYTES 40u
struct exchange_place {
	uint64_t address_word_offset; /* of a word peer_connect wrote into the card's arena, or EXCHANGE_OWN_ARENA */
	uint64_t offset;	      /* from the address the word holds */
};
struct exchange_copy_arguments {
	struct exchange_place source;
	struct exchange_place destination;
	uint64_t byte_count; /* 1 or more */
};
#ifdef __cplusplus
static_assert(sizeof(struct exchange_copy_arguments) == EXCHANGE_COPY_ARGUMENT_BYTES, "a copy launch's record");
#else
_Static_assert(sizeof(struct exchange_copy_arguments) == EXCHANGE_COPY_ARGUMENT_BYTES, "a copy launch's record");
#endif

/* The launches a launch of a table waits for in a graph: CHAIN behind the launch before it; a run of SIDE launches
 * behind the launch before the run (the fork), each behind the one before it; SIDE_MORE behind the fork alone (another
 * side run of one launch, at most LAUNCH_MOST_SIDE_RUNS runs a fork); RESUME behind the fork, not the side runs; JOIN
 * behind the launch before it and every side run's last. A side run at the head of the table forks at the graph's
 * root (behind nothing, as RESUME then is). */
struct launch_order {
	uint32_t behind_count;
	uint32_t behind[1u + LAUNCH_MOST_SIDE_RUNS]; /* indices into the table, ascending, none twice */
};

/* include/anemone/backend_seam.h:206-308, member for member. */
struct backend_operations {
	const char *name;
	MUST_CHECK result_status (*card_count)(uint32_t *card_count_out);
	MUST_CHECK result_status (*card_describe)(uint32_t card_index,
						  struct card_description_record *description_out);
	MUST_CHECK result_status (*card_open)(uint32_t card_index, uint64_t arena_byte_count,
					      struct device_card **card_out);
	void (*card_close)(struct device_card *card, uint64_t wait_limit_nanoseconds);
	MUST_CHECK result_status (*staging_allocate)(uint64_t byte_count, void **page_locked_memory_out);
	void (*staging_free)(void *page_locked_memory);
	MUST_CHECK result_status (*upload_begin)(struct device_card *card, uint64_t arena_byte_offset,
						 const void *page_locked_source, uint64_t byte_count,
						 uint64_t *upload_ticket_out);
	MUST_CHECK result_status (*upload_wait)(struct device_card *card, uint64_t upload_ticket,
						uint64_t wait_limit_nanoseconds);
	MUST_CHECK result_status (*digest)(struct device_card *card, uint64_t arena_byte_offset, uint64_t byte_count,
					   uint64_t wait_limit_nanoseconds, uint64_t *digest_out);
	MUST_CHECK result_status (*download_begin)(struct device_card *card, uint64_t arena_byte_offset,
						   void *page_locked_destination, uint64_t byte_count,
						   uint64_t *download_ticket_out);
	MUST_CHECK result_status (*kernel_prepare)(struct device_card *card, const char *kernel_file_name,
						   const char *function_name, uint32_t argument_byte_count,
						   uint32_t *kernel_out);
	MUST_CHECK result_status (*launch_run)(struct device_card *card, const struct kernel_launch *launches,
					       uint32_t launch_count);
	MUST_CHECK result_status (*launch_wait)(struct device_card *card, uint64_t wait_limit_nanoseconds);
	bool (*format_supported)(uint32_t card_index, enum weight_format_code format);
	MUST_CHECK result_status (*exchange_allocate)(uint64_t byte_count, void **exchange_out);
	void (*exchange_free)(void *exchange);
	MUST_CHECK result_status (*exchange_attach)(struct device_card *card, const void *exchange,
						    uint64_t address_word_offset);
	MUST_CHECK result_status (*peer_attach)(struct device_card *accessor, struct device_card *owner,
						const char *gate_record_path, uint64_t address_word_offset);
	MUST_CHECK result_status (*graph_capture)(struct device_card *card, const struct kernel_launch *launches,
						  uint32_t launch_count, uint32_t *graph_out);
	MUST_CHECK result_status (*graph_run)(struct device_card *card, uint32_t graph);
	MUST_CHECK result_status (*mark_record)(struct device_card *card, uint32_t mark);
	MUST_CHECK result_status (*mark_follow)(struct device_card *card, struct device_card *owner, uint32_t mark);
	void (*staging_retire)(void *page_locked_memory);
	MUST_CHECK result_status (*peer_connect)(struct device_card *accessor, struct device_card *owner,
						 uint64_t owner_offset, uint64_t address_word_offset);
	MUST_CHECK result_status (*measure_begin)(struct device_card *card);
	MUST_CHECK result_status (*measure_end)(struct device_card *card);
	MUST_CHECK result_status (*measure_elapsed_us)(struct device_card *card, uint64_t wait_limit_nanoseconds,
						       double *microseconds_out);
};

/* Replaces backend_cuda_value (include/anemone/backend_seam.h:310; source/backend_cuda.c:1321-1349). */
extern const struct backend_operations backend_cuda_value;

/* ---- B200 extensions: no counterpart in the reference, which drives all its cards from one process ---- */

/* The table above, for callers that bind by function (a foreign-function interface cannot read a data symbol's
 * function pointers portably). */
const struct backend_operations *backend_b200_operations(void);

/* One process per GPU: the owner exports its arena as a 64-byte inter-process handle ... */
#define BACKEND_B200_IPC_HANDLE_BYTES 64u
MUST_CHECK result_status backend_b200_ipc_export(struct device_card *card,
						 unsigned char handle_out[BACKEND_B200_IPC_HANDLE_BYTES]);
/* ... and an accessor in another process maps it and writes the address of (owner arena + owner_offset), as its own
 * kernels reach it, into its arena at address_word_offset: peer_connect across processes. The mapping lives until the
 * accessor card is closed. At most BACKEND_MAXIMUM_CARDS mappings a card; the same handle maps once. */
MUST_CHECK result_status backend_b200_ipc_connect(struct device_card *accessor,
						  const unsigned char handle[BACKEND_B200_IPC_HANDLE_BYTES],
						  uint64_t owner_offset, uint64_t address_word_offset);
/* Queue a fill of arena bytes (zeroing signal lines and scratch at load), behind everything queued before. */
MUST_CHECK result_status backend_b200_fill(struct device_card *card, uint64_t arena_byte_offset, unsigned char value,
					   uint64_t byte_count);
/* Registers one more kernel file for kernel_prepare: an sm_100a cubin image the caller built (the bytes are copied;
 * at most four, never under the name of a file the library embeds or of one registered before). Kernels of such a file
 * follow the same contract: extern "C" __global__ f(record, arena address). Cards opened before or after see it. */
MUST_CHECK result_status backend_b200_image_register(const char *kernel_file_name, const void *image,
						     uint64_t image_byte_count);
/* Waits for the card's queue, then reports whether any kernel of the library's kernel files gave up a bounded wait
 * since the files were loaded (a shared-memory barrier of the prefill products; a signal line of the push and the
 * exchange, whose kernels also report a replayed sequence, 2, and a row count beyond the prepared rows, 4). Such a CTA
 * stores nothing more and returns; nothing traps. *expired_out is 0, or the kernels' bits or-ed. */
MUST_CHECK result_status backend_b200_waits_expired(struct device_card *card, uint32_t *expired_out);
/* One step in ONE call, for a serving loop that must not pay a foreign-function call, a ticket and a polled wait per
 * transfer: queue the copy of input_byte_count bytes from page-locked memory to the arena, the captured graph, the
 * copy of output_byte_count arena bytes back to page-locked memory, then block (the driver's stream wait, which
 * returns as the last copy completes) until all of it is done. Both host ranges lie in staging blocks of
 * staging_allocate; either byte count may be 0 (no such copy). Equivalent to upload_begin + graph_run +
 * download_begin + upload_wait of the table. */
MUST_CHECK result_status backend_b200_step_run(struct device_card *card, uint32_t graph,
					       uint64_t input_arena_offset, const void *page_locked_input,
					       uint64_t input_byte_count, uint64_t output_arena_offset,
					       void *page_locked_output, uint64_t output_byte_count);
/* The same step as ONE graph: the copy in, the chain of launches and the copy out are captured together (memcpy nodes
 * at fixed page-locked addresses, read and written when the graph runs), so that a step is a single graph launch and a
 * wait: backend_b200_graph_run_wait. For tables of LAUNCH_CHAIN kernel launches (STATUS_UNSUPPORTED otherwise: such a
 * table goes through graph_capture and backend_b200_step_run). The caller writes its inputs to the same page-locked
 * range before every run and reads the output range after the wait. */
MUST_CHECK result_status backend_b200_step_capture(struct device_card *card, const struct kernel_launch *launches,
						   uint32_t launch_count, uint64_t input_arena_offset,
						   const void *page_locked_input, uint64_t input_byte_count,
						   uint64_t output_arena_offset, void *page_locked_output,
						   uint64_t output_byte_count, uint32_t *graph_out);
/* graph_run of the table, then the driver's stream wait: returns when the graph has run (any captured graph). */
MUST_CHECK result_status backend_b200_graph_run_wait(struct device_card *card, uint32_t graph);
/* Kernel launches this card has queued since it was opened, graph launches counted by their kernel nodes. */
/* The dependencies graph_capture gives every launch of a table (order_out[launch_count]), from the branches alone: no
 * card is needed. STATUS_INVALID_ARGUMENT for a NULL, an empty table, a branch that is none of LAUNCH_* or a table
 * outside the grammar (SIDE right behind SIDE_MORE; SIDE_MORE or RESUME not behind a side run; a fifth side run; JOIN
 * without a side run); order_out is then untouched. */
MUST_CHECK result_status backend_b200_launch_order(const struct kernel_launch *launches, uint32_t launch_count,
						   struct launch_order *order_out);

uint64_t backend_b200_launch_count(const struct device_card *card);
/* The device address of the arena (diagnostics and interoperation with other libraries of the same process). */
uint64_t backend_b200_arena_address(const struct device_card *card);

#ifdef __cplusplus
}
#endif
#endif
