/*
 * anemone_b200_collective.h: load-time preparation of the fixed-order reductions over ranks, and the host function that
 * defines their order. Host C11. A refusal leaves every output unchanged.
 *
 * Protocol kept from the reference (include/anemone/ordered_collective_records.h:5-38): every rank launches the same
 * kernel with the same strictly increasing 64-bit sequence, read on the device from the step block, so one prepared
 * launch (or captured graph) serves every step; two parity slots per rank; a signal line is written only by its owner,
 * after its payload, with a system-scope release, and read with a system-scope acquire; sums are
 * ((+0 + rank 0) + rank 1) + ... in FP32 with one rounded add per rank; no atomics on data.
 * Changed for NVLink/NVSwitch: all routes are direct peer loads (no host mirrors); a line holds the owner's step
 * sequence itself instead of a generation counter plus sequence words; a wait that runs out reports through a status
 * block (B200 entries) and never traps.
 */
#ifndef ANEMONE_B200_COLLECTIVE_H
#define ANEMONE_B200_COLLECTIVE_H

#include "anemone_b200_backend.h"
#include "anemone_b200_records.h"

#ifdef __cplusplus
extern "C" {
#endif

/* include/anemone/ordered_collective.h:25-33 */
struct ordered_collective_kernels {
	uint32_t handles[ORDERED_COLLECTIVE_OPERATIONS];
};

struct ordered_collective_description {
	struct ordered_collective_arguments arguments;
	uint64_t arena_byte_count;
	enum ordered_collective_operation operation;
};

/* include/anemone/ordered_collective.h:57-68 */
struct ordered_collective_route_description {
	const struct card_description_record *cards;
	const uint32_t *direct_reader_masks;
	uint32_t rank_count, element_count;
	enum ordered_collective_operation operation;
	bool common_numa_root;
	bool paired_scatter_gather;
};

/* include/anemone/ordered_collective.h:67-69. host_reader_masks_out[source] = the readers of `source` that lack
 * direct access (they would need a host mirror). The reference's PCIe preferences for its CMP cards do not apply to
 * NVLink: a reader with direct access is always direct. This library's kernels refuse host routes, so a caller must
 * see all-zero masks before it prepares a launch. */
MUST_CHECK result_status ordered_collective_routes_prepare(
	const struct ordered_collective_route_description *description, uint32_t *host_reader_masks_out);

/* include/anemone/ordered_collective.h:70-100 (source/ordered_routes_measured.c): routes with a caller-qualified table
 * of measured overrides. A row names one operation at one exact size in caller rank order: the direct reader masks
 * it was measured under, the cards' arithmetic class and link fields, and the host reader masks to use. Malformed
 * rows (counts, operation, a mask outside the group, a source that does not read itself or mirrors itself, a denied
 * reader without a mirror), duplicate keys and unequal rows of one scatter/gather pair: STATUS_INVALID_ARGUMENT;
 * a row whose key matches the description but whose masks, class or link fields do not: STATUS_UNSUPPORTED; no
 * matching row: the qualified-direct / denied-host masks of ordered_collective_routes_prepare. Errors leave the
 * output untouched. Pure preparation: no allocation, no backend call. */
#define ORDERED_ROUTE_POLICY_MAXIMUM_ROWS 256u
struct ordered_collective_route_policy {
	uint32_t rank_count, element_count;
	enum ordered_collective_operation operation;
	bool paired_scatter_gather;
	uint32_t arithmetic_classes[ORDERED_COLLECTIVE_MAXIMUM_RANKS];
	uint32_t link_generations[ORDERED_COLLECTIVE_MAXIMUM_RANKS];
	uint32_t link_lane_counts[ORDERED_COLLECTIVE_MAXIMUM_RANKS];
	uint32_t expected_direct_reader_masks[ORDERED_COLLECTIVE_MAXIMUM_RANKS];
	uint32_t host_reader_masks[ORDERED_COLLECTIVE_MAXIMUM_RANKS];
};
MUST_CHECK result_status ordered_collective_routes_prepare_measured(
	const struct ordered_collective_route_description *description,
	const struct ordered_collective_route_policy *rows, uint32_t row_count, uint32_t *host_reader_masks_out);

/* include/anemone/ordered_collective.h:101-103 (source/ordered_collective.c:117-142): the four FP32 kernels. */
MUST_CHECK result_status ordered_collective_kernels_prepare(const struct backend_operations *backend,
							    struct device_card *card,
							    struct ordered_collective_kernels *kernels_out);

/* include/anemone/ordered_collective.h:104-107 (source/ordered_collective.c:208-282): one block of 256 threads. */
MUST_CHECK result_status ordered_collective_prepare(const struct ordered_collective_description *description,
						    const struct ordered_collective_kernels *kernels,
						    struct kernel_launch *launch_out);

/* include/anemone/ordered_collective.h:108-110 (source/ordered_collective.c:144-206): the same four operations on host
 * arrays, which DEFINE the order the kernels must reproduce bit for bit. A staging utility for callers and tests;
 * nothing in this library calls it. Refuses overlapping buffers and a rounding mode other than to-nearest. */
MUST_CHECK result_status ordered_collective_host(const float *const *inputs, float *const *outputs,
						 uint32_t rank_count, uint32_t element_count,
						 enum ordered_collective_operation operation);

/* ---- B200 extension: the expert layer's reduction, FP32 partial rows -> one bfloat16 result ---- */

struct ordered_reduce_bf16_description {
	struct ordered_reduce_bf16_arguments reduce; /* .collective as above; output_offset an ARENA offset */
	uint64_t pair_output_offset; /* FP32 [row_capacity * pairs_per_row][width]: the finished pair outputs */
	uint64_t arena_byte_count;
	uint32_t pairs_per_row;
	uint32_t row_capacity; /* collective.element_count = row_capacity * width */
};

/* No reference counterpart as one call; the arithmetic is tp_exchange_owner_sum's (source/kernel_tp_exchange.cu:
 * 190-247). Writes two launches: ordered_row_sum_publish, ordered_reduce_bf16 (kernel file "kernel_ordered_b200").
 * Validates what ordered_collective_prepare validates (region, slots, table, step block, disjointness), that width is a
 * multiple of 4, the result and status ranges, and that no peer entry will be a host route. */
#define ORDERED_REDUCE_BF16_LAUNCHES 2u
MUST_CHECK result_status ordered_reduce_bf16_prepare(const struct ordered_reduce_bf16_description *description,
						     const struct backend_operations *backend,
						     struct device_card *card, struct kernel_launch *launches_out);
/* B200 extension: the same reduction for pair outputs that are bfloat16, in ONE launch
 * ("ordered_publish_reduce_flags_bf16", struct ordered_publish_reduce_bf16_arguments): row sums, the optional
 * bfloat16 addend row (0: none), the optional FP32 copy of the rank's own rows (0: none), READY and the rank-ordered
 * sum with one rounding, with flags that arrive in the reader's own memory. The description is
 * ordered_reduce_bf16_prepare's with pair outputs of 2 bytes an element; mode ORDERED_REDUCE_EVERY_RANK; the slot
 * layout is the EXL3 layer step's (input_offset at least EXL3_LAYER_SIGNAL_BYTES), at most
 * ORDERED_COLLECTIVE_MAXIMUM_ELEMENTS elements. */
MUST_CHECK result_status ordered_publish_reduce_bf16_prepare(const struct ordered_reduce_bf16_description *description,
							     uint64_t addend_offset, uint64_t row_output_offset,
							     const struct backend_operations *backend,
							     struct device_card *card, struct kernel_launch *launch_out);

/* ---- one-shot push all-reduce (include/anemone/ordered_push.h:37-59) ---- */

struct ordered_push_description {
	struct ordered_push_arguments arguments;
	uint64_t arena_byte_count;
};

/* include/anemone/ordered_push.h:42-44: the handle of ("kernel_ordered_push", "ordered_push"). */
MUST_CHECK result_status ordered_push_kernel_prepare(const struct backend_operations *backend,
						     struct device_card *card, uint32_t *kernel_out);

/* include/anemone/ordered_push.h:45-47 (source/ordered_push.c:63-161): the reference's checks and refusals, its
 * record copied unchanged into the launch. The launch is groups x blocks CTAs of 256 threads (the reference: one CTA).
 * A record that is well formed but names a host mirror (incoming_host_mask != 0) is STATUS_UNSUPPORTED. The slot's
 * signal lines, ORDERED_PUSH_PHASES * rank_count * 128 bytes, must be zero before the first launch. */
MUST_CHECK result_status ordered_push_prepare(const struct ordered_push_description *description, uint32_t kernel,
					      struct kernel_launch *launch_out);

/* include/anemone/ordered_push.h:54-59: host_writer_masks_out[owner] = the sources that lack direct access to
 * `owner` (direct_reader_masks[owner] then names the accessors qualified to WRITE the owner). All-reduce only. */
MUST_CHECK result_status ordered_push_routes_prepare(const struct ordered_collective_route_description *description,
						     uint32_t *host_writer_masks_out);

/* ---- the exchange of a tensor-parallel layer site (include/anemone/tp_exchange.h:49-63) ---- */

/* include/anemone/tp_exchange.h:49-51: the handle of ("kernel_tp_exchange", "tp_exchange"). */
MUST_CHECK result_status tp_exchange_kernel_prepare(const struct backend_operations *backend,
						    struct device_card *card, uint32_t *kernel_out);

/* include/anemone/tp_exchange.h:52-55 (source/tp_exchange.c:26-48): the push of the step's live rows under the
 * layer's own sequence, one launch. element_count is a whole number of rows; the reference's row is its model's 5120
 * elements, and that is what this entry assumes; tp_exchange_rows_prepare takes the width. layer < layer_count <=
 * TP_EXCHANGE_MAXIMUM_PHASES; element_count <= TP_EXCHANGE_MAXIMUM_ELEMENTS. */
MUST_CHECK result_status tp_exchange_prepare(const struct ordered_push_description *description, uint32_t layer,
					     uint32_t layer_count, uint32_t kernel, struct kernel_launch *launch_out);
MUST_CHECK result_status tp_exchange_rows_prepare(const struct ordered_push_description *description,
						  uint32_t row_width, uint32_t layer, uint32_t layer_count,
						  uint32_t kernel, struct kernel_launch *launch_out);

/* include/anemone/tp_exchange.h:56-58 (source/tp_exchange.c:50-88): the four handles of a form. Forms
 * TP_EXCHANGE_FORM_PUSH and TP_EXCHANGE_FORM_OWNER_SUMS; the ring and copy-engine forms are STATUS_UNSUPPORTED. */
MUST_CHECK result_status tp_exchange_wide_kernels_prepare(const struct backend_operations *backend,
							  struct device_card *card, uint32_t form,
							  uint32_t kernels_out[TP_EXCHANGE_WIDE_LAUNCHES]);

/* include/anemone/tp_exchange.h:59-63 (source/tp_exchange.c:90-136): four launches a caller queues in order, as the
 * reference's PUBLISH, READY, SUM, DONE are. Here the first launch is the whole exchange (values out, READY, the
 * ordered sums, for the owner sums the one rounding to bfloat16 and the stores into every rank's output array, DONE)
 * and the other three are empty kernels of one small CTA, kept so a caller's table keeps its four entries. The owner
 * sums want every offset and stride a multiple of 16 bytes and no host route, as the reference does. */
MUST_CHECK result_status tp_exchange_wide_prepare(const struct ordered_push_description *description, uint32_t layer,
						  uint32_t layer_count,
						  const uint32_t kernels[TP_EXCHANGE_WIDE_LAUNCHES], uint32_t form,
						  struct kernel_launch launches_out[TP_EXCHANGE_WIDE_LAUNCHES]);
MUST_CHECK result_status tp_exchange_wide_rows_prepare(const struct ordered_push_description *description,
						       uint32_t row_width, uint32_t layer, uint32_t layer_count,
						       const uint32_t kernels[TP_EXCHANGE_WIDE_LAUNCHES], uint32_t form,
						       struct kernel_launch launches_out[TP_EXCHANGE_WIDE_LAUNCHES]);

/* ---- local completion around the exchange (include/anemone/tp2_join.h:36-59) ---- */

struct tp2_join_range { /* the reference's struct linear_range */
	uint64_t byte_offset;
	uint64_t byte_count;
};

struct tp2_join_description {
	struct tp2_join_range source;
	struct tp2_join_range routed_sums; /* {0, 0}: none; else FP32 rows added first (operations 0, 4, 5 only) */
	struct tp2_join_range output;
	struct tp2_join_range step; /* {0, 0} unless a slot stride is given */
	uint64_t source_slot_stride;
	uint64_t output_slot_stride;
	uint32_t width;
	uint32_t row_count;
	uint32_t source_row_stride;
	uint32_t routed_row_stride;
	uint32_t output_row_stride;
	uint32_t operation;
	uint32_t reserved_zero;
};

/* include/anemone/tp2_join.h:52-54: the handle of ("kernel_tp2_join", "tp2_join"). *kernel_out only on STATUS_OK. */
MUST_CHECK result_status tp2_join_kernel_prepare(const struct backend_operations *backend, struct device_card *card,
						 uint32_t *kernel_out);

/* include/anemone/tp2_join.h:55-58 (source/tp2_join.c:47-205): 1 to 1024 rows of 1 to 32768 elements, every row
 * stride at least the width; ranges on 16-byte multiples, inside the arena, large enough for the last strided row in
 * both parity slots; used spans, both parities and the step block disjoint (so no conversion in place); a routed array
 * only where the operation adds one; a static operation with step exactly {0, 0}; the ring orders with a width that
 * is a multiple of 4 and dense ring rows. A refusal leaves the launch untouched. */
MUST_CHECK result_status tp2_join_prepare(const struct tp2_join_description *description, uint64_t arena_byte_count,
					  uint32_t kernel, struct kernel_launch *launch_out);

/* ---- B200 extension: the expert layer's reduction of a decode step as one launch ---- */

struct ordered_rows_push_description {
	struct ordered_rows_push_arguments arguments;
	uint64_t arena_byte_count;
};

/* No reference counterpart as one call: the push's stores and waits (source/kernel_ordered_push.cuh) around the owner
 * sums' arithmetic (source/kernel_tp_exchange.cu:190-247). One launch of ("kernel_ordered_b200", "ordered_rows_push").
 * Validates the push record (its inbox the only array inside the slot), width a multiple of 4, element_count a whole
 * number of rows, the FP32 wire, 16-byte offsets, the result and pair output ranges. Fewer bytes cross NVLink with
 * ordered_reduce_bf16's owner runs once a step has many rows; this form is the one for decode steps. */
MUST_CHECK result_status ordered_rows_push_prepare(const struct ordered_rows_push_description *description,
						   const struct backend_operations *backend, struct device_card *card,
						   struct kernel_launch *launch_out);

/* ---- the output-axis exchanges (struct exact_ring_arguments of the records header) ----
 * The reference's model program fills these launches itself (source/model_v41_program.c:8445); this library offers a
 * preparer with the usual checks. kind: which of the three entries. blocks: the grid, 1 to EXACT_RING_BLOCKS (0: 16).
 * Checks: 2, 4 or 8 ranks, the rank, a mode the entry has, packs_per_owner a positive multiple of 32, vectors as the
 * mode needs them, a positive deadline; input and output of rank_count * packs_per_owner packs each, 16-byte aligned,
 * inside the arena, disjoint (the sums may also work in place: input_offset == output_offset); the bank of
 * ring_exchange_bank_bytes bytes, disjoint from both; the peer table. The bank's bytes for four ranks never exceed
 * what the reference's formulas reserve (round once: 128 + 128 packs + 512; exact sum: 128 + 192 packs; gather: 128
 * + 120 packs; compressed: 128 + 6 (packs / 32) 544). */
enum ring_exchange_kind { RING_EXCHANGE_EXACT = 0, RING_EXCHANGE_COMPRESSED = 1, RING_EXCHANGE_ROUND_ONCE = 2 };
uint64_t ring_exchange_bank_bytes(enum ring_exchange_kind kind, uint32_t mode, uint32_t rank_count,
				  uint32_t packs_per_owner);
struct ring_exchange_description {
	struct exact_ring_arguments arguments;
	uint64_t arena_byte_count;
	enum ring_exchange_kind kind;
	uint32_t blocks;
};
MUST_CHECK result_status ring_exchange_prepare(const struct ring_exchange_description *description,
					       const struct backend_operations *backend, struct device_card *card,
					       struct kernel_launch *launch_out);

#ifdef __cplusplus
}
#endif
#endif
