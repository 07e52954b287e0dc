/*
 * ring_exchange.c: load-time preparation of the three output-axis exchanges (anemone_b200_collective.h; the records
 * header describes them). The reference has no preparer for these launches (its model program fills them itself,
 * source/model_v41_program.c:8445); the checks are the contract of include/anemone/exact_ring_records.h,
 * round_once_ring_records.h and compressed_ring_records.h, for 2, 4 or 8 ranks.
 */
#include "anemone_b200_collective.h"

#include <stddef.h>

#include "prepare_common.h"

static uint32_t rank_count_of(const struct exact_ring_arguments *arguments)
{
	return arguments->reserved_words[0] == 0 ? EXACT_RING_RANKS : (uint32_t)arguments->reserved_words[0];
}

uint64_t ring_exchange_bank_bytes(enum ring_exchange_kind kind, uint32_t mode, uint32_t rank_count,
				  uint32_t packs_per_owner)
{
	const uint64_t flags = 2u * (uint64_t)rank_count * EXACT_RING_BLOCKS * 4u; /* two meetings, a word a rank and block */
	const uint64_t plane = (uint64_t)rank_count * packs_per_owner * EXACT_RING_PACK_BYTES;
	if (kind == RING_EXCHANGE_COMPRESSED)
		return EXACT_RING_METADATA_BYTES + 2u * ((uint64_t)rank_count - 1u) * (packs_per_owner / COMPRESSED_RING_PACKS) *
							   COMPRESSED_RING_PACKET_BYTES;
	if (kind == RING_EXCHANGE_EXACT && mode == EXACT_RING_GATHER)
		return EXACT_RING_METADATA_BYTES + plane + flags;
	return EXACT_RING_METADATA_BYTES + 2u * plane + flags; /* the ranks' packs, the owners' results */
}

result_status ring_exchange_prepare(const struct ring_exchange_description *description,
				    const struct backend_operations *backend, struct device_card *card,
				    struct kernel_launch *launch_out)
{
	if (description == NULL || backend == NULL || backend->kernel_prepare == NULL || card == NULL || launch_out == NULL ||
	    (uint32_t)description->kind > RING_EXCHANGE_ROUND_ONCE || description->blocks > EXACT_RING_BLOCKS)
		return STATUS_INVALID_ARGUMENT;
	const struct exact_ring_arguments *const a = &description->arguments;
	const uint32_t ranks = rank_count_of(a);
	const bool gather = a->mode == EXACT_RING_GATHER, columns = a->mode == EXACT_RING_BF16_SUM_COLUMNS;
	if ((ranks != 2u && ranks != 4u && ranks != 8u) || a->reserved_words[0] > 8u || a->reserved_words[1] != 0 ||
	    a->rank >= ranks || a->mode > EXACT_RING_BF16_SUM_COLUMNS ||
	    (gather && description->kind != RING_EXCHANGE_EXACT) || a->packs_per_owner == 0 ||
	    a->packs_per_owner % COMPRESSED_RING_PACKS != 0 || a->packs_per_owner > (1u << 24) ||
	    (columns && (a->vectors == 0 || a->packs_per_owner % a->vectors != 0)) ||
	    (gather && a->vectors != 0 && a->packs_per_owner % a->vectors != 0) ||
	    (a->mode == EXACT_RING_BF16_SUM && a->vectors != 0) || a->deadline_cycles == 0 ||
	    a->deadline_cycles > ((uint64_t)1 << 62))
		return STATUS_INVALID_ARGUMENT;
	const uint64_t bytes = (uint64_t)ranks * a->packs_per_owner * EXACT_RING_PACK_BYTES;
	const bool in_place = !gather && a->input_offset == a->output_offset;
	const struct checked_range ranges[4] = {
		{ "input", a->input_offset, bytes },
		{ "output", a->output_offset, in_place ? 0u : bytes },
		{ "bank", a->bank_offset, ring_exchange_bank_bytes(description->kind, a->mode, ranks, a->packs_per_owner) },
		{ "peer table", a->peer_table_offset, (uint64_t)ranks * sizeof(struct ordered_collective_peer) }
	};
	if (!prepare_ranges_are_valid("ring exchange", ranges, 4, description->arena_byte_count))
		return STATUS_INVALID_ARGUMENT;
	static const char *const files[3] = { KERNEL_FILE_EXACT_RING, KERNEL_FILE_COMPRESSED_RING,
					      KERNEL_FILE_ROUND_ONCE_RING };
	static const char *const names[3] = { KERNEL_EXACT_RING, KERNEL_COMPRESSED_RING, KERNEL_ROUND_ONCE_RING };
	uint32_t kernel = BACKEND_NO_KERNEL;
	const result_status status =
		backend->kernel_prepare(card, files[description->kind], names[description->kind], sizeof(*a), &kernel);
	if (status != STATUS_OK)
		return status;
	if (kernel == BACKEND_NO_KERNEL)
		return STATUS_UNSUPPORTED;
	prepare_launch_fill(launch_out, kernel, description->blocks == 0 ? EXACT_RING_BLOCKS : description->blocks, 1, 1,
			    EXACT_RING_THREADS, 0, a, sizeof(*a));
	return STATUS_OK;
}
