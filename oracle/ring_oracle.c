/*
 * ring_oracle.c: CPU restatement of the reference's output-axis exchanges between the ranks of a tensor-parallel group.
 * TEST INFRASTRUCTURE: only tests/, the smoke check and the bench's CPU legs may call it; the product never does.
 *
 * What is restated (reference files by their path in its project):
 *   - the gather's output order (source/kernel_exact_ring.cu; include/anemone/exact_ring_records.h:17-31);
 *   - the BF16 sum of the exact and the compressed ring: owner o's part starts at the rank behind o, passes round the
 *     ring with one bfloat16 addition (fma.rn.bf16x2 with ones: the exact sum rounded once) a rank, and ends at o; the
 *     ring's transport carries a +0 half as -0, in both directions, so every travelling partial and every result a
 *     rank other than its owner receives has no +0 (source/kernel_cut_through.cuh:277-307, 368-431);
 *   - the round-once sum: FP32 additions in rank order from +0, one rounding to bfloat16, the same bits on every rank
 *     (source/kernel_bf16_round_once_ring.cu:70-195; the independent model of tests/compressed_ring_card_test.c:217-241);
 *   - the exponent-delta wire code of a group of 32 packs (source/bf16_wire_codec.h:38-70,
 *     source/kernel_bf16_compressed_ring.cu; include/anemone/compressed_ring_records.h).
 * Pins: the round-once model against the four known answers of tests/compressed_ring_card_test.c:500-520; the wire
 * code against the reference's own header where it was compiled (oracle/_ref), exhaustively. The hop order of the BF16
 * sum has no CPU vector in the reference (its card test compares two GPU forms with one another): parity unpinned for
 * that order beyond this reading.
 */
#include <math.h>
#include <string.h>

#include "anemone_oracle.h"

#define PACK_VALUES 8u

static double bf16_as_double(uint16_t bits)
{
	return (double)orc_bfloat16_value(bits);
}

/* a double to the nearest bfloat16, ties to even, subnormals kept, overflow to infinity, not-a-number 0x7FFF (the
 * canonical one of the card's bfloat16 arithmetic) */
static uint16_t bf16_of_double(double value)
{
	if (isnan(value))
		return 0x7FFFu;
	const uint16_t sign = signbit(value) ? 0x8000u : 0u;
	const double magnitude = fabs(value);
	if (magnitude == 0.0)
		return sign;
	if (isinf(magnitude))
		return sign | 0x7F80u;
	int exponent;
	(void)frexp(magnitude, &exponent); /* magnitude = f 2^exponent, f in [0.5, 1) */
	const int leading = exponent - 1;
	const int last_place = leading < -126 ? -133 : leading - 7;
	const double steps = nearbyint(ldexp(magnitude, -last_place)); /* to nearest, ties to even */
	const float rounded = (float)ldexp(steps, last_place);	       /* exact, or an infinity from 2^128 */
	uint32_t bits;
	memcpy(&bits, &rounded, sizeof(bits));
	return sign | (uint16_t)(bits >> 16);
}

uint16_t orc_ring_bf16_add(uint16_t left, uint16_t right)
{
	return bf16_of_double(bf16_as_double(left) + bf16_as_double(right));
}

static uint16_t travelling(uint16_t bits)
{
	return bits == 0 ? 0x8000u : bits;
}

static uint64_t place_of(uint32_t rank_count, uint32_t packs, uint32_t row_packs, uint32_t owner, uint32_t pack)
{
	if (row_packs == 0)
		return (uint64_t)owner * packs + pack;
	const uint32_t row = pack / row_packs;
	return ((uint64_t)row * rank_count + owner) * row_packs + pack % row_packs;
}

void orc_ring_bf16_sum(const uint16_t *const *inputs, uint32_t rank_count, uint32_t packs_per_owner, uint32_t vectors,
		       uint16_t *const *outputs)
{
	const uint32_t row_packs = vectors == 0 ? 0u : packs_per_owner / vectors;
	for (uint32_t owner = 0; owner < rank_count; owner++)
		for (uint32_t pack = 0; pack < packs_per_owner; pack++) {
			const uint64_t at = place_of(rank_count, packs_per_owner, row_packs, owner, pack) * PACK_VALUES;
			for (uint32_t value = 0; value < PACK_VALUES; value++) {
				uint16_t sum = travelling(inputs[(owner + 1u) % rank_count][at + value]);
				for (uint32_t hop = 2; hop < rank_count; hop++)
					sum = travelling(orc_ring_bf16_add(sum, inputs[(owner + hop) % rank_count][at + value]));
				sum = orc_ring_bf16_add(sum, inputs[owner][at + value]);
				for (uint32_t rank = 0; rank < rank_count; rank++)
					outputs[rank][at + value] = rank == owner ? sum : travelling(sum);
			}
		}
}

void orc_ring_round_once(const uint16_t *const *inputs, uint32_t rank_count, uint64_t value_count, uint16_t *output)
{
	for (uint64_t index = 0; index < value_count; index++) {
		float sum = 0.0f;
		for (uint32_t rank = 0; rank < rank_count; rank++)
			sum = sum + orc_bfloat16_value(inputs[rank][index]);
		output[index] = orc_bfloat16_bits(sum);
	}
}

void orc_ring_gather(const uint16_t *const *inputs, uint32_t rank_count, uint32_t packs_per_owner, uint32_t vectors,
		     uint16_t *output)
{
	const uint32_t row_packs = vectors == 0 ? 0u : packs_per_owner / vectors;
	for (uint32_t owner = 0; owner < rank_count; owner++)
		for (uint32_t pack = 0; pack < packs_per_owner; pack++)
			memcpy(output + place_of(rank_count, packs_per_owner, row_packs, owner, pack) * PACK_VALUES,
			       inputs[owner] + ((uint64_t)owner * packs_per_owner + pack) * PACK_VALUES,
			       PACK_VALUES * sizeof(uint16_t));
}

/* ---- the wire code ---- */

static uint32_t exponent_of(uint16_t bits)
{
	return (bits >> 7) & 0xFFu;
}

/* a group's 32 packs ([32][8] bfloat16) as one packet of 136 words: word 0 the largest exponent, word 1 a bit a lane
 * that is sent as it is, from word 4 the lanes' words one after the other (three for a coded lane: the eight
 * sign-and-mantissa bytes, then the eight distances from the largest exponent, a nibble each; four for a raw one) */
void orc_ring_packet_encode(const uint16_t *values, uint32_t *packet)
{
	uint32_t top = 0;
	for (uint32_t index = 0; index < 32u * PACK_VALUES; index++)
		top = exponent_of(values[index]) > top ? exponent_of(values[index]) : top;
	memset(packet, 0, 136u * sizeof(uint32_t));
	uint32_t mask = 0, word = 4;
	for (uint32_t lane = 0; lane < 32; lane++) {
		const uint16_t *const pack = values + lane * PACK_VALUES;
		bool raw = false;
		for (uint32_t value = 0; value < PACK_VALUES; value++)
			raw = raw || top - exponent_of(pack[value]) > 15u;
		if (raw) {
			mask |= 1u << lane;
			for (uint32_t pair = 0; pair < 4; pair++)
				packet[word++] = pack[2 * pair] | (uint32_t)pack[2 * pair + 1] << 16;
			continue;
		}
		uint64_t bytes = 0;
		uint32_t nibbles = 0;
		for (uint32_t value = 0; value < PACK_VALUES; value++) {
			bytes |= (uint64_t)((pack[value] & 0x7Fu) | (pack[value] >> 15) << 7) << (8 * value);
			nibbles |= (top - exponent_of(pack[value])) << (4 * value);
		}
		packet[word++] = (uint32_t)bytes;
		packet[word++] = (uint32_t)(bytes >> 32);
		packet[word++] = nibbles;
	}
	packet[0] = top;
	packet[1] = mask;
}

void orc_ring_packet_decode(const uint32_t *packet, uint16_t *values)
{
	const uint32_t top = packet[0], mask = packet[1];
	uint32_t word = 4;
	for (uint32_t lane = 0; lane < 32; lane++) {
		uint16_t *const pack = values + lane * PACK_VALUES;
		if ((mask >> lane) & 1u) {
			for (uint32_t pair = 0; pair < 4; pair++, word++) {
				pack[2 * pair] = (uint16_t)packet[word];
				pack[2 * pair + 1] = (uint16_t)(packet[word] >> 16);
			}
			continue;
		}
		const uint64_t bytes = packet[word] | (uint64_t)packet[word + 1] << 32;
		const uint32_t nibbles = packet[word + 2];
		word += 3;
		for (uint32_t value = 0; value < PACK_VALUES; value++) {
			const uint32_t byte = (uint32_t)(bytes >> (8 * value)) & 0xFFu;
			pack[value] = (uint16_t)((byte & 0x7Fu) | (byte >> 7) << 15 |
						 (top - ((nibbles >> (4 * value)) & 15u)) << 7);
		}
	}
}
