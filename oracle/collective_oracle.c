/*
 * collective_oracle.c: CPU restatement of the reference's fixed-order reduction and of the router's conventions.
 * TEST INFRASTRUCTURE ONLY (see anemone_oracle.h): never linked into or called by the shipped library.
 */
#include "anemone_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* source/ordered_collective.c:187-196: sum = +0; for each rank ascending: sum = sum + input[rank][element] */
void orc_ordered_sum(const float *const *inputs, uint32_t rank_count, uint32_t element_count, float *output)
{
	for (uint32_t element = 0; element < element_count; element++) {
		float sum = 0.0f;
		for (uint32_t rank = 0; rank < rank_count; rank++)
			sum = sum + inputs[rank][element];
		output[element] = sum;
	}
}

/* source/kernel_tp_exchange.cu:223-237: the same sum, then one rounding to bfloat16 */
void orc_ordered_reduce_bf16(const float *const *inputs, uint32_t rank_count, uint32_t element_count,
			     uint16_t *output)
{
	for (uint32_t element = 0; element < element_count; element++) {
		float sum = 0.0f;
		for (uint32_t rank = 0; rank < rank_count; rank++)
			sum = sum + inputs[rank][element];
		output[element] = orc_bfloat16_bits(sum);
	}
}

/* source/ordered_collective.c:144-206. Slices are ceil(n / ranks) elements; reduce-scatter writes only the owner's
 * output at full-array indices; gather copies slice owner's input. Returns 0, or 1 for arguments it refuses. */
/* cvt.rn.bf16.f32 as the push's bfloat16 wire applies it to every rank's value (source/kernel_ordered_push.cuh:
 * 143-158): to nearest even, a finite value beyond the format to infinity, a not-a-number to 0x7FFF. */
static float push_wire_value(float value, uint32_t payload_format)
{
	if (payload_format == 0)
		return value;
	uint32_t bits;
	memcpy(&bits, &value, sizeof(bits));
	bits = (bits & 0x7FFFFFFFu) > 0x7F800000u ? 0x7FFF0000u : (bits + 0x7FFFu + ((bits >> 16) & 1u)) & 0xFFFF0000u;
	memcpy(&value, &bits, sizeof(bits));
	return value;
}

void orc_ordered_push(const float *const *inputs, uint32_t rank_count, uint32_t element_count, uint32_t payload_format,
		      float *output)
{
	for (uint32_t element = 0; element < element_count; element++) {
		volatile float sum = 0.0f;
		for (uint32_t rank = 0; rank < rank_count; rank++)
			sum = sum + push_wire_value(inputs[rank][element], payload_format);
		output[element] = sum;
	}
}

void orc_owner_sums(const float *const *inputs, uint32_t rank_count, uint32_t element_count, uint32_t payload_format,
		    uint16_t *output)
{
	for (uint32_t element = 0; element < element_count; element++) {
		volatile float sum = 0.0f;
		for (uint32_t rank = 0; rank < rank_count; rank++)
			sum = sum + push_wire_value(inputs[rank][element], payload_format);
		output[element] = orc_bfloat16_bits(sum);
	}
}

/* The local completion, element by element as source/kernel_tp2_join.cu:43-108 states it. The ring orders are built
 * from their definition (owner o holds quarter o of every slab of 8 rows, counted row by row; slab after slab, owner
 * after owner), not from the kernel's closed form. */
void orc_tp2_join(const struct tp2_join_arguments *record, unsigned char *arena)
{
	const uint32_t rows = record->row_count, width = record->width, operation = record->operation;
	const uint64_t parity = record->source_slot_stride != 0 || record->output_slot_stride != 0 ?
					((const struct step_block *)(arena + record->step_offset))->sequence & 1u :
					0u;
	const unsigned char *const source = arena + record->source_offset + parity * record->source_slot_stride;
	unsigned char *const output = arena + record->output_offset + parity * record->output_slot_stride;
	uint64_t *place = NULL;
	if (operation == TP2_JOIN_RING_PACK || operation == TP2_JOIN_RING_UNPACK) {
		place = malloc((size_t)rows * width * sizeof(*place));
		uint64_t next = 0;
		for (uint32_t owner = 0; owner < TP2_JOIN_RING_OWNERS; owner++)
			for (uint32_t first = 0; first < rows; first += TP2_JOIN_RING_SLAB_ROWS) {
				const uint32_t slab_rows = rows - first < TP2_JOIN_RING_SLAB_ROWS ? rows - first :
												    TP2_JOIN_RING_SLAB_ROWS;
				const uint32_t quarter = slab_rows * width / TP2_JOIN_RING_OWNERS;
				for (uint32_t index = owner * quarter; index < (owner + 1u) * quarter; index++)
					place[(uint64_t)(first + index / width) * width + index % width] = next++;
			}
	}
	for (uint32_t row = 0; row < rows; row++)
		for (uint32_t column = 0; column < width; column++) {
			const uint64_t from = (uint64_t)row * record->source_row_stride + column;
			const uint64_t to = (uint64_t)row * record->output_row_stride + column;
			if (operation == TP2_JOIN_BFLOAT16_COPY) {
				((uint16_t *)output)[to] = ((const uint16_t *)source)[from];
			} else if (operation == TP2_JOIN_FLOAT32_COPY) {
				((uint32_t *)output)[to] = ((const uint32_t *)source)[from];
			} else if (operation == TP2_JOIN_RING_UNPACK) {
				((uint16_t *)output)[to] = ((const uint16_t *)source)[place[(uint64_t)row * width + column]];
			} else if (operation == TP2_JOIN_FLOAT32_TO_BFLOAT16) {
				((uint16_t *)output)[to] = orc_bfloat16_bits(((const float *)source)[from]);
			} else {
				volatile float value = orc_bfloat16_value(((const uint16_t *)source)[from]);
				if (record->has_routed_sums != 0)
					value = ((const float *)(arena + record->routed_sums_offset))
							[(uint64_t)row * record->routed_row_stride + column] +
						value;
				if (operation == TP2_JOIN_BFLOAT16_TO_FLOAT32)
					((float *)output)[to] = value;
				else if (operation == TP2_JOIN_BFLOAT16_SUM_TO_BFLOAT16)
					((uint16_t *)output)[to] = orc_bfloat16_bits(value);
				else
					((uint16_t *)output)[place[(uint64_t)row * width + column]] = orc_bfloat16_bits(value);
			}
		}
	free(place);
}

int orc_ordered_collective(const float *const *inputs, float *const *outputs, uint32_t rank_count,
			   uint32_t element_count, int operation)
{
	if (inputs == NULL || outputs == NULL || rank_count == 0 || rank_count > ORDERED_COLLECTIVE_MAXIMUM_RANKS ||
	    element_count == 0 || element_count > ORDERED_COLLECTIVE_MAXIMUM_ELEMENTS || operation < 0 ||
	    operation >= (int)ORDERED_COLLECTIVE_OPERATIONS)
		return 1;
	const uint32_t slice = (element_count + rank_count - 1u) / rank_count;
	for (uint32_t element = 0; element < element_count; element++) {
		float sum = 0.0f;
		if (operation == ORDERED_GATHER) {
			sum = inputs[element / slice][element];
		} else {
			for (uint32_t rank = 0; rank < rank_count; rank++)
				sum = sum + inputs[rank][element];
		}
		if (operation == ORDERED_REDUCE_SCATTER) {
			outputs[element / slice][element] = sum;
		} else {
			for (uint32_t rank = 0; rank < rank_count; rank++)
				outputs[rank][element] = sum;
		}
	}
	return 0;
}

/* ---------------------------------------------------------------- router */

/* source/kernel_router.cuh:36-46: a float's bits mapped so that unsigned order is numeric order, -0 below +0, a
 * not-a-number above everything; ties go to the lower expert (its complement is larger). */
static uint64_t router_key(float score, uint32_t expert)
{
	uint32_t bits;
	memcpy(&bits, &score, sizeof(bits));
	const uint32_t ordered = score != score ? 0xFFFFFFFFu : (bits & 0x80000000u) ? ~bits : bits | 0x80000000u;
	return (uint64_t)ordered << 32 | (uint32_t)~expert;
}

/* e^a in FP32 by a fixed sequence of single roundings (the router's own definition, the same on the card): nothing
 * of the mathematics library, so the host and the card give the same bits. a is a number; below -104 the result is
 * +0, above 88.75 +infinity. n = rint(a log2 e); r = a - n ln 2 in two exact-product steps; a degree-7 polynomial;
 * the scale 2^n as two powers of two, so that only the last product can round (a subnormal result). */
static float router_power_of_two(int32_t exponent)
{
	const uint32_t bits = (uint32_t)(exponent + 127) << 23;
	float value;
	memcpy(&value, &bits, sizeof(value));
	return value;
}

static float router_exponential(float a)
{
	if (a < -104.0f)
		return 0.0f;
	if (a > 88.75f)
		return INFINITY;
	const float n = rintf(a * 1.44269504f);
	float r = a - n * 0.693359375f;
	r = r - n * -2.12194440e-4f;
	float p = 1.9875691500e-4f;
	p = p * r + 1.3981999507e-3f;
	p = p * r + 8.3334519073e-3f;
	p = p * r + 4.1665795894e-2f;
	p = p * r + 1.6666665459e-1f;
	p = p * r + 5.0000001201e-1f;
	p = p * (r * r) + r;
	p = p + 1.0f;
	const int32_t whole = (int32_t)n, first = whole >> 1;
	return p * router_power_of_two(first) * router_power_of_two(whole - first);
}

/* log(1 + t) for 0 <= t <= 1 as 2 atanh(z), z = t / (2 + t) <= 1/3, by nine terms of its series in z^2 */
static float router_log_one_plus(float t)
{
	const float z = t / (2.0f + t), w = z * z;
	float p = 1.0f / 17.0f;
	p = p * w + 1.0f / 15.0f;
	p = p * w + 1.0f / 13.0f;
	p = p * w + 1.0f / 11.0f;
	p = p * w + 1.0f / 9.0f;
	p = p * w + 1.0f / 7.0f;
	p = p * w + 1.0f / 5.0f;
	p = p * w + 1.0f / 3.0f;
	p = p * w + 1.0f;
	return 2.0f * z * p;
}

/* The affinity of a router score. SQRT_SOFTPLUS (include/anemone/router_records.h:10-12): sqrt(softplus(s)),
 * softplus(s) = s above 20, else max(s, 0) + log(1 + e^-|s|); SIGMOID: 1 / (1 + e^-s). A not-a-number stays one. */
float orc_router_affinity(float score, uint32_t scoring)
{
	if (score != score)
		return score;
	if (scoring == ROUTER_SCORING_SQRT_SOFTPLUS) {
		if (score > 20.0f)
			return sqrtf(score);
		const float magnitude = score < 0.0f ? -score : score;
		const float tail = router_log_one_plus(router_exponential(-magnitude));
		return sqrtf((score > 0.0f ? score : 0.0f) + tail);
	}
	return 1.0f / (1.0f + router_exponential(-score));
}

/* source/kernel_router.cuh:47-119 and tests/router_reference.c:150-190: the `picks` experts of the largest
 * affinity + bias (bias may be NULL: none), one at a time, the lower expert first among equals; slots in ascending
 * expert order; weights from the unbiased affinities, their sum from +0 in ascending expert order. */
void orc_router_row_biased(const float *scores, const float *bias, uint32_t expert_count, uint32_t picks,
			   uint32_t scoring, float route_scale, uint32_t *experts_out, float *weights_out)
{
	uint64_t keys[ROUTER_B200_MAXIMUM_EXPERTS];
	float affinities[ROUTER_B200_MAXIMUM_EXPERTS];
	uint32_t chosen[ROUTER_B200_MAXIMUM_PICKS];
	for (uint32_t expert = 0; expert < expert_count; expert++) {
		affinities[expert] = orc_router_affinity(scores[expert], scoring);
		keys[expert] = router_key(bias != NULL ? affinities[expert] + bias[expert] : affinities[expert], expert);
	}
	for (uint32_t pick = 0; pick < picks; pick++) {
		uint32_t best = 0;
		for (uint32_t expert = 1; expert < expert_count; expert++)
			if (keys[expert] > keys[best])
				best = expert;
		chosen[pick] = best;
		keys[best] = 0; /* below every live key */
	}
	/* slots in ascending expert order */
	for (uint32_t pick = 0; pick < picks; pick++) {
		uint32_t slot = 0;
		for (uint32_t other = 0; other < picks; other++)
			slot += chosen[other] < chosen[pick] ? 1u : 0u;
		experts_out[slot] = chosen[pick];
	}
	float sum = 0.0f;
	for (uint32_t slot = 0; slot < picks; slot++) {
		weights_out[slot] = affinities[experts_out[slot]];
		sum += weights_out[slot];
	}
	for (uint32_t slot = 0; slot < picks; slot++)
		weights_out[slot] = weights_out[slot] / (sum + 1e-20f) * route_scale;
}

void orc_router_row(const float *scores, uint32_t expert_count, uint32_t picks, uint32_t scoring, float route_scale,
		    uint32_t *experts_out, float *weights_out)
{
	orc_router_row_biased(scores, NULL, expert_count, picks, scoring, route_scale, experts_out, weights_out);
}

uint32_t orc_router_jobs(const uint32_t *experts, const float *weights, uint32_t live_rows, uint32_t picks,
			 uint32_t expert_count, uint32_t shared_count, const uint64_t *expert_table,
			 uint32_t job_capacity, struct expert_job_record *jobs_out)
{
	const uint32_t pairs_per_row = picks + shared_count;
	uint32_t job_count = 0;
	memset(jobs_out, 0, (size_t)job_capacity * sizeof(*jobs_out));
	for (uint32_t expert = 0; expert < expert_count + shared_count; expert++) {
		struct expert_job_record *job = NULL;
		for (uint32_t row = 0; row < live_rows; row++) {
			uint32_t slot = UINT32_MAX;
			float weight = 1.0f;
			if (expert >= expert_count) {
				slot = picks + (expert - expert_count);
			} else {
				for (uint32_t pick = 0; pick < picks; pick++)
					if (experts[row * picks + pick] == expert) {
						slot = pick;
						weight = weights[row * picks + pick];
					}
			}
			if (slot == UINT32_MAX)
				continue;
			if (job == NULL || job->row_count == LINEAR_MAXIMUM_ROWS) {
				if (job_count == job_capacity)
					return UINT32_MAX;
				job = &jobs_out[job_count++];
				job->gate_offset = expert_table[3u * expert];
				job->up_offset = expert_table[3u * expert + 1u];
				job->down_offset = expert_table[3u * expert + 2u];
				job->expert = expert;
			}
			job->pair_index[job->row_count] = row * pairs_per_row + slot;
			job->route_weight[job->row_count] = weight;
			job->row_count++;
		}
	}
	return job_count;
}
