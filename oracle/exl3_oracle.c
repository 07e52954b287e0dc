/*
 * exl3_oracle.c: CPU restatement of the reference's EXL3 decode and expert chain.
 * TEST INFRASTRUCTURE ONLY (see anemone_oracle.h): never linked into or called by the shipped library.
 * Parity pinned against the reference's known-answer vectors and its own compiled oracle (oracle/_ref).
 */
#include "anemone_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ---------------------------------------------------------------- numeric helpers */

float orc_half_value(uint16_t bits)
{
	const uint32_t sign = bits >> 15, exponent = (bits >> 10) & 31u, fraction = bits & 1023u;
	double magnitude;
	if (exponent == 0)
		magnitude = ldexp((double)fraction, -24);
	else if (exponent == 31)
		magnitude = fraction == 0 ? INFINITY : NAN;
	else
		magnitude = ldexp((double)(fraction | 1024u), (int)exponent - 25);
	return (float)(sign ? -magnitude : magnitude);
}

uint16_t orc_half_nearest(double value)
{
	if (value != value)
		return 0x7E00u;
	const uint16_t sign = signbit(value) ? 0x8000u : 0u;
	const double magnitude = fabs(value);
	if (magnitude >= 65520.0) /* halfway between the largest finite FP16 and 2^16 rounds up to infinity */
		return sign | 0x7C00u;
	if (magnitude < ldexp(1.0, -14)) {
		/* subnormal: multiples of 2^-24, nearest even */
		const double scaled = ldexp(magnitude, 24);
		const double rounded = nearbyint(scaled); /* round-to-nearest-even under the default mode */
		return sign | (uint16_t)rounded; /* 1024 becomes the smallest normal, as it should */
	}
	int exponent;
	const double fraction = frexp(magnitude, &exponent); /* magnitude = fraction * 2^exponent, 0.5 <= fraction < 1 */
	double mantissa = nearbyint(ldexp(fraction, 11)); /* 1024 .. 2048 */
	int biased = exponent - 1 + 15;
	if (mantissa == 2048.0) {
		mantissa = 1024.0;
		biased++;
	}
	if (biased >= 31)
		return sign | 0x7C00u;
	return sign | (uint16_t)(biased << 10) | (uint16_t)((uint32_t)mantissa - 1024u);
}

float orc_bfloat16_value(uint16_t bits)
{
	const uint32_t word = (uint32_t)bits << 16;
	float value;
	memcpy(&value, &word, sizeof(value));
	return value;
}

/* source/kernel_linear_common.cuh:186-191: add 0x7FFF plus the kept bit's parity, cut; any NaN -> 0x7FC0 */
uint16_t orc_bfloat16_bits(float value)
{
	uint32_t bits;
	memcpy(&bits, &value, sizeof(bits));
	if ((bits & 0x7FFFFFFFu) > 0x7F800000u)
		return 0x7FC0u;
	return (uint16_t)((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16);
}

/* ---------------------------------------------------------------- decode */

/* include/anemone/exl3_records.h:69-72; tests/exl3_reference.c:25-37. The product of the FP16 fused multiply-add
 * is exact in double (11-bit x 11-bit significands), as is its sum with the bias, so one rounding remains. */
uint16_t orc_exl3_codebook(uint32_t state)
{
	const uint32_t hashed = (state & 0xFFFFu) * EXL3_MUL1_MULTIPLIER;
	const uint32_t byte_sum = (hashed & 255u) + ((hashed >> 8) & 255u) + ((hashed >> 16) & 255u) + (hashed >> 24);
	const double base = (double)orc_half_value((uint16_t)(EXL3_MUL1_BASE + byte_sum));
	return orc_half_nearest(base * (double)orc_half_value(EXL3_MUL1_SCALE) +
				(double)orc_half_value(EXL3_MUL1_BIAS));
}

static uint16_t codebook_table[65536];
static int codebook_ready;

static const uint16_t *codebook(void)
{
	if (!codebook_ready) {
#ifdef _OPENMP
#pragma omp critical(orc_codebook)
#endif
		{
			if (!codebook_ready) {
				for (uint32_t state = 0; state < 65536u; state++)
					codebook_table[state] = orc_exl3_codebook(state);
				codebook_ready = 1;
			}
		}
	}
	return codebook_table;
}

static uint32_t tile_words(uint32_t bits_x2)
{
	return EXL3_TILE_VALUES * bits_x2 / 2u / EXL3_WORD_BITS;
}

static uint32_t load_word(const unsigned char *bytes)
{
	return (uint32_t)bytes[0] | (uint32_t)bytes[1] << 8 | (uint32_t)bytes[2] << 16 | (uint32_t)bytes[3] << 24;
}

/* tests/exl3_reference.c:66-99: one bit at a time, MSB-first inside little-endian 32-bit words, cyclic. */
uint16_t orc_exl3_state(const unsigned char *codes, uint32_t inputs, uint32_t outputs, uint32_t stored_width,
			uint32_t input, uint32_t output)
{
	(void)inputs;
	const uint32_t bits_x2 = exl3_bits_x2(stored_width);
	const uint32_t ring_bits = EXL3_TILE_VALUES * bits_x2 / 2u;
	const uint64_t tile = (uint64_t)(input / EXL3_TILE) * (outputs / EXL3_TILE) + output / EXL3_TILE;
	const unsigned char *const bytes = codes + tile * (ring_bits / 8u);
	const uint32_t position = exl3_tile_position(input % EXL3_TILE, output % EXL3_TILE);
	const uint32_t end = exl3_window_end(position, bits_x2);
	uint32_t state = 0;
	for (uint32_t bit = 0; bit < EXL3_STATE_BITS; bit++) {
		const uint32_t ring_bit = (end + ring_bits - EXL3_STATE_BITS + bit) % ring_bits;
		const uint32_t word = load_word(bytes + ring_bit / 32u * 4u);
		state = state << 1 | ((word >> (31u - ring_bit % 32u)) & 1u);
	}
	return (uint16_t)state;
}

/* 16 bits starting at ring bit `begin` of a tile of `words` words */
static inline uint32_t ring_window(const unsigned char *tile, uint32_t words, uint32_t begin)
{
	const uint32_t word = begin / 32u, shift = begin % 32u;
	const uint64_t both = (uint64_t)load_word(tile + 4u * word) << 32 | load_word(tile + 4u * ((word + 1u) % words));
	return (uint32_t)(both >> (48u - shift)) & 0xFFFFu;
}

/* The 256 states of one tile into [16 inputs][16 outputs] with row stride `stride`. */
static void tile_states(const unsigned char *tile, uint32_t bits_x2, uint16_t *out, uint32_t stride)
{
	const uint32_t words = tile_words(bits_x2), ring_bits = words * 32u;
	for (uint32_t position = 0; position < EXL3_TILE_VALUES; position++) {
		const uint32_t lane = position >> 3, element = position & 7u;
		const uint32_t input = (lane & 3u) * 2u + (element & 1u) + ((element & 2u) ? 8u : 0u);
		const uint32_t output = (lane >> 2) + ((element & 4u) ? 8u : 0u);
		const uint32_t begin =
			(exl3_window_end(position, bits_x2) + ring_bits - EXL3_STATE_BITS) % ring_bits;
		out[input * stride + output] = (uint16_t)ring_window(tile, words, begin);
	}
}

void orc_exl3_states(const unsigned char *codes, uint32_t inputs, uint32_t outputs, uint32_t stored_width,
		     uint16_t *states_out)
{
	const uint32_t bits_x2 = exl3_bits_x2(stored_width);
	const uint32_t tile_bytes = tile_words(bits_x2) * 4u;
	const uint32_t tile_columns = outputs / EXL3_TILE;
	for (uint32_t tile_row = 0; tile_row < inputs / EXL3_TILE; tile_row++)
		for (uint32_t tile_column = 0; tile_column < tile_columns; tile_column++)
			tile_states(codes + ((uint64_t)tile_row * tile_columns + tile_column) * tile_bytes, bits_x2,
				    states_out + (uint64_t)tile_row * EXL3_TILE * outputs + tile_column * EXL3_TILE,
				    outputs);
}

void orc_exl3_decode(const unsigned char *codes, uint32_t inputs, uint32_t outputs, uint32_t stored_width,
		     uint16_t *weights_out)
{
	const uint16_t *const table = codebook();
	orc_exl3_states(codes, inputs, outputs, stored_width, weights_out);
	const uint64_t count = (uint64_t)inputs * outputs;
	for (uint64_t index = 0; index < count; index++)
		weights_out[index] = table[weights_out[index]];
}

uint64_t orc_exl3_states_digest(const unsigned char *codes, uint32_t inputs, uint32_t outputs, uint32_t stored_width)
{
	uint64_t digest = 0xCBF29CE484222325ull;
	for (uint32_t input = 0; input < inputs; input++)
		for (uint32_t output = 0; output < outputs; output++) {
			const uint16_t state = orc_exl3_state(codes, inputs, outputs, stored_width, input, output);
			digest = (digest ^ (state & 255u)) * 0x100000001B3ull;
			digest = (digest ^ (uint32_t)(state >> 8)) * 0x100000001B3ull;
		}
	return digest;
}

uint64_t orc_exl3_slice(const unsigned char *source, uint32_t inputs, uint32_t outputs, uint32_t stored_width,
			uint32_t in_begin, uint32_t in_count, uint32_t out_begin, uint32_t out_count,
			unsigned char *destination)
{
	const uint32_t bits_x2 = exl3_bits_x2(stored_width);
	const uint64_t tile_bytes = tile_words(bits_x2) * 4u;
	const uint64_t source_row = outputs / EXL3_TILE * tile_bytes, kept_row = out_count / EXL3_TILE * tile_bytes;
	unsigned char *cursor = destination;
	for (uint32_t row = 0; row < in_count / EXL3_TILE; row++) {
		memcpy(cursor,
		       source + (uint64_t)(in_begin / EXL3_TILE + row) * source_row +
			       out_begin / EXL3_TILE * tile_bytes,
		       kept_row);
		cursor += kept_row;
	}
	const unsigned char *const scales = source + exl3_code_bytes(inputs, outputs, bits_x2);
	memcpy(cursor, scales + (uint64_t)in_begin * 2u, (uint64_t)in_count * 2u);
	cursor += (uint64_t)in_count * 2u;
	memcpy(cursor, scales + ((uint64_t)inputs + out_begin) * 2u, (uint64_t)out_count * 2u);
	cursor += (uint64_t)out_count * 2u;
	return (uint64_t)(cursor - destination);
}

/* ---------------------------------------------------------------- expert chain */

/* source/kernel_exl3.cu:104-124: value = (column & stride) == 0 ? value + other : other - value */
void orc_hadamard128(float *values)
{
	float next[EXL3_TRANSFORM];
	for (uint32_t stride = 1; stride < EXL3_TRANSFORM; stride *= 2u) {
		for (uint32_t column = 0; column < EXL3_TRANSFORM; column++) {
			const float value = values[column], other = values[column ^ stride];
			next[column] = (column & stride) == 0 ? value + other : other - value;
		}
		memcpy(values, next, sizeof(next));
	}
}

static uint16_t load_half(const unsigned char *bytes, uint64_t index)
{
	return (uint16_t)(bytes[2u * index] | bytes[2u * index + 1u] << 8);
}

struct product_shape {
	uint32_t inputs, outputs;
};

/* FP32 [column][outputs] products of one job's matrix against its columns' FP16 operands, one 16-output tile column:
 * double accumulation over the whole K, one rounding to FP32. */
static void product_tile_column(const unsigned char *matrix, uint32_t bits_x2, struct product_shape shape,
				uint32_t tile_column, const uint16_t *const *operand_rows, uint32_t columns,
				float *const *product_rows)
{
	const uint16_t *const table = codebook();
	const uint32_t tile_bytes = tile_words(bits_x2) * 4u;
	double sums[LINEAR_MAXIMUM_ROWS][EXL3_TILE] = { { 0 } };
	uint16_t states[EXL3_TILE * EXL3_TILE];
	float weights[EXL3_TILE * EXL3_TILE];
	for (uint32_t tile_row = 0; tile_row < shape.inputs / EXL3_TILE; tile_row++) {
		tile_states(matrix + ((uint64_t)tile_row * (shape.outputs / EXL3_TILE) + tile_column) * tile_bytes,
			    bits_x2, states, EXL3_TILE);
		for (uint32_t index = 0; index < EXL3_TILE * EXL3_TILE; index++)
			weights[index] = orc_half_value(table[states[index]]);
		for (uint32_t column = 0; column < columns; column++) {
			const uint16_t *const operands = operand_rows[column] + (uint64_t)tile_row * EXL3_TILE;
			for (uint32_t input = 0; input < EXL3_TILE; input++) {
				const double fed = (double)orc_half_value(operands[input]);
				for (uint32_t output = 0; output < EXL3_TILE; output++)
					sums[column][output] += (double)weights[input * EXL3_TILE + output] * fed;
			}
		}
	}
	for (uint32_t column = 0; column < columns; column++)
		for (uint32_t output = 0; output < EXL3_TILE; output++)
			product_rows[column][tile_column * EXL3_TILE + output] = (float)sums[column][output];
}

static uint32_t job_bits_x2(const struct exl3_expert_record *record, const struct expert_job_record *job,
			    const uint32_t *widths)
{
	return exl3_bits_x2(widths != NULL ? widths[job->expert] : record->bits_per_weight);
}

void orc_exl3_experts(const struct exl3_expert_record *record, unsigned char *arena, const uint32_t *widths,
		      uint32_t threads)
{
	const struct expert_job_record *const jobs = (const struct expert_job_record *)(arena + record->jobs_offset);
	const uint32_t H = record->input_size, I = record->inner_size, pairs = record->pair_count;
	const unsigned char *const input = arena + record->input_offset;
	uint16_t *const operands = (uint16_t *)(arena + record->operands_offset);
	float *const products = (float *)(arena + record->products_offset);
	uint16_t *const hidden = (uint16_t *)(arena + record->hidden_offset);
	const float N = EXL3_NORMALIZATION, L = record->activation_limit;
#ifdef _OPENMP
	const int workers = threads == 0 ? omp_get_max_threads() : (int)threads;
#else
	(void)threads;
#endif
	(void)codebook();

	/* input pass (source/kernel_exl3.cu:133-167): operands [projection][pair][H] */
	for (uint32_t j = 0; j < record->job_count; j++) {
		const struct expert_job_record *const job = &jobs[j];
		const uint64_t codes = exl3_code_bytes(H, I, job_bits_x2(record, job, widths));
		for (uint32_t projection = 0; projection < EXL3_PROJECTIONS; projection++) {
			const unsigned char *const suh =
				arena + (projection == 0 ? job->gate_offset : job->up_offset) + codes;
			for (uint32_t column = 0; column < job->row_count; column++) {
				const uint32_t pair = job->pair_index[column], row = pair / record->pairs_per_row;
				for (uint32_t block = 0; block < H / EXL3_TRANSFORM; block++) {
					float values[EXL3_TRANSFORM];
					for (uint32_t lane = 0; lane < EXL3_TRANSFORM; lane++) {
						const uint32_t channel = block * EXL3_TRANSFORM + lane;
						values[lane] =
							orc_bfloat16_value(load_half(input, (uint64_t)row * H + channel)) *
							orc_half_value(load_half(suh, channel));
					}
					orc_hadamard128(values);
					for (uint32_t lane = 0; lane < EXL3_TRANSFORM; lane++)
						operands[((uint64_t)projection * pairs + pair) * H +
							 block * EXL3_TRANSFORM + lane] =
							orc_half_nearest((double)(values[lane] * N));
				}
			}
		}
	}

	/* gate/up products (source/kernel_exl3.cu:178-293): FP32 [projection][pair][I] */
	{
		const uint32_t tile_columns = I / EXL3_TILE;
		const int64_t items = (int64_t)record->job_count * EXL3_PROJECTIONS * tile_columns;
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 8) num_threads(workers)
#endif
		for (int64_t item = 0; item < items; item++) {
			const uint32_t tile_column = (uint32_t)(item % tile_columns);
			const uint32_t projection = (uint32_t)(item / tile_columns % EXL3_PROJECTIONS);
			const struct expert_job_record *const job = &jobs[item / tile_columns / EXL3_PROJECTIONS];
			if (job->row_count == 0)
				continue;
			const uint16_t *fed[LINEAR_MAXIMUM_ROWS];
			float *out[LINEAR_MAXIMUM_ROWS];
			for (uint32_t column = 0; column < job->row_count; column++) {
				const uint64_t plane = (uint64_t)projection * pairs + job->pair_index[column];
				fed[column] = operands + plane * H;
				out[column] = products + plane * I;
			}
			product_tile_column(arena + (projection == 0 ? job->gate_offset : job->up_offset),
					    job_bits_x2(record, job, widths), (struct product_shape){ H, I },
					    tile_column, fed, job->row_count, out);
		}
	}

	/* activation (source/kernel_exl3.cu:314-372): bfloat16 hidden [pair][I], FP16 down operands [pair][I] */
	for (uint32_t j = 0; j < record->job_count; j++) {
		const struct expert_job_record *const job = &jobs[j];
		const uint32_t bits_x2 = job_bits_x2(record, job, widths);
		const unsigned char *const gate_svh = arena + job->gate_offset + exl3_code_bytes(H, I, bits_x2) + 2u * H;
		const unsigned char *const up_svh = arena + job->up_offset + exl3_code_bytes(H, I, bits_x2) + 2u * H;
		const unsigned char *const down_suh = arena + job->down_offset + exl3_code_bytes(I, H, bits_x2);
		for (uint32_t column = 0; column < job->row_count; column++) {
			const uint32_t pair = job->pair_index[column];
			for (uint32_t block = 0; block < I / EXL3_TRANSFORM; block++) {
				float gate[EXL3_TRANSFORM], up[EXL3_TRANSFORM], fed[EXL3_TRANSFORM];
				const uint64_t base = (uint64_t)pair * I + block * EXL3_TRANSFORM;
				memcpy(gate, products + base, sizeof(gate));
				memcpy(up, products + (uint64_t)pairs * I + base, sizeof(up));
				orc_hadamard128(gate);
				orc_hadamard128(up);
				for (uint32_t lane = 0; lane < EXL3_TRANSFORM; lane++) {
					const uint32_t channel = block * EXL3_TRANSFORM + lane;
					const float gate_value = gate[lane] * N * orc_half_value(load_half(gate_svh, channel));
					const float up_value = up[lane] * N * orc_half_value(load_half(up_svh, channel));
					const float bounded_gate = fminf(gate_value, L);
					const float bounded_up = fminf(fmaxf(up_value, -L), L);
					const float value = bounded_gate / (1.0f + expf(-bounded_gate)) * bounded_up;
					hidden[base + lane] = orc_bfloat16_bits(value);
					fed[lane] = value * orc_half_value(load_half(down_suh, channel));
				}
				orc_hadamard128(fed);
				for (uint32_t lane = 0; lane < EXL3_TRANSFORM; lane++)
					operands[base + lane] = orc_half_nearest((double)(fed[lane] * N));
			}
		}
	}

	/* down products: FP32 [pair][H] */
	{
		const uint32_t tile_columns = H / EXL3_TILE;
		const int64_t items = (int64_t)record->job_count * tile_columns;
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 8) num_threads(workers)
#endif
		for (int64_t item = 0; item < items; item++) {
			const uint32_t tile_column = (uint32_t)(item % tile_columns);
			const struct expert_job_record *const job = &jobs[item / tile_columns];
			if (job->row_count == 0)
				continue;
			const uint16_t *fed[LINEAR_MAXIMUM_ROWS];
			float *out[LINEAR_MAXIMUM_ROWS];
			for (uint32_t column = 0; column < job->row_count; column++) {
				fed[column] = operands + (uint64_t)job->pair_index[column] * I;
				out[column] = products + (uint64_t)job->pair_index[column] * H;
			}
			product_tile_column(arena + job->down_offset, job_bits_x2(record, job, widths),
					    (struct product_shape){ I, H }, tile_column, fed, job->row_count, out);
		}
	}

	/* finish (source/kernel_exl3.cu:374-402): in place, FP32 [pair][H], route weight last */
	float *const outputs = (float *)(arena + record->output_offset);
	for (uint32_t j = 0; j < record->job_count; j++) {
		const struct expert_job_record *const job = &jobs[j];
		const unsigned char *const down_svh =
			arena + job->down_offset + exl3_code_bytes(I, H, job_bits_x2(record, job, widths)) + 2u * I;
		for (uint32_t column = 0; column < job->row_count; column++) {
			const uint32_t pair = job->pair_index[column];
			for (uint32_t block = 0; block < H / EXL3_TRANSFORM; block++) {
				float values[EXL3_TRANSFORM];
				const uint64_t base = (uint64_t)pair * H + block * EXL3_TRANSFORM;
				memcpy(values, products + base, sizeof(values));
				orc_hadamard128(values);
				for (uint32_t lane = 0; lane < EXL3_TRANSFORM; lane++) {
					const float value = values[lane] * N *
							    orc_half_value(load_half(down_svh, block * EXL3_TRANSFORM + lane));
					outputs[base + lane] = value * job->route_weight[column];
				}
			}
		}
	}
}

/* source/kernel_exl3.cu:406-424 */
void orc_exl3_row_sum(const struct expert_row_sum_arguments *record, uint32_t rows, unsigned char *arena)
{
	const float *const pairs = (const float *)(arena + record->pair_output_offset);
	float *const sums = (float *)(arena + record->row_output_offset);
	for (uint64_t row = 0; row < rows; row++)
		for (uint32_t channel = 0; channel < record->width; channel++) {
			float sum = 0.0f;
			for (uint32_t slot = 0; slot < record->pairs_per_row; slot++)
				sum += pairs[(row * record->pairs_per_row + slot) * record->width + channel];
			sums[row * record->width + channel] = sum;
		}
}
