/*
 * mx_oracle.c: CPU restatement of the reference's original-weights expert arithmetic: E4M3 block quantization of
 * activations, E2M1 weights with E8M0 scales, the sliced FP32 chains and the bfloat16 roundings
 * (include/anemone/linear_records.h:36-99; include/anemone/weight_format_seam.h:23-46; tests/linear_reference.c).
 * TEST INFRASTRUCTURE ONLY (see anemone_oracle.h): never linked into or called by the shipped library.
 * Pinned against the reference's own test references compiled from its sources (oracle/_ref): test_linear_quantize,
 * test_weight_format_lay_out, test_weight_format_*_value, test_linear_products' tolerance.
 */
#include "anemone_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

double orc_e2m1_value(uint32_t code)
{
	static const double magnitudes[8] = { 0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0 };
	return (code & 8u) ? -magnitudes[code & 7u] : magnitudes[code & 7u];
}

double orc_e4m3_value(uint32_t code)
{
	const uint32_t exponent = (code >> 3) & 15u, fraction = code & 7u;
	const double magnitude = exponent == 0 ? ldexp((double)fraction, -9) : ldexp((double)(8u + fraction), (int)exponent - 10);
	return (code & 0x80u) ? -magnitude : magnitude;
}

double orc_e8m0_value(uint32_t code)
{
	return ldexp(1.0, (int)code - 127);
}

/* tests/linear_reference.c:249-288: all in FP32 up to the scale, the division by a power of two exact */
void orc_mx_quantize(const uint16_t *values, uint32_t width, uint8_t *codes_out, uint8_t *exponents_out)
{
	for (uint32_t block = 0; block < width / 32u; block++) {
		const uint16_t *const in = values + 32u * block;
		float largest = 1.0e-4f;
		for (uint32_t index = 0; index < 32u; index++) {
			const float magnitude = orc_bfloat16_value((uint16_t)(in[index] & 0x7FFFu));
			largest = magnitude > largest ? magnitude : largest;
		}
		const float ratio = largest * (1.0f / 448.0f);
		uint32_t code = 0;
		while (code < 255u && orc_e8m0_value(code) < (double)ratio)
			code++;
		exponents_out[block] = (uint8_t)code;
		for (uint32_t index = 0; index < 32u; index++) {
			double scaled = (double)orc_bfloat16_value((uint16_t)(in[index] & 0x7FFFu)) * ldexp(1.0, 127 - (int)code);
			if (scaled > 448.0)
				scaled = 448.0;
			uint32_t nearest = 0;
			double distance = scaled;
			for (uint32_t candidate = 1; candidate < 127u; candidate++) {
				const double d = fabs(orc_e4m3_value(candidate) - scaled);
				if (d < distance || (d == distance && candidate % 2u == 0)) {
					nearest = candidate;
					distance = d;
				}
			}
			codes_out[32u * block + index] = (uint8_t)(nearest | ((in[index] & 0x8000u) ? 0x80u : 0u));
		}
	}
}

/* include/anemone/linear_records.h:20-25: natural order -> lane order */
void orc_mx_codes_lay_out(const uint8_t *codes, uint32_t width, uint8_t *stored_out)
{
	for (uint32_t byte = 0; byte < width; byte++) {
		const uint32_t j = byte % 4u, s = byte / 4u % 4u, t = byte / 16u % 4u, l = byte / 64u;
		stored_out[byte] = codes[64u * l + 16u * s + 2u * t + j / 2u + 8u * (j % 2u)];
	}
}

/* the operand of a code on this library's class: the E4M3 byte placed as FP16 bits; operand order */
void orc_mx_operands_lay_out(const uint8_t *codes, uint32_t width, uint16_t *operands_out)
{
	for (uint32_t half = 0; half < width; half++) {
		const uint32_t h = half % 2u, r = half / 2u % 2u, s = half / 4u % 4u, t = half / 16u % 4u, l = half / 64u;
		const uint8_t code = codes[64u * l + 16u * s + 2u * t + h + 8u * r];
		operands_out[half] = (uint16_t)(((uint32_t)(code & 0x80u) << 8) | ((uint32_t)(code & 0x7Fu) << 7));
	}
}

/* include/anemone/weight_format_seam.h:29-35: codes [output][input] (4-bit), scales [output][input / 32] -> stored */
void orc_mx_weights_lay_out(const uint8_t *codes, const uint8_t *scales, uint32_t outputs, uint32_t inputs,
			    uint8_t *stored_out)
{
	uint32_t *const words = (uint32_t *)stored_out;
	const uint32_t loads = inputs / 64u;
	memset(stored_out, 0, (size_t)outputs * inputs / 2u + (size_t)outputs * inputs / 32u);
	for (uint32_t tile = 0; tile < outputs / 16u; tile++)
		for (uint32_t load = 0; load < loads; load++)
			for (uint32_t lane = 0; lane < 32u; lane++)
				for (uint32_t step = 0; step < 4u; step++) {
					const uint32_t g = lane / 4u, t = lane % 4u;
					uint32_t word = 0;
					for (uint32_t r = 0; r < 4u; r++)
						for (uint32_t h = 0; h < 2u; h++) {
							const uint32_t output = 16u * tile + g + 8u * (r % 2u);
							const uint32_t input = 64u * load + 16u * step + 2u * t + 8u * (r / 2u) + h;
							word |= (uint32_t)(codes[(size_t)output * inputs + input] & 15u) << (4u * r + 16u * h);
						}
					words[(((size_t)tile * loads + load) * 32u + lane) * 4u + step] = word;
				}
	uint8_t *const stored_scales = stored_out + (size_t)outputs * inputs / 2u;
	for (uint32_t tile = 0; tile < outputs / 16u; tile++)
		for (uint32_t load = 0; load < loads; load++)
			for (uint32_t g = 0; g < 8u; g++)
				for (uint32_t q = 0; q < 2u; q++)
					for (uint32_t r = 0; r < 2u; r++)
						stored_scales[(((size_t)tile * loads + load) * 8u + g) * 4u + 2u * q + r] =
							scales[(size_t)(16u * tile + g + 8u * r) * (inputs / 32u) + 2u * load + q];
}

static uint32_t stored_weight(const uint8_t *stored, uint32_t inputs, uint32_t output, uint32_t input)
{
	const uint32_t tile = output / 16u, row = output % 16u, g = row % 8u, load = input / 64u, within = input % 64u;
	const uint32_t step = within / 16u, k = within % 16u, t = (k % 8u) / 2u, h = k % 2u, r = (row / 8u) + 2u * (k / 8u);
	const uint32_t *const words = (const uint32_t *)stored;
	const uint32_t word = words[(((size_t)tile * (inputs / 64u) + load) * 32u + 4u * g + t) * 4u + step];
	return (word >> (4u * r + 16u * h)) & 15u;
}

static uint32_t stored_scale(const uint8_t *stored, uint32_t outputs, uint32_t inputs, uint32_t output, uint32_t block)
{
	const uint8_t *const scales = stored + (size_t)outputs * inputs / 2u;
	const uint32_t tile = output / 16u, row = output % 16u;
	return scales[(((size_t)tile * (inputs / 64u) + block / 2u) * 8u + row % 8u) * 4u + 2u * (block % 2u) + row / 8u];
}

/* One output of one vector: S chains of FP32 fused multiply-adds, one per block of 32 inputs, p the exact sum of the
 * block's 32 products rounded once to FP32; the chains added from +0; rounded once to bfloat16. codes/exponents: the
 * vector's NATURAL-order E4M3 codes and its block exponents. */
uint16_t orc_mx_output(const uint8_t *stored, uint32_t outputs, uint32_t inputs, uint32_t output, const uint8_t *codes,
		       const uint8_t *exponents, uint32_t slices)
{
	const uint32_t loads = inputs / 64u;
	float sum = 0.0f;
	for (uint32_t slice = 0; slice < slices; slice++) {
		float chain = 0.0f;
		for (uint32_t load = loads * slice / slices; load < loads * (slice + 1u) / slices; load++)
			for (uint32_t q = 0; q < 2u; q++) {
				const uint32_t block = 2u * load + q;
				double exact = 0.0;
				for (uint32_t index = 0; index < 32u; index++)
					exact += orc_e2m1_value(stored_weight(stored, inputs, output, 32u * block + index)) *
						 orc_e4m3_value(codes[32u * block + index]);
				const float p = (float)exact;
				const float scale = (float)ldexp(1.0, (int)stored_scale(stored, outputs, inputs, output, block) - 127 +
									      (int)exponents[block] - 127);
				chain = fmaf(p, scale, chain);
			}
		sum = sum + chain;
	}
	return orc_bfloat16_bits(sum);
}

/* linear_records.h:94-99 with gate and up already bfloat16: the bits of the hidden value */
uint16_t orc_mx_hidden(uint16_t gate_bits, uint16_t up_bits, float limit, float route_weight)
{
	const float gate = orc_bfloat16_value(gate_bits), up = orc_bfloat16_value(up_bits);
	const float bounded_gate = gate > limit ? limit : gate;
	const float bounded_up = up > limit ? limit : (up < -limit ? -limit : up);
	const float gated = bounded_gate / (1.0f + expf(-bounded_gate));
	return orc_bfloat16_bits(gated * bounded_up * route_weight);
}

/* The routed experts on an arena image, launch for launch (gate/up with the hidden step; quantization of every pair's
 * hidden vector; down; FP32 row sum of the bfloat16 pair outputs). input codes/exponents: LANE-order codes and block
 * exponents of the rows, as activation_quantize_entry leaves them. */
void orc_mx_experts(const struct expert_gate_up_arguments *gate_up, const struct expert_down_arguments *down,
		    uint32_t job_count, uint32_t slices_gate_up, uint32_t slices_down, uint64_t hidden_codes_offset,
		    uint64_t hidden_exponents_offset, uint64_t hidden_operands_offset, unsigned char *arena)
{
	const struct expert_job_record *const jobs = (const struct expert_job_record *)(arena + gate_up->jobs_offset);
	const uint32_t H = gate_up->input_size, I = gate_up->output_size;
	uint8_t *const natural = malloc(H > I ? H : I);
	uint16_t *const hidden = (uint16_t *)(arena + gate_up->hidden_offset);
	for (uint32_t j = 0; j < job_count; j++) {
		const struct expert_job_record *const job = &jobs[j];
		for (uint32_t column = 0; column < job->row_count; column++) {
			const uint32_t pair = job->pair_index[column], row = pair / gate_up->pairs_per_row;
			const uint8_t *const lane_codes = arena + gate_up->codes_offset + (size_t)row * H;
			for (uint32_t byte = 0; byte < H; byte++) { /* lane order back to natural order */
				const uint32_t jj = byte % 4u, s = byte / 4u % 4u, t = byte / 16u % 4u, l = byte / 64u;
				natural[64u * l + 16u * s + 2u * t + jj / 2u + 8u * (jj % 2u)] = lane_codes[byte];
			}
			const uint8_t *const exponents = arena + gate_up->exponents_offset + (size_t)row * (H / 32u);
#pragma omp parallel for
			for (uint32_t output = 0; output < I; output++) {
				const uint16_t gate = orc_mx_output(arena + job->gate_offset, I, H, output, natural, exponents,
								    slices_gate_up);
				const uint16_t up = orc_mx_output(arena + job->up_offset, I, H, output, natural, exponents,
								  slices_gate_up);
				hidden[(size_t)pair * I + output] =
					orc_mx_hidden(gate, up, gate_up->activation_limit, job->route_weight[column]);
			}
		}
	}
	/* quantize the hidden vector of every pair */
	uint8_t *const codes = malloc(I);
	for (uint32_t pair = 0; pair < gate_up->pair_count; pair++) {
		orc_mx_quantize(hidden + (size_t)pair * I, I, codes, arena + hidden_exponents_offset + (size_t)pair * (I / 32u));
		orc_mx_codes_lay_out(codes, I, arena + hidden_codes_offset + (size_t)pair * I);
		orc_mx_operands_lay_out(codes, I, (uint16_t *)(arena + hidden_operands_offset) + (size_t)pair * I);
	}
	uint16_t *const outputs = (uint16_t *)(arena + down->output_offset);
	for (uint32_t j = 0; j < job_count; j++) {
		const struct expert_job_record *const job = &jobs[j];
		for (uint32_t column = 0; column < job->row_count; column++) {
			const uint32_t pair = job->pair_index[column];
			orc_mx_quantize(hidden + (size_t)pair * I, I, natural, codes); /* codes: scratch for the exponents */
			const uint8_t *const exponents = arena + hidden_exponents_offset + (size_t)pair * (I / 32u);
#pragma omp parallel for
			for (uint32_t output = 0; output < H; output++)
				outputs[(size_t)pair * H + output] = orc_mx_output(arena + job->down_offset, H, I, output, natural,
										   exponents, slices_down);
		}
	}
	free(codes);
	free(natural);
}

/* expert_row_sum_entry: FP32 sums of bfloat16 pair outputs from +0 in ascending slot order */
void orc_mx_row_sum(const struct expert_row_sum_arguments *record, uint32_t rows, unsigned char *arena)
{
	const uint16_t *const pairs = (const uint16_t *)(arena + record->pair_output_offset);
	float *const sums = (float *)(arena + record->row_output_offset);
	for (uint64_t row = 0; row < rows; row++)
		for (uint32_t channel = 0; channel < record->width; channel++) {
			float sum = 0.0f;
			for (uint32_t slot = 0; slot < record->pairs_per_row; slot++)
				sum += orc_bfloat16_value(pairs[(row * record->pairs_per_row + slot) * record->width + channel]);
			sums[row * record->width + channel] = sum;
		}
}

/* ---- the always-on expert: WEIGHT_FORMAT_E4M3_SCALED (include/anemone/weight_format_seam.h:36-42) ---- */

/* the byte of a stored matrix that holds W[output][input], by the format's own sentence: byte b of lane 4 g + t of
 * (tile, group) is W[16 tile + g + 8 (b % 2)][32 group + 8 (b / 4) + 2 t + (b / 2) % 2] */
static size_t e4m3_place(uint32_t inputs, uint32_t output, uint32_t input)
{
	const uint32_t tile = output / 16u, g = output % 8u, upper = output % 16u / 8u;
	const uint32_t group = input / 32u, within = input % 32u;
	const uint32_t quarter = within / 8u, t = within % 8u / 2u, odd = within % 2u;
	const uint32_t b = 4u * quarter + 2u * odd + upper;
	return (((size_t)tile * (inputs / 32u) + group) * 32u + 4u * g + t) * 16u + b;
}

/* codes [output][input] E4M3 bytes and scales [(outputs + 31) / 32][inputs / 32] E8M0 codes -> the stored matrix */
void orc_e4m3_weights_lay_out(const uint8_t *codes, const uint8_t *scales, uint32_t outputs, uint32_t inputs,
			      uint8_t *stored_out)
{
	for (uint32_t output = 0; output < outputs; output++)
		for (uint32_t input = 0; input < inputs; input++)
			stored_out[e4m3_place(inputs, output, input)] = codes[(size_t)output * inputs + input];
	memcpy(stored_out + (size_t)outputs * inputs, scales, (size_t)((outputs + 31u) / 32u) * (inputs / 32u));
}

/* One output of one row of trunk_linear_quantized_<S>: as orc_mx_output with E4M3 weights and one scale per 32 outputs
 * by 32 inputs (block128 0), or one FP32 scale per 128 outputs by 128 inputs behind the same bytes (block128 1: the
 * original-weights checkpoints' block-scaled FP8, which the reference does not have; the chain rule is the
 * reference's, include/anemone/linear_records.h:45-99, with that scale in the place of 2^(weight code - 127)).
 * codes/exponents: the row's NATURAL-order E4M3 codes and its block exponents. */
static uint16_t trunk_output(const uint8_t *stored, uint32_t outputs, uint32_t inputs, uint32_t output,
			     const uint8_t *codes, const uint8_t *exponents, uint32_t slices, int block128)
{
	const uint32_t loads = inputs / 64u;
	const uint8_t *const scales = stored + (size_t)outputs * inputs + (size_t)(output / 32u) * (inputs / 32u);
	const float *const scales128 =
		(const float *)(const void *)(stored + (size_t)outputs * inputs) + (size_t)(output / 128u) * (inputs / 128u);
	float sum = 0.0f;
	for (uint32_t slice = 0; slice < slices; slice++) {
		float chain = 0.0f;
		for (uint32_t load = loads * slice / slices; load < loads * (slice + 1u) / slices; load++)
			for (uint32_t q = 0; q < 2u; q++) {
				const uint32_t block = 2u * load + q;
				double exact = 0.0;
				for (uint32_t index = 0; index < 32u; index++)
					exact += orc_e4m3_value(stored[e4m3_place(inputs, output, 32u * block + index)]) *
						 orc_e4m3_value(codes[32u * block + index]);
				const float p = (float)exact;
				const float scale = block128 ? scales128[block / 4u] * (float)ldexp(1.0, (int)exponents[block] - 127) :
							       (float)ldexp(1.0, (int)scales[block] - 127 + (int)exponents[block] - 127);
				chain = fmaf(p, scale, chain);
			}
		sum = sum + chain;
	}
	return orc_bfloat16_bits(sum);
}

uint16_t orc_trunk_output(const uint8_t *stored, uint32_t outputs, uint32_t inputs, uint32_t output, const uint8_t *codes,
			  const uint8_t *exponents, uint32_t slices)
{
	return trunk_output(stored, outputs, inputs, output, codes, exponents, slices, 0);
}

uint16_t orc_trunk_output_block128(const uint8_t *stored, uint32_t outputs, uint32_t inputs, uint32_t output,
				   const uint8_t *codes, const uint8_t *exponents, uint32_t slices)
{
	return trunk_output(stored, outputs, inputs, output, codes, exponents, slices, 1);
}

/* E4M3 codes [output][input] in natural order and FP32 scales [ceil(outputs / 128)][inputs / 128] -> the stored matrix
 * of WEIGHT_FORMAT_E4M3_BLOCK128 */
void orc_e4m3_block128_lay_out(const uint8_t *codes, const float *scales, uint32_t outputs, uint32_t inputs,
			       uint8_t *stored_out)
{
	for (uint32_t output = 0; output < outputs; output++)
		for (uint32_t input = 0; input < inputs; input++)
			stored_out[e4m3_place(inputs, output, input)] = codes[(size_t)output * inputs + input];
	memcpy(stored_out + (size_t)outputs * inputs, scales, (size_t)((outputs + 127u) / 128u) * (inputs / 128u) * 4u);
}

/* The always-on expert on an arena image, launch for launch (linear_shared_expert_prepare's four): gate and up,
 * the hidden step with a route weight of 1, quantization of the hidden rows, down. */
static void shared_expert(const struct trunk_linear_quantized_arguments *gate_up, const struct trunk_hidden_arguments *hidden,
			  const struct activation_quantize_arguments *quantize,
			  const struct trunk_linear_quantized_arguments *down, uint32_t slices_gate_up, uint32_t slices_down,
			  unsigned char *arena, int block128)
{
	const uint32_t H = gate_up->input_size, I = gate_up->output_size[0], O = down->output_size[0];
	const uint32_t rows = gate_up->row_count;
	uint8_t *const natural = malloc(H > I ? H : I);
	uint8_t *const scratch = malloc(I);
	for (uint32_t row = 0; row < rows; row++) {
		const uint8_t *const lane_codes = arena + gate_up->codes_offset + (size_t)row * H;
		for (uint32_t byte = 0; byte < H; byte++) {
			const uint32_t jj = byte % 4u, s = byte / 4u % 4u, t = byte / 16u % 4u, l = byte / 64u;
			natural[64u * l + 16u * s + 2u * t + jj / 2u + 8u * (jj % 2u)] = lane_codes[byte];
		}
		const uint8_t *const exponents = arena + gate_up->exponents_offset + (size_t)row * (H / 32u);
		uint16_t *const gate_out = (uint16_t *)(arena + gate_up->output_offset[0]) + (size_t)row * I;
		uint16_t *const up_out = (uint16_t *)(arena + gate_up->output_offset[1]) + (size_t)row * I;
		uint16_t *const hidden_out = (uint16_t *)(arena + hidden->hidden_offset) + (size_t)row * I;
#pragma omp parallel for
		for (uint32_t output = 0; output < I; output++) {
			gate_out[output] = trunk_output(arena + gate_up->weights_offset[0], I, H, output, natural, exponents,
							slices_gate_up, block128);
			up_out[output] = trunk_output(arena + gate_up->weights_offset[1], I, H, output, natural, exponents,
						      slices_gate_up, block128);
			hidden_out[output] = orc_mx_hidden(gate_out[output], up_out[output], hidden->activation_limit, 1.0f);
		}
		uint8_t *const hidden_exponents = arena + quantize->exponents_offset + (size_t)row * (I / 32u);
		orc_mx_quantize(hidden_out, I, scratch, hidden_exponents);
		orc_mx_codes_lay_out(scratch, I, arena + quantize->codes_offset + (size_t)row * I);
		orc_mx_operands_lay_out(scratch, I, (uint16_t *)(arena + quantize->operands_offset) + (size_t)row * I);
		uint16_t *const out = (uint16_t *)(arena + down->output_offset[0]) + (size_t)row * O;
#pragma omp parallel for
		for (uint32_t output = 0; output < O; output++)
			out[output] = trunk_output(arena + down->weights_offset[0], O, I, output, scratch, hidden_exponents,
						   slices_down, block128);
	}
	free(scratch);
	free(natural);
}

void orc_shared_expert(const struct trunk_linear_quantized_arguments *gate_up, const struct trunk_hidden_arguments *hidden,
		       const struct activation_quantize_arguments *quantize,
		       const struct trunk_linear_quantized_arguments *down, uint32_t slices_gate_up, uint32_t slices_down,
		       unsigned char *arena)
{
	shared_expert(gate_up, hidden, quantize, down, slices_gate_up, slices_down, arena, 0);
}

void orc_shared_expert_block128(const struct trunk_linear_quantized_arguments *gate_up,
				const struct trunk_hidden_arguments *hidden,
				const struct activation_quantize_arguments *quantize,
				const struct trunk_linear_quantized_arguments *down, uint32_t slices_gate_up,
				uint32_t slices_down, unsigned char *arena)
{
	shared_expert(gate_up, hidden, quantize, down, slices_gate_up, slices_down, arena, 1);
}
