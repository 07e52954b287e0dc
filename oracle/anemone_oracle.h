/*
 * anemone_oracle.h: CPU restatement of the reference's arithmetic for the quantized MoE expert-layer path.
 *
 * THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE. Only the tests, the smoke check and the benchmark's CPU-baseline
 * legs may link or call it, and only as the checker or as the timed CPU baseline. The shipped library never calls
 * into this directory and has no CPU fallback.
 *
 * Parity is PINNED: the decode functions are checked against the reference's own known-answer vectors
 * (tests/exl3_widths_test.c:67-88, tests/exl3_sm120_reference_test.c:12-14, tests/exl3_test.c:13-14) and, where the
 * reference sources are present, against the reference's own oracle compiled from them (oracle/_ref, built by
 * oracle/Makefile); the ordered reduction against source/ordered_collective.c:144-206 compiled the same way and the
 * cancellation-sensitive vectors of tests/ordered_collective_test.c:190-272.
 *
 * Every function operates on the same bytes the device sees: a host image of the arena and the same by-value records.
 * All floating-point steps are single FP32 operations with one rounding each (build with -ffp-contract=off), in the
 * order the reference's kernels state, except the products, which are accumulated in double precision and rounded
 * once (the reference's tensor-core association is card-specific; the layer tolerance absorbs it).
 */
#ifndef ANEMONE_ORACLE_H
#define ANEMONE_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#include "anemone_b200_records.h"

/* ---- numeric helpers ---- */
float orc_half_value(uint16_t bits); /* FP16 bits -> value */
uint16_t orc_half_nearest(double value); /* value -> FP16 bits, to nearest, ties to even */
float orc_bfloat16_value(uint16_t bits);
/* FP32 -> bfloat16 bits, nearest-even, not-a-number -> 0x7FC0 (source/kernel_linear_common.cuh:186-191) */
uint16_t orc_bfloat16_bits(float value);

/* ---- EXL3 decode (tests/exl3_reference.c:25-107, include/anemone/exl3_records.h:69-72, 104-110) ---- */
/* FP16 bits of a 16-bit trellis state: b = byte sum of state * 0x83DCD12D; fma(fp16(1024 + b), 0x1EEE, 0xC931). */
uint16_t orc_exl3_codebook(uint32_t state);
/* The state of weight (input, output) by walking the tile's ring bit by bit (slow, independent of the table path). */
uint16_t orc_exl3_state(const unsigned char *codes, uint32_t inputs, uint32_t outputs, uint32_t stored_width,
			uint32_t input, uint32_t output);
/* All states / all FP16 weights of a matrix, [input][output]; sliding-window, table-driven (the timed CPU path). */
void orc_exl3_states(const unsigned char *codes, uint32_t inputs, uint32_t outputs, uint32_t stored_width,
		     uint16_t *states_out);
void orc_exl3_decode(const unsigned char *codes, uint32_t inputs, uint32_t outputs, uint32_t stored_width,
		     uint16_t *weights_out);
/* FNV-1a 64 over the states, input-major, low byte first (the digest of tests/exl3_widths_test.c:182-213). */
uint64_t orc_exl3_states_digest(const unsigned char *codes, uint32_t inputs, uint32_t outputs, uint32_t stored_width);
/* Lossless slice of a stored matrix (source/exl3_layout.c:45-106): codes of inputs [in_begin, +in_count) x outputs
 * [out_begin, +out_count), then the matching parts of suh and svh. All multiples of 128. Returns bytes written. */
uint64_t orc_exl3_slice(const unsigned char *source, uint32_t inputs, uint32_t outputs, uint32_t stored_width,
			uint32_t in_begin, uint32_t in_count, uint32_t out_begin, uint32_t out_count,
			unsigned char *destination);

/* ---- the expert chain on an arena image (source/kernel_exl3.cu:104-124, 133-167, 178-293, 314-402, 406-424) ---- */
/* In-place 128-point Sylvester butterfly in the kernel's order: stride 1..64, lower = a + b, upper = a - b. */
void orc_hadamard128(float *values);
/* The five passes on the host image, writing the same arrays the launches write (operands, products, hidden,
 * pair outputs). widths: NULL, or per-expert stored widths (then record->bits_per_weight is ignored).
 * threads: worker threads over jobs x output tiles (0 = all cores). */
void orc_exl3_experts(const struct exl3_expert_record *record, unsigned char *arena, const uint32_t *widths,
		      uint32_t threads);
/* exl3_row_sum: rows x width FP32 sums of pairs_per_row pair outputs from +0 in ascending slot order. */
void orc_exl3_row_sum(const struct expert_row_sum_arguments *record, uint32_t rows, unsigned char *arena);

/* ---- ordered reduction (source/ordered_collective.c:187-204, source/kernel_tp_exchange.cu:223-237) ---- */
/* outputs[e] = ((+0 + in[0][e]) + in[1][e]) + ... */
void orc_ordered_sum(const float *const *inputs, uint32_t rank_count, uint32_t element_count, float *output);
/* The same sum rounded once to bfloat16. */
void orc_ordered_reduce_bf16(const float *const *inputs, uint32_t rank_count, uint32_t element_count,
			     uint16_t *output);
/* The one-shot push (source/kernel_ordered_push.cuh:121-290): payload_format 0 = FP32 wire, the sum above; 1 = every
 * rank's value (its own too) rounded to bfloat16 to nearest even (cvt.rn.bf16.f32) before the same adds. */
void orc_ordered_push(const float *const *inputs, uint32_t rank_count, uint32_t element_count, uint32_t payload_format,
		      float *output);
/* The owner sums (source/kernel_tp_exchange.cu:190-247): the push's sum rounded once to bfloat16. */
void orc_owner_sums(const float *const *inputs, uint32_t rank_count, uint32_t element_count, uint32_t payload_format,
		    uint16_t *output);
/* The local completion around the exchange (source/kernel_tp2_join.cu:43-108) on a host copy of the arena. */
void orc_tp2_join(const struct tp2_join_arguments *record, unsigned char *arena);
/* The four operations of the reference's host twin, same argument meaning as ordered_collective_host. */
int orc_ordered_collective(const float *const *inputs, float *const *outputs, uint32_t rank_count,
			   uint32_t element_count, int operation);

/* ---- router (source/kernel_router.cuh:36-119; include/anemone/router_records.h:10-30) ---- */
/* One row: `picks` experts by slot (ascending expert) and their weights. scoring: ROUTER_SCORING_*. */
void orc_router_row(const float *scores, uint32_t expert_count, uint32_t picks, uint32_t scoring, float route_scale,
		    uint32_t *experts_out, float *weights_out);
/* The same with a per-expert selection bias (NULL: none): picks by affinity + bias, weights from the affinity alone. */
void orc_router_row_biased(const float *scores, const float *bias, uint32_t expert_count, uint32_t picks,
			   uint32_t scoring, float route_scale, uint32_t *experts_out, float *weights_out);
/* The affinity of one score: a fixed sequence of FP32 roundings with no library function, so the card's bits equal
 * the host's. */
float orc_router_affinity(float score, uint32_t scoring);
/* The job table of the live rows (same bytes as router_select_b200 writes). Returns the number of non-empty jobs. */
uint32_t orc_router_jobs(const uint32_t *experts, const float *weights, uint32_t live_rows, uint32_t picks,
			 uint32_t expert_count, uint32_t shared_count, const uint64_t *expert_table,
			 uint32_t job_capacity, struct expert_job_record *jobs_out);

/* ---- original-weights experts: MXFP4 weights by E4M3 block-quantized activations (mx_oracle.c) ---- */
double orc_e2m1_value(uint32_t code);
double orc_e4m3_value(uint32_t code);
double orc_e8m0_value(uint32_t code);
/* bfloat16 values -> natural-order E4M3 codes and block exponents (tests/linear_reference.c:249-288) */
void orc_mx_quantize(const uint16_t *values, uint32_t width, uint8_t *codes_out, uint8_t *exponents_out);
void orc_mx_codes_lay_out(const uint8_t *codes, uint32_t width, uint8_t *stored_out);
void orc_mx_operands_lay_out(const uint8_t *codes, uint32_t width, uint16_t *operands_out);
/* 4-bit codes [output][input] and E8M0 scales [output][input / 32] -> the stored matrix */
void orc_mx_weights_lay_out(const uint8_t *codes, const uint8_t *scales, uint32_t outputs, uint32_t inputs,
			    uint8_t *stored_out);
uint16_t orc_mx_output(const uint8_t *stored, uint32_t outputs, uint32_t inputs, uint32_t output, const uint8_t *codes,
		       const uint8_t *exponents, uint32_t slices);
uint16_t orc_mx_hidden(uint16_t gate_bits, uint16_t up_bits, float limit, float route_weight);
void orc_mx_experts(const struct expert_gate_up_arguments *gate_up, const struct expert_down_arguments *down,
		    uint32_t job_count, uint32_t slices_gate_up, uint32_t slices_down, uint64_t hidden_codes_offset,
		    uint64_t hidden_exponents_offset, uint64_t hidden_operands_offset, unsigned char *arena);
void orc_mx_row_sum(const struct expert_row_sum_arguments *record, uint32_t rows, unsigned char *arena);
/* the always-on expert: E4M3 weights, one E8M0 scale per 32 outputs by 32 inputs (tests/weight_format_reference.h:8-16,
 * tests/linear_reference.h:30-37) */
void orc_e4m3_weights_lay_out(const uint8_t *codes, const uint8_t *scales, uint32_t outputs, uint32_t inputs,
			      uint8_t *stored_out);
uint16_t orc_trunk_output(const uint8_t *stored, uint32_t outputs, uint32_t inputs, uint32_t output, const uint8_t *codes,
			  const uint8_t *exponents, uint32_t slices);
void orc_shared_expert(const struct trunk_linear_quantized_arguments *gate_up, const struct trunk_hidden_arguments *hidden,
		       const struct activation_quantize_arguments *quantize,
		       const struct trunk_linear_quantized_arguments *down, uint32_t slices_gate_up, uint32_t slices_down,
		       unsigned char *arena);
/* the same three for WEIGHT_FORMAT_E4M3_BLOCK128 (one FP32 scale per 128 outputs by 128 inputs; not a format of the
 * reference: the chain rule is its own with that scale in the place of 2^(weight code - 127)) */
void orc_e4m3_block128_lay_out(const uint8_t *codes, const float *scales, uint32_t outputs, uint32_t inputs,
			       uint8_t *stored_out);
uint16_t orc_trunk_output_block128(const uint8_t *stored, uint32_t outputs, uint32_t inputs, uint32_t output,
				   const uint8_t *codes, const uint8_t *exponents, uint32_t slices);
void orc_shared_expert_block128(const struct trunk_linear_quantized_arguments *gate_up,
				const struct trunk_hidden_arguments *hidden,
				const struct activation_quantize_arguments *quantize,
				const struct trunk_linear_quantized_arguments *down, uint32_t slices_gate_up,
				uint32_t slices_down, unsigned char *arena);

/* ---- the output-axis exchanges (ring_oracle.c) ----
 * inputs[rank]: that rank's bfloat16 values, rank_count * packs_per_owner packs of eight. vectors: 0 for owner-major
 * parts, else the rows of [row][owner][the row's packs]. */
uint16_t orc_ring_bf16_add(uint16_t left, uint16_t right);
void orc_ring_bf16_sum(const uint16_t *const *inputs, uint32_t rank_count, uint32_t packs_per_owner, uint32_t vectors,
		       uint16_t *const *outputs);
void orc_ring_round_once(const uint16_t *const *inputs, uint32_t rank_count, uint64_t value_count, uint16_t *output);
void orc_ring_gather(const uint16_t *const *inputs, uint32_t rank_count, uint32_t packs_per_owner, uint32_t vectors,
		     uint16_t *output);
void orc_ring_packet_encode(const uint16_t *values, uint32_t *packet);
void orc_ring_packet_decode(const uint32_t *packet, uint16_t *values);

#endif
