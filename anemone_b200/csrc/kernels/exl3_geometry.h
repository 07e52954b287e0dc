/*
 * exl3_geometry.h: launch geometry the EXL3 kernels and the host preparers must agree on. C11 and CUDA.
 */
#ifndef AB_EXL3_GEOMETRY_H
#define AB_EXL3_GEOMETRY_H

#include "anemone_b200_records.h"

#define EXL3_WARP 32u
#define EXL3_PRODUCT_WARPS 4u
#define EXL3_PRODUCT_THREADS (EXL3_PRODUCT_WARPS * EXL3_WARP)
#define EXL3_GROUP_TILES 8u /* adjacent output tiles of a product CTA: 128 outputs, one Hadamard block */
#define EXL3_STAGE_STEPS 4u /* K steps (tile rows) of one round of a product CTA: one a warp */
#define EXL3_TRANSFORM_WARPS 4u /* a transform CTA: one warp per 128-channel block */
#define EXL3_TRANSFORM_THREADS (EXL3_TRANSFORM_WARPS * EXL3_WARP)
#define EXL3_RECONSTRUCT_THREADS 256u
#define EXL3_ROW_SUM_THREADS 128u

/* bytes of the cross-warp partial sums of a product CTA: [warp][tile][lane] float4 */
#define EXL3_PRODUCT_PARTIAL_BYTES (EXL3_PRODUCT_WARPS * EXL3_GROUP_TILES * EXL3_WARP * 16u)

/* Dynamic shared memory of a product CTA: the partial sums (the same for every width). */
AB_INLINE uint32_t exl3_product_dynamic_bytes(uint32_t bits_x2)
{
	(void)bits_x2;
	return EXL3_PRODUCT_PARTIAL_BYTES;
}

/* Split K of the fused B200 launches: a product of `outputs` outputs over `inputs` inputs is cut in this many equal
 * runs of whole 128-input blocks, each its own CTA; the last CTA to finish a (job, 128 outputs) adds the runs in
 * ascending order from +0. A CTA that streams all of K is the cheapest (no partial sums to store and add), but a rank
 * with few outputs then starts too few CTAs to fill the card: the smallest power of two, at most 8, that gives a job
 * at least 32 work items (groups of 128 outputs times runs), dividing inputs / 128 and leaving a run at least 4
 * blocks (32 K steps). */
AB_INLINE uint32_t exl3_moe_splits(uint32_t inputs, uint32_t outputs)
{
	const uint32_t blocks = inputs / EXL3_TRANSFORM, groups = outputs / EXL3_TRANSFORM;
	uint32_t splits = 1u;
	while (splits < 8u && groups * splits < 32u && blocks % (2u * splits) == 0u && blocks / (2u * splits) >= 4u)
		splits *= 2u;
	return splits;
}

/* ---- the decode step's three launches (kernel_exl3_layer) ---- */
#define EXL3_LAYER_DEFAULT_SMS 148u
#define EXL3_LAYER_WORD_LIVE_JOBS 0u
#define EXL3_LAYER_WORD_TICKET 1u /* the next item of the products' list; zero between steps */
/* The default cut of the layer's products, measured on one to eight ranks' shapes of a hidden width of 4096 and an
 * intermediate width of 2048 (a CTA an item; an item's fixed cost, the chain of dependent loads from its ticket to its
 * first weights, is about 2.5 us of its place on the card): gate and up in 4 runs of K where the rank holds at least
 * 1024 inner channels, in 8 below (more items of the fewer outputs); down in one run. Halved while it does not divide
 * the K blocks of 128. */
AB_INLINE uint32_t exl3_layer_gate_up_runs(uint32_t input_size, uint32_t inner_size)
{
	uint32_t runs = inner_size >= 1024u ? 4u : 8u;
	while (runs > 1u && (input_size / EXL3_TRANSFORM) % runs != 0)
		runs /= 2u;
	return runs;
}

/* uint32 words of the moe record's counters that lie before the layer's own words */
AB_INLINE uint64_t exl3_layer_counter_begin(uint32_t job_count, uint32_t input_size, uint32_t inner_size)
{
	return (uint64_t)job_count * (inner_size / EXL3_TRANSFORM + input_size / EXL3_TRANSFORM);
}

/* bytes at counters_offset in the layer form: the per-(job, group) counters, then the layer's words, then a word a
 * job: how many groups of 128 inner channels of the job have their down operands in place (the router's launch
 * zeroes them, the gate and up items count, the down items, which run beside the last of those, read) */
AB_INLINE uint64_t exl3_layer_counter_bytes(uint32_t job_count, uint32_t input_size, uint32_t inner_size)
{
	return (exl3_layer_counter_begin(job_count, input_size, inner_size) + EXL3_LAYER_COUNTER_WORDS + job_count) * 4u;
}

/* the FP32 partial sums of the layer form: gate/up's [2][runs][pairs][inner], then, in a range of their own (down
 * items write while gate and up items still read), down's [runs][pairs][input] */
AB_INLINE uint64_t exl3_layer_gate_up_product_bytes(uint32_t pair_count, uint32_t inner_size)
{
	return (uint64_t)EXL3_PROJECTIONS * EXL3_LAYER_MAXIMUM_RUNS * pair_count * inner_size * 4u;
}

/* ---- prefill (kernel_exl3_prefill) ---- */
#define EXL3_PREFILL_GEMM_THREADS 576u /* a copy warp, an issuing warp, sixteen decode warps */
#define EXL3_PREFILL_OPERAND_PARTS 4u /* an operand CTA takes a quarter of a tile's rows */
#define EXL3_PREFILL_GATE_UP_STEPS 2u /* steps of 16 inputs of one stage: two matrices */
#define EXL3_PREFILL_DOWN_STEPS 4u /* one matrix */
/* ring depths: operand blocks (bulk copies, mostly from L2), decoded weights (made on the SM) */
#define EXL3_PREFILL_A_STAGES 4u
#define EXL3_PREFILL_B_STAGES 4u
/* the largest of the product CTAs' forms: a stage is 32 KB of one ring and 16 KB of the other */
#define EXL3_PREFILL_W_STAGE 8192u /* trellis words of one stage at most: 16 x 16 x 64 weights x 4 bits */
#define EXL3_PREFILL_DYNAMIC_BYTES \
	(EXL3_PREFILL_A_STAGES * 32768u + EXL3_PREFILL_B_STAGES * (16384u + EXL3_PREFILL_W_STAGE))
#define EXL3_PREFILL_STAGING_ROW 132u /* floats of a staged accumulator row */

#endif
