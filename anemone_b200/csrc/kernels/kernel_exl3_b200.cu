/*
 * kernel_exl3_b200.cu: the routed-expert layer of one rank in four launches (struct exl3_moe_record), with a stored
 * width per expert. No counterpart in the reference, whose chain is five launches of one width plus a row sum; the
 * arithmetic of every value is the same chain's (exl3_passes.cuh) except that a product is cut in exl3_moe_splits(K, outputs)
 * runs of K whose FP32 sums are added in ascending order from +0.
 *   exl3_moe_input    grid (ceil(H / 128 / 4), jobs, 2) x 128   x . suh, Hadamard, FP16 operands of gate and of up
 *   exl3_moe_gate_up  grid (I / 128 * S, jobs, 2) x 128        a CTA streams one run of K of 128 gate or up outputs of
 *                                                               its job and writes FP32 partial sums; the LAST CTA of a
 *                                                               (job, 128 outputs) to finish adds the runs, transforms,
 *                                                               applies SwiGLU and the down-side scale and transform:
 *                                                               bfloat16 hidden, FP16 down operands
 *   exl3_moe_down     grid (H / 128 * S', jobs) x 128          the same for down; the last CTA applies the output
 *                                                               transform, scale and route weight: FP32 pair outputs
 *   exl3_moe_row_sum  grid (ceil(H / 128), rows) x 128         FP32 row sums from +0 in ascending slot order
 * "Last" is found with a counter per (job, 128 outputs) in the arena (zero at load, reset by the CTA that finds it full):
 * which CTA is last varies from run to run, what it computes does not. Many short work items instead of one long one
 * per (job, 128 outputs) keep every SM busy to the end of a decode step, where only ~58 experts are active.
 */
#include "exl3_fused.cuh"

extern "C" __global__ void __launch_bounds__(EXL3_TRANSFORM_THREADS)
	exl3_moe_input(struct exl3_moe_record record, unsigned char *arena)
{
	exl3_input_pass(record.base, arena, moe_widths(record, arena));
}

extern "C" __global__ void __launch_bounds__(EXL3_PRODUCT_THREADS)
	exl3_moe_gate_up(struct exl3_moe_record record, unsigned char *arena)
{
	extern __shared__ __align__(128) unsigned char dynamic_shared[];
	__shared__ exl3_product_shared shared;
	__shared__ uint32_t flag;
	exl3_moe_gate_up_block(record, arena, exl3_moe_splits(record.base.input_size, record.base.inner_size),
			       dynamic_shared, &shared, &flag);
}

extern "C" __global__ void __launch_bounds__(EXL3_PRODUCT_THREADS)
	exl3_moe_down(struct exl3_moe_record record, unsigned char *arena)
{
	extern __shared__ __align__(128) unsigned char dynamic_shared[];
	__shared__ exl3_product_shared shared;
	__shared__ uint32_t flag;
	exl3_moe_down_block(record, arena, exl3_moe_splits(record.base.inner_size, record.base.input_size),
			    dynamic_shared, &shared, &flag);
}

extern "C" __global__ void exl3_moe_row_sum(struct exl3_moe_record record, unsigned char *arena)
{
	const uint32_t channel = blockIdx.x * blockDim.x + threadIdx.x;
	if (channel >= record.base.input_size)
		return;
	const uint64_t row = blockIdx.y;
	const uint32_t width = record.base.input_size, slots = record.base.pairs_per_row;
	const float *const pairs = reinterpret_cast<const float *>(arena + record.base.output_offset);
	float sum = 0.0f;
	for (uint32_t slot = 0; slot < slots; slot++)
		sum = __fadd_rn(sum, pairs[(row * slots + slot) * width + channel]);
	reinterpret_cast<float *>(arena + record.row_output_offset)[row * width + channel] = sum;
}
