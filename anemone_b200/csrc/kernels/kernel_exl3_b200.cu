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

template <uint32_t BX2>
__device__ __forceinline__ void moe_gate_up(const struct exl3_moe_record &moe, unsigned char *arena,
					    const struct expert_job_record *job, unsigned char *dynamic_shared,
					    exl3_product_shared *shared, uint32_t *flag)
{
	const struct exl3_expert_record &record = moe.base;
	const uint32_t lane = threadIdx.x % EXL3_WARP, warp = threadIdx.x / EXL3_WARP;
	const uint32_t H = record.input_size, I = record.inner_size, pairs = record.pair_count;
	const uint32_t runs = exl3_moe_splits(H, I), groups = I / EXL3_TRANSFORM;
	const uint32_t group = blockIdx.x / runs, run = blockIdx.x % runs, projection = blockIdx.z;
	const uint32_t steps = H / EXL3_TILE / runs;
	const uint32_t fed_column = lane / 4u < job->row_count ? lane / 4u : 0u;
	const __half *const operands = reinterpret_cast<const __half *>(arena + record.operands_offset);
	float sums[2][4];
	if (!exl3_product_core<BX2>(arena + (projection == 0 ? job->gate_offset : job->up_offset), I, group, run * steps,
				    steps, operands + ((uint64_t)projection * pairs + job->pair_index[fed_column]) * H,
				    dynamic_shared, shared, sums))
		return;
	/* partial sums: FP32 [projection][run][pair][I] */
	float *const partials = reinterpret_cast<float *>(arena + record.products_offset);
	const uint64_t run_stride = (uint64_t)pairs * I;
	float *rows[LINEAR_MAXIMUM_ROWS];
#pragma unroll
	for (uint32_t column = 0; column < LINEAR_MAXIMUM_ROWS; column++)
		rows[column] = partials + ((uint64_t)projection * runs + run) * run_stride +
			       (uint64_t)job->pair_index[column < job->row_count ? column : 0u] * I + group * EXL3_TRANSFORM;
	store_partial(sums, rows, job->row_count);
	uint32_t *const counter = reinterpret_cast<uint32_t *>(arena + moe.counters_offset) + blockIdx.y * groups + group;
	if (!last_of(counter, EXL3_PROJECTIONS * runs, flag))
		return;
	exl3_gate_up_epilogue<BX2>(moe, arena, job, group, partials, partials + (uint64_t)runs * run_stride, run_stride, runs,
				   runs);
}

template <uint32_t BX2>
__device__ __forceinline__ void moe_down(const struct exl3_moe_record &moe, unsigned char *arena,
					 const struct expert_job_record *job, unsigned char *dynamic_shared,
					 exl3_product_shared *shared, uint32_t *flag)
{
	const struct exl3_expert_record &record = moe.base;
	const uint32_t lane = threadIdx.x % EXL3_WARP, warp = threadIdx.x / EXL3_WARP;
	const uint32_t H = record.input_size, I = record.inner_size, pairs = record.pair_count;
	const uint32_t runs = exl3_moe_splits(I, H), groups = H / EXL3_TRANSFORM;
	const uint32_t group = blockIdx.x / runs, run = blockIdx.x % runs;
	const uint32_t steps = I / EXL3_TILE / runs;
	const uint32_t fed_column = lane / 4u < job->row_count ? lane / 4u : 0u;
	const __half *const operands =
		reinterpret_cast<const __half *>(arena + record.operands_offset) + (uint64_t)EXL3_PROJECTIONS * pairs * H;
	float sums[2][4];
	if (!exl3_product_core<BX2>(arena + job->down_offset, H, group, run * steps, steps,
				    operands + (uint64_t)job->pair_index[fed_column] * I, dynamic_shared, shared, sums))
		return;
	/* partial sums: FP32 [run][pair][H]; run 0's rows are also where the pair outputs go */
	float *const partials = reinterpret_cast<float *>(arena + record.products_offset);
	const uint64_t run_stride = (uint64_t)pairs * H;
	float *rows[LINEAR_MAXIMUM_ROWS];
#pragma unroll
	for (uint32_t column = 0; column < LINEAR_MAXIMUM_ROWS; column++)
		rows[column] = partials + run * run_stride +
			       (uint64_t)job->pair_index[column < job->row_count ? column : 0u] * H + group * EXL3_TRANSFORM;
	store_partial(sums, rows, job->row_count);
	uint32_t *const counter = reinterpret_cast<uint32_t *>(arena + moe.counters_offset) +
				  (uint64_t)record.job_count * (I / EXL3_TRANSFORM) + blockIdx.y * groups + group;
	if (!last_of(counter, runs, flag))
		return;
	exl3_down_epilogue<BX2>(moe, arena, job, group, partials, run_stride, runs);
}

#define MOE_WIDTH_SWITCH(function)                                                         \
	switch (exl3_job_bits_x2(record.base, job, moe_widths(record, arena))) {           \
	case EXL3_BITS_X2_K2:                                                              \
		function<EXL3_BITS_X2_K2>(record, arena, job, dynamic_shared, &shared, &flag);   \
		break;                                                                     \
	case EXL3_BITS_X2_K2_5:                                                            \
		function<EXL3_BITS_X2_K2_5>(record, arena, job, dynamic_shared, &shared, &flag); \
		break;                                                                     \
	case EXL3_BITS_X2_K3:                                                              \
		function<EXL3_BITS_X2_K3>(record, arena, job, dynamic_shared, &shared, &flag);   \
		break;                                                                     \
	case EXL3_BITS_X2_K4:                                                              \
		function<EXL3_BITS_X2_K4>(record, arena, job, dynamic_shared, &shared, &flag);   \
		break;                                                                     \
	default:                                                                           \
		break;                                                                     \
	}

extern "C" __global__ void __launch_bounds__(EXL3_PRODUCT_THREADS)
	exl3_moe_gate_up(struct exl3_moe_record record, unsigned char *arena)
{
	extern __shared__ __align__(128) unsigned char dynamic_shared[];
	__shared__ exl3_product_shared shared;
	__shared__ uint32_t flag;
	const struct expert_job_record *const job = exl3_job(record.base, arena, blockIdx.y);
	if (job->row_count == 0)
		return;
	MOE_WIDTH_SWITCH(moe_gate_up)
}

extern "C" __global__ void __launch_bounds__(EXL3_PRODUCT_THREADS)
	exl3_moe_down(struct exl3_moe_record record, unsigned char *arena)
{
	extern __shared__ __align__(128) unsigned char dynamic_shared[];
	__shared__ exl3_product_shared shared;
	__shared__ uint32_t flag;
	const struct expert_job_record *const job = exl3_job(record.base, arena, blockIdx.y);
	if (job->row_count == 0)
		return;
	MOE_WIDTH_SWITCH(moe_down)
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
