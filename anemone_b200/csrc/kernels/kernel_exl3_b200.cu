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
#include "exl3_passes.cuh"

#define STAGED_ROW 132u /* floats of one staged column: 128 outputs and a pad that spreads the columns over the banks */

__device__ __forceinline__ const uint32_t *moe_widths(const struct exl3_moe_record &record, const unsigned char *arena)
{
	return record.base.bits_per_weight == EXL3_WIDTH_PER_EXPERT ?
		       reinterpret_cast<const uint32_t *>(arena + record.widths_offset) :
		       nullptr;
}

extern "C" __global__ void __launch_bounds__(EXL3_TRANSFORM_THREADS)
	exl3_moe_input(struct exl3_moe_record record, unsigned char *arena)
{
	exl3_input_pass(record.base, arena, moe_widths(record, arena));
}

/* this thread's sums (exl3_product_core's layout) to partial rows: row(column) + 128 group + output */
__device__ __forceinline__ void store_partial(const float sums[2][4], float *const rows[LINEAR_MAXIMUM_ROWS],
					      uint32_t row_count)
{
	const uint32_t lane = threadIdx.x % EXL3_WARP, warp = threadIdx.x / EXL3_WARP;
	const uint32_t group_lane = lane / 4u, place = lane % 4u;
#pragma unroll
	for (uint32_t mine = 0; mine < 2; mine++)
#pragma unroll
		for (uint32_t c = 0; c < 4; c++) {
			const uint32_t column = place * 2u + (c & 1u);
			if (column < row_count)
				rows[column][(warp * 2u + mine) * EXL3_TILE + group_lane + (c >> 1) * 8u] = sums[mine][c];
		}
}

/* true in exactly one CTA of the `expected` that work on this counter: the last to arrive. Every CTA's partial sums are
 * visible to it. The counter is left at zero for the next launch. */
__device__ __forceinline__ bool last_of(uint32_t *counter, uint32_t expected, uint32_t *flag)
{
	__threadfence();
	__syncthreads();
	if (threadIdx.x == 0) {
		const uint32_t arrived = atomicAdd(counter, 1u) + 1u;
		*flag = arrived == expected ? 1u : 0u;
		if (arrived == expected)
			*counter = 0u;
		__threadfence();
	}
	__syncthreads();
	return *flag != 0u;
}

/* FP32 sum over the runs, in ascending order from +0, of this lane's four channels of one partial row */
__device__ __forceinline__ void sum_runs(const float *first_run, uint64_t run_stride, uint32_t runs, float out[4])
{
	float4 total = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
	for (uint32_t run = 0; run < runs; run++) {
		const float4 part = __ldcg(reinterpret_cast<const float4 *>(first_run + run * run_stride));
		total.x = __fadd_rn(total.x, part.x);
		total.y = __fadd_rn(total.y, part.y);
		total.z = __fadd_rn(total.z, part.z);
		total.w = __fadd_rn(total.w, part.w);
	}
	out[0] = total.x, out[1] = total.y, out[2] = total.z, out[3] = total.w;
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
	/* the last CTA of this (job, 128 outputs): activation of the job's rows, a warp a row */
	const uint32_t channel = group * EXL3_TRANSFORM + lane * 4u;
	const uint64_t codes = exl3_code_bytes(H, I, BX2);
	float gate_scale[4], up_scale[4], down_scale[4];
	load_half4(reinterpret_cast<const __half *>(arena + job->gate_offset + codes) + H + channel, gate_scale);
	load_half4(reinterpret_cast<const __half *>(arena + job->up_offset + codes) + H + channel, up_scale);
	load_half4(reinterpret_cast<const __half *>(arena + job->down_offset + exl3_code_bytes(I, H, BX2)) + channel,
		   down_scale);
	for (uint32_t column = warp; column < job->row_count; column += EXL3_PRODUCT_WARPS) {
		const uint64_t at = (uint64_t)job->pair_index[column] * I + channel;
		float gate[4], up[4];
		sum_runs(partials + at, run_stride, runs, gate);
		sum_runs(partials + (uint64_t)runs * run_stride + at, run_stride, runs, up);
		hadamard128_warp(gate, lane);
		hadamard128_warp(up, lane);
		float hidden[4];
		exl3_swiglu4(gate, up, gate_scale, up_scale, record.activation_limit, hidden);
		const __nv_bfloat162 low = __halves2bfloat162(__float2bfloat16_rn(hidden[0]), __float2bfloat16_rn(hidden[1]));
		const __nv_bfloat162 high = __halves2bfloat162(__float2bfloat16_rn(hidden[2]), __float2bfloat16_rn(hidden[3]));
		uint2 stored;
		stored.x = *reinterpret_cast<const uint32_t *>(&low);
		stored.y = *reinterpret_cast<const uint32_t *>(&high);
		*reinterpret_cast<uint2 *>(reinterpret_cast<__nv_bfloat16 *>(arena + record.hidden_offset) + at) = stored;
		float fed[4];
#pragma unroll
		for (uint32_t i = 0; i < 4; i++)
			fed[i] = __fmul_rn(hidden[i], down_scale[i]);
		hadamard128_warp(fed, lane);
#pragma unroll
		for (uint32_t i = 0; i < 4; i++)
			fed[i] = __fmul_rn(fed[i], EXL3_NORMALIZATION);
		/* the down operands live behind the gate/up operands, which other CTAs of this launch still read */
		store_half4(reinterpret_cast<__half *>(arena + record.operands_offset) + (uint64_t)EXL3_PROJECTIONS * pairs * H +
				    at,
			    fed);
	}
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
	const uint32_t channel = group * EXL3_TRANSFORM + lane * 4u;
	float scale[4];
	load_half4(reinterpret_cast<const __half *>(arena + job->down_offset + exl3_code_bytes(I, H, BX2)) + I + channel,
		   scale);
	for (uint32_t column = warp; column < job->row_count; column += EXL3_PRODUCT_WARPS) {
		const uint64_t at = (uint64_t)job->pair_index[column] * H + channel;
		float v[4];
		sum_runs(partials + at, run_stride, runs, v);
		hadamard128_warp(v, lane);
		const float weight = job->route_weight[column];
#pragma unroll
		for (uint32_t i = 0; i < 4; i++)
			v[i] = __fmul_rn(__fmul_rn(__fmul_rn(v[i], EXL3_NORMALIZATION), scale[i]), weight);
		*reinterpret_cast<float4 *>(reinterpret_cast<float *>(arena + record.output_offset) + at) =
			make_float4(v[0], v[1], v[2], v[3]);
	}
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
