/*
 * kernel_exl3_b200.cu: the routed-expert layer of one rank in four launches (struct exl3_moe_record), with a stored
 * width per expert. No counterpart in the reference, whose chain is five launches of one width plus a row sum; the
 * arithmetic of every value is the same chain's (exl3_passes.cuh), only the round trips through global memory between
 * products and transforms are gone:
 *   exl3_moe_input    grid (ceil(H / 128 / 4), jobs, 2) x 128   x . suh, Hadamard, FP16 operands of gate and of up
 *   exl3_moe_gate_up  grid (I / 128, jobs) x 128               a CTA computes 128 gate and 128 up outputs of its job,
 *                                                               transforms them, applies SwiGLU, the down-side scale
 *                                                               and transform: bfloat16 hidden, FP16 down operands
 *   exl3_moe_down     grid (H / 128, jobs) x 128               128 down outputs, output transform, scale, route weight:
 *                                                               FP32 pair outputs
 *   exl3_moe_row_sum  grid (ceil(H / 128), rows) x 128         FP32 row sums from +0 in ascending slot order
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

/* this thread's sums (exl3_product_core's layout) into staged[column][output] */
__device__ __forceinline__ void stage_sums(float *staged, const float sums[2][4])
{
	const uint32_t lane = threadIdx.x % EXL3_WARP, warp = threadIdx.x / EXL3_WARP;
	const uint32_t group_lane = lane / 4u, place = lane % 4u;
#pragma unroll
	for (uint32_t mine = 0; mine < 2; mine++)
#pragma unroll
		for (uint32_t c = 0; c < 4; c++)
			staged[(place * 2u + (c & 1u)) * STAGED_ROW + (warp * 2u + mine) * EXL3_TILE + group_lane +
			       (c >> 1) * 8u] = sums[mine][c];
}

template <uint32_t BX2>
__device__ __forceinline__ void moe_gate_up(const struct exl3_expert_record &record, unsigned char *arena,
					    const struct expert_job_record *job, unsigned char *dynamic_shared,
					    exl3_product_shared *shared)
{
	const uint32_t lane = threadIdx.x % EXL3_WARP, warp = threadIdx.x / EXL3_WARP;
	const uint32_t fed_column = lane / 4u < job->row_count ? lane / 4u : 0u;
	float gate_sums[2][4], up_sums[2][4];
	const __half *const operands = reinterpret_cast<const __half *>(arena + record.operands_offset);
	if (!exl3_product_core<BX2>(arena + job->gate_offset, record.input_size, record.inner_size, blockIdx.x,
				    operands + (uint64_t)job->pair_index[fed_column] * record.input_size, dynamic_shared,
				    shared, gate_sums))
		return;
	__syncthreads();
	if (!exl3_product_core<BX2>(arena + job->up_offset, record.input_size, record.inner_size, blockIdx.x,
				    operands + ((uint64_t)record.pair_count + job->pair_index[fed_column]) * record.input_size,
				    dynamic_shared, shared, up_sums))
		return;
	float *const staged = reinterpret_cast<float *>(dynamic_shared); /* [2][8][STAGED_ROW] */
	stage_sums(staged, gate_sums);
	stage_sums(staged + LINEAR_MAXIMUM_ROWS * STAGED_ROW, up_sums);
	__syncthreads();
	const uint32_t channel = blockIdx.x * EXL3_TRANSFORM + lane * 4u;
	const uint64_t codes = exl3_code_bytes(record.input_size, record.inner_size, BX2);
	float gate_scale[4], up_scale[4], down_scale[4];
	load_half4(reinterpret_cast<const __half *>(arena + job->gate_offset + codes) + record.input_size + channel,
		   gate_scale);
	load_half4(reinterpret_cast<const __half *>(arena + job->up_offset + codes) + record.input_size + channel, up_scale);
	load_half4(reinterpret_cast<const __half *>(arena + job->down_offset +
						    exl3_code_bytes(record.inner_size, record.input_size, BX2)) +
			   channel,
		   down_scale);
	for (uint32_t column = warp; column < job->row_count; column += EXL3_PRODUCT_WARPS) {
		const float4 gate_raw = *reinterpret_cast<const float4 *>(staged + column * STAGED_ROW + lane * 4u);
		const float4 up_raw =
			*reinterpret_cast<const float4 *>(staged + (LINEAR_MAXIMUM_ROWS + column) * STAGED_ROW + lane * 4u);
		float gate[4] = { gate_raw.x, gate_raw.y, gate_raw.z, gate_raw.w };
		float up[4] = { up_raw.x, up_raw.y, up_raw.z, up_raw.w };
		hadamard128_warp(gate, lane);
		hadamard128_warp(up, lane);
		float hidden[4];
		exl3_swiglu4(gate, up, gate_scale, up_scale, record.activation_limit, hidden);
		const uint64_t at = (uint64_t)job->pair_index[column] * record.inner_size + channel;
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
		store_half4(reinterpret_cast<__half *>(arena + record.operands_offset) +
				    (uint64_t)EXL3_PROJECTIONS * record.pair_count * record.input_size + at,
			    fed);
	}
}

template <uint32_t BX2>
__device__ __forceinline__ void moe_down(const struct exl3_expert_record &record, unsigned char *arena,
					 const struct expert_job_record *job, unsigned char *dynamic_shared,
					 exl3_product_shared *shared)
{
	const uint32_t lane = threadIdx.x % EXL3_WARP, warp = threadIdx.x / EXL3_WARP;
	const uint32_t fed_column = lane / 4u < job->row_count ? lane / 4u : 0u;
	float sums[2][4];
	const __half *const operands = reinterpret_cast<const __half *>(arena + record.operands_offset) +
				       (uint64_t)EXL3_PROJECTIONS * record.pair_count * record.input_size;
	if (!exl3_product_core<BX2>(arena + job->down_offset, record.inner_size, record.input_size, blockIdx.x,
				    operands + (uint64_t)job->pair_index[fed_column] * record.inner_size, dynamic_shared,
				    shared, sums))
		return;
	float *const staged = reinterpret_cast<float *>(dynamic_shared);
	stage_sums(staged, sums);
	__syncthreads();
	const uint32_t channel = blockIdx.x * EXL3_TRANSFORM + lane * 4u;
	float scale[4];
	load_half4(reinterpret_cast<const __half *>(arena + job->down_offset +
						    exl3_code_bytes(record.inner_size, record.input_size, BX2)) +
			   record.inner_size + channel,
		   scale);
	for (uint32_t column = warp; column < job->row_count; column += EXL3_PRODUCT_WARPS) {
		const float4 raw = *reinterpret_cast<const float4 *>(staged + column * STAGED_ROW + lane * 4u);
		float v[4] = { raw.x, raw.y, raw.z, raw.w };
		hadamard128_warp(v, lane);
		const float weight = job->route_weight[column];
#pragma unroll
		for (uint32_t i = 0; i < 4; i++)
			v[i] = __fmul_rn(__fmul_rn(__fmul_rn(v[i], EXL3_NORMALIZATION), scale[i]), weight);
		*reinterpret_cast<float4 *>(reinterpret_cast<float *>(arena + record.output_offset) +
					    (uint64_t)job->pair_index[column] * record.input_size + channel) =
			make_float4(v[0], v[1], v[2], v[3]);
	}
}

#define MOE_WIDTH_SWITCH(function)                                                          \
	switch (exl3_job_bits_x2(record.base, job, moe_widths(record, arena))) {            \
	case EXL3_BITS_X2_K2:                                                               \
		function<EXL3_BITS_X2_K2>(record.base, arena, job, dynamic_shared, &shared);   \
		break;                                                                      \
	case EXL3_BITS_X2_K2_5:                                                             \
		function<EXL3_BITS_X2_K2_5>(record.base, arena, job, dynamic_shared, &shared); \
		break;                                                                      \
	case EXL3_BITS_X2_K3:                                                               \
		function<EXL3_BITS_X2_K3>(record.base, arena, job, dynamic_shared, &shared);   \
		break;                                                                      \
	case EXL3_BITS_X2_K4:                                                               \
		function<EXL3_BITS_X2_K4>(record.base, arena, job, dynamic_shared, &shared);   \
		break;                                                                      \
	default:                                                                            \
		break;                                                                      \
	}

extern "C" __global__ void __launch_bounds__(EXL3_PRODUCT_THREADS)
	exl3_moe_gate_up(struct exl3_moe_record record, unsigned char *arena)
{
	extern __shared__ __align__(128) unsigned char dynamic_shared[];
	__shared__ exl3_product_shared shared;
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
