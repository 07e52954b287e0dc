/*
 * exl3_passes.cuh: the passes of the routed-expert chain as device functions, shared by the entries that keep the
 * reference's names (kernel_exl3.cu) and by the fused B200 entries (kernel_exl3_b200.cu). Arithmetic follows the
 * reference's retained chain step for step (source/kernel_exl3.cu:133-167, 314-402, 406-424): every FP32 operation
 * is one rounding (the kernel files are built with --fmad=false), transforms run in the same stage order.
 *
 * Transform passes: one warp per 128-channel block, four channels a lane (channel = 128 block + 4 lane + i).
 */
#ifndef AB_EXL3_PASSES_CUH
#define AB_EXL3_PASSES_CUH

#include "exl3_device.cuh"

__device__ __forceinline__ const struct expert_job_record *exl3_job(const struct exl3_expert_record &record,
								      const unsigned char *arena, uint32_t index)
{
	return reinterpret_cast<const struct expert_job_record *>(arena + record.jobs_offset) + index;
}

/* bits_x2 of a job's matrices: the record's width, or the expert's entry of the width table */
__device__ __forceinline__ uint32_t exl3_job_bits_x2(const struct exl3_expert_record &record,
						     const struct expert_job_record *job, const uint32_t *widths)
{
	return exl3_bits_x2(widths != nullptr ? widths[job->expert] : record.bits_per_weight);
}

__device__ __forceinline__ void load_half4(const __half *source, float out[4])
{
	const uint2 raw = *reinterpret_cast<const uint2 *>(source);
	const __half2 low = *reinterpret_cast<const __half2 *>(&raw.x), high = *reinterpret_cast<const __half2 *>(&raw.y);
	out[0] = __low2float(low);
	out[1] = __high2float(low);
	out[2] = __low2float(high);
	out[3] = __high2float(high);
}

__device__ __forceinline__ void store_half4(__half *destination, const float v[4])
{
	const __half2 low = __halves2half2(__float2half_rn(v[0]), __float2half_rn(v[1]));
	const __half2 high = __halves2half2(__float2half_rn(v[2]), __float2half_rn(v[3]));
	uint2 raw;
	raw.x = *reinterpret_cast<const uint32_t *>(&low);
	raw.y = *reinterpret_cast<const uint32_t *>(&high);
	*reinterpret_cast<uint2 *>(destination) = raw;
}

/* input pass: grid (ceil(H / 128 / 4), jobs, 2), block 128 */
__device__ __forceinline__ void exl3_input_pass(const struct exl3_expert_record &record, unsigned char *arena,
						const uint32_t *widths)
{
	const struct expert_job_record *const job = exl3_job(record, arena, blockIdx.y);
	const uint32_t lane = threadIdx.x % EXL3_WARP;
	const uint32_t block = blockIdx.x * EXL3_TRANSFORM_WARPS + threadIdx.x / EXL3_WARP;
	if (job->row_count == 0 || block >= record.input_size / EXL3_TRANSFORM)
		return;
	const uint32_t channel = block * EXL3_TRANSFORM + lane * 4u;
	const uint64_t matrix = blockIdx.z == 0 ? job->gate_offset : job->up_offset;
	const __half *const suh = reinterpret_cast<const __half *>(
		arena + matrix + exl3_code_bytes(record.input_size, record.inner_size, exl3_job_bits_x2(record, job, widths)));
	float scale[4];
	load_half4(suh + channel, scale);
	const __nv_bfloat16 *const input = reinterpret_cast<const __nv_bfloat16 *>(arena + record.input_offset);
	__half *const operands = reinterpret_cast<__half *>(arena + record.operands_offset);
	for (uint32_t column = 0; column < job->row_count; column++) {
		const uint32_t pair = job->pair_index[column], row = pair / record.pairs_per_row;
		const uint2 raw = *reinterpret_cast<const uint2 *>(input + (uint64_t)row * record.input_size + channel);
		float v[4] = { __uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xFFFF0000u),
			       __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xFFFF0000u) };
#pragma unroll
		for (uint32_t i = 0; i < 4; i++)
			v[i] = __fmul_rn(v[i], scale[i]);
		hadamard128_warp(v, lane);
#pragma unroll
		for (uint32_t i = 0; i < 4; i++)
			v[i] = __fmul_rn(v[i], EXL3_NORMALIZATION);
		store_half4(operands + ((uint64_t)blockIdx.z * record.pair_count + pair) * record.input_size + channel, v);
	}
}

/* The SwiGLU step of one lane's four channels: gate and up are transformed products; returns the FP32 hidden values
 * (source/kernel_exl3.cu:336-352). */
__device__ __forceinline__ void exl3_swiglu4(float gate[4], float up[4], const float gate_scale[4],
					     const float up_scale[4], float limit, float hidden[4])
{
#pragma unroll
	for (uint32_t i = 0; i < 4; i++) {
		const float gate_value = __fmul_rn(__fmul_rn(gate[i], EXL3_NORMALIZATION), gate_scale[i]);
		const float up_value = __fmul_rn(__fmul_rn(up[i], EXL3_NORMALIZATION), up_scale[i]);
		const float bounded_gate = fminf(gate_value, limit);
		const float bounded_up = fminf(fmaxf(up_value, -limit), limit);
		hidden[i] = __fmul_rn(__fdiv_rn(bounded_gate, __fadd_rn(1.0f, expf(-bounded_gate))), bounded_up);
	}
}

/* activation pass: grid (ceil(I / 128 / 4), jobs), block 128. down_suh_begin: where this rank's inner columns start
 * in the down matrix's suh (0 unless the down matrix is wider than the launch's inner size), down_inputs/down_outputs
 * the resident down matrix's shape. */
__device__ __forceinline__ void exl3_activate_pass(const struct exl3_expert_record &record, unsigned char *arena,
						   const uint32_t *widths, uint32_t down_inputs,
						   uint32_t down_outputs, uint32_t down_suh_begin)
{
	const struct expert_job_record *const job = exl3_job(record, arena, blockIdx.y);
	const uint32_t lane = threadIdx.x % EXL3_WARP;
	const uint32_t block = blockIdx.x * EXL3_TRANSFORM_WARPS + threadIdx.x / EXL3_WARP;
	if (job->row_count == 0 || block >= record.inner_size / EXL3_TRANSFORM)
		return;
	const uint32_t channel = block * EXL3_TRANSFORM + lane * 4u;
	const uint32_t bits_x2 = exl3_job_bits_x2(record, job, widths);
	const uint64_t codes = exl3_code_bytes(record.input_size, record.inner_size, bits_x2);
	float gate_scale[4], up_scale[4], down_scale[4];
	load_half4(reinterpret_cast<const __half *>(arena + job->gate_offset + codes) + record.input_size + channel,
		   gate_scale);
	load_half4(reinterpret_cast<const __half *>(arena + job->up_offset + codes) + record.input_size + channel,
		   up_scale);
	load_half4(reinterpret_cast<const __half *>(arena + job->down_offset +
						    exl3_code_bytes(down_inputs, down_outputs, bits_x2)) +
			   down_suh_begin + channel,
		   down_scale);
	const float *const products = reinterpret_cast<const float *>(arena + record.products_offset);
	for (uint32_t column = 0; column < job->row_count; column++) {
		const uint32_t pair = job->pair_index[column];
		const uint64_t at = (uint64_t)pair * record.inner_size + channel;
		const float4 gate_raw = *reinterpret_cast<const float4 *>(products + at);
		const float4 up_raw =
			*reinterpret_cast<const float4 *>(products + (uint64_t)record.pair_count * record.inner_size + at);
		float gate[4] = { gate_raw.x, gate_raw.y, gate_raw.z, gate_raw.w };
		float up[4] = { up_raw.x, up_raw.y, up_raw.z, up_raw.w };
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
		store_half4(reinterpret_cast<__half *>(arena + record.operands_offset) + at, fed);
	}
}

/* finish pass: grid (ceil(H / 128 / 4), jobs), block 128; in place on the down products */
__device__ __forceinline__ void exl3_finish_pass(const struct exl3_expert_record &record, unsigned char *arena,
						 const uint32_t *widths)
{
	const struct expert_job_record *const job = exl3_job(record, arena, blockIdx.y);
	const uint32_t lane = threadIdx.x % EXL3_WARP;
	const uint32_t block = blockIdx.x * EXL3_TRANSFORM_WARPS + threadIdx.x / EXL3_WARP;
	if (job->row_count == 0 || block >= record.input_size / EXL3_TRANSFORM)
		return;
	const uint32_t channel = block * EXL3_TRANSFORM + lane * 4u;
	float scale[4];
	load_half4(reinterpret_cast<const __half *>(arena + job->down_offset +
						    exl3_code_bytes(record.inner_size, record.input_size,
								    exl3_job_bits_x2(record, job, widths))) +
			   record.inner_size + channel,
		   scale);
	for (uint32_t column = 0; column < job->row_count; column++) {
		const uint64_t at = (uint64_t)job->pair_index[column] * record.input_size + channel;
		const float4 raw = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(arena + record.products_offset) + at);
		float v[4] = { raw.x, raw.y, raw.z, raw.w };
		hadamard128_warp(v, lane);
		const float weight = job->route_weight[column];
#pragma unroll
		for (uint32_t i = 0; i < 4; i++)
			v[i] = __fmul_rn(__fmul_rn(__fmul_rn(v[i], EXL3_NORMALIZATION), scale[i]), weight);
		*reinterpret_cast<float4 *>(reinterpret_cast<float *>(arena + record.output_offset) + at) =
			make_float4(v[0], v[1], v[2], v[3]);
	}
}

/* product pass: grid (outputs / 128, jobs, projections), block 128, dynamic shared exl3_product_dynamic_bytes.
 * DOWN false: gate (z = 0) or up (z = 1), inputs = H, outputs = inner, operands [z][pair][H], products [z][pair][I];
 * DOWN true: inputs = inner, outputs = H, operands [pair][I], products [pair][H]. */
template <uint32_t BX2, bool DOWN>
__device__ __forceinline__ void exl3_product_pass(const struct exl3_expert_record &record, unsigned char *arena,
						  const struct expert_job_record *job, unsigned char *dynamic_shared,
						  exl3_product_shared *shared)
{
	const uint32_t inputs = DOWN ? record.inner_size : record.input_size;
	const uint32_t outputs = DOWN ? record.input_size : record.inner_size;
	const uint32_t projection = DOWN ? 0u : blockIdx.z;
	const uint32_t lane = threadIdx.x % EXL3_WARP, warp = threadIdx.x / EXL3_WARP;
	const uint32_t group_lane = lane / 4u, place = lane % 4u;
	const uint64_t matrix = DOWN ? job->down_offset : projection == 0 ? job->gate_offset : job->up_offset;
	const uint32_t fed_column = group_lane < job->row_count ? group_lane : 0u;
	const __half *const operand_row =
		reinterpret_cast<const __half *>(arena + record.operands_offset) +
		((uint64_t)projection * record.pair_count + job->pair_index[fed_column]) * inputs;
	float sums[2][4];
	if (!exl3_product_core<BX2>(arena + matrix, outputs, blockIdx.x, 0u, inputs / EXL3_TILE, operand_row,
				    dynamic_shared, shared, sums))
		return;
	float *const products = reinterpret_cast<float *>(arena + record.products_offset);
#pragma unroll
	for (uint32_t mine = 0; mine < 2; mine++) {
		const uint32_t output = blockIdx.x * EXL3_TRANSFORM + (warp * 2u + mine) * EXL3_TILE + group_lane;
#pragma unroll
		for (uint32_t c = 0; c < 4; c++) {
			const uint32_t column = place * 2u + (c & 1u);
			if (column < job->row_count)
				products[((uint64_t)projection * record.pair_count + job->pair_index[column]) * outputs +
					 output + (c >> 1) * 8u] = sums[mine][c];
		}
	}
}

/* The product pass for a width known only at run time: one uniform branch per CTA. */
template <bool DOWN>
__device__ __forceinline__ void exl3_product_any_width(const struct exl3_expert_record &record, unsigned char *arena,
							const uint32_t *widths, unsigned char *dynamic_shared,
							exl3_product_shared *shared)
{
	const struct expert_job_record *const job = exl3_job(record, arena, blockIdx.y);
	if (job->row_count == 0)
		return;
	switch (exl3_job_bits_x2(record, job, widths)) {
	case EXL3_BITS_X2_K2:
		exl3_product_pass<EXL3_BITS_X2_K2, DOWN>(record, arena, job, dynamic_shared, shared);
		break;
	case EXL3_BITS_X2_K2_5:
		exl3_product_pass<EXL3_BITS_X2_K2_5, DOWN>(record, arena, job, dynamic_shared, shared);
		break;
	case EXL3_BITS_X2_K3:
		exl3_product_pass<EXL3_BITS_X2_K3, DOWN>(record, arena, job, dynamic_shared, shared);
		break;
	case EXL3_BITS_X2_K4:
		exl3_product_pass<EXL3_BITS_X2_K4, DOWN>(record, arena, job, dynamic_shared, shared);
		break;
	default:
		break;
	}
}

#endif
