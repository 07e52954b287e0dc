/*
 * kernel_exl3.cu: the EXL3 entries under the names the reference's preparers ask for (kernel file "kernel_exl3":
 * source/kernel_exl3.cu:67-89, 133-167, 295-312, 314-424, 428-492), implemented anew for sm_100a. One record by value
 * and the arena's address; offsets only; no atomics on data. Launch shapes are the ones this library's preparers write
 * (csrc/host/exl3.c), not the reference's.
 */
#include "exl3_passes.cuh"

/* Bit-exact diagnostic decode: FP16 [input][output]. One thread a weight: grid ceil(values / 256), block 256. */
extern "C" __global__ void exl3_reconstruct(struct exl3_reconstruct_record record, unsigned char *arena)
{
	const uint64_t element = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
	if (element >= (uint64_t)record.input_size * record.output_size)
		return;
	const uint32_t input = (uint32_t)(element / record.output_size), output = (uint32_t)(element % record.output_size);
	const uint32_t bits_x2 = exl3_bits_x2(record.bits_per_weight);
	const uint32_t words = 4u * bits_x2, ring_bits = 128u * bits_x2;
	const uint32_t *const tile = reinterpret_cast<const uint32_t *>(arena + record.matrix_offset) +
				     ((uint64_t)(input / EXL3_TILE) * (record.output_size / EXL3_TILE) + output / EXL3_TILE) * words;
	const uint32_t position = exl3_tile_position(input % EXL3_TILE, output % EXL3_TILE);
	const uint32_t begin = (exl3_window_end(position, bits_x2) + ring_bits - EXL3_STATE_BITS) % ring_bits;
	const uint32_t word = begin / 32u, shift = begin % 32u;
	const uint32_t window = __funnelshift_l(tile[(word + 1u) % words], tile[word], shift);
	const uint32_t bits = exl3_value_bits(window >> 16);
	const __half value = __hfma(__ushort_as_half((unsigned short)bits), __ushort_as_half(EXL3_MUL1_SCALE),
				    __ushort_as_half(EXL3_MUL1_BIAS));
	reinterpret_cast<__half *>(arena + record.output_offset)[element] = value;
}

extern "C" __global__ void __launch_bounds__(EXL3_TRANSFORM_THREADS)
	exl3_input(struct exl3_expert_record record, unsigned char *arena)
{
	exl3_input_pass(record, arena, nullptr);
}

extern "C" __global__ void __launch_bounds__(EXL3_TRANSFORM_THREADS)
	exl3_activate(struct exl3_expert_record record, unsigned char *arena)
{
	exl3_activate_pass(record, arena, nullptr, record.inner_size, record.input_size, 0u);
}

extern "C" __global__ void __launch_bounds__(EXL3_TRANSFORM_THREADS)
	bb_exl3_activate_output_shard(struct bb_exl3_shard_activation_record arguments, unsigned char *arena)
{
	exl3_activate_pass(arguments.base, arena, nullptr, arguments.down_input_size, arguments.down_output_size,
			   arguments.down_input_begin);
}

extern "C" __global__ void __launch_bounds__(EXL3_TRANSFORM_THREADS)
	exl3_finish(struct exl3_expert_record record, unsigned char *arena)
{
	exl3_finish_pass(record, arena, nullptr);
}

/* grid (ceil(width / 128), rows), block 128: FP32 sums from +0 in ascending slot order */
extern "C" __global__ void exl3_row_sum(struct expert_row_sum_arguments record, unsigned char *arena)
{
	const uint32_t channel = blockIdx.x * blockDim.x + threadIdx.x;
	if (channel >= record.width)
		return;
	const uint64_t row = blockIdx.y;
	const float *const pairs = reinterpret_cast<const float *>(arena + record.pair_output_offset);
	float sum = 0.0f;
	for (uint32_t slot = 0; slot < record.pairs_per_row; slot++)
		sum = __fadd_rn(sum, pairs[(row * record.pairs_per_row + slot) * record.width + channel]);
	reinterpret_cast<float *>(arena + record.row_output_offset)[row * record.width + channel] = sum;
}

#define EXL3_PRODUCT_ENTRIES(width, bits_x2)                                                                  \
	extern "C" __global__ void __launch_bounds__(EXL3_PRODUCT_THREADS)                                    \
		exl3_gate_up_##width(struct exl3_expert_record record, unsigned char *arena)                  \
	{                                                                                                     \
		extern __shared__ __align__(128) unsigned char dynamic_shared[];                              \
		__shared__ exl3_product_shared shared;                                                        \
		const struct expert_job_record *const job = exl3_job(record, arena, blockIdx.y);              \
		if (job->row_count != 0)                                                                      \
			exl3_product_pass<bits_x2, false>(record, arena, job, dynamic_shared, &shared);       \
	}                                                                                                     \
	extern "C" __global__ void __launch_bounds__(EXL3_PRODUCT_THREADS)                                    \
		exl3_down_##width(struct exl3_expert_record record, unsigned char *arena)                     \
	{                                                                                                     \
		extern __shared__ __align__(128) unsigned char dynamic_shared[];                              \
		__shared__ exl3_product_shared shared;                                                        \
		const struct expert_job_record *const job = exl3_job(record, arena, blockIdx.y);              \
		if (job->row_count != 0)                                                                      \
			exl3_product_pass<bits_x2, true>(record, arena, job, dynamic_shared, &shared);        \
	}
EXL3_PRODUCT_ENTRIES(k2, EXL3_BITS_X2_K2)
EXL3_PRODUCT_ENTRIES(k2_5, EXL3_BITS_X2_K2_5)
EXL3_PRODUCT_ENTRIES(k3, EXL3_BITS_X2_K3)
EXL3_PRODUCT_ENTRIES(k4, EXL3_BITS_X2_K4)
