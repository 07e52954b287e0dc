/*
 * kernel_trunk_linear.cu: the always-on (shared) expert of the original-weights profile: y = W x for one or two
 * matrices of E4M3 weights (WEIGHT_FORMAT_E4M3_SCALED, one E8M0 scale per 32 by 32 weights) and 1 to 8 rows of E4M3
 * block-quantized activations, under the reference's entry names and records (source/kernel_trunk_linear.cu:82-133,
 * 467-539; contract include/anemone/linear_records.h:100-118, 308-330, 352-362), new for sm_100a.
 *
 *   trunk_linear_quantized_<S>  grid ((output_size[0] + output_size[1]) / 16), block 32 S: bfloat16 [row][output]
 *   trunk_linear_block128_<S>   the same for WEIGHT_FORMAT_E4M3_BLOCK128 (no counterpart in the reference): the same
 *                               bytes, one FP32 scale per 128 outputs by 128 inputs instead of the E8M0 codes; chain =
 *                               fma(p, scale * 2^(activation code - 127 + 16), chain)
 *   trunk_hidden_entry          grid (ceil(width / 256), vectors), block 256: the hidden step, route weight 1
 *   trunk_rows_add_entry        grid (ceil(width / 256), rows), block 256: FP32 row sums += bfloat16 rows
 * A block owns one tile of 16 outputs of one of the matrices; the tile's bytes for all of K are contiguous in the
 * stored format (lane order), so a warp streams its slice with two 128-bit loads a lane per 64 inputs, and a byte
 * becomes an FP16 operand by bit placement alone (its value times 2^-8, as the activation operands are). Per block of
 * 32 inputs the tensor cores add the 32 products from zero (two m16n8k16 instructions), and chain = fma(p, 2^e, chain)
 * with e = weight code + activation code - 254 + 16. A slice is one chain; the S chains are added from +0 in ascending
 * order; one rounding to bfloat16. Rows stand in the columns of the instruction: column c carries row c, a column
 * from row_count on carries row 0 again and is stored nowhere.
 */
#include <stdint.h>

#include "anemone_b200_records.h"

#define WARP 32u
#define TRUNK_AHEAD 4u /* groups of 32 inputs of a lane in flight */

__device__ __forceinline__ uint32_t bfloat16_bits(float value)
{
	const uint32_t bits = __float_as_uint(value);
	return (bits & 0x7FFFFFFFu) > 0x7F800000u ? 0x7FC0u : (bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16;
}

__device__ __forceinline__ float bfloat16_value(uint32_t bits)
{
	return __uint_as_float(bits << 16);
}

/* bytes 0 and 2 of a word placed as two FP16: sign to bit 15, the seven low bits to bits 7..13 */
__device__ __forceinline__ uint32_t place_even_bytes(uint32_t word)
{
	return ((word << 7) & 0x3F803F80u) | ((word << 8) & 0x80008000u);
}

/* bytes 1 and 3 of a word: their signs already stand at bits 15 and 31 */
__device__ __forceinline__ uint32_t place_odd_bytes(uint32_t word)
{
	return ((word >> 1) & 0x3F803F80u) | (word & 0x80008000u);
}

__device__ __forceinline__ void mma_f16(float accumulator[4], const uint32_t a[4], uint32_t b0, uint32_t b1)
{
	asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
		     "{%0,%1,%2,%3};"
		     : "+f"(accumulator[0]), "+f"(accumulator[1]), "+f"(accumulator[2]), "+f"(accumulator[3])
		     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

/* 2^(weight code + activation code - 254 + 16) as an FP32: nothing below the normal numbers, at most 2^127 */
__device__ __forceinline__ float block_scale(uint32_t weight_code, uint32_t activation_code)
{
	const int32_t field = (int32_t)(weight_code + activation_code) - 111;
	return field < 1 ? 0.0f : __uint_as_float((uint32_t)(field > 254 ? 254 : field) << 23);
}

/* the same factor for a weight scale that is an FP32 number (one per 128 by 128 weights): scale * 2^(activation code
 * - 127 + 16); the product of a number and a power of two is exact unless it leaves the normal range */
__device__ __forceinline__ float block128_scale(float weight_scale, uint32_t activation_code)
{
	const uint32_t field = activation_code + 16u;
	return __fmul_rn(weight_scale, __uint_as_float((field > 254u ? 254u : field) << 23));
}

/* BLOCK128 false: WEIGHT_FORMAT_E4M3_SCALED (the reference's: one E8M0 code per 32 by 32 weights behind the bytes);
 * true: WEIGHT_FORMAT_E4M3_BLOCK128 (one FP32 scale per 128 outputs by 128 inputs behind the same bytes). */
template <uint32_t S, bool BLOCK128>
__device__ __forceinline__ void trunk_linear_quantized(const struct trunk_linear_quantized_arguments &arguments,
						       unsigned char *arena)
{
	__shared__ float parts[S][WARP][4];
	const uint32_t lane = threadIdx.x % WARP, slice = threadIdx.x / WARP, group_lane = lane / 4u, place = lane % 4u;
	const uint32_t first_tiles = arguments.output_size[0] / LINEAR_OUTPUTS_PER_TILE;
	const bool second = blockIdx.x >= first_tiles;
	const uint32_t tile = second ? blockIdx.x - first_tiles : blockIdx.x;
	const uint32_t outputs = arguments.output_size[second ? 1 : 0], inputs = arguments.input_size;
	const unsigned char *const matrix = arena + arguments.weights_offset[second ? 1 : 0];
	const uint32_t groups = inputs / LINEAR_VALUES_PER_BLOCK, loads = inputs / LINEAR_VALUES_PER_LOAD;
	/* eight rows a block column (blockIdx.y; the reference's launches have one: at most eight rows) */
	const uint32_t row_base = blockIdx.y * LINEAR_MAXIMUM_ROWS;
	const uint32_t rows = min(arguments.row_count - row_base, LINEAR_MAXIMUM_ROWS);
	const uint32_t fed_row = row_base + (group_lane < rows ? group_lane : 0u);
	const uint32_t even_row = row_base + (2u * place < rows ? 2u * place : 0u);
	const uint32_t odd_row = row_base + (2u * place + 1u < rows ? 2u * place + 1u : 0u);
	const uint4 *const bytes = reinterpret_cast<const uint4 *>(matrix) + ((uint64_t)tile * groups) * WARP + lane;
	const unsigned char *const scales = matrix + (uint64_t)outputs * inputs + (uint64_t)(tile / 2u) * groups;
	const float *const scales128 =
		reinterpret_cast<const float *>(matrix + (uint64_t)outputs * inputs) + (uint64_t)(tile / 8u) * (groups / 4u);
	/* operand order of a vector: per load of 64 values, lane place t holds eight 32-bit registers (two 128-bit loads) */
	const uint4 *const fed =
		reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(arena + arguments.operands_offset) +
						(uint64_t)fed_row * inputs) +
		place * 2u;
	const unsigned char *const exponents = arena + arguments.exponents_offset;
	const unsigned char *const exponents_even = exponents + (uint64_t)even_row * groups;
	const unsigned char *const exponents_odd = exponents + (uint64_t)odd_row * groups;
	/* the slice's groups: whole loads, as the routed experts' slices are cut */
	const uint32_t first = loads * slice / S * 2u, last = loads * (slice + 1u) / S * 2u;
	float chains[4] = { 0.0f, 0.0f, 0.0f, 0.0f };
	uint4 ahead[TRUNK_AHEAD];
#pragma unroll
	for (uint32_t slot = 0; slot < TRUNK_AHEAD; slot++)
		if (first + slot < last)
			ahead[slot] = __ldcs(bytes + (uint64_t)(first + slot) * WARP);
	for (uint32_t base = first; base < last; base += TRUNK_AHEAD) {
#pragma unroll
		for (uint32_t slot = 0; slot < TRUNK_AHEAD; slot++) {
			const uint32_t group = base + slot;
			if (group >= last)
				break;
			const uint4 current = ahead[slot];
			if (group + TRUNK_AHEAD < last)
				ahead[slot] = __ldcs(bytes + (uint64_t)(group + TRUNK_AHEAD) * WARP);
			/* the group's two steps of 16 inputs are registers 4 (group % 2) .. + 3 of its load's eight */
			const uint4 fed_registers = __ldg(fed + (uint64_t)(group / 2u) * 8u + (group % 2u));
			const uint32_t words[4] = { current.x, current.y, current.z, current.w };
			const uint32_t fed_words[4] = { fed_registers.x, fed_registers.y, fed_registers.z, fed_registers.w };
			float sum[4] = { 0.0f, 0.0f, 0.0f, 0.0f };
#pragma unroll
			for (uint32_t step = 0; step < 2u; step++) {
				const uint32_t a[4] = { place_even_bytes(words[2u * step]), place_odd_bytes(words[2u * step]),
							place_even_bytes(words[2u * step + 1u]),
							place_odd_bytes(words[2u * step + 1u]) };
				mma_f16(sum, a, fed_words[2u * step], fed_words[2u * step + 1u]);
			}
			float even, odd;
			if (BLOCK128) {
				const float weight_scale = __ldg(scales128 + group / 4u);
				even = block128_scale(weight_scale, exponents_even[group]);
				odd = block128_scale(weight_scale, exponents_odd[group]);
			} else {
				const uint32_t weight_code = scales[group];
				even = block_scale(weight_code, exponents_even[group]);
				odd = block_scale(weight_code, exponents_odd[group]);
			}
			chains[0] = __fmaf_rn(sum[0], even, chains[0]);
			chains[1] = __fmaf_rn(sum[1], odd, chains[1]);
			chains[2] = __fmaf_rn(sum[2], even, chains[2]);
			chains[3] = __fmaf_rn(sum[3], odd, chains[3]);
		}
	}
#pragma unroll
	for (uint32_t c = 0; c < 4; c++)
		parts[slice][lane][c] = chains[c];
	__syncthreads();
	if (slice != 0)
		return;
	uint16_t *const output = reinterpret_cast<uint16_t *>(arena + arguments.output_offset[second ? 1 : 0]);
#pragma unroll
	for (uint32_t c = 0; c < 4; c++) {
		const uint32_t row = 2u * place + (c & 1u);
		if (row >= rows)
			continue;
		float sum = 0.0f;
#pragma unroll
		for (uint32_t part = 0; part < S; part++)
			sum = __fadd_rn(sum, parts[part][lane][c]);
		output[(uint64_t)(row_base + row) * outputs + tile * LINEAR_OUTPUTS_PER_TILE + group_lane + (c >> 1) * 8u] =
			(uint16_t)bfloat16_bits(sum);
	}
}

#define TRUNK_ENTRIES(S)                                                                                       \
	extern "C" __global__ void __launch_bounds__(32 * S)                                                   \
		trunk_linear_quantized_##S(struct trunk_linear_quantized_arguments arguments, unsigned char *arena) \
	{                                                                                                      \
		trunk_linear_quantized<S, false>(arguments, arena);                                            \
	}                                                                                                      \
	extern "C" __global__ void __launch_bounds__(32 * S)                                                   \
		trunk_linear_block128_##S(struct trunk_linear_quantized_arguments arguments, unsigned char *arena) \
	{                                                                                                      \
		trunk_linear_quantized<S, true>(arguments, arena);                                             \
	}
TRUNK_ENTRIES(1)
TRUNK_ENTRIES(2)
TRUNK_ENTRIES(4)
TRUNK_ENTRIES(8)
TRUNK_ENTRIES(16)

extern "C" __global__ void __launch_bounds__(LINEAR_ELEMENT_THREADS)
	trunk_hidden_entry(struct trunk_hidden_arguments arguments, unsigned char *arena)
{
	const uint32_t channel = blockIdx.x * blockDim.x + threadIdx.x;
	if (channel >= arguments.width)
		return;
	const uint64_t at = (uint64_t)blockIdx.y * arguments.width + channel;
	const float g = bfloat16_value(reinterpret_cast<const uint16_t *>(arena + arguments.gate_offset)[at]);
	const float u = bfloat16_value(reinterpret_cast<const uint16_t *>(arena + arguments.up_offset)[at]);
	const float limit = arguments.activation_limit;
	const float bounded_gate = g > limit ? limit : g;
	const float bounded_up = u > limit ? limit : (u < -limit ? -limit : u);
	const float gated = __fdiv_rn(bounded_gate, __fadd_rn(1.0f, expf(-bounded_gate)));
	const float value = __fmul_rn(__fmul_rn(gated, bounded_up), 1.0f);
	reinterpret_cast<uint16_t *>(arena + arguments.hidden_offset)[at] = (uint16_t)bfloat16_bits(value);
}

extern "C" __global__ void __launch_bounds__(LINEAR_ELEMENT_THREADS)
	trunk_rows_add_entry(struct trunk_rows_add_arguments arguments, unsigned char *arena)
{
	const uint32_t channel = blockIdx.x * blockDim.x + threadIdx.x;
	if (channel >= arguments.width)
		return;
	const uint64_t at = (uint64_t)blockIdx.y * arguments.width + channel;
	float *const sums = reinterpret_cast<float *>(arena + arguments.sums_offset);
	sums[at] = __fadd_rn(sums[at], bfloat16_value(reinterpret_cast<const uint16_t *>(arena + arguments.values_offset)[at]));
}
