/*
 * kernel_expert_linear.cu: the routed experts of the original-weights profile: MXFP4 (E2M1 with one E8M0 scale per
 * 32 inputs) weights by E4M3 block-quantized activations, under the reference's entry names and records
 * (source/kernel_expert_linear.cu:344-435; contract include/anemone/linear_records.h:45-99, 245-299), new for sm_100a.
 *
 *   expert_gate_up_<S>  grid (output_size / 16, jobs), block 64 S: warps 0 .. S-1 take the S slices of gate, warps
 *                       S .. 2S-1 those of up; then the hidden step: bfloat16 [pair][output_size]
 *   expert_down_<S>     grid (output_size / 16, jobs), block 32 S: bfloat16 [pair][output_size]
 *   expert_row_sum_entry  grid (ceil(width / block), rows): FP32 sums of bfloat16 pair outputs, ascending slots
 * A block owns one tile of 16 outputs of one job; the tile's words for all of K are contiguous in the stored format
 * (lane order), so a warp streams its slice with one 128-bit load a lane per 64 inputs, four loads ahead, and a code
 * becomes an FP16 operand by bit placement alone: the E2M1 nibble placed is its value times 2^-14, the activation
 * operand (written by activation_quantize_entry) its E4M3 value times 2^-8. Per block of 32 inputs the tensor cores add
 * the 32 products from zero (two m16n8k16 instructions), and chain = fma(p, 2^e, chain) with 2^e the exact power of
 * two that applies both scales and undoes the placements (e = weight code + activation code - 254 + 22). A slice is one
 * chain; the S chains are added from +0 in ascending order; one rounding to bfloat16.
 */
#include <stdint.h>

#include "anemone_b200_records.h"

#define WARP 32u
#define EXPERT_AHEAD 4u /* loads of a lane in flight */

__device__ __forceinline__ uint32_t bfloat16_bits(float value)
{
	const uint32_t bits = __float_as_uint(value);
	return (bits & 0x7FFFFFFFu) > 0x7F800000u ? 0x7FC0u : (bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16;
}

__device__ __forceinline__ float bfloat16_value(uint32_t bits)
{
	return __uint_as_float(bits << 16);
}

/* the two nibbles of register r of a stored word (bits 4 r and 4 r + 16) placed as two FP16: sign to bit 15, the three
 * magnitude bits to bits 9..11 */
template <uint32_t R> __device__ __forceinline__ uint32_t place_e2m1(uint32_t word)
{
	const uint32_t sign = word << (12u - 4u * R);
	const uint32_t magnitude = R < 3u ? word << (9u - 4u * R) : word >> 3;
	return (sign & 0x80008000u) | (magnitude & 0x0E000E00u);
}

__device__ __forceinline__ void mma_f16(float accumulator[4], const uint32_t a[4], uint32_t b0, uint32_t b1)
{
	asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
		     "{%0,%1,%2,%3};"
		     : "+f"(accumulator[0]), "+f"(accumulator[1]), "+f"(accumulator[2]), "+f"(accumulator[3])
		     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

/* 2^(weight code + activation code - 254 + 22) as an FP32: nothing below the normal numbers (the block then adds
 * nothing), at most 2^127 */
__device__ __forceinline__ float block_scale(uint32_t weight_code, uint32_t activation_code)
{
	const int32_t field = (int32_t)(weight_code + activation_code) - 105;
	return field < 1 ? 0.0f : __uint_as_float((uint32_t)(field > 254 ? 254 : field) << 23);
}

/* True if every byte of `word` is an E8M0 code from 53 to 179. Where the two codes of a block's scale both are,
 * block_scale(w, a) is the product of the normal numbers 2^(w - 127) and 2^(a - 105) and is formed that way (two
 * multiply-adds of the integer multiplier and one FP32 multiplication instead of the clamped sum on the ALU pipe, which
 * bounds these kernels): field = w + a - 105 lies in 1 .. 253, nothing is clamped, the product is exact. */
__device__ __forceinline__ bool codes_are_central(uint32_t word)
{
	const uint32_t even = (word & 0x00FF00FFu) + 0x004B004Bu, odd = ((word >> 8) & 0x00FF00FFu) + 0x004B004Bu;
	return (((even ^ 0x00800080u) | (odd ^ 0x00800080u)) & 0x01800180u) == 0u;
}

/* the four scales of one block of 32 inputs: (low row, high row) x (even column, odd column). central: every code
 * involved passed codes_are_central (a lane decides for itself: the products lie outside the branch) */
__device__ __forceinline__ void block_scales(bool central, uint32_t low_row, uint32_t high_row, uint32_t even_code,
					     uint32_t odd_code, float scales[4])
{
	if (central) {
		const float low = __uint_as_float(low_row * 0x00800000u), high = __uint_as_float(high_row * 0x00800000u);
		const float even = __uint_as_float(even_code * 0x00800000u + 0x0B000000u),
			    odd = __uint_as_float(odd_code * 0x00800000u + 0x0B000000u); /* 2^(code - 127 + 22) */
		scales[0] = __fmul_rn(low, even);
		scales[1] = __fmul_rn(low, odd);
		scales[2] = __fmul_rn(high, even);
		scales[3] = __fmul_rn(high, odd);
	} else {
		scales[0] = block_scale(low_row, even_code);
		scales[1] = block_scale(low_row, odd_code);
		scales[2] = block_scale(high_row, even_code);
		scales[3] = block_scale(high_row, odd_code);
	}
}

/* One slice of one tile: the chains of this lane's four (output, column) results. matrix: the stored matrix of
 * `outputs` x `inputs`; operands / exponents: per column's vector (this lane feeds column lane / 4 and collects columns
 * 2 t, 2 t + 1). */
__device__ __forceinline__ void slice_chains(const unsigned char *matrix, uint32_t outputs, uint32_t inputs,
					     uint32_t tile, uint32_t first_load, uint32_t last_load,
					     const uint16_t *fed_operands, const unsigned char *exponents_even,
					     const unsigned char *exponents_odd, float chains[4])
{
	const uint32_t lane = threadIdx.x % WARP, group = lane / 4u, place = lane % 4u;
	const uint32_t loads = inputs / LINEAR_VALUES_PER_LOAD;
	const uint4 *const words = reinterpret_cast<const uint4 *>(matrix) + ((uint64_t)tile * loads) * WARP + lane;
	const uint32_t *const scales =
		reinterpret_cast<const uint32_t *>(matrix + (uint64_t)outputs * inputs / 2u) + (uint64_t)tile * loads * 8u + group;
	const uint4 *const fed = reinterpret_cast<const uint4 *>(fed_operands) + place * 2u;
	chains[0] = chains[1] = chains[2] = chains[3] = 0.0f;
	if (first_load >= last_load)
		return;
	/* EXPERT_AHEAD loads in flight a lane: a slice is short (a few KB a warp), so the depth of the prefetch, not the
	 * occupancy, decides how much of the memory system a launch keeps busy */
	uint4 ahead_words[EXPERT_AHEAD];
	uint32_t ahead_scales[EXPERT_AHEAD];
#pragma unroll
	for (uint32_t slot = 0; slot < EXPERT_AHEAD; slot++)
		if (first_load + slot < last_load) {
			ahead_words[slot] = __ldcs(words + (uint64_t)(first_load + slot) * WARP);
			ahead_scales[slot] = __ldcs(scales + (uint64_t)(first_load + slot) * 8u);
		}
	for (uint32_t base = first_load; base < last_load; base += EXPERT_AHEAD) {
#pragma unroll
		for (uint32_t slot = 0; slot < EXPERT_AHEAD; slot++) {
			const uint32_t load = base + slot;
			if (load >= last_load)
				break;
			const uint4 current = ahead_words[slot];
			const uint32_t scale_word = ahead_scales[slot];
			if (load + EXPERT_AHEAD < last_load) {
				ahead_words[slot] = __ldcs(words + (uint64_t)(load + EXPERT_AHEAD) * WARP);
				ahead_scales[slot] = __ldcs(scales + (uint64_t)(load + EXPERT_AHEAD) * 8u);
			}
			const uint4 fed_low = __ldg(fed + (uint64_t)load * 8u), fed_high = __ldg(fed + (uint64_t)load * 8u + 1u);
			const uint32_t fed_registers[8] = { fed_low.x, fed_low.y, fed_low.z, fed_low.w,
							    fed_high.x, fed_high.y, fed_high.z, fed_high.w };
			const uint32_t step_words[4] = { current.x, current.y, current.z, current.w };
			const uint32_t even = *reinterpret_cast<const uint16_t *>(exponents_even + 2u * load);
			const uint32_t odd = *reinterpret_cast<const uint16_t *>(exponents_odd + 2u * load);
			const bool central = codes_are_central(scale_word) && codes_are_central(even | odd << 16);
#pragma unroll
			for (uint32_t q = 0; q < 2u; q++) {
				float sum[4] = { 0.0f, 0.0f, 0.0f, 0.0f };
#pragma unroll
				for (uint32_t half = 0; half < 2u; half++) {
					const uint32_t step = 2u * q + half, word = step_words[step];
					const uint32_t a[4] = { place_e2m1<0>(word), place_e2m1<1>(word), place_e2m1<2>(word),
								place_e2m1<3>(word) };
					mma_f16(sum, a, fed_registers[2u * step], fed_registers[2u * step + 1u]);
				}
				float scales[4];
				block_scales(central, (scale_word >> (16u * q)) & 0xFFu, (scale_word >> (16u * q + 8u)) & 0xFFu,
					     (even >> (8u * q)) & 0xFFu, (odd >> (8u * q)) & 0xFFu, scales);
#pragma unroll
				for (uint32_t c = 0; c < 4; c++)
					chains[c] = __fmaf_rn(sum[c], scales[c], chains[c]);
			}
		}
	}
}

/* the vector (a row for gate/up, a pair for down) of column c of a job; columns beyond its rows repeat column 0 */
__device__ __forceinline__ uint32_t column_pair(const struct expert_job_record *job, uint32_t column)
{
	return job->pair_index[column < job->row_count ? column : 0u];
}

template <uint32_t S>
__device__ __forceinline__ void gate_up(const struct expert_gate_up_arguments &arguments, unsigned char *arena)
{
	__shared__ float parts[2][S][WARP][4];
	const struct expert_job_record *const job =
		reinterpret_cast<const struct expert_job_record *>(arena + arguments.jobs_offset) + blockIdx.y;
	if (job->row_count == 0)
		return;
	const uint32_t lane = threadIdx.x % WARP, warp = threadIdx.x / WARP, group = lane / 4u, place = lane % 4u;
	const uint32_t which = warp / S, slice = warp % S;
	const uint32_t H = arguments.input_size, loads = H / LINEAR_VALUES_PER_LOAD;
	const uint32_t fed_row = column_pair(job, group) / arguments.pairs_per_row;
	const uint32_t even_row = column_pair(job, 2u * place) / arguments.pairs_per_row;
	const uint32_t odd_row = column_pair(job, 2u * place + 1u) / arguments.pairs_per_row;
	const unsigned char *const exponents = arena + arguments.exponents_offset;
	float chains[4];
	slice_chains(arena + (which == 0 ? job->gate_offset : job->up_offset), arguments.output_size, H, blockIdx.x,
		     loads * slice / S, loads * (slice + 1u) / S,
		     reinterpret_cast<const uint16_t *>(arena + arguments.operands_offset) + (uint64_t)fed_row * H,
		     exponents + (uint64_t)even_row * (H / 32u), exponents + (uint64_t)odd_row * (H / 32u), chains);
#pragma unroll
	for (uint32_t c = 0; c < 4; c++)
		parts[which][slice][lane][c] = chains[c];
	__syncthreads();
	if (warp != 0)
		return;
	uint16_t *const hidden = reinterpret_cast<uint16_t *>(arena + arguments.hidden_offset);
#pragma unroll
	for (uint32_t c = 0; c < 4; c++) {
		const uint32_t column = 2u * place + (c & 1u);
		if (column >= job->row_count)
			continue;
		float gate = 0.0f, up = 0.0f;
#pragma unroll
		for (uint32_t part = 0; part < S; part++) {
			gate = __fadd_rn(gate, parts[0][part][lane][c]);
			up = __fadd_rn(up, parts[1][part][lane][c]);
		}
		/* gate and up are bfloat16 first, as the reference's linear returns them */
		const float g = bfloat16_value(bfloat16_bits(gate)), u = bfloat16_value(bfloat16_bits(up));
		const float limit = arguments.activation_limit;
		const float bounded_gate = g > limit ? limit : g;
		const float bounded_up = u > limit ? limit : (u < -limit ? -limit : u);
		const float gated = __fdiv_rn(bounded_gate, __fadd_rn(1.0f, expf(-bounded_gate)));
		const float value = __fmul_rn(__fmul_rn(gated, bounded_up), job->route_weight[column]);
		hidden[(uint64_t)job->pair_index[column] * arguments.output_size + blockIdx.x * LINEAR_OUTPUTS_PER_TILE + group +
		       (c >> 1) * 8u] = (uint16_t)bfloat16_bits(value);
	}
}

template <uint32_t S>
__device__ __forceinline__ void down(const struct expert_down_arguments &arguments, unsigned char *arena)
{
	__shared__ float parts[S][WARP][4];
	const struct expert_job_record *const job =
		reinterpret_cast<const struct expert_job_record *>(arena + arguments.jobs_offset) + blockIdx.y;
	if (job->row_count == 0)
		return;
	const uint32_t lane = threadIdx.x % WARP, slice = threadIdx.x / WARP, group = lane / 4u, place = lane % 4u;
	const uint32_t I = arguments.input_size, loads = I / LINEAR_VALUES_PER_LOAD;
	const unsigned char *const exponents = arena + arguments.exponents_offset;
	float chains[4];
	slice_chains(arena + job->down_offset, arguments.output_size, I, blockIdx.x, loads * slice / S,
		     loads * (slice + 1u) / S,
		     reinterpret_cast<const uint16_t *>(arena + arguments.operands_offset) + (uint64_t)column_pair(job, group) * I,
		     exponents + (uint64_t)column_pair(job, 2u * place) * (I / 32u),
		     exponents + (uint64_t)column_pair(job, 2u * place + 1u) * (I / 32u), chains);
#pragma unroll
	for (uint32_t c = 0; c < 4; c++)
		parts[slice][lane][c] = chains[c];
	__syncthreads();
	if (slice != 0)
		return;
	uint16_t *const output = reinterpret_cast<uint16_t *>(arena + arguments.output_offset);
#pragma unroll
	for (uint32_t c = 0; c < 4; c++) {
		const uint32_t column = 2u * place + (c & 1u);
		if (column >= job->row_count)
			continue;
		float sum = 0.0f;
#pragma unroll
		for (uint32_t part = 0; part < S; part++)
			sum = __fadd_rn(sum, parts[part][lane][c]);
		output[(uint64_t)job->pair_index[column] * arguments.output_size + blockIdx.x * LINEAR_OUTPUTS_PER_TILE + group +
		       (c >> 1) * 8u] = (uint16_t)bfloat16_bits(sum);
	}
}

#define EXPERT_ENTRIES(S)                                                                                  \
	extern "C" __global__ void __launch_bounds__(64 * S)                                               \
		expert_gate_up_##S(struct expert_gate_up_arguments arguments, unsigned char *arena)        \
	{                                                                                                  \
		gate_up<S>(arguments, arena);                                                              \
	}                                                                                                  \
	extern "C" __global__ void __launch_bounds__(32 * S)                                               \
		expert_down_##S(struct expert_down_arguments arguments, unsigned char *arena)              \
	{                                                                                                  \
		down<S>(arguments, arena);                                                                 \
	}
EXPERT_ENTRIES(1)
EXPERT_ENTRIES(2)
EXPERT_ENTRIES(4)
EXPERT_ENTRIES(8)
EXPERT_ENTRIES(16)

/* ------------------------------------------------------------------ many rows: a group of jobs a block
 *
 * expert_gate_up_many / expert_down_many: the same products for a job table of many rows. A warp owns one tile of 16
 * outputs for ALL of K and for up to LINEAR_MANY_JOBS consecutive jobs of one expert: it places a load's words once
 * and multiplies them with every job's columns; a job's slices are walked one after the other (a slice one chain, the
 * chains added from +0 in ascending order), so every value goes through the thin instances' operations in their order.
 * The warps of a block take neighbouring tiles and the same jobs: the rows' operands come from L2 once a block. */

/* The chains of R jobs over one slice of one tile. fed[r], exponents_even[r], exponents_odd[r]: as slice_chains'
 * fed, exponents_even, exponents_odd, of job r. */
template <uint32_t R>
__device__ __forceinline__ void slice_chains_many(const unsigned char *matrix, uint32_t outputs, uint32_t inputs,
						   uint32_t tile, uint32_t first_load, uint32_t last_load,
						   const uint4 *const (&fed)[R], const unsigned char *const (&exponents_even)[R],
						   const unsigned char *const (&exponents_odd)[R], float (&chains)[R][4])
{
	const uint32_t lane = threadIdx.x % WARP, group = lane / 4u;
	const uint32_t loads = inputs / LINEAR_VALUES_PER_LOAD;
	const uint4 *const words = reinterpret_cast<const uint4 *>(matrix) + ((uint64_t)tile * loads) * WARP + lane;
	const uint32_t *const scales =
		reinterpret_cast<const uint32_t *>(matrix + (uint64_t)outputs * inputs / 2u) + (uint64_t)tile * loads * 8u + group;
#pragma unroll
	for (uint32_t r = 0; r < R; r++)
		chains[r][0] = chains[r][1] = chains[r][2] = chains[r][3] = 0.0f;
	if (first_load >= last_load)
		return;
	uint4 ahead_words[EXPERT_AHEAD];
	uint32_t ahead_scales[EXPERT_AHEAD];
#pragma unroll
	for (uint32_t slot = 0; slot < EXPERT_AHEAD; slot++)
		if (first_load + slot < last_load) {
			ahead_words[slot] = __ldcs(words + (uint64_t)(first_load + slot) * WARP);
			ahead_scales[slot] = __ldcs(scales + (uint64_t)(first_load + slot) * 8u);
		}
	for (uint32_t base = first_load; base < last_load; base += EXPERT_AHEAD) {
#pragma unroll
		for (uint32_t slot = 0; slot < EXPERT_AHEAD; slot++) {
			const uint32_t load = base + slot;
			if (load >= last_load)
				break;
			const uint4 current = ahead_words[slot];
			const uint32_t scale_word = ahead_scales[slot];
			if (load + EXPERT_AHEAD < last_load) {
				ahead_words[slot] = __ldcs(words + (uint64_t)(load + EXPERT_AHEAD) * WARP);
				ahead_scales[slot] = __ldcs(scales + (uint64_t)(load + EXPERT_AHEAD) * 8u);
			}
			const uint32_t step_words[4] = { current.x, current.y, current.z, current.w };
			uint32_t a[4][4];
#pragma unroll
			for (uint32_t step = 0; step < 4u; step++) {
				a[step][0] = place_e2m1<0>(step_words[step]);
				a[step][1] = place_e2m1<1>(step_words[step]);
				a[step][2] = place_e2m1<2>(step_words[step]);
				a[step][3] = place_e2m1<3>(step_words[step]);
			}
#pragma unroll
			for (uint32_t r = 0; r < R; r++) {
				const uint4 fed_low = __ldg(fed[r] + (uint64_t)load * 8u), fed_high = __ldg(fed[r] + (uint64_t)load * 8u + 1u);
				const uint32_t fed_registers[8] = { fed_low.x, fed_low.y, fed_low.z, fed_low.w,
								    fed_high.x, fed_high.y, fed_high.z, fed_high.w };
				const uint32_t even = *reinterpret_cast<const uint16_t *>(exponents_even[r] + 2u * load);
				const uint32_t odd = *reinterpret_cast<const uint16_t *>(exponents_odd[r] + 2u * load);
#pragma unroll
				for (uint32_t q = 0; q < 2u; q++) {
					float sum[4] = { 0.0f, 0.0f, 0.0f, 0.0f };
#pragma unroll
					for (uint32_t half = 0; half < 2u; half++) {
						const uint32_t step = 2u * q + half;
						mma_f16(sum, a[step], fed_registers[2u * step], fed_registers[2u * step + 1u]);
					}
					/* the clamped sums here: with two jobs' chains live the branch of block_scales costs more than
					 * it saves */
					const uint32_t low_row = (scale_word >> (16u * q)) & 0xFFu,
						       high_row = (scale_word >> (16u * q + 8u)) & 0xFFu;
					const uint32_t even_code = (even >> (8u * q)) & 0xFFu, odd_code = (odd >> (8u * q)) & 0xFFu;
					chains[r][0] = __fmaf_rn(sum[0], block_scale(low_row, even_code), chains[r][0]);
					chains[r][1] = __fmaf_rn(sum[1], block_scale(low_row, odd_code), chains[r][1]);
					chains[r][2] = __fmaf_rn(sum[2], block_scale(high_row, even_code), chains[r][2]);
					chains[r][3] = __fmaf_rn(sum[3], block_scale(high_row, odd_code), chains[r][3]);
				}
			}
		}
	}
}

/* the sums of R jobs for one tile of one matrix: every slice's chains, added from +0 in ascending order. vectors: the
 * divisor that makes a pair index a vector of the operand arrays (pairs_per_row for gate/up, 1 for down) */
template <uint32_t R>
__device__ __forceinline__ void sums_many(const unsigned char *matrix, uint32_t outputs, uint32_t inputs, uint32_t tile,
					   uint32_t slices, const struct expert_job_record *jobs, uint32_t vectors,
					   const unsigned char *operands, const unsigned char *exponents, float (&totals)[R][4])
{
	const uint32_t lane = threadIdx.x % WARP, group = lane / 4u, place = lane % 4u;
	const uint32_t loads = inputs / LINEAR_VALUES_PER_LOAD;
	const uint4 *fed[R];
	const unsigned char *even[R], *odd[R];
#pragma unroll
	for (uint32_t r = 0; r < R; r++) {
		fed[r] = reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(operands) +
							 (uint64_t)(column_pair(&jobs[r], group) / vectors) * inputs) +
			 place * 2u;
		even[r] = exponents + (uint64_t)(column_pair(&jobs[r], 2u * place) / vectors) * (inputs / 32u);
		odd[r] = exponents + (uint64_t)(column_pair(&jobs[r], 2u * place + 1u) / vectors) * (inputs / 32u);
		totals[r][0] = totals[r][1] = totals[r][2] = totals[r][3] = 0.0f;
	}
	for (uint32_t slice = 0; slice < slices; slice++) {
		float chains[R][4];
		slice_chains_many<R>(matrix, outputs, inputs, tile, loads * slice / slices, loads * (slice + 1u) / slices, fed,
				     even, odd, chains);
#pragma unroll
		for (uint32_t r = 0; r < R; r++)
#pragma unroll
			for (uint32_t c = 0; c < 4; c++)
				totals[r][c] = __fadd_rn(totals[r][c], chains[r][c]);
	}
}

#define MANY_GATE_UP_TILES 4u /* tiles of 16 outputs of a block, of gate and of up */
#define MANY_DOWN_TILES 8u

template <uint32_t R>
__device__ __forceinline__ void gate_up_many(const struct expert_gate_up_many_arguments &many, unsigned char *arena,
					     const struct expert_job_record *jobs,
					     float (&parts)[MANY_GATE_UP_TILES][LINEAR_MANY_JOBS][WARP][4])
{
	const struct expert_gate_up_arguments &arguments = many.base;
	const uint32_t lane = threadIdx.x % WARP, warp = threadIdx.x / WARP, group = lane / 4u, place = lane % 4u;
	const uint32_t which = warp / MANY_GATE_UP_TILES, mine = warp % MANY_GATE_UP_TILES;
	const uint32_t tile = blockIdx.x * MANY_GATE_UP_TILES + mine;
	float totals[R][4];
	sums_many<R>(arena + (which == 0 ? jobs[0].gate_offset : jobs[0].up_offset), arguments.output_size,
		     arguments.input_size, tile, many.slice_count, jobs, arguments.pairs_per_row,
		     arena + arguments.operands_offset, arena + arguments.exponents_offset, totals);
	__syncthreads(); /* the run before this one has read its parts */
	if (which == 1u) {
#pragma unroll
		for (uint32_t r = 0; r < R; r++)
#pragma unroll
			for (uint32_t c = 0; c < 4; c++)
				parts[mine][r][lane][c] = totals[r][c];
	}
	__syncthreads();
	if (which != 0u)
		return;
	uint16_t *const hidden = reinterpret_cast<uint16_t *>(arena + arguments.hidden_offset);
#pragma unroll
	for (uint32_t r = 0; r < R; r++)
#pragma unroll
		for (uint32_t c = 0; c < 4; c++) {
			const uint32_t column = 2u * place + (c & 1u);
			if (column >= jobs[r].row_count)
				continue;
			/* gate and up are bfloat16 first, as the reference's linear returns them */
			const float g = bfloat16_value(bfloat16_bits(totals[r][c])),
				    u = bfloat16_value(bfloat16_bits(parts[mine][r][lane][c]));
			const float limit = arguments.activation_limit;
			const float bounded_gate = g > limit ? limit : g;
			const float bounded_up = u > limit ? limit : (u < -limit ? -limit : u);
			const float gated = __fdiv_rn(bounded_gate, __fadd_rn(1.0f, expf(-bounded_gate)));
			const float value = __fmul_rn(__fmul_rn(gated, bounded_up), jobs[r].route_weight[column]);
			hidden[(uint64_t)jobs[r].pair_index[column] * arguments.output_size + tile * LINEAR_OUTPUTS_PER_TILE + group +
			       (c >> 1) * 8u] = (uint16_t)bfloat16_bits(value);
		}
}

template <uint32_t R>
__device__ __forceinline__ void down_many(const struct expert_down_many_arguments &many, unsigned char *arena,
					  const struct expert_job_record *jobs)
{
	const struct expert_down_arguments &arguments = many.base;
	const uint32_t lane = threadIdx.x % WARP, warp = threadIdx.x / WARP, group = lane / 4u, place = lane % 4u;
	const uint32_t tile = blockIdx.x * MANY_DOWN_TILES + warp;
	float totals[R][4];
	sums_many<R>(arena + jobs[0].down_offset, arguments.output_size, arguments.input_size, tile, many.slice_count, jobs, 1u,
		     arena + arguments.operands_offset, arena + arguments.exponents_offset, totals);
	uint16_t *const output = reinterpret_cast<uint16_t *>(arena + arguments.output_offset);
#pragma unroll
	for (uint32_t r = 0; r < R; r++)
#pragma unroll
		for (uint32_t c = 0; c < 4; c++) {
			const uint32_t column = 2u * place + (c & 1u);
			if (column >= jobs[r].row_count)
				continue;
			output[(uint64_t)jobs[r].pair_index[column] * arguments.output_size + tile * LINEAR_OUTPUTS_PER_TILE + group +
			       (c >> 1) * 8u] = (uint16_t)bfloat16_bits(totals[r][c]);
		}
}

/* the jobs of the block's group from `first` that are live and of one expert (at most LINEAR_MANY_JOBS - first) */
__device__ __forceinline__ uint32_t many_run(const struct expert_job_record *jobs, uint32_t first, uint32_t count)
{
	uint32_t run = 0;
	while (first + run < count && jobs[first + run].row_count != 0 && jobs[first + run].expert == jobs[first].expert)
		run++;
	return run;
}

#if LINEAR_MANY_JOBS >= 3
#define MANY_CASE_3(call) \
	case 3:           \
		call(3);  \
		break;
#else
#define MANY_CASE_3(call)
#endif
#if LINEAR_MANY_JOBS >= 4
#define MANY_CASE_4(call) \
	case 4:           \
		call(4);  \
		break;
#else
#define MANY_CASE_4(call)
#endif
#define MANY_RUNS(call)                                                                  \
	const uint32_t first_job = blockIdx.y * LINEAR_MANY_JOBS;                         \
	const struct expert_job_record *const group_jobs =                                \
		reinterpret_cast<const struct expert_job_record *>(arena + many.base.jobs_offset) + first_job; \
	const uint32_t count = min(LINEAR_MANY_JOBS, many.job_count - first_job);         \
	for (uint32_t first = 0; first < count;) {                                        \
		const uint32_t run = many_run(group_jobs, first, count);                  \
		const struct expert_job_record *const jobs = group_jobs + first;          \
		switch (run) {                                                            \
		case 0:                                                                   \
			first++; /* an empty job */                                       \
			break;                                                            \
		case 1:                                                                   \
			call(1);                                                          \
			break;                                                            \
		case 2:                                                                   \
			call(2);                                                          \
			break;                                                            \
		MANY_CASE_3(call)                                                         \
		MANY_CASE_4(call)                                                         \
		default:                                                                  \
			break;                                                            \
		}                                                                         \
		first += run;                                                             \
	}

extern "C" __global__ void __launch_bounds__(2u * MANY_GATE_UP_TILES * WARP, 2)
	expert_gate_up_many(struct expert_gate_up_many_arguments many, unsigned char *arena)
{
	__shared__ float parts[MANY_GATE_UP_TILES][LINEAR_MANY_JOBS][WARP][4];
	if (blockIdx.y * LINEAR_MANY_JOBS >= many.job_count)
		return;
#define MANY_CALL(R) gate_up_many<R>(many, arena, jobs, parts)
	MANY_RUNS(MANY_CALL)
#undef MANY_CALL
}

extern "C" __global__ void __launch_bounds__(MANY_DOWN_TILES * WARP, 2)
	expert_down_many(struct expert_down_many_arguments many, unsigned char *arena)
{
	if (blockIdx.y * LINEAR_MANY_JOBS >= many.job_count)
		return;
#define MANY_CALL(R) down_many<R>(many, arena, jobs)
	MANY_RUNS(MANY_CALL)
#undef MANY_CALL
}

extern "C" __global__ void expert_row_sum_entry(struct expert_row_sum_arguments arguments, unsigned char *arena)
{
	const uint32_t channel = blockIdx.x * blockDim.x + threadIdx.x;
	if (channel >= arguments.width)
		return;
	const uint64_t row = blockIdx.y;
	const uint16_t *const pairs = reinterpret_cast<const uint16_t *>(arena + arguments.pair_output_offset);
	float sum = 0.0f;
	for (uint32_t slot = 0; slot < arguments.pairs_per_row; slot++)
		sum = __fadd_rn(sum, bfloat16_value(pairs[(row * arguments.pairs_per_row + slot) * arguments.width + channel]));
	reinterpret_cast<float *>(arena + arguments.row_output_offset)[row * arguments.width + channel] = sum;
}
