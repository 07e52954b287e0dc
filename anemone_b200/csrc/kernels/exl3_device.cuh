/*
 * exl3_device.cuh: device building blocks of the EXL3 expert kernels for sm_100a.
 *
 *   - trellis decode of a lane's eight weights of a 16 x 16 tile straight into the A-fragment registers of
 *     mma.sync.m16n8k16 (the stream order of the format IS that fragment order);
 *   - the 128-point Hadamard butterfly on one warp, four values a lane, in the stage order of the reference's
 *     transform (source/kernel_exl3.cu:104-124), so the FP32 bits are the same;
 *   - a product core: one CTA computes 128 outputs of one job for up to eight rows. Four warps take interleaved K
 *     steps; a lane loads its ring words straight from global memory into registers one round ahead, decodes them in
 *     registers and accumulates in FP32 on the tensor cores; the four partial sums are added in warp order from +0. A
 *     CTA may take a part of K only (split K): the caller then adds the parts in a fixed order.
 *   - mbarrier and bulk-copy helpers for the prefill kernels' rings. Every mbarrier wait is bounded: a wait that runs
 *     out raises exl3_wait_expired (a module global the host can read); nothing traps.
 */
#ifndef AB_EXL3_DEVICE_CUH
#define AB_EXL3_DEVICE_CUH

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "exl3_geometry.h"

#define EXL3_WAIT_CYCLES 1500000000ll /* of the device clock: under a second */

__device__ unsigned int exl3_wait_expired;

/* ------------------------------------------------------------------ mbarrier and bulk copy (PTX) */

__device__ __forceinline__ uint32_t smem_address(const void *pointer)
{
	return (uint32_t)__cvta_generic_to_shared(pointer);
}

__device__ __forceinline__ void barrier_init(uint64_t *barrier, uint32_t arrivals)
{
	asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_address(barrier)), "r"(arrivals) : "memory");
}

__device__ __forceinline__ void barrier_invalidate(uint64_t *barrier)
{
	asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_address(barrier)) : "memory");
}

__device__ __forceinline__ void barrier_expect(uint64_t *barrier, uint32_t bytes)
{
	asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_address(barrier)), "r"(bytes)
		     : "memory");
}

__device__ __forceinline__ void barrier_arrive(uint64_t *barrier)
{
	asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_address(barrier)) : "memory");
}

/* true once the phase of the given parity has completed; false if the bounded wait ran out. The wait spins on
 * try_wait (which itself suspends the thread for a short, hardware-chosen time) and never sleeps: a sleep's wake-up
 * is far coarser than the hand-offs of a pipeline stage. The bound is a count of device clock cycles. */
__device__ __forceinline__ bool barrier_wait(uint64_t *barrier, uint32_t parity)
{
	const uint32_t address = smem_address(barrier);
	long long begun = 0;
	for (uint32_t poll = 1;; poll++) {
		uint32_t complete;
		asm volatile("{\n\t.reg .pred p;\n\t"
			     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
			     "selp.u32 %0, 1, 0, p;\n\t}"
			     : "=r"(complete)
			     : "r"(address), "r"(parity)
			     : "memory");
		if (complete != 0)
			return true;
		if ((poll & 255u) == 0u) {
			const long long now = clock64();
			if (begun == 0)
				begun = now;
			else if (now - begun > EXL3_WAIT_CYCLES)
				break;
		}
	}
	atomicExch(&exl3_wait_expired, 1u);
	return false;
}

/* bytes a multiple of 16, both addresses 16-byte aligned; completes `bytes` of the barrier's transaction count */
__device__ __forceinline__ void bulk_load(void *shared_destination, const void *global_source, uint32_t bytes,
					  uint64_t *barrier)
{
	asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
			     smem_address(shared_destination)),
		     "l"(global_source), "r"(bytes), "r"(smem_address(barrier))
		     : "memory");
}

/* ------------------------------------------------------------------ decode */

template <uint32_t BX2> struct exl3_ring {
	static constexpr uint32_t ring_bits = 128u * BX2;
	static constexpr uint32_t words = ring_bits / 32u;
	static constexpr uint32_t tile_bytes = ring_bits / 8u;
	/* bits from the start of the lane's first window to the start of the window of its symbol e */
	__host__ __device__ static constexpr uint32_t offset(uint32_t e)
	{
		return (((e + 1u) * BX2) >> 1) - (BX2 >> 1);
	}
	/* ring bit where lane l's first window starts */
	__host__ __device__ static constexpr uint32_t begin(uint32_t lane)
	{
		return ((((8u * lane + 1u) * BX2) >> 1) + ring_bits - 16u) % ring_bits;
	}
};

/* FP16 bits (in the low half) of a state: dp4a sums the four bytes of state * multiplier onto 0x6400 */
__device__ __forceinline__ uint32_t exl3_value_bits(uint32_t state)
{
	return __dp4a(state * EXL3_MUL1_MULTIPLIER, 0x01010101u, EXL3_MUL1_BASE);
}

__device__ __forceinline__ uint32_t exl3_pair(uint32_t low_state, uint32_t high_state)
{
	/* low | high << 16 as a multiply-add: the integer multiplier's pipe instead of the ALU's, which the window
	 * shifts and masks keep busy */
	const uint32_t packed = exl3_value_bits(high_state) * 65536u + exl3_value_bits(low_state);
	const __half2 scale = __halves2half2(__ushort_as_half(EXL3_MUL1_SCALE), __ushort_as_half(EXL3_MUL1_SCALE));
	const __half2 bias = __halves2half2(__ushort_as_half(EXL3_MUL1_BIAS), __ushort_as_half(EXL3_MUL1_BIAS));
	const __half2 value = __hfma2(*reinterpret_cast<const __half2 *>(&packed), scale, bias);
	return *reinterpret_cast<const uint32_t *>(&value);
}

/* state of the lane's symbol e from its two ring words, already shifted so that its first window starts at the top.
 * Widths whose windows start on a few distinct bit positions modulo 8 (K2: four, K4: two) take a state as two bytes of
 * the word shifted by that position (one shift serves every state that shares it, one byte permute a state: the
 * compiler keeps the shifted word); the other widths shift and mask. */
template <uint32_t BX2>
__device__ __forceinline__ uint32_t exl3_state_of(uint32_t high, uint32_t low, uint32_t e)
{
	const uint32_t offset = exl3_ring<BX2>::offset(e);
	if (offset == 0u)
		return high >> 16;
	if (BX2 == 4u || BX2 == 8u) {
		/* the 32 bits the state lies in: the first word, or the window that begins 16 bits into it */
		const uint32_t word = offset <= 16u ? high : __funnelshift_r(low, high, 16);
		const uint32_t distance = (offset <= 16u ? 16u : 32u) - offset; /* of the state's last bit from the word's */
		const uint32_t byte = distance / 8u; /* 0, 1 or 2: the state is bytes byte, byte + 1 of the shifted word */
		return __byte_perm(word >> (distance % 8u), 0u, byte == 0u ? 0x4410u : byte == 1u ? 0x4421u : 0x4432u);
	}
	if (offset <= 16u)
		return (high >> (16u - offset)) & 0xFFFFu;
	return __funnelshift_r(low, high, 48u - offset) & 0xFFFFu;
}

/* The four A registers of m16n8k16 for one tile: symbols {0,1}, {4,5}, {2,3}, {6,7} of the lane. */
template <uint32_t BX2>
__device__ __forceinline__ void exl3_decode_fragment(uint32_t word0, uint32_t word1, uint32_t shift,
						      uint32_t fragment[4])
{
	const uint32_t high = __funnelshift_l(word1, word0, shift);
	const uint32_t low = word1 << shift;
	fragment[0] = exl3_pair(exl3_state_of<BX2>(high, low, 0), exl3_state_of<BX2>(high, low, 1));
	fragment[1] = exl3_pair(exl3_state_of<BX2>(high, low, 4), exl3_state_of<BX2>(high, low, 5));
	fragment[2] = exl3_pair(exl3_state_of<BX2>(high, low, 2), exl3_state_of<BX2>(high, low, 3));
	fragment[3] = exl3_pair(exl3_state_of<BX2>(high, low, 6), exl3_state_of<BX2>(high, low, 7));
}

__device__ __forceinline__ void mma_f16(float accumulator[4], const uint32_t a[4], uint32_t b0, uint32_t b1)
{
	asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
		     "{%0,%1,%2,%3};"
		     : "+f"(accumulator[0]), "+f"(accumulator[1]), "+f"(accumulator[2]), "+f"(accumulator[3])
		     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

/* ------------------------------------------------------------------ Hadamard, one warp, values 4 lane + i */

__device__ __forceinline__ void hadamard128_warp(float v[4], uint32_t lane)
{
	/* strides 1 and 2 inside the lane */
	float a = __fadd_rn(v[0], v[1]), b = __fsub_rn(v[0], v[1]);
	float c = __fadd_rn(v[2], v[3]), d = __fsub_rn(v[2], v[3]);
	v[0] = __fadd_rn(a, c);
	v[1] = __fadd_rn(b, d);
	v[2] = __fsub_rn(a, c);
	v[3] = __fsub_rn(b, d);
	/* strides 4 .. 64 across lanes: the lower partner takes a + b, the upper one (lower - upper) */
#pragma unroll
	for (uint32_t distance = 1; distance < EXL3_WARP; distance <<= 1) {
		const bool upper = (lane & distance) != 0;
#pragma unroll
		for (uint32_t i = 0; i < 4; i++) {
			const float other = __shfl_xor_sync(0xFFFFFFFFu, v[i], distance);
			v[i] = upper ? __fsub_rn(other, v[i]) : __fadd_rn(v[i], other);
		}
	}
}

/* ------------------------------------------------------------------ the product core */

struct exl3_product_shared {
	uint32_t failed; /* kept for the callers' sake: the core has no wait that could fail */
};

/* Dynamic shared memory of a product CTA (exl3_geometry.h): the warps' partial sums after the K loop. */

/* sums[tile][c]: this thread's share of the CTA's 128 outputs x 8 columns after the cross-warp reduction: thread
 * (warp w, lane (g, t)) returns, for tiles j = 2 w and 2 w + 1, the m16n8 accumulator layout
 *   c0: (output 16 j + g, column 2 t)   c1: (16 j + g, 2 t + 1)   c2: (16 j + g + 8, 2 t)   c3: (16 j + g + 8, 2 t + 1).
 * matrix: the codes of a matrix of `outputs` outputs; group: which 128 outputs; the K steps (tile rows)
 * [step_begin, step_begin + step_count), a multiple of EXL3_STAGE_STEPS; operand_row: FP16 [inputs] of the pair that
 * stands in this lane's column (lane / 4; columns beyond the job's rows repeat column 0 and are ignored by the caller).
 * Warp w takes step 4 r + w of round r. A lane reads its two ring words of each of the eight tiles of a step straight
 * from global memory into registers (the warp's 16 loads of a step cover 8 x 16 bits_x2 contiguous bytes), one round
 * ahead of the round it decodes, together with that round's operands: no shared memory, no barrier and no producer
 * stand between the memory system and the decode, whose instruction issue is what bounds the kernel. The operands are
 * read past the L1 (they may have been written by a launch that still runs beside this one); the weights through it.
 * Returns true (the signature keeps a verdict for callers written for a core with bounded waits). All 128 threads
 * call it. */
template <uint32_t BX2>
__device__ __forceinline__ bool exl3_product_core(const unsigned char *matrix, uint32_t outputs, uint32_t group,
						  uint32_t step_begin, uint32_t step_count,
						  const __half *const operand_row, unsigned char *dynamic_shared,
						  exl3_product_shared *shared, float sums[2][4])
{
	typedef exl3_ring<BX2> ring;
	(void)shared;
	const uint32_t lane = threadIdx.x % EXL3_WARP, warp = threadIdx.x / EXL3_WARP;
	const uint32_t rounds = step_count / EXL3_STAGE_STEPS;
	const uint64_t step_words = (uint64_t)(outputs / EXL3_TILE) * ring::words; /* of one tile row of the matrix */
	const uint32_t begin = ring::begin(lane);
	const uint32_t word_index = begin / 32u, shift = begin % 32u, next_index = (word_index + 1u) % ring::words;
	/* this warp's first step, the CTA's first tile */
	const uint32_t *const words = reinterpret_cast<const uint32_t *>(matrix) + (step_begin + warp) * step_words +
				      (uint64_t)group * EXL3_GROUP_TILES * ring::words;
	const uint64_t round_words = EXL3_STAGE_STEPS * step_words;
	/* this lane's B operand of round r: inputs 2 t, 2 t + 1 and 2 t + 8, 2 t + 9 of step 4 r + warp */
	const uint32_t *const fed = reinterpret_cast<const uint32_t *>(operand_row + (step_begin + warp) * EXL3_TILE +
								      (lane % 4u) * 2u);
	constexpr uint32_t fed_round_words = EXL3_STAGE_STEPS * EXL3_TILE / 2u;
	float accumulators[EXL3_GROUP_TILES][4];
#pragma unroll
	for (uint32_t tile = 0; tile < EXL3_GROUP_TILES; tile++)
#pragma unroll
		for (uint32_t c = 0; c < 4; c++)
			accumulators[tile][c] = 0.0f;

	uint32_t first[EXL3_GROUP_TILES][2], second[EXL3_GROUP_TILES][2], first_fed[2], second_fed[2];
#define EXL3_ROUND_LOAD(set, set_fed, round)                                                                  \
	do {                                                                                                   \
		const uint32_t *const from = words + (uint64_t)(round) * round_words;                          \
		_Pragma("unroll") for (uint32_t tile = 0; tile < EXL3_GROUP_TILES; tile++)                     \
		{                                                                                              \
			set[tile][0] = __ldg(from + tile * ring::words + word_index);                          \
			set[tile][1] = __ldg(from + tile * ring::words + next_index);                          \
		}                                                                                              \
		set_fed[0] = __ldcg(fed + (uint64_t)(round) * fed_round_words);                                \
		set_fed[1] = __ldcg(fed + (uint64_t)(round) * fed_round_words + 4);                            \
	} while (0)
#define EXL3_ROUND_MULTIPLY(set, set_fed)                                                                     \
	do {                                                                                                   \
		_Pragma("unroll") for (uint32_t tile = 0; tile < EXL3_GROUP_TILES; tile++)                     \
		{                                                                                              \
			uint32_t fragment[4];                                                                  \
			exl3_decode_fragment<BX2>(set[tile][0], set[tile][1], shift, fragment);                \
			mma_f16(accumulators[tile], fragment, set_fed[0], set_fed[1]);                         \
		}                                                                                              \
	} while (0)
	EXL3_ROUND_LOAD(first, first_fed, 0u);
	for (uint32_t round = 0; round < rounds; round += 2u) {
		if (round + 1u < rounds)
			EXL3_ROUND_LOAD(second, second_fed, round + 1u);
		EXL3_ROUND_MULTIPLY(first, first_fed);
		if (round + 1u >= rounds)
			break;
		if (round + 2u < rounds)
			EXL3_ROUND_LOAD(first, first_fed, round + 2u);
		EXL3_ROUND_MULTIPLY(second, second_fed);
	}
#undef EXL3_ROUND_LOAD
#undef EXL3_ROUND_MULTIPLY

	float4 *const partial = reinterpret_cast<float4 *>(dynamic_shared); /* [warp][tile][lane] */
#pragma unroll
	for (uint32_t tile = 0; tile < EXL3_GROUP_TILES; tile++)
		partial[(warp * EXL3_GROUP_TILES + tile) * EXL3_WARP + lane] = make_float4(
			accumulators[tile][0], accumulators[tile][1], accumulators[tile][2], accumulators[tile][3]);
	__syncthreads();
#pragma unroll
	for (uint32_t mine = 0; mine < 2; mine++) {
		const uint32_t tile = warp * 2u + mine;
		float total[4] = { 0.0f, 0.0f, 0.0f, 0.0f };
#pragma unroll
		for (uint32_t slice = 0; slice < EXL3_PRODUCT_WARPS; slice++) {
			const float4 part = partial[(slice * EXL3_GROUP_TILES + tile) * EXL3_WARP + lane];
			total[0] = __fadd_rn(total[0], part.x);
			total[1] = __fadd_rn(total[1], part.y);
			total[2] = __fadd_rn(total[2], part.z);
			total[3] = __fadd_rn(total[3], part.w);
		}
#pragma unroll
		for (uint32_t c = 0; c < 4; c++)
			sums[mine][c] = total[c];
	}
	__syncthreads(); /* the partial sums are consumed: the caller may reuse the dynamic shared memory */
	return true;
}

#endif
