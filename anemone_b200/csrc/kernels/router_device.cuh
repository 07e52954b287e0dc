/*
 * router_device.cuh: the per-row part of the router, shared by the decode router (kernel_router_b200.cu) and the
 * prefill router (kernel_exl3_prefill.cu). One warp a row. Conventions: the reference's router_select_entry
 * (source/kernel_router.cuh:36-119): keys order scores as its top-k orders float32 (a not-a-number above every number,
 * -0 below +0), the lower expert first among equals; slots in ascending expert order; the weight sum from +0 in
 * ascending expert order, every operation one FP32 rounding.
 */
#ifndef AB_ROUTER_DEVICE_CUH
#define AB_ROUTER_DEVICE_CUH

#include <stdint.h>

#include "anemone_b200_records.h"

#define WARP 32u
#define EXPERTS_PER_LANE (ROUTER_B200_MAXIMUM_EXPERTS / WARP)

__device__ __forceinline__ uint64_t router_key(float score, uint32_t expert)
{
	const uint32_t bits = __float_as_uint(score);
	const uint32_t ordered = score != score ? 0xFFFFFFFFu : (bits & 0x80000000u) != 0 ? ~bits : bits | 0x80000000u;
	return (uint64_t)ordered << 32 | (uint64_t)(uint32_t)~expert;
}

__device__ __forceinline__ float router_affinity(float score, uint32_t scoring)
{
	if (scoring == ROUTER_SCORING_SQRT_SOFTPLUS)
		return __fsqrt_rn(score > 20.0f ? score : log1pf(expf(score)));
	return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-score)));
}

/* One row by one warp: `picks` rounds of a warp-wide maximum over 64-bit keys. chosen and weight: the row's
 * ROUTER_B200_MAXIMUM_PICKS entries in shared memory, filled by slot; the same values go to picks_out and weights_out
 * (the row's entries in the arena). All 32 lanes call. */
__device__ __forceinline__ void router_row(const float *scores, uint32_t experts, uint32_t picks, uint32_t scoring,
					   float route_scale, uint32_t lane, uint32_t *chosen, float *weight,
					   uint32_t *picks_out, float *weights_out)
{
	uint64_t keys[EXPERTS_PER_LANE];
#pragma unroll
	for (uint32_t place = 0; place < EXPERTS_PER_LANE; place++) {
		const uint32_t expert = place * WARP + lane;
		keys[place] = expert < experts ? router_key(scores[expert], expert) : 0ull;
	}
	uint32_t mine = 0; /* lane p keeps pick p */
	for (uint32_t pick = 0; pick < picks; pick++) {
		uint64_t best = 0;
#pragma unroll
		for (uint32_t place = 0; place < EXPERTS_PER_LANE; place++)
			best = keys[place] > best ? keys[place] : best;
		for (uint32_t distance = WARP / 2u; distance != 0; distance >>= 1) {
			const uint64_t other = __shfl_xor_sync(0xFFFFFFFFu, best, distance);
			best = other > best ? other : best;
		}
#pragma unroll
		for (uint32_t place = 0; place < EXPERTS_PER_LANE; place++)
			keys[place] = keys[place] == best ? 0ull : keys[place];
		if (lane == pick)
			mine = ~(uint32_t)best;
	}
	/* slot = the number of picked experts below mine */
	uint32_t slot = 0;
	for (uint32_t pick = 0; pick < picks; pick++) {
		const uint32_t other = __shfl_sync(0xFFFFFFFFu, mine, pick);
		slot += lane < picks && other < mine ? 1u : 0u;
	}
	if (lane < picks) {
		chosen[slot] = mine;
		weight[slot] = router_affinity(scores[mine], scoring);
	}
	__syncwarp();
	float sum = 0.0f;
	for (uint32_t place = 0; place < picks; place++)
		sum = __fadd_rn(sum, weight[place]);
	__syncwarp();
	if (lane < picks) {
		const float value = __fmul_rn(__fdiv_rn(weight[lane], __fadd_rn(sum, 1e-20f)), route_scale);
		weight[lane] = value;
		picks_out[lane] = chosen[lane];
		weights_out[lane] = value;
	}
	__syncwarp();
}

#endif
