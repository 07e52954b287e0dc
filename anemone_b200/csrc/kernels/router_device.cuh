/*
 * router_device.cuh: the per-row part of the router, shared by the decode router (kernel_router_b200.cu) and the
 * prefill router (kernel_exl3_prefill.cu). One warp a row. Conventions: the reference's router_select_entry
 * (source/kernel_router.cuh:36-119): the picks are the largest affinity + bias; keys order them as its top-k orders
 * float32 (a not-a-number above every number, -0 below +0), the lower expert first among equals; slots in ascending
 * expert order; the weights from the affinities without the bias, their sum from +0 in ascending expert order, every
 * operation one FP32 rounding. The affinity itself is a fixed sequence of FP32 roundings (no library function), so a
 * host restatement reproduces it bit for bit.
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

/* e^a in FP32 by a fixed sequence of single roundings: no function of the mathematics library, so that a host
 * restatement gives the same bits (every operation below is one IEEE rounding; the file is built without fused
 * multiply-adds). Below -104: +0; above 88.75: +infinity. n = rint(a log2 e); r = a - n ln 2 in two steps whose
 * products are exact; a degree-7 polynomial; the scale 2^n as two powers of two, so that only the last product can
 * round (a subnormal result). */
__device__ __forceinline__ float router_power_of_two(int32_t exponent)
{
	return __uint_as_float((uint32_t)(exponent + 127) << 23);
}

__device__ __forceinline__ float router_exponential(float a)
{
	if (a < -104.0f)
		return 0.0f;
	if (a > 88.75f)
		return __uint_as_float(0x7F800000u);
	const float n = rintf(__fmul_rn(a, 1.44269504f));
	float r = __fsub_rn(a, __fmul_rn(n, 0.693359375f));
	r = __fsub_rn(r, __fmul_rn(n, -2.12194440e-4f));
	float p = 1.9875691500e-4f;
	p = __fadd_rn(__fmul_rn(p, r), 1.3981999507e-3f);
	p = __fadd_rn(__fmul_rn(p, r), 8.3334519073e-3f);
	p = __fadd_rn(__fmul_rn(p, r), 4.1665795894e-2f);
	p = __fadd_rn(__fmul_rn(p, r), 1.6666665459e-1f);
	p = __fadd_rn(__fmul_rn(p, r), 5.0000001201e-1f);
	p = __fadd_rn(__fmul_rn(p, __fmul_rn(r, r)), r);
	p = __fadd_rn(p, 1.0f);
	const int32_t whole = (int32_t)n, first = whole >> 1;
	return __fmul_rn(__fmul_rn(p, router_power_of_two(first)), router_power_of_two(whole - first));
}

/* log(1 + t) for 0 <= t <= 1 as 2 atanh(z), z = t / (2 + t) <= 1/3, by nine terms of its series in z^2 */
__device__ __forceinline__ float router_log_one_plus(float t)
{
	const float z = __fdiv_rn(t, __fadd_rn(2.0f, t)), w = __fmul_rn(z, z);
	float p = __fdiv_rn(1.0f, 17.0f);
	p = __fadd_rn(__fmul_rn(p, w), __fdiv_rn(1.0f, 15.0f));
	p = __fadd_rn(__fmul_rn(p, w), __fdiv_rn(1.0f, 13.0f));
	p = __fadd_rn(__fmul_rn(p, w), __fdiv_rn(1.0f, 11.0f));
	p = __fadd_rn(__fmul_rn(p, w), __fdiv_rn(1.0f, 9.0f));
	p = __fadd_rn(__fmul_rn(p, w), __fdiv_rn(1.0f, 7.0f));
	p = __fadd_rn(__fmul_rn(p, w), __fdiv_rn(1.0f, 5.0f));
	p = __fadd_rn(__fmul_rn(p, w), __fdiv_rn(1.0f, 3.0f));
	p = __fadd_rn(__fmul_rn(p, w), 1.0f);
	return __fmul_rn(__fmul_rn(2.0f, z), p);
}

/* The affinity of a router score. SQRT_SOFTPLUS (include/anemone/router_records.h:10-12): sqrt(softplus(s)),
 * softplus(s) = s above 20, else max(s, 0) + log(1 + e^-|s|); SIGMOID: 1 / (1 + e^-s). A not-a-number stays one.
 * Within the reference's own tolerance for a card's affinity (tests/router_reference.h: four last places). */
__device__ __forceinline__ float router_affinity(float score, uint32_t scoring)
{
	if (score != score)
		return score;
	if (scoring == ROUTER_SCORING_SQRT_SOFTPLUS) {
		if (score > 20.0f)
			return __fsqrt_rn(score);
		const float tail = router_log_one_plus(router_exponential(-fabsf(score)));
		return __fsqrt_rn(__fadd_rn(score > 0.0f ? score : 0.0f, tail));
	}
	return __fdiv_rn(1.0f, __fadd_rn(1.0f, router_exponential(-score)));
}

/* One row by one warp: `picks` rounds of a warp-wide maximum over 64-bit keys of affinity + bias (bias may be null:
 * none), as the reference's router_row (source/kernel_router.cuh:47-119); the weights come from the affinities alone.
 * chosen and weight: the row's ROUTER_B200_MAXIMUM_PICKS entries in shared memory, filled by slot; the same values go
 * to picks_out and weights_out (the row's entries in the arena) unless those are null. All 32 lanes call. */
__device__ __forceinline__ void router_row(const float *scores, const float *bias, uint32_t experts, uint32_t picks,
					   uint32_t scoring, float route_scale, uint32_t lane, uint32_t *chosen,
					   float *weight, uint32_t *picks_out, float *weights_out)
{
	uint64_t keys[EXPERTS_PER_LANE];
#pragma unroll
	for (uint32_t place = 0; place < EXPERTS_PER_LANE; place++) {
		const uint32_t expert = place * WARP + lane;
		if (expert < experts) {
			const float affinity = router_affinity(scores[expert], scoring);
			keys[place] = router_key(bias != nullptr ? __fadd_rn(affinity, bias[expert]) : affinity, expert);
		} else {
			keys[place] = 0ull;
		}
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
		if (picks_out != nullptr) {
			picks_out[lane] = chosen[lane];
			weights_out[lane] = value;
		}
	}
	__syncwarp();
}

/* the largest of the warp's keys (0: none), by two 32-bit reductions: the ordered score, then the expert among those
 * that hold it */
__device__ __forceinline__ uint64_t router_warp_largest(uint64_t key)
{
	const uint32_t high = __reduce_max_sync(0xFFFFFFFFu, (uint32_t)(key >> 32));
	const uint32_t low = __reduce_max_sync(0xFFFFFFFFu, (uint32_t)(key >> 32) == high ? (uint32_t)key : 0u);
	return (uint64_t)high << 32 | low;
}

/* One row by a TEAM of ROUTER_TEAM_WARPS warps (member: 0 ..), for a launch whose time is this chain of dependent
 * instructions: every member takes a quarter of the experts (interleaved by runs of 32), finds its `picks` largest
 * keys and leaves them in `candidates` (shared memory, ROUTER_TEAM_WARPS x ROUTER_B200_MAXIMUM_PICKS keys of this row's
 * team); behind the team's barrier (a named barrier `barrier` of the team's threads alone) member 0 picks the
 * largest `picks` of the candidates. The picks are router_row's: the largest keys are the largest keys however they
 * are found; slots, weights and their sum are formed as there. All lanes of all members call. */
#define ROUTER_TEAM_WARPS 4u
#define ROUTER_TEAM_SLOTS (ROUTER_B200_MAXIMUM_EXPERTS / (ROUTER_TEAM_WARPS * WARP))
__device__ __forceinline__ void router_row_team(const float *scores, const float *bias, uint32_t experts, uint32_t picks,
						uint32_t scoring, float route_scale, uint32_t lane, uint32_t member,
						uint32_t barrier, uint64_t *candidates, uint32_t *chosen, float *weight,
						uint32_t *picks_out, float *weights_out)
{
	uint64_t keys[ROUTER_TEAM_SLOTS];
#pragma unroll
	for (uint32_t place = 0; place < ROUTER_TEAM_SLOTS; place++) {
		const uint32_t expert = (place * ROUTER_TEAM_WARPS + member) * WARP + lane;
		if (expert < experts) {
			const float affinity = router_affinity(scores[expert], scoring);
			keys[place] = router_key(bias != nullptr ? __fadd_rn(affinity, bias[expert]) : affinity, expert);
		} else {
			keys[place] = 0ull;
		}
	}
	for (uint32_t pick = 0; pick < picks; pick++) {
		uint64_t best = 0;
#pragma unroll
		for (uint32_t place = 0; place < ROUTER_TEAM_SLOTS; place++)
			best = keys[place] > best ? keys[place] : best;
		best = router_warp_largest(best);
#pragma unroll
		for (uint32_t place = 0; place < ROUTER_TEAM_SLOTS; place++)
			keys[place] = keys[place] == best ? 0ull : keys[place];
		if (lane == pick)
			candidates[member * ROUTER_B200_MAXIMUM_PICKS + pick] = best;
	}
	asm volatile("bar.sync %0, %1;" ::"r"(barrier), "n"(ROUTER_TEAM_WARPS * WARP) : "memory");
	if (member != 0)
		return;
	/* the team's candidates: two a lane */
	uint64_t held[2];
#pragma unroll
	for (uint32_t place = 0; place < 2; place++) {
		const uint32_t index = place * WARP + lane;
		held[place] = index % ROUTER_B200_MAXIMUM_PICKS < picks ? candidates[index] : 0ull;
	}
	uint32_t mine = 0; /* lane p keeps pick p */
	for (uint32_t pick = 0; pick < picks; pick++) {
		const uint64_t best = router_warp_largest(held[0] > held[1] ? held[0] : held[1]);
		held[0] = held[0] == best ? 0ull : held[0];
		held[1] = held[1] == best ? 0ull : held[1];
		if (lane == pick)
			mine = ~(uint32_t)best;
	}
	uint32_t slot = 0; /* the number of picked experts below mine */
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
		if (picks_out != nullptr) {
			picks_out[lane] = chosen[lane];
			weights_out[lane] = value;
		}
	}
	__syncwarp();
}

/* The job table of `live` rows' choices, by one block of any whole number of warps (every thread calls; the block's
 * barriers are passed by all). chosen and weight: [row][ROUTER_B200_MAXIMUM_PICKS] by slot; row_mask and first_job:
 * ROUTER_B200_MAXIMUM_EXPERTS entries of shared memory each. Jobs in ascending expert order, an expert's rows
 * ascending, at most eight rows a job, the always-on experts' jobs behind the routed ones; every other byte of the
 * table zero (include/anemone/router_records.h:20-26). The only atomic is an OR into a shared-memory bit mask, whose
 * result does not depend on order. job_count_out (may be null): where the number of non-empty jobs goes. */
__device__ __forceinline__ void router_job_table(uint32_t live, uint32_t experts, uint32_t picks, uint32_t shared,
						 uint32_t job_capacity,
						 const uint32_t (*chosen)[ROUTER_B200_MAXIMUM_PICKS],
						 const float (*weight)[ROUTER_B200_MAXIMUM_PICKS],
						 unsigned long long *row_mask, uint32_t *first_job,
						 struct expert_job_record *jobs, const uint64_t *offsets,
						 uint32_t *job_count_out)
{
	const uint32_t lane = threadIdx.x % WARP, warp = threadIdx.x / WARP;
	/* every byte of the job table starts zero */
	uint4 *const table = reinterpret_cast<uint4 *>(jobs);
	for (uint32_t index = threadIdx.x; index < job_capacity * (uint32_t)(sizeof(struct expert_job_record) / 16u);
	     index += blockDim.x)
		table[index] = make_uint4(0, 0, 0, 0);
	for (uint32_t expert = threadIdx.x; expert < ROUTER_B200_MAXIMUM_EXPERTS; expert += blockDim.x)
		row_mask[expert] = 0ull;
	__syncthreads();
	/* which rows chose each expert: a 64-bit mask per expert, then the first job of every expert by a warp-wide
	 * prefix sum over the experts' job counts */
	for (uint32_t pair = threadIdx.x; pair < live * picks; pair += blockDim.x)
		atomicOr(&row_mask[chosen[pair / picks][pair % picks]], 1ull << (pair / picks));
	__syncthreads();
	if (warp == 0) {
		const unsigned long long everyone = live >= 64u ? ~0ull : (1ull << live) - 1ull;
		uint32_t local[EXPERTS_PER_LANE], total = 0;
#pragma unroll
		for (uint32_t place = 0; place < EXPERTS_PER_LANE; place++) {
			const uint32_t expert = lane * EXPERTS_PER_LANE + place;
			const uint32_t rows = expert < experts	       ? (uint32_t)__popcll(row_mask[expert]) :
					      expert < experts + shared ? live :
									  0u;
			if (expert >= experts && expert < experts + shared)
				row_mask[expert] = everyone;
			local[place] = total;
			total += (rows + LINEAR_MAXIMUM_ROWS - 1u) / LINEAR_MAXIMUM_ROWS;
		}
		uint32_t before = total; /* inclusive scan over the lanes, then made exclusive */
		for (uint32_t distance = 1; distance < WARP; distance <<= 1) {
			const uint32_t other = __shfl_up_sync(0xFFFFFFFFu, before, distance);
			if (lane >= distance)
				before += other;
		}
		if (lane == WARP - 1u && job_count_out != nullptr)
			*job_count_out = before < job_capacity ? before : job_capacity;
		before -= total;
#pragma unroll
		for (uint32_t place = 0; place < EXPERTS_PER_LANE; place++)
			first_job[lane * EXPERTS_PER_LANE + place] = before + local[place];
	}
	__syncthreads();
	/* a thread a pair: its place among its expert's rows decides its job and column */
	const uint32_t pairs_per_row = picks + shared;
	for (uint32_t pair = threadIdx.x; pair < live * pairs_per_row; pair += blockDim.x) {
		const uint32_t row = pair / pairs_per_row, slot = pair % pairs_per_row;
		const uint32_t expert = slot < picks ? chosen[row][slot] : experts + (slot - picks);
		const unsigned long long mask = row_mask[expert];
		const uint32_t place = (uint32_t)__popcll(mask & ((1ull << row) - 1ull)); /* rows below mine in the expert */
		const uint32_t job_index = first_job[expert] + place / LINEAR_MAXIMUM_ROWS;
		if (job_index >= job_capacity)
			continue;
		struct expert_job_record *const job = &jobs[job_index];
		const uint32_t column = place % LINEAR_MAXIMUM_ROWS;
		job->pair_index[column] = pair;
		job->route_weight[column] = slot < picks ? weight[row][slot] : 1.0f;
		if (column == 0) {
			const uint32_t remaining = (uint32_t)__popcll(mask) - place;
			job->gate_offset = offsets[3u * expert];
			job->up_offset = offsets[3u * expert + 1u];
			job->down_offset = offsets[3u * expert + 2u];
			job->expert = expert;
			job->row_count = remaining < LINEAR_MAXIMUM_ROWS ? remaining : LINEAR_MAXIMUM_ROWS;
		}
	}
}

#endif
