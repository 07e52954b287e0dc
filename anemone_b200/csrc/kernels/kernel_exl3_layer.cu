/*
 * kernel_exl3_layer.cu: one decode step of a rank's expert layer in four launches (struct exl3_layer_route_record,
 * struct exl3_moe_record; the fourth launch is ordered_publish_reduce_flags of kernel_ordered_b200.cu). No counterpart file in the reference, whose step is a router launch, five expert launches,
 * a row sum and an exchange of one CTA; the arithmetic of every value is its retained chain's (exl3_passes.cuh), the
 * router's conventions its router_select_entry's (router_device.cuh), the reduction's order its owner sums'.
 *
 * The two product launches are the fused products of the fixed cut (exl3_fused.cuh) with a cut the preparer chooses
 * for the step's size and the rank's share of the columns (the grid tells it): a CTA streams one run of K of 128
 * outputs of one job; the runs leave FP32 partial sums in the arena and the CTA that completes a (job, 128 outputs),
 * found with a counter, adds them in ascending K order from +0. The cut depends on the prepared shapes alone.
 */
#include "exl3_fused.cuh"
#include "router_device.cuh"

#define EXL3_LAYER_READY_POLLS 2048u /* of about 200 ns each, before a down CTA waits for the whole launch before it */

__device__ __forceinline__ uint32_t *layer_words(const struct exl3_moe_record &moe, unsigned char *arena)
{
	return reinterpret_cast<uint32_t *>(arena + moe.counters_offset) +
	       exl3_layer_counter_begin(moe.base.job_count, moe.base.input_size, moe.base.inner_size);
}

/* ------------------------------------------------------------------ router and input transform */

extern "C" __global__ void __launch_bounds__(EXL3_LAYER_ROUTE_THREADS)
	exl3_layer_route_input(struct exl3_layer_route_record record, unsigned char *arena)
{
	__shared__ uint32_t chosen[ROUTER_B200_MAXIMUM_ROWS][ROUTER_B200_MAXIMUM_PICKS]; /* by slot */
	__shared__ float weight[ROUTER_B200_MAXIMUM_ROWS][ROUTER_B200_MAXIMUM_PICKS];
	__shared__ unsigned long long row_mask[ROUTER_B200_MAXIMUM_EXPERTS];
	__shared__ uint32_t first_job[ROUTER_B200_MAXIMUM_EXPERTS];
	const struct exl3_expert_record &base = record.moe.base;
	/* the gate/up launch may take its place on the card now: it waits for the whole of this launch before it reads */
	asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
	const struct step_block step = *reinterpret_cast<const struct step_block *>(arena + record.step_offset);
	const uint32_t live = min(step.row_count, record.row_capacity);
	const uint32_t routed = record.routed_count, picks = record.picks, shared = record.shared_count;
	const uint32_t lane = threadIdx.x % WARP, warp = threadIdx.x / WARP, warps = blockDim.x / WARP;
	const bool writer = blockIdx.x == 0;
	const float *const scores = reinterpret_cast<const float *>(arena + record.scores_offset);
	const float *const bias =
		record.bias_offset != 0 ? reinterpret_cast<const float *>(arena + record.bias_offset) : nullptr;
	/* every CTA chooses every live row's experts itself: the same arithmetic, the same picks */
	for (uint32_t row = warp; row < live; row += warps)
		router_row(scores + (uint64_t)row * routed, bias, routed, picks, record.scoring, record.route_scale, lane,
			   chosen[row], weight[row],
			   writer ? reinterpret_cast<uint32_t *>(arena + record.picks_offset) + (uint64_t)row * picks : nullptr,
			   writer ? reinterpret_cast<float *>(arena + record.weights_offset) + (uint64_t)row * picks : nullptr);
	__syncthreads();
	const uint64_t *const table = reinterpret_cast<const uint64_t *>(arena + record.expert_table_offset);
	if (writer) {
		uint32_t *const words = layer_words(record.moe, arena);
		for (uint32_t job = threadIdx.x; job < base.job_count; job += blockDim.x)
			words[EXL3_LAYER_COUNTER_WORDS + job] = 0u; /* no job's down operands are in place yet */
		router_job_table(live, routed, picks, shared, base.job_count, chosen, weight, row_mask, first_job,
				 reinterpret_cast<struct expert_job_record *>(arena + base.jobs_offset), table,
				 &words[EXL3_LAYER_WORD_LIVE_JOBS]);
		return;
	}
	/* the others: a warp a (pair, gate or up, block of 128 inputs): x . suh, Hadamard, FP16 operand */
	const uint32_t H = base.input_size, blocks = H / EXL3_TRANSFORM, slots = picks + shared;
	const uint32_t tasks = live * slots * EXL3_PROJECTIONS * blocks;
	const uint32_t *const widths = moe_widths(record.moe, arena);
	const __nv_bfloat16 *const input = reinterpret_cast<const __nv_bfloat16 *>(arena + base.input_offset);
	__half *const operands = reinterpret_cast<__half *>(arena + base.operands_offset);
	for (uint32_t task = (blockIdx.x - 1u) * warps + warp; task < tasks; task += (gridDim.x - 1u) * warps) {
		const uint32_t block = task % blocks, projection = task / blocks % EXL3_PROJECTIONS;
		const uint32_t pair = task / (blocks * EXL3_PROJECTIONS), row = pair / slots, slot = pair % slots;
		const uint32_t expert = slot < picks ? chosen[row][slot] : routed + (slot - picks);
		const uint32_t bits_x2 = exl3_bits_x2(widths != nullptr ? widths[expert] : base.bits_per_weight);
		const uint32_t channel = block * EXL3_TRANSFORM + lane * 4u;
		float scale[4];
		load_half4(reinterpret_cast<const __half *>(arena + table[3u * expert + projection] +
							    exl3_code_bytes(H, base.inner_size, bits_x2)) +
				   channel,
			   scale);
		const uint2 raw = *reinterpret_cast<const uint2 *>(input + (uint64_t)row * H + channel);
		float v[4] = { __uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xFFFF0000u),
			       __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xFFFF0000u) };
#pragma unroll
		for (uint32_t i = 0; i < 4; i++)
			v[i] = __fmul_rn(v[i], scale[i]);
		hadamard128_warp(v, lane);
#pragma unroll
		for (uint32_t i = 0; i < 4; i++)
			v[i] = __fmul_rn(v[i], EXL3_NORMALIZATION);
		store_half4(operands + ((uint64_t)projection * base.pair_count + pair) * H + channel, v);
	}
}

/* ------------------------------------------------------------------ gate/up products */

/* grid (inner_size / 128 * runs, jobs, 2) x 128: exl3_moe_gate_up's CTAs with the cut of K the preparer chose
 * (gridDim.x tells it) */
extern "C" __global__ void __launch_bounds__(EXL3_PRODUCT_THREADS)
	exl3_layer_gate_up(struct exl3_moe_record record, unsigned char *arena)
{
	extern __shared__ __align__(128) unsigned char dynamic_shared[];
	__shared__ exl3_product_shared shared;
	__shared__ uint32_t flag;
	/* This launch may have begun while the router's still runs: everything it reads is that launch's, so it waits for
	 * the whole of it. Only then may the down launch be given the card's free room (once every CTA of this grid has
	 * said so or ended, which is when the last of them has begun): its CTAs read the job table, which must be this
	 * step's, and wait for their job's operands themselves. */
	asm volatile("griddepcontrol.wait;" ::: "memory");
	asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
	exl3_moe_gate_up_block(record, arena, gridDim.x / (record.base.inner_size / EXL3_TRANSFORM), dynamic_shared, &shared,
			       &flag, layer_words(record, arena) + EXL3_LAYER_COUNTER_WORDS);
}

/* ------------------------------------------------------------------ down products */

/* grid (input_size / 128 * runs, jobs) x 128: exl3_moe_down's CTAs with the cut the preparer chose */
extern "C" __global__ void __launch_bounds__(EXL3_PRODUCT_THREADS)
	exl3_layer_down(struct exl3_moe_record record, unsigned char *arena)
{
	extern __shared__ __align__(128) unsigned char dynamic_shared[];
	__shared__ exl3_product_shared shared;
	__shared__ uint32_t flag;
	/* This launch may have begun while the gate/up launch still runs. The job table is older than both; the job's
	 * down operands are in place once every group of its inner channels has been counted. A CTA looks for that a
	 * bounded number of times, then waits for the whole gate/up launch (which is all a launch that began behind it
	 * does anyway): it cannot wait in vain. */
	asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); /* the reduction's launch waits for all of this one */
	if (exl3_job(record.base, arena, blockIdx.y)->row_count == 0)
		return;
	if (threadIdx.x == 0) {
		const uint32_t *const ready = layer_words(record, arena) + EXL3_LAYER_COUNTER_WORDS + blockIdx.y;
		const uint32_t wanted = record.base.inner_size / EXL3_TRANSFORM;
		uint32_t seen = 0;
		for (uint32_t poll = 0; poll < EXL3_LAYER_READY_POLLS; poll++) {
			asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(ready) : "memory");
			if (seen == wanted)
				break;
			__nanosleep(200);
		}
		if (seen != wanted)
			asm volatile("griddepcontrol.wait;" ::: "memory");
	}
	__syncthreads();
	exl3_moe_down_block(record, arena, gridDim.x / (record.base.input_size / EXL3_TRANSFORM), dynamic_shared, &shared,
			    &flag);
}
