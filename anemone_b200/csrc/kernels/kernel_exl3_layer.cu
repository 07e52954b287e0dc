/*
 * kernel_exl3_layer.cu: one decode step of a rank's expert layer in three launches (struct exl3_layer_route_record,
 * struct exl3_layer_products_record; the third launch is ordered_publish_reduce_flags of kernel_ordered_b200.cu). No
 * counterpart file in the reference, whose step is a router launch, five expert launches, a row sum and an exchange of
 * one CTA; the arithmetic of every value is its retained chain's (exl3_passes.cuh), the router's conventions its
 * router_select_entry's (router_device.cuh), the reduction's order its owner sums'.
 *
 * The products are one launch. The step's work is a list of items of the fused products of the fixed cut
 * (exl3_fused.cuh): one run of K of 128 outputs of one matrix of one job; the runs leave FP32 partial sums in the
 * arena and the CTA that completes a (job, 128 outputs), found with a counter, adds them in ascending K order from +0.
 * Gate and up items come first, in job order, then the down items, which wait for their job's activation; a CTA takes
 * the next item of the list when it begins. The cut depends on the prepared shapes alone, and so does every sum: which
 * CTA computes an item, and when, does not matter to its bits.
 */
#include "exl3_fused.cuh"
#include "router_device.cuh"

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
	__shared__ uint64_t candidates[EXL3_LAYER_ROUTE_THREADS / WARP / ROUTER_TEAM_WARPS]
				      [ROUTER_TEAM_WARPS * ROUTER_B200_MAXIMUM_PICKS];
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
	/* every CTA chooses every live row's experts itself (the same arithmetic, the same picks), a team of four warps
	 * a row: the launch lasts as long as one row's chain of dependent instructions */
	const uint32_t team = warp / ROUTER_TEAM_WARPS, teams = warps / ROUTER_TEAM_WARPS;
	for (uint32_t first = 0; first < live; first += teams) { /* a whole team leaves the loop together */
		const uint32_t row = first + team;
		if (row < live)
			router_row_team(scores + (uint64_t)row * routed, bias, routed, picks, record.scoring, record.route_scale,
					lane, warp % ROUTER_TEAM_WARPS, 1u + team, candidates[team], chosen[row], weight[row],
					writer ? reinterpret_cast<uint32_t *>(arena + record.picks_offset) + (uint64_t)row * picks :
						 nullptr,
					writer ? reinterpret_cast<float *>(arena + record.weights_offset) + (uint64_t)row * picks :
						 nullptr);
	}
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

/* ------------------------------------------------------------------ the products */

/* one thread: true once *word == wanted, false after EXL3_WAIT_CYCLES (the expiry is recorded) */
__device__ __forceinline__ bool layer_word_wait(const uint32_t *word, uint32_t wanted)
{
	long long begun = 0;
	for (uint32_t poll = 1;; poll++) {
		uint32_t seen;
		asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(word) : "memory");
		if (seen == wanted)
			return true;
		if ((poll & 63u) == 0u) {
			const long long now = clock64();
			if (begun == 0)
				begun = now;
			else if (now - begun > EXL3_WAIT_CYCLES)
				break;
		}
		__nanosleep(100);
	}
	atomicExch(&exl3_wait_expired, 1u);
	return false;
}

/* grid (job_count * items a job) x 128: a CTA an item. A CTA takes a ticket as its first act and works on the item of
 * that number: the gate and up items of every live job in job order, then the down items (tickets beyond the step's
 * items end at once). Tickets are handed out in the order the CTAs begin, so every gate/up item has begun before any
 * down item begins; a down item's CTA waits for its job's word to reach the number of groups of inner channels, which
 * the gate/up items count up without waiting for anything, so the wait ends. It is bounded all the same: an item whose
 * wait ran out is skipped and the host finds exl3_wait_expired set. The card hands a freed place to the next CTA, so
 * its room is filled to the last item whatever the step's size. (A grid that walks the items in a loop keeps the
 * loop's words alive through the products and spills: a CTA an item does not.) */
extern "C" __global__ void __launch_bounds__(EXL3_PRODUCT_THREADS)
	exl3_layer_products(struct exl3_layer_products_record record, unsigned char *arena)
{
	extern __shared__ __align__(128) unsigned char dynamic_shared[];
	__shared__ exl3_product_shared shared;
	__shared__ uint32_t flag;
	__shared__ struct moe_item taken; /* the CTA's item; job UINT32_MAX: none */
	__shared__ uint32_t kind; /* 0: gate or up, 1: down, 2: a down item whose wait ran out */
	/* This launch may have been given its place while the router's still runs: everything it reads is that launch's,
	 * so it waits for the whole of it; the reduction's launch may then take its place behind this one. */
	asm volatile("griddepcontrol.wait;" ::: "memory");
	asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
	const struct exl3_moe_record &moe = record.moe;
	if (threadIdx.x == 0) {
		/* one thread takes the ticket and finds its item (the divisions are its alone), and waits where the item must */
		uint32_t *const words = layer_words(moe, arena);
		const uint32_t index = atomicAdd(&words[EXL3_LAYER_WORD_TICKET], 1u);
		if (index == gridDim.x - 1u)
			words[EXL3_LAYER_WORD_TICKET] = 0u; /* the last one: the word is zero again for the next step */
		const uint32_t jobs = min(words[EXL3_LAYER_WORD_LIVE_JOBS], moe.base.job_count);
		const uint32_t inner_groups = moe.base.inner_size / EXL3_TRANSFORM;
		const uint32_t gate_up_a_matrix = inner_groups * record.gate_up_runs;
		const uint32_t gate_up_a_job = EXL3_PROJECTIONS * gate_up_a_matrix;
		const uint32_t down_a_job = moe.base.input_size / EXL3_TRANSFORM * record.down_runs;
		const uint32_t gate_up_items = jobs * gate_up_a_job, items = gate_up_items + jobs * down_a_job;
		struct moe_item item = { UINT32_MAX, 0u, 0u, 0u };
		uint32_t what = 0;
		if (index < gate_up_items) {
			const uint32_t within = index % gate_up_a_job, of_matrix = within % gate_up_a_matrix;
			item.job = index / gate_up_a_job;
			item.group = of_matrix / record.gate_up_runs;
			item.run = of_matrix % record.gate_up_runs;
			item.projection = within / gate_up_a_matrix;
		} else if (index < items) {
			const uint32_t behind = index - gate_up_items, within = behind % down_a_job;
			item.job = behind / down_a_job;
			item.group = within / record.down_runs;
			item.run = within % record.down_runs;
			what = layer_word_wait(words + EXL3_LAYER_COUNTER_WORDS + item.job, inner_groups) ? 1u : 2u;
		}
		taken = item;
		kind = what;
	}
	__syncthreads();
	/* through a lane's register, so that the compiler knows every lane of a warp holds the same item (what depends on
	 * it then lives in the warp's uniform registers, not in every lane's) */
	const struct moe_item item = { (uint32_t)__shfl_sync(0xFFFFFFFFu, taken.job, 0),
				       (uint32_t)__shfl_sync(0xFFFFFFFFu, taken.group, 0),
				       (uint32_t)__shfl_sync(0xFFFFFFFFu, taken.run, 0),
				       (uint32_t)__shfl_sync(0xFFFFFFFFu, taken.projection, 0) };
	const uint32_t what = (uint32_t)__shfl_sync(0xFFFFFFFFu, kind, 0);
	if (item.job == UINT32_MAX || what == 2u)
		return;
	if (what == 0u) {
		exl3_moe_gate_up_item(moe, arena, item, record.gate_up_runs, dynamic_shared, &shared, &flag,
				      layer_words(moe, arena) + EXL3_LAYER_COUNTER_WORDS);
		return;
	}
	exl3_moe_down_item(moe, arena, item, record.down_runs, dynamic_shared, &shared, &flag,
				   record.down_products_offset);
}
