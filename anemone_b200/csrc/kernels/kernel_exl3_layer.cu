/*
 * kernel_exl3_layer.cu: one decode step of a rank's expert layer in four launches (struct exl3_layer_route_record,
 * struct exl3_moe_record, struct exl3_layer_down_record; the fourth launch is ordered_reduce_flags of
 * kernel_ordered_b200.cu). No counterpart file in the reference, whose step is a router launch, five expert launches,
 * a row sum and an exchange of one CTA; the arithmetic of every value is its retained chain's (exl3_passes.cuh), the
 * router's conventions its router_select_entry's (router_device.cuh), the reduction's order its owner sums'.
 *
 * The two product launches treat the step's live (job, matrix, 128 outputs) items as ONE sequence of K rounds and cut
 * it in gridDim.x equal runs: a CTA streams its run, which may end one item and begin the next. Every SM therefore
 * has the same work whatever the number of live experts and however few columns a rank holds, and a CTA's set-up is
 * paid once per run instead of once per short item. An item's runs leave FP32 partial sums in the arena; the CTA that
 * completes the item (found with a counter) adds them in ascending K order from +0. The cut depends on the live job
 * count and the grid alone.
 */
#include "exl3_fused.cuh"
#include "ordered_device.cuh"
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
	const struct exl3_expert_record &base = record.moe.base;
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
		router_job_table(live, routed, picks, shared, base.job_count, chosen, weight, row_mask, first_job,
				 reinterpret_cast<struct expert_job_record *>(arena + base.jobs_offset), table,
				 &words[EXL3_LAYER_WORD_LIVE_JOBS]);
		if (threadIdx.x == 0)
			words[EXL3_LAYER_WORD_FAILED] = 0u;
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

/* ------------------------------------------------------------------ products: one sequence of rounds, cut evenly */

struct layer_run {
	uint32_t item; /* of the launch's live items */
	uint32_t round_begin, round_count; /* of the item's rounds */
	uint32_t index; /* of this run among the item's runs, in ascending K order */
};

/* runs the sequence's cut leaves of an item: the CTAs whose rounds meet the item's */
__device__ __forceinline__ uint32_t layer_runs_of(uint32_t item, uint32_t item_rounds, uint32_t quantum)
{
	return (item * item_rounds + item_rounds - 1u) / quantum - item * item_rounds / quantum + 1u;
}

template <uint32_t BX2>
__device__ __noinline__ void layer_gate_up_run(const struct exl3_moe_record &moe, unsigned char *arena,
						  const struct expert_job_record *job, uint32_t job_index,
						  uint32_t projection, uint32_t group, const struct layer_run &run,
						  uint32_t gate_runs, uint32_t up_runs, unsigned char *dynamic_shared,
						  exl3_product_shared *shared, uint32_t *flag)
{
	const struct exl3_expert_record &record = moe.base;
	const uint32_t lane = threadIdx.x % EXL3_WARP;
	const uint32_t H = record.input_size, I = record.inner_size, pairs = record.pair_count;
	const uint32_t fed_column = lane / 4u < job->row_count ? lane / 4u : 0u;
	const __half *const operands = reinterpret_cast<const __half *>(arena + record.operands_offset);
	float sums[2][4];
	if (!exl3_product_core<BX2>(arena + (projection == 0 ? job->gate_offset : job->up_offset), I, group,
				    run.round_begin * EXL3_STAGE_STEPS, run.round_count * EXL3_STAGE_STEPS,
				    operands + ((uint64_t)projection * pairs + job->pair_index[fed_column]) * H,
				    dynamic_shared, shared, sums))
		return;
	/* partial sums: FP32 [projection][EXL3_LAYER_MAXIMUM_RUNS][pair][I] */
	float *const partials = reinterpret_cast<float *>(arena + record.products_offset);
	const uint64_t run_stride = (uint64_t)pairs * I;
	float *rows[LINEAR_MAXIMUM_ROWS];
#pragma unroll
	for (uint32_t column = 0; column < LINEAR_MAXIMUM_ROWS; column++)
		rows[column] = partials + ((uint64_t)projection * EXL3_LAYER_MAXIMUM_RUNS + run.index) * run_stride +
			       (uint64_t)job->pair_index[column < job->row_count ? column : 0u] * I + group * EXL3_TRANSFORM;
	store_partial(sums, rows, job->row_count);
	uint32_t *const counter =
		reinterpret_cast<uint32_t *>(arena + moe.counters_offset) + job_index * (I / EXL3_TRANSFORM) + group;
	if (!last_of(counter, gate_runs + up_runs, flag))
		return;
	exl3_gate_up_epilogue<BX2>(moe, arena, job, group, partials,
				   partials + (uint64_t)EXL3_LAYER_MAXIMUM_RUNS * run_stride, run_stride, gate_runs, up_runs);
}

/* true in the one CTA that completed the item (it has written the pair outputs) */
template <uint32_t BX2>
__device__ __noinline__ bool layer_down_run(const struct exl3_moe_record &moe, unsigned char *arena,
					       const struct expert_job_record *job, uint32_t job_index, uint32_t group,
					       const struct layer_run &run, uint32_t runs, unsigned char *dynamic_shared,
					       exl3_product_shared *shared, uint32_t *flag)
{
	const struct exl3_expert_record &record = moe.base;
	const uint32_t lane = threadIdx.x % EXL3_WARP;
	const uint32_t H = record.input_size, I = record.inner_size, pairs = record.pair_count;
	const uint32_t fed_column = lane / 4u < job->row_count ? lane / 4u : 0u;
	const __half *const operands =
		reinterpret_cast<const __half *>(arena + record.operands_offset) + (uint64_t)EXL3_PROJECTIONS * pairs * H;
	float sums[2][4];
	if (!exl3_product_core<BX2>(arena + job->down_offset, H, group, run.round_begin * EXL3_STAGE_STEPS,
				    run.round_count * EXL3_STAGE_STEPS, operands + (uint64_t)job->pair_index[fed_column] * I,
				    dynamic_shared, shared, sums))
		return false;
	/* partial sums: FP32 [EXL3_LAYER_MAXIMUM_RUNS][pair][H]; run 0's rows are also where the pair outputs go */
	float *const partials = reinterpret_cast<float *>(arena + record.products_offset);
	const uint64_t run_stride = (uint64_t)pairs * H;
	float *rows[LINEAR_MAXIMUM_ROWS];
#pragma unroll
	for (uint32_t column = 0; column < LINEAR_MAXIMUM_ROWS; column++)
		rows[column] = partials + run.index * run_stride +
			       (uint64_t)job->pair_index[column < job->row_count ? column : 0u] * H + group * EXL3_TRANSFORM;
	store_partial(sums, rows, job->row_count);
	uint32_t *const counter = reinterpret_cast<uint32_t *>(arena + moe.counters_offset) +
				  (uint64_t)record.job_count * (I / EXL3_TRANSFORM) + job_index * (H / EXL3_TRANSFORM) + group;
	if (!last_of(counter, runs, flag))
		return false;
	exl3_down_epilogue<BX2>(moe, arena, job, group, partials, run_stride, runs);
	return true;
}

/* This CTA's runs of the sequence of `items` items of item_rounds rounds each: calls body(run) for each in order. */
template <typename BODY>
__device__ __forceinline__ void layer_for_each_run(uint32_t items, uint32_t item_rounds, uint32_t quantum, BODY body)
{
	const uint32_t total = items * item_rounds;
	const uint32_t begin = blockIdx.x * quantum;
	if (begin >= total)
		return;
	const uint32_t end = min(begin + quantum, total);
	for (uint32_t position = begin; position < end;) {
		struct layer_run run;
		run.item = position / item_rounds;
		run.round_begin = position % item_rounds;
		run.round_count = min(item_rounds - run.round_begin, end - position);
		run.index = blockIdx.x - run.item * item_rounds / quantum;
		body(run);
		position += run.round_count;
	}
}

#define LAYER_WIDTH_SWITCH(bits_x2, call)               \
	switch (bits_x2) {                              \
	case EXL3_BITS_X2_K2: {                         \
		constexpr uint32_t BX2 = EXL3_BITS_X2_K2;   \
		call;                                   \
		break;                                  \
	}                                               \
	case EXL3_BITS_X2_K2_5: {                       \
		constexpr uint32_t BX2 = EXL3_BITS_X2_K2_5; \
		call;                                   \
		break;                                  \
	}                                               \
	case EXL3_BITS_X2_K3: {                         \
		constexpr uint32_t BX2 = EXL3_BITS_X2_K3;   \
		call;                                   \
		break;                                  \
	}                                               \
	case EXL3_BITS_X2_K4: {                         \
		constexpr uint32_t BX2 = EXL3_BITS_X2_K4;   \
		call;                                   \
		break;                                  \
	}                                               \
	default:                                        \
		break;                                  \
	}

extern "C" __global__ void __launch_bounds__(EXL3_PRODUCT_THREADS, EXL3_LAYER_PRODUCT_CTAS_PER_SM)
	exl3_layer_gate_up(struct exl3_moe_record record, unsigned char *arena)
{
	extern __shared__ __align__(128) unsigned char dynamic_shared[];
	__shared__ exl3_product_shared shared;
	__shared__ uint32_t flag;
	const uint32_t live_jobs = min(layer_words(record, arena)[EXL3_LAYER_WORD_LIVE_JOBS], record.base.job_count);
	const uint32_t groups = record.base.inner_size / EXL3_TRANSFORM;
	const uint32_t item_rounds = exl3_layer_item_rounds(record.base.input_size);
	const uint32_t items = live_jobs * EXL3_PROJECTIONS * groups;
	const uint32_t quantum = exl3_layer_quantum(items * item_rounds, item_rounds, gridDim.x);
	const uint32_t *const widths = moe_widths(record, arena);
	layer_for_each_run(items, item_rounds, quantum, [&](const struct layer_run &run) {
		/* items: job-major, then gate and up, then the group of 128 outputs */
		const uint32_t group = run.item % groups, projection = run.item / groups % EXL3_PROJECTIONS;
		const uint32_t job_index = run.item / (groups * EXL3_PROJECTIONS);
		const struct expert_job_record *const job = exl3_job(record.base, arena, job_index);
		if (job->row_count == 0)
			return;
		const uint32_t gate_item = (job_index * EXL3_PROJECTIONS) * groups + group;
		const uint32_t gate_runs = layer_runs_of(gate_item, item_rounds, quantum);
		const uint32_t up_runs = layer_runs_of(gate_item + groups, item_rounds, quantum);
		LAYER_WIDTH_SWITCH(exl3_job_bits_x2(record.base, job, widths),
				   layer_gate_up_run<BX2>(record, arena, job, job_index, projection, group, run, gate_runs,
							  up_runs, dynamic_shared, &shared, &flag))
	});
}

/* ------------------------------------------------------------------ down, row sums into the slot, READY to everyone */

__device__ __forceinline__ unsigned char *layer_slot(const struct exl3_layer_publish_arguments &publish,
						     unsigned char *arena, uint32_t rank, uint64_t sequence)
{
	unsigned char *region;
	if (rank == publish.rank) {
		region = arena + publish.region_offset;
	} else {
		const struct ordered_collective_peer *const peers =
			reinterpret_cast<const struct ordered_collective_peer *>(arena + publish.peer_table_offset);
		region = reinterpret_cast<unsigned char *>(peers[rank].arena_address) + peers[rank].region_offset;
	}
	return region + (sequence & 1u) * publish.parity_stride;
}

/* The CTA that completed a group of 128 columns over all live jobs: this rank's row sums of the group (slots added
 * from +0 in ascending order) into its rows of the slot, once every rank has said it is done with the slot's
 * previous use (their DONE words arrive in this rank's own memory); the CTA that completes the last group stores
 * READY into every rank's slot. A wait that runs out sets the status block and the failed word: nothing is published
 * and the peers' own deadlines report it. All 128 threads call. */
__device__ __forceinline__ void layer_publish_group(const struct exl3_layer_down_record &record, unsigned char *arena,
						    uint32_t group, uint32_t live_rows, uint64_t sequence, uint32_t *flag)
{
	const struct exl3_layer_publish_arguments &publish = record.publish;
	const struct exl3_expert_record &base = record.moe.base;
	const uint32_t lane = threadIdx.x % EXL3_WARP, warp = threadIdx.x / EXL3_WARP;
	uint32_t *const words = layer_words(record.moe, arena);
	unsigned char *const mine = layer_slot(publish, arena, publish.rank, sequence);
	unsigned char *const local = mine + EXL3_LAYER_LOCAL_LINE * ORDERED_COLLECTIVE_LINE_BYTES;
	unsigned char *const status = arena + publish.status_offset;
	const uint64_t previous = *reinterpret_cast<const volatile uint64_t *>(local + ORDERED_LOCAL_PREVIOUS_OFFSET);
	if (threadIdx.x == 0)
		*flag = 1u;
	__syncthreads();
	if (previous >= sequence) {
		if (threadIdx.x == 0) {
			ordered_status_set(status, ORDERED_STATUS_BAD_SEQUENCE, ORDERED_READY_PHASE, publish.rank);
			*flag = 0u;
		}
	} else if (previous != 0 && threadIdx.x < publish.rank_count) {
		const unsigned char *const line =
			mine + (EXL3_LAYER_DONE_LINE + threadIdx.x) * ORDERED_COLLECTIVE_LINE_BYTES;
		const long long begin = clock64();
		while (signal_load(line) < previous) {
			if ((uint64_t)(clock64() - begin) > publish.deadline_cycles) {
				ordered_status_set(status, ORDERED_STATUS_TIMED_OUT, ORDERED_DONE_PHASE, threadIdx.x);
				atomicExch(flag, 0u);
				break;
			}
			__nanosleep(100);
		}
	}
	__syncthreads();
	const bool alive = *flag != 0u;
	if (alive) {
		const uint32_t H = base.input_size, slots = base.pairs_per_row;
		const float *const pairs = reinterpret_cast<const float *>(arena + base.output_offset);
		float *const rows = reinterpret_cast<float *>(mine + publish.input_offset);
		const uint32_t channel = group * EXL3_TRANSFORM + lane * 4u;
		for (uint32_t row = warp; row < live_rows; row += EXL3_PRODUCT_WARPS) {
			float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
			for (uint32_t slot = 0; slot < slots; slot++) {
				const float4 value = __ldcg(
					reinterpret_cast<const float4 *>(pairs + ((uint64_t)row * slots + slot) * H + channel));
				sum.x = __fadd_rn(sum.x, value.x);
				sum.y = __fadd_rn(sum.y, value.y);
				sum.z = __fadd_rn(sum.z, value.z);
				sum.w = __fadd_rn(sum.w, value.w);
			}
			*reinterpret_cast<float4 *>(rows + (uint64_t)row * H + channel) = sum;
		}
	} else if (threadIdx.x == 0) {
		atomicExch(&words[EXL3_LAYER_WORD_FAILED], 1u);
	}
	if (!last_of(&words[EXL3_LAYER_WORD_GROUPS_DONE], base.input_size / EXL3_TRANSFORM, flag))
		return;
	if (atomicAdd(&words[EXL3_LAYER_WORD_FAILED], 0u) != 0u)
		return;
	if (threadIdx.x == 0)
		*reinterpret_cast<volatile uint64_t *>(local + ORDERED_LOCAL_PREVIOUS_OFFSET) = sequence;
	if (threadIdx.x < publish.rank_count) {
		__threadfence_system();
		signal_store(layer_slot(publish, arena, threadIdx.x, sequence) +
				     (EXL3_LAYER_READY_LINE + publish.rank) * ORDERED_COLLECTIVE_LINE_BYTES,
			     sequence);
	}
}

extern "C" __global__ void __launch_bounds__(EXL3_PRODUCT_THREADS, EXL3_LAYER_PRODUCT_CTAS_PER_SM)
	exl3_layer_down_publish(struct exl3_layer_down_record record, unsigned char *arena)
{
	extern __shared__ __align__(128) unsigned char dynamic_shared[];
	__shared__ exl3_product_shared shared;
	__shared__ uint32_t flag;
	const struct exl3_moe_record &moe = record.moe;
	const struct step_block step = *reinterpret_cast<const struct step_block *>(arena + record.publish.step_offset);
	uint32_t *const words = layer_words(moe, arena);
	const uint32_t live_jobs = min(words[EXL3_LAYER_WORD_LIVE_JOBS], moe.base.job_count);
	const uint32_t live_rows = min(step.row_count, record.publish.row_capacity);
	const uint32_t groups = moe.base.input_size / EXL3_TRANSFORM;
	if (live_jobs == 0) {
		/* no live row: nothing to add, but the ranks still meet in the reduction */
		if (blockIdx.x < groups && step.sequence != 0)
			layer_publish_group(record, arena, blockIdx.x, 0u, step.sequence, &flag);
		return;
	}
	const uint32_t item_rounds = exl3_layer_item_rounds(moe.base.inner_size);
	const uint32_t items = live_jobs * groups;
	const uint32_t quantum = exl3_layer_quantum(items * item_rounds, item_rounds, gridDim.x);
	const uint32_t *const widths = moe_widths(moe, arena);
	layer_for_each_run(items, item_rounds, quantum, [&](const struct layer_run &run) {
		/* items: job-major, then the group of 128 outputs */
		const uint32_t group = run.item % groups, job_index = run.item / groups;
		const struct expert_job_record *const job = exl3_job(moe.base, arena, job_index);
		bool completed = false;
		if (job->row_count != 0) {
			const uint32_t runs = layer_runs_of(run.item, item_rounds, quantum);
			LAYER_WIDTH_SWITCH(exl3_job_bits_x2(moe.base, job, widths),
					   completed = layer_down_run<BX2>(moe, arena, job, job_index, group, run, runs,
									   dynamic_shared, &shared, &flag))
		}
		if (!completed || step.sequence == 0)
			return;
		/* this CTA wrote the item's pair outputs: count the job in on the group's columns */
		if (last_of(&words[EXL3_LAYER_COUNTER_WORDS + group], live_jobs, &flag))
			layer_publish_group(record, arena, group, live_rows, step.sequence, &flag);
	});
}
