/*
 * kernel_router_b200.cu: router select and job-table builder for up to 64 live rows (struct
 * router_select_b200_arguments). One block of 1024 threads, a row's picks depend on that row alone (a team of four
 * warps a row for up to eight live rows, a warp a row beyond).
 * (The only atomic is an OR into a shared-memory bit mask, whose result does not depend on order.)
 * Conventions are the reference's router_select_entry (source/kernel_router.cuh:36-119, include/anemone/
 * router_records.h:7-30): keys order scores as the reference's top-k orders float32 (a not-a-number above every
 * number, -0 below +0), the lower expert first among equals; slots in ascending expert order; the weight sum from +0
 * in ascending expert order, every operation one FP32 rounding; jobs in ascending expert order, rows ascending, at
 * most eight rows a job. The picks are the largest affinity + bias (bias_offset 0: no bias), the weights come from
 * the affinities alone, as in the reference. Differences: expert count, picks and scoring are record fields instead
 * of the reference model's constants; the affinity is a fixed sequence of FP32 roundings without a library function
 * (router_device.cuh), so that the choice can be restated bit for bit on a host; always-on shared experts get jobs
 * behind the routed ones.
 */
#include "activation_quantize_device.cuh"
#include "router_device.cuh"

/* router_select_b200's one block */
__device__ __forceinline__ void router_select_block(const struct router_select_b200_arguments &arguments,
						    unsigned char *arena)
{
	__shared__ uint32_t chosen[ROUTER_B200_MAXIMUM_ROWS][ROUTER_B200_MAXIMUM_PICKS]; /* by slot */
	__shared__ float weight[ROUTER_B200_MAXIMUM_ROWS][ROUTER_B200_MAXIMUM_PICKS];
	__shared__ unsigned long long row_mask[ROUTER_B200_MAXIMUM_EXPERTS]; /* bit r: row r stands in the expert */
	__shared__ uint32_t first_job[ROUTER_B200_MAXIMUM_EXPERTS];
	__shared__ uint64_t candidates[ROUTER_B200_THREADS / WARP / ROUTER_TEAM_WARPS]
				      [ROUTER_TEAM_WARPS * ROUTER_B200_MAXIMUM_PICKS];
	const struct step_block step = *reinterpret_cast<const struct step_block *>(arena + arguments.step_offset);
	const uint32_t live = min(step.row_count, arguments.row_capacity);
	const uint32_t experts = arguments.expert_count, picks = arguments.picks, shared = arguments.shared_count;
	const uint32_t lane = threadIdx.x % WARP, warp = threadIdx.x / WARP;
	const float *const scores = reinterpret_cast<const float *>(arena + arguments.scores_offset);

	const float *const bias =
		arguments.bias_offset != 0 ? reinterpret_cast<const float *>(arena + arguments.bias_offset) : nullptr;
	uint32_t *const picks_out = reinterpret_cast<uint32_t *>(arena + arguments.picks_offset);
	float *const weights_out = reinterpret_cast<float *>(arena + arguments.weights_offset);
	const uint32_t team = warp / ROUTER_TEAM_WARPS, teams = blockDim.x / WARP / ROUTER_TEAM_WARPS;
	if (live <= teams) {
		/* a team of four warps a row (the same picks and weights): the launch lasts as long as one row's chain of
		 * dependent instructions, which a team shortens */
		if (team < live)
			router_row_team(scores + (uint64_t)team * experts, bias, experts, picks, arguments.scoring,
					arguments.route_scale, lane, warp % ROUTER_TEAM_WARPS, 1u + team, candidates[team],
					chosen[team], weight[team], picks_out + (uint64_t)team * picks,
					weights_out + (uint64_t)team * picks);
	} else {
		/* one warp a row */
		for (uint32_t row = warp; row < live; row += blockDim.x / WARP)
			router_row(scores + (uint64_t)row * experts, bias, experts, picks, arguments.scoring,
				   arguments.route_scale, lane, chosen[row], weight[row], picks_out + (uint64_t)row * picks,
				   weights_out + (uint64_t)row * picks);
	}
	__syncthreads();
	router_job_table(live, experts, picks, shared, arguments.job_capacity, chosen, weight, row_mask, first_job,
			 reinterpret_cast<struct expert_job_record *>(arena + arguments.jobs_offset),
			 reinterpret_cast<const uint64_t *>(arena + arguments.expert_table_offset), nullptr);
}

extern "C" __global__ void __launch_bounds__(ROUTER_B200_THREADS)
	router_select_b200(struct router_select_b200_arguments arguments, unsigned char *arena)
{
	router_select_block(arguments, arena);
}

/* grid (1 + quantizer blocks) x ROUTER_B200_THREADS: block 0 is the router's block, the warps of the others take the
 * quantizer's loads of 64 values, row after row */
extern "C" __global__ void __launch_bounds__(ROUTER_B200_THREADS)
	router_select_quantize(struct router_select_quantize_arguments arguments, unsigned char *arena)
{
	if (blockIdx.x == 0) {
		router_select_block(arguments.router, arena);
		return;
	}
	const uint32_t warps = blockDim.x / WARP, loads = arguments.quantize.width / 64u;
	const uint32_t tasks = arguments.vector_count * loads;
	for (uint32_t task = (blockIdx.x - 1u) * warps + threadIdx.x / WARP; task < tasks; task += (gridDim.x - 1u) * warps)
		activation_quantize_load(arguments.quantize, arena, task / loads, task % loads, threadIdx.x % WARP);
}

/* One block: copy the pool entry the cursor names into the step input area, then advance the cursor. */
extern "C" __global__ void __launch_bounds__(ROUTER_B200_THREADS)
	step_input_select(struct step_input_select_arguments arguments, unsigned char *arena)
{
	uint64_t *const cursor = reinterpret_cast<uint64_t *>(arena + arguments.cursor_offset);
	const uint64_t entry = *cursor % arguments.pool_count;
	const uint4 *const source = reinterpret_cast<const uint4 *>(arena + arguments.pool_offset + entry * arguments.pool_stride);
	uint4 *const destination = reinterpret_cast<uint4 *>(arena + arguments.destination_offset);
	for (uint32_t index = threadIdx.x; index < arguments.byte_count / 16u; index += blockDim.x)
		destination[index] = source[index];
	__syncthreads();
	if (threadIdx.x == 0)
		*cursor = *cursor + 1u;
}

/* ------------------------------------------------------------------ the job table of many rows */

/* One block of ROUTER_B200_THREADS. The grouping launch has left, per expert, its rows' entries (pair, route weight)
 * in ascending row order and their count. Thread e counts expert e's jobs of eight rows; a block-wide prefix sum gives
 * every expert its first job; then a warp an expert (in turns) writes that expert's jobs, lane c the job's column c.
 * The table's bytes are those router_select_b200 writes for the same choices. */
extern "C" __global__ void __launch_bounds__(ROUTER_B200_THREADS)
	router_wide_jobs(struct router_wide_arguments arguments, unsigned char *arena)
{
	__shared__ uint32_t first_job[ROUTER_B200_MAXIMUM_EXPERTS + 1u];
	__shared__ uint32_t warp_total[ROUTER_B200_THREADS / WARP];
	const struct exl3_prefill_record &routing = arguments.routing;
	const struct exl3_prefill_parts parts = exl3_prefill_parts_of(routing.row_capacity, routing.picks, 0u,
								      routing.expert_count, routing.input_size,
								      routing.inner_size);
	unsigned char *const workspace = arena + routing.workspace_offset;
	const uint32_t *const counts = reinterpret_cast<const uint32_t *>(workspace + parts.counts);
	const struct exl3_prefill_entry *const entries =
		reinterpret_cast<const struct exl3_prefill_entry *>(workspace + parts.entries);
	const uint64_t *const table = reinterpret_cast<const uint64_t *>(arena + routing.expert_table_offset);
	struct expert_job_record *const jobs = reinterpret_cast<struct expert_job_record *>(arena + arguments.jobs_offset);
	const uint32_t lane = threadIdx.x % WARP, warp = threadIdx.x / WARP, warps = blockDim.x / WARP;
	const uint32_t experts = routing.expert_count;
	/* jobs of expert `threadIdx.x`, and the block's exclusive prefix sum of them */
	const uint32_t mine = threadIdx.x < experts ? (counts[threadIdx.x] + LINEAR_MAXIMUM_ROWS - 1u) / LINEAR_MAXIMUM_ROWS : 0u;
	uint32_t before = mine;
	for (uint32_t distance = 1; distance < WARP; distance <<= 1) {
		const uint32_t other = __shfl_up_sync(0xFFFFFFFFu, before, distance);
		if (lane >= distance)
			before += other;
	}
	if (lane == WARP - 1u)
		warp_total[warp] = before;
	__syncthreads();
	uint32_t earlier = 0;
	for (uint32_t other = 0; other < warp; other++)
		earlier += warp_total[other];
	if (threadIdx.x < experts)
		first_job[threadIdx.x] = earlier + before - mine;
	if (threadIdx.x == blockDim.x - 1u)
		first_job[ROUTER_B200_MAXIMUM_EXPERTS] = earlier + before; /* every expert's jobs together */
	__syncthreads();
	const uint32_t live_jobs = min(first_job[ROUTER_B200_MAXIMUM_EXPERTS], arguments.job_capacity);
	/* every byte of the jobs behind the live ones is zero */
	uint4 *const words = reinterpret_cast<uint4 *>(jobs + live_jobs);
	const uint32_t spare = (arguments.job_capacity - live_jobs) * (uint32_t)(sizeof(struct expert_job_record) / 16u);
	for (uint32_t index = threadIdx.x; index < spare; index += blockDim.x)
		words[index] = make_uint4(0, 0, 0, 0);
	for (uint32_t expert = warp; expert < experts; expert += warps) {
		const uint32_t rows = counts[expert];
		const struct exl3_prefill_entry *const of_expert = entries + (uint64_t)expert * routing.row_capacity;
		for (uint32_t first = 0, job_index = first_job[expert]; first < rows && job_index < arguments.job_capacity;
		     first += LINEAR_MAXIMUM_ROWS, job_index++) {
			struct expert_job_record *const job = &jobs[job_index];
			if (lane < LINEAR_MAXIMUM_ROWS) {
				const bool held = first + lane < rows;
				const struct exl3_prefill_entry entry =
					held ? of_expert[first + lane] : exl3_prefill_entry{ 0u, 0.0f };
				job->pair_index[lane] = entry.pair;
				job->route_weight[lane] = entry.route_weight;
			}
			if (lane == 0) {
				job->gate_offset = table[3u * expert];
				job->up_offset = table[3u * expert + 1u];
				job->down_offset = table[3u * expert + 2u];
				job->expert = expert;
				job->row_count = min(rows - first, LINEAR_MAXIMUM_ROWS);
			}
		}
	}
}
