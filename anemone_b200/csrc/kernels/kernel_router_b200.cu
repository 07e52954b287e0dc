/*
 * kernel_router_b200.cu: router select and job-table builder for up to 64 live rows (struct
 * router_select_b200_arguments). One block of 1024 threads, a row's picks depend on that row alone.
 * (The only atomic is an OR into a shared-memory bit mask, whose result does not depend on order.)
 * Conventions are the reference's router_select_entry (source/kernel_router.cuh:36-119, include/anemone/
 * router_records.h:7-30): keys order scores as the reference's top-k orders float32 (a not-a-number above every
 * number, -0 below +0), the lower expert first among equals; slots in ascending expert order; the weight sum from +0
 * in ascending expert order, every operation one FP32 rounding; jobs in ascending expert order, rows ascending, at
 * most eight rows a job. Differences: expert count, picks and scoring are record fields instead of the reference
 * model's constants; the picks are the largest SCORES (the affinity is monotone in the score), so that the chosen
 * experts do not depend on the last bit of expf; always-on shared experts get jobs behind the routed ones.
 */
#include "router_device.cuh"

extern "C" __global__ void __launch_bounds__(ROUTER_B200_THREADS)
	router_select_b200(struct router_select_b200_arguments arguments, unsigned char *arena)
{
	__shared__ uint32_t chosen[ROUTER_B200_MAXIMUM_ROWS][ROUTER_B200_MAXIMUM_PICKS]; /* by slot */
	__shared__ float weight[ROUTER_B200_MAXIMUM_ROWS][ROUTER_B200_MAXIMUM_PICKS];
	__shared__ unsigned long long row_mask[ROUTER_B200_MAXIMUM_EXPERTS]; /* bit r: row r stands in the expert */
	__shared__ uint32_t first_job[ROUTER_B200_MAXIMUM_EXPERTS];
	const struct step_block step = *reinterpret_cast<const struct step_block *>(arena + arguments.step_offset);
	const uint32_t live = min(step.row_count, arguments.row_capacity);
	const uint32_t experts = arguments.expert_count, picks = arguments.picks, shared = arguments.shared_count;
	const uint32_t lane = threadIdx.x % WARP, warp = threadIdx.x / WARP;
	const float *const scores = reinterpret_cast<const float *>(arena + arguments.scores_offset);

	/* every byte of the job table starts zero */
	uint4 *const table = reinterpret_cast<uint4 *>(arena + arguments.jobs_offset);
	for (uint32_t index = threadIdx.x; index < arguments.job_capacity * (uint32_t)(sizeof(struct expert_job_record) / 16u);
	     index += blockDim.x)
		table[index] = make_uint4(0, 0, 0, 0);
	for (uint32_t expert = threadIdx.x; expert < ROUTER_B200_MAXIMUM_EXPERTS; expert += blockDim.x)
		row_mask[expert] = 0ull;

	/* one warp a row */
	for (uint32_t row = warp; row < live; row += blockDim.x / WARP)
		router_row(scores + (uint64_t)row * experts, experts, picks, arguments.scoring, arguments.route_scale, lane,
			   chosen[row], weight[row],
			   reinterpret_cast<uint32_t *>(arena + arguments.picks_offset) + (uint64_t)row * picks,
			   reinterpret_cast<float *>(arena + arguments.weights_offset) + (uint64_t)row * picks);
	__syncthreads();

	/* which rows chose each expert: a 64-bit mask per expert (an OR is the same in any order), then the first job of
	 * every expert by a warp-wide prefix sum over the experts' job counts */
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
		before -= total;
#pragma unroll
		for (uint32_t place = 0; place < EXPERTS_PER_LANE; place++)
			first_job[lane * EXPERTS_PER_LANE + place] = before + local[place];
	}
	__syncthreads();

	/* a thread a pair: its place among its expert's rows decides its job and column */
	const uint32_t pairs_per_row = picks + shared;
	struct expert_job_record *const jobs = reinterpret_cast<struct expert_job_record *>(arena + arguments.jobs_offset);
	const uint64_t *const offsets = reinterpret_cast<const uint64_t *>(arena + arguments.expert_table_offset);
	for (uint32_t pair = threadIdx.x; pair < live * pairs_per_row; pair += blockDim.x) {
		const uint32_t row = pair / pairs_per_row, slot = pair % pairs_per_row;
		const uint32_t expert = slot < picks ? chosen[row][slot] : experts + (slot - picks);
		const unsigned long long mask = row_mask[expert];
		const uint32_t place = (uint32_t)__popcll(mask & ((1ull << row) - 1ull)); /* rows below mine in the expert */
		const uint32_t job_index = first_job[expert] + place / LINEAR_MAXIMUM_ROWS;
		if (job_index >= arguments.job_capacity)
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
