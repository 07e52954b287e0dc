/*
 * kernel_router_b200.cu: router select and job-table builder for up to 64 live rows (struct
 * router_select_b200_arguments). One block of 1024 threads, a row's picks depend on that row alone.
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

	/* one warp a row */
	const float *const bias =
		arguments.bias_offset != 0 ? reinterpret_cast<const float *>(arena + arguments.bias_offset) : nullptr;
	for (uint32_t row = warp; row < live; row += blockDim.x / WARP)
		router_row(scores + (uint64_t)row * experts, bias, experts, picks, arguments.scoring, arguments.route_scale,
			   lane, chosen[row], weight[row],
			   reinterpret_cast<uint32_t *>(arena + arguments.picks_offset) + (uint64_t)row * picks,
			   reinterpret_cast<float *>(arena + arguments.weights_offset) + (uint64_t)row * picks);
	__syncthreads();
	router_job_table(live, experts, picks, shared, arguments.job_capacity, chosen, weight, row_mask, first_job,
			 reinterpret_cast<struct expert_job_record *>(arena + arguments.jobs_offset),
			 reinterpret_cast<const uint64_t *>(arena + arguments.expert_table_offset), nullptr);
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
