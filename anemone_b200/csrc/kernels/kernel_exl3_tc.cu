/*
 * kernel_exl3_tc.cu: the kernels behind the reference's default entry points of the routed experts
 * (anemone_b200_exl3_tc.h): they take the reference's own records (struct exl3_tc_record, struct exl3_tcp_record), derive
 * this library's struct exl3_moe_record and scratch layout from them (exl3_tc_layout.h) and run the fused products
 * of the fixed cut (exl3_fused.cuh). Arithmetic: the retained chain's (FP32 transforms, FP16 operands, exactly
 * decoded weights, FP32 accumulation), the rows' sums from +0 in ascending slot order.
 *   exl3_tc_operands   grid (ceil(5120 / 128 / 4), jobs, 2) x 128: the scratch's counters and routed marks set to zero,
 *                      then x . suh, Hadamard, FP16 operands of gate and of up
 *   exl3_tc_gate_up    grid (intermediate / 128 * runs, jobs, 2) x 128
 *   exl3_tc_mark       grid (ceil(jobs / 128)) x 128: marks the pairs the job table holds
 *   exl3_tc_down       grid (5120 / 128 * runs, jobs) x 128
 *   exl3_tc_combine    grid (5120 / 512, rows) x 128: a row's sum over its routed pairs, FP32 out or added to the
 *                      bfloat16 row of the always-on expert and rounded once (shared_sum)
 *   exl3_tcp_route     one block x 1024: struct router_pick [rows][6] -> the job table inside the workspace (experts
 *                      ascending, an expert's rows ascending, eight rows a job), every mark set
 *   exl3_tcp_*         the four launches above for a struct exl3_tcp_record
 */
#include "exl3_fused.cuh"
#include "exl3_tc_layout.h"
#include "ordered_device.cuh"

struct tc_view {
	struct exl3_moe_record moe;
	struct exl3_tc_layout layout;
	uint64_t workspace_offset;
	uint32_t rows;
};

__device__ __forceinline__ struct tc_view tc_view_of(const struct exl3_tc_record &record)
{
	struct tc_view view;
	const uint64_t pairs = (uint64_t)record.row_count * EXL3_TC_PAIRS_PER_ROW;
	view.layout = exl3_tc_layout_of(pairs, record.job_capacity, record.intermediate, 0u,
					exl3_tc_workspace_bytes(pairs, record.intermediate));
	view.moe = exl3_tc_moe_record(record.jobs_offset, record.hidden_offset, record.workspace_offset,
				      record.output_offset, record.row_count, record.intermediate, record.bits_x2,
				      record.activation_limit, &view.layout);
	view.workspace_offset = record.workspace_offset;
	view.rows = record.row_count;
	return view;
}

/* A prefill record's launches take the call in chunks of at most EXL3_TCP_JOINT_ROWS rows, one after the other in the
 * same workspace (the caller's workspace formula does not grow beyond that many rows' worth of this library's
 * scratch); record.part names the chunk of a prepared launch. */
__device__ __forceinline__ struct tc_view tcp_view_of(const struct exl3_tcp_record &record)
{
	struct tc_view view;
	const uint32_t first = record.part * EXL3_TCP_JOINT_ROWS;
	const uint32_t rows = min(record.row_count - first, EXL3_TCP_JOINT_ROWS);
	const uint64_t pairs = (uint64_t)rows * EXL3_TC_PAIRS_PER_ROW;
	/* the cut of the products follows the CHUNK's own workspace size (never more than the call's), so that a row's
	 * sums do not depend on how many rows follow it in the call */
	view.layout = exl3_tc_layout_of(pairs, 0u, record.intermediate, exl3_tcp_job_capacity(pairs),
					exl3_tcp_workspace_bytes(rows, record.intermediate));
	view.moe = exl3_tc_moe_record(record.workspace_offset + view.layout.jobs,
				      record.hidden_offset + (uint64_t)first * EXL3_TC_HIDDEN * 2u, record.workspace_offset,
				      record.output_offset + (uint64_t)first * EXL3_TC_HIDDEN * 4u, rows, record.intermediate,
				      record.bits_x2, record.activation_limit, &view.layout);
	view.workspace_offset = record.workspace_offset;
	view.rows = rows;
	return view;
}

/* every block of the launch zeroes its share of the counters (and, for a decode record, of the marks) */
__device__ __forceinline__ void tc_clear(const struct tc_view &view, unsigned char *arena, bool marks_too)
{
	const uint32_t blocks = gridDim.x * gridDim.y * gridDim.z;
	const uint32_t block = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
	const uint64_t words = (uint64_t)view.layout.job_capacity *
			       (view.moe.base.inner_size / EXL3_TRANSFORM + EXL3_TC_HIDDEN / EXL3_TRANSFORM);
	uint32_t *const counters = reinterpret_cast<uint32_t *>(arena + view.moe.counters_offset);
	for (uint64_t word = (uint64_t)block * blockDim.x + threadIdx.x; word < words; word += (uint64_t)blocks * blockDim.x)
		counters[word] = 0u;
	if (!marks_too)
		return;
	uint32_t *const routed = reinterpret_cast<uint32_t *>(arena + view.workspace_offset + view.layout.routed);
	for (uint64_t pair = (uint64_t)block * blockDim.x + threadIdx.x; pair < view.moe.base.pair_count;
	     pair += (uint64_t)blocks * blockDim.x)
		routed[pair] = 0u;
}

__device__ __forceinline__ void tc_mark(const struct tc_view &view, unsigned char *arena)
{
	const uint32_t index = blockIdx.x * blockDim.x + threadIdx.x;
	if (index >= view.layout.job_capacity)
		return;
	const struct expert_job_record *const job = exl3_job(view.moe.base, arena, index);
	uint32_t *const routed = reinterpret_cast<uint32_t *>(arena + view.workspace_offset + view.layout.routed);
	for (uint32_t column = 0; column < job->row_count && column < LINEAR_MAXIMUM_ROWS; column++)
		if (job->pair_index[column] < view.moe.base.pair_count)
			routed[job->pair_index[column]] = 1u;
}

/* grid (5120 / 512, rows) x 128: four channels a thread */
__device__ __forceinline__ void tc_combine(const struct tc_view &view, unsigned char *arena, uint32_t shared_sum,
					   uint64_t shared_offset)
{
	const uint32_t vector = blockIdx.x * blockDim.x + threadIdx.x, vectors = EXL3_TC_HIDDEN / 4u;
	const uint32_t row = blockIdx.y;
	if (vector >= vectors || row >= view.rows)
		return;
	const float4 *const pairs = reinterpret_cast<const float4 *>(arena + view.moe.base.output_offset);
	const uint32_t *const routed =
		reinterpret_cast<const uint32_t *>(arena + view.workspace_offset + view.layout.routed);
	float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
	for (uint32_t slot = 0; slot < EXL3_TC_PAIRS_PER_ROW; slot++) {
		const uint64_t pair = (uint64_t)row * EXL3_TC_PAIRS_PER_ROW + slot;
		if (routed[pair] == 0u)
			continue; /* no job holds the pair: it adds nothing */
		const float4 value = pairs[pair * vectors + vector];
		sum.x = __fadd_rn(sum.x, value.x);
		sum.y = __fadd_rn(sum.y, value.y);
		sum.z = __fadd_rn(sum.z, value.z);
		sum.w = __fadd_rn(sum.w, value.w);
	}
	if (shared_sum == 0u) {
		reinterpret_cast<float4 *>(arena + view.moe.row_output_offset)[(uint64_t)row * vectors + vector] = sum;
		return;
	}
	/* the always-on expert's bfloat16 row plus the sum, rounded once (the reference's combine with shared_sum,
	 * source/kernel_exl3_tc.cu:466-474) */
	uint2 *const place = reinterpret_cast<uint2 *>(arena + shared_offset) + (uint64_t)row * vectors + vector;
	const uint2 held = *place;
	const float x = __fadd_rn(sum.x, __uint_as_float(held.x << 16));
	const float y = __fadd_rn(sum.y, __uint_as_float(held.x & 0xFFFF0000u));
	const float z = __fadd_rn(sum.z, __uint_as_float(held.y << 16));
	const float w = __fadd_rn(sum.w, __uint_as_float(held.y & 0xFFFF0000u));
	*place = make_uint2(bfloat16_bits(x) | bfloat16_bits(y) << 16, bfloat16_bits(z) | bfloat16_bits(w) << 16);
}

/* ------------------------------------------------------------------ decode records */

extern "C" __global__ void __launch_bounds__(EXL3_TRANSFORM_THREADS)
	exl3_tc_operands(struct exl3_tc_record record, unsigned char *arena)
{
	const struct tc_view view = tc_view_of(record);
	tc_clear(view, arena, true);
	exl3_input_pass(view.moe.base, arena, nullptr);
}

extern "C" __global__ void __launch_bounds__(EXL3_PRODUCT_THREADS)
	exl3_tc_gate_up(struct exl3_tc_record record, unsigned char *arena)
{
	extern __shared__ __align__(128) unsigned char dynamic_shared[];
	__shared__ exl3_product_shared shared;
	__shared__ uint32_t flag;
	const struct tc_view view = tc_view_of(record);
	exl3_moe_gate_up_block(view.moe, arena, view.layout.gate_up_runs, dynamic_shared, &shared, &flag);
}

extern "C" __global__ void __launch_bounds__(128) exl3_tc_mark(struct exl3_tc_record record, unsigned char *arena)
{
	tc_mark(tc_view_of(record), arena);
}

extern "C" __global__ void __launch_bounds__(EXL3_PRODUCT_THREADS)
	exl3_tc_down(struct exl3_tc_record record, unsigned char *arena)
{
	extern __shared__ __align__(128) unsigned char dynamic_shared[];
	__shared__ exl3_product_shared shared;
	__shared__ uint32_t flag;
	const struct tc_view view = tc_view_of(record);
	exl3_moe_down_block(view.moe, arena, view.layout.down_runs, dynamic_shared, &shared, &flag);
}

extern "C" __global__ void __launch_bounds__(128) exl3_tc_combine(struct exl3_tc_record record, unsigned char *arena)
{
	tc_combine(tc_view_of(record), arena, record.shared_sum, record.shared_offset);
}

/* ------------------------------------------------------------------ prefill records */

#define TCP_ROUTE_THREADS 1024u

/* One block. The picks of a row name its experts in ascending order, each at most once. Expert e's pairs in
 * ascending row order (a warp an expert at a time, ballots give each row's place: no atomics, a fixed order), cut in
 * jobs of eight; jobs in ascending expert order, the rest of the table zero. */
extern "C" __global__ void __launch_bounds__(TCP_ROUTE_THREADS)
	exl3_tcp_route(struct exl3_tcp_record record, unsigned char *arena)
{
	__shared__ uint32_t pair_count[EXL3_TCP_EXPERTS], first_job[EXL3_TCP_EXPERTS];
	const struct tc_view view = tcp_view_of(record);
	const uint32_t lane = threadIdx.x % EXL3_WARP, warp = threadIdx.x / EXL3_WARP, warps = blockDim.x / EXL3_WARP;
	const uint32_t pairs = view.moe.base.pair_count;
	const struct router_pick *const picks =
		reinterpret_cast<const struct router_pick *>(arena + record.picks_offset) +
		(uint64_t)record.part * EXL3_TCP_JOINT_ROWS * EXL3_TC_PAIRS_PER_ROW;
	const uint64_t *const offsets = reinterpret_cast<const uint64_t *>(arena + record.expert_offsets_offset);
	struct expert_job_record *const jobs = reinterpret_cast<struct expert_job_record *>(arena + view.moe.base.jobs_offset);
	uint4 *const table = reinterpret_cast<uint4 *>(jobs);
	for (uint32_t index = threadIdx.x; index < view.layout.job_capacity * (uint32_t)(sizeof(*jobs) / 16u);
	     index += blockDim.x)
		table[index] = make_uint4(0, 0, 0, 0);
	uint32_t *const routed = reinterpret_cast<uint32_t *>(arena + view.workspace_offset + view.layout.routed);
	for (uint32_t pair = threadIdx.x; pair < pairs; pair += blockDim.x)
		routed[pair] = picks[pair].expert < EXL3_TCP_EXPERTS ? 1u : 0u;
	/* the pairs of each expert: a warp an expert, its lanes over the pairs */
	for (uint32_t expert = warp; expert < EXL3_TCP_EXPERTS; expert += warps) {
		uint32_t count = 0;
		for (uint32_t pair = lane; pair < pairs; pair += EXL3_WARP)
			count += picks[pair].expert == expert ? 1u : 0u;
		for (uint32_t distance = EXL3_WARP / 2u; distance != 0; distance >>= 1)
			count += __shfl_xor_sync(0xFFFFFFFFu, count, distance);
		if (lane == 0)
			pair_count[expert] = count;
	}
	__syncthreads();
	if (threadIdx.x == 0) { /* 384 additions: the first job of every expert */
		uint32_t next = 0;
		for (uint32_t expert = 0; expert < EXL3_TCP_EXPERTS; expert++) {
			first_job[expert] = next;
			next += (pair_count[expert] + LINEAR_MAXIMUM_ROWS - 1u) / LINEAR_MAXIMUM_ROWS;
		}
	}
	__syncthreads();
	for (uint32_t expert = warp; expert < EXL3_TCP_EXPERTS; expert += warps) {
		if (pair_count[expert] == 0)
			continue;
		uint32_t placed = 0; /* the expert's pairs before this stretch of 32 */
		for (uint32_t begin = 0; begin < pairs; begin += EXL3_WARP) {
			const uint32_t pair = begin + lane;
			const bool mine = pair < pairs && picks[pair].expert == expert;
			const uint32_t ballot = __ballot_sync(0xFFFFFFFFu, mine);
			if (mine) {
				const uint32_t place = placed + __popc(ballot & ((1u << lane) - 1u));
				const uint32_t job_index = first_job[expert] + place / LINEAR_MAXIMUM_ROWS;
				if (job_index < view.layout.job_capacity) {
					struct expert_job_record *const job = &jobs[job_index];
					const uint32_t column = place % LINEAR_MAXIMUM_ROWS;
					job->pair_index[column] = pair;
					job->route_weight[column] = picks[pair].route_weight;
					if (column == 0) {
						const uint32_t remaining = pair_count[expert] - place;
						job->gate_offset = offsets[3u * expert];
						job->up_offset = offsets[3u * expert + 1u];
						job->down_offset = offsets[3u * expert + 2u];
						job->expert = expert;
						job->row_count = remaining < LINEAR_MAXIMUM_ROWS ? remaining : LINEAR_MAXIMUM_ROWS;
					}
				}
			}
			placed += __popc(ballot);
		}
	}
}

extern "C" __global__ void __launch_bounds__(EXL3_TRANSFORM_THREADS)
	exl3_tcp_operands(struct exl3_tcp_record record, unsigned char *arena)
{
	const struct tc_view view = tcp_view_of(record);
	tc_clear(view, arena, false);
	exl3_input_pass(view.moe.base, arena, nullptr);
}

extern "C" __global__ void __launch_bounds__(EXL3_PRODUCT_THREADS)
	exl3_tcp_gate_up(struct exl3_tcp_record record, unsigned char *arena)
{
	extern __shared__ __align__(128) unsigned char dynamic_shared[];
	__shared__ exl3_product_shared shared;
	__shared__ uint32_t flag;
	const struct tc_view view = tcp_view_of(record);
	exl3_moe_gate_up_block(view.moe, arena, view.layout.gate_up_runs, dynamic_shared, &shared, &flag);
}

extern "C" __global__ void __launch_bounds__(EXL3_PRODUCT_THREADS)
	exl3_tcp_down(struct exl3_tcp_record record, unsigned char *arena)
{
	extern __shared__ __align__(128) unsigned char dynamic_shared[];
	__shared__ exl3_product_shared shared;
	__shared__ uint32_t flag;
	const struct tc_view view = tcp_view_of(record);
	exl3_moe_down_block(view.moe, arena, view.layout.down_runs, dynamic_shared, &shared, &flag);
}

extern "C" __global__ void __launch_bounds__(128) exl3_tcp_combine(struct exl3_tcp_record record, unsigned char *arena)
{
	tc_combine(tcp_view_of(record), arena, 0u, 0u);
}
