/*
 * exl3_fused.cuh: what the fused expert launches share (kernel_exl3_b200.cu: a fixed cut of K per CTA;
 * kernel_exl3_layer.cu: one sequence of K rounds cut evenly over the grid): partial sums of a run of K in the arena,
 * the counter that finds the CTA completing a (job, 128 outputs), the sum of the runs in ascending order from +0, and
 * the two epilogues (activation with the down-side transform; output transform, scale and route weight). The
 * arithmetic of every value is the retained chain's (exl3_passes.cuh).
 */
#ifndef AB_EXL3_FUSED_CUH
#define AB_EXL3_FUSED_CUH

#include "exl3_passes.cuh"

__device__ __forceinline__ const uint32_t *moe_widths(const struct exl3_moe_record &record, const unsigned char *arena)
{
	return record.base.bits_per_weight == EXL3_WIDTH_PER_EXPERT ?
		       reinterpret_cast<const uint32_t *>(arena + record.widths_offset) :
		       nullptr;
}

/* this thread's sums (exl3_product_core's layout) to partial rows: row(column) + 128 group + output */
__device__ __forceinline__ void store_partial(const float sums[2][4], float *const rows[LINEAR_MAXIMUM_ROWS],
					      uint32_t row_count)
{
	const uint32_t lane = threadIdx.x % EXL3_WARP, warp = threadIdx.x / EXL3_WARP;
	const uint32_t group_lane = lane / 4u, place = lane % 4u;
#pragma unroll
	for (uint32_t mine = 0; mine < 2; mine++)
#pragma unroll
		for (uint32_t c = 0; c < 4; c++) {
			const uint32_t column = place * 2u + (c & 1u);
			if (column < row_count)
				rows[column][(warp * 2u + mine) * EXL3_TILE + group_lane + (c >> 1) * 8u] = sums[mine][c];
		}
}

/* true in exactly one CTA of the `expected` that work on this counter: the last to arrive. Every CTA's partial sums are
 * visible to it. The counter is left at zero for the next launch. */
__device__ __forceinline__ bool last_of(uint32_t *counter, uint32_t expected, uint32_t *flag)
{
	__threadfence();
	__syncthreads();
	if (threadIdx.x == 0) {
		const uint32_t arrived = atomicAdd(counter, 1u) + 1u;
		*flag = arrived == expected ? 1u : 0u;
		if (arrived == expected)
			*counter = 0u;
		__threadfence();
	}
	__syncthreads();
	return *flag != 0u;
}

/* FP32 sum over the runs, in ascending order from +0, of this lane's four channels of one partial row */
__device__ __forceinline__ void sum_runs(const float *first_run, uint64_t run_stride, uint32_t runs, float out[4])
{
	float4 total = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
	for (uint32_t run = 0; run < runs; run++) {
		const float4 part = __ldcg(reinterpret_cast<const float4 *>(first_run + run * run_stride));
		total.x = __fadd_rn(total.x, part.x);
		total.y = __fadd_rn(total.y, part.y);
		total.z = __fadd_rn(total.z, part.z);
		total.w = __fadd_rn(total.w, part.w);
	}
	out[0] = total.x, out[1] = total.y, out[2] = total.z, out[3] = total.w;
}

/* The activation of a job's rows for one group of 128 inner channels, a warp a row, by the CTA that completed the
 * group's gate and up products: gate_first / up_first: run 0 of the FP32 partial rows [pair][inner] of each, the
 * further runs run_stride floats apart. Writes the bfloat16 hidden values and the FP16 down operands (behind the
 * gate/up operands, which other CTAs of the launch still read). All 128 threads call. */
template <uint32_t BX2>
__device__ __forceinline__ void exl3_gate_up_epilogue(const struct exl3_moe_record &moe, unsigned char *arena,
						      const struct expert_job_record *job, uint32_t group,
						      const float *gate_first, const float *up_first, uint64_t run_stride,
						      uint32_t gate_runs, uint32_t up_runs)
{
	const struct exl3_expert_record &record = moe.base;
	const uint32_t lane = threadIdx.x % EXL3_WARP, warp = threadIdx.x / EXL3_WARP;
	const uint32_t H = record.input_size, I = record.inner_size, pairs = record.pair_count;
	const uint32_t channel = group * EXL3_TRANSFORM + lane * 4u;
	const uint64_t codes = exl3_code_bytes(H, I, BX2);
	float gate_scale[4], up_scale[4], down_scale[4];
	load_half4(reinterpret_cast<const __half *>(arena + job->gate_offset + codes) + H + channel, gate_scale);
	load_half4(reinterpret_cast<const __half *>(arena + job->up_offset + codes) + H + channel, up_scale);
	load_half4(reinterpret_cast<const __half *>(arena + job->down_offset + exl3_code_bytes(I, H, BX2)) + channel,
		   down_scale);
	for (uint32_t column = warp; column < job->row_count; column += EXL3_PRODUCT_WARPS) {
		const uint64_t at = (uint64_t)job->pair_index[column] * I + channel;
		float gate[4], up[4];
		sum_runs(gate_first + at, run_stride, gate_runs, gate);
		sum_runs(up_first + at, run_stride, up_runs, up);
		hadamard128_warp(gate, lane);
		hadamard128_warp(up, lane);
		float hidden[4];
		exl3_swiglu4(gate, up, gate_scale, up_scale, record.activation_limit, hidden);
		const __nv_bfloat162 low = __halves2bfloat162(__float2bfloat16_rn(hidden[0]), __float2bfloat16_rn(hidden[1]));
		const __nv_bfloat162 high = __halves2bfloat162(__float2bfloat16_rn(hidden[2]), __float2bfloat16_rn(hidden[3]));
		uint2 stored;
		stored.x = *reinterpret_cast<const uint32_t *>(&low);
		stored.y = *reinterpret_cast<const uint32_t *>(&high);
		*reinterpret_cast<uint2 *>(reinterpret_cast<__nv_bfloat16 *>(arena + record.hidden_offset) + at) = stored;
		float fed[4];
#pragma unroll
		for (uint32_t i = 0; i < 4; i++)
			fed[i] = __fmul_rn(hidden[i], down_scale[i]);
		hadamard128_warp(fed, lane);
#pragma unroll
		for (uint32_t i = 0; i < 4; i++)
			fed[i] = __fmul_rn(fed[i], EXL3_NORMALIZATION);
		store_half4(reinterpret_cast<__half *>(arena + record.operands_offset) + (uint64_t)EXL3_PROJECTIONS * pairs * H +
				    at,
			    fed);
	}
}

/* The finish of a job's rows for one group of 128 outputs by the CTA that completed the group's down products:
 * first: run 0 of the FP32 partial rows [pair][input_size]; writes the pair outputs (transform, scale, route
 * weight) at output_offset. All 128 threads call. */
template <uint32_t BX2>
__device__ __forceinline__ void exl3_down_epilogue(const struct exl3_moe_record &moe, unsigned char *arena,
						   const struct expert_job_record *job, uint32_t group, const float *first,
						   uint64_t run_stride, uint32_t runs, uint64_t output_offset)
{
	const struct exl3_expert_record &record = moe.base;
	const uint32_t lane = threadIdx.x % EXL3_WARP, warp = threadIdx.x / EXL3_WARP;
	const uint32_t H = record.input_size, I = record.inner_size;
	const uint32_t channel = group * EXL3_TRANSFORM + lane * 4u;
	float scale[4];
	load_half4(reinterpret_cast<const __half *>(arena + job->down_offset + exl3_code_bytes(I, H, BX2)) + I + channel,
		   scale);
	for (uint32_t column = warp; column < job->row_count; column += EXL3_PRODUCT_WARPS) {
		const uint64_t at = (uint64_t)job->pair_index[column] * H + channel;
		float v[4];
		sum_runs(first + at, run_stride, runs, v);
		hadamard128_warp(v, lane);
		const float weight = job->route_weight[column];
#pragma unroll
		for (uint32_t i = 0; i < 4; i++)
			v[i] = __fmul_rn(__fmul_rn(__fmul_rn(v[i], EXL3_NORMALIZATION), scale[i]), weight);
		*reinterpret_cast<float4 *>(reinterpret_cast<float *>(arena + output_offset) + at) =
			make_float4(v[0], v[1], v[2], v[3]);
	}
}

/* what one pass of a product CTA works on: run `run` of the cut of K, of 128 outputs (`group`) of one matrix
 * (`projection`: gate or up; 0 for down) of job `job` */
struct moe_item {
	uint32_t job, group, run, projection;
};

/* One item of gate or up: run item.run of K of 128 outputs of the job; the CTA that completes the (job, 128 outputs)
 * applies the activation. ready (may be null): a word a job that counts the groups whose down operands are in place. */
template <uint32_t BX2>
__device__ __forceinline__ void moe_gate_up(const struct exl3_moe_record &moe, unsigned char *arena,
					    const struct expert_job_record *job, uint32_t runs,
					    unsigned char *dynamic_shared, exl3_product_shared *shared, uint32_t *flag,
					    uint32_t *ready, const struct moe_item &item, uint64_t)
{
	const struct exl3_expert_record &record = moe.base;
	const uint32_t lane = threadIdx.x % EXL3_WARP;
	const uint32_t H = record.input_size, I = record.inner_size, pairs = record.pair_count;
	const uint32_t groups = I / EXL3_TRANSFORM;
	const uint32_t group = item.group, run = item.run, projection = item.projection;
	const uint32_t steps = H / EXL3_TILE / runs;
	const uint32_t fed_column = lane / 4u < job->row_count ? lane / 4u : 0u;
	const __half *const operands = reinterpret_cast<const __half *>(arena + record.operands_offset);
	float sums[2][4];
	if (!exl3_product_core<BX2>(arena + (projection == 0 ? job->gate_offset : job->up_offset), I, group, run * steps,
				    steps, operands + ((uint64_t)projection * pairs + job->pair_index[fed_column]) * H,
				    dynamic_shared, shared, sums))
		return;
	/* partial sums: FP32 [projection][run][pair][I] */
	float *const partials = reinterpret_cast<float *>(arena + record.products_offset);
	const uint64_t run_stride = (uint64_t)pairs * I;
	float *rows[LINEAR_MAXIMUM_ROWS];
#pragma unroll
	for (uint32_t column = 0; column < LINEAR_MAXIMUM_ROWS; column++)
		rows[column] = partials + ((uint64_t)projection * runs + run) * run_stride +
			       (uint64_t)job->pair_index[column < job->row_count ? column : 0u] * I + group * EXL3_TRANSFORM;
	store_partial(sums, rows, job->row_count);
	uint32_t *const counter = reinterpret_cast<uint32_t *>(arena + moe.counters_offset) + item.job * groups + group;
	if (!last_of(counter, EXL3_PROJECTIONS * runs, flag))
		return;
	exl3_gate_up_epilogue<BX2>(moe, arena, job, group, partials, partials + (uint64_t)runs * run_stride, run_stride, runs,
				   runs);
	if (ready != nullptr) { /* one more group of the job's down operands is in place, for a launch that runs beside */
		__threadfence();
		__syncthreads();
		if (threadIdx.x == 0)
			atomicAdd(ready + item.job, 1u);
	}
}

/* The same for down: grid (input_size / 128 * runs, jobs). */
template <uint32_t BX2>
__device__ __forceinline__ void moe_down(const struct exl3_moe_record &moe, unsigned char *arena,
					 const struct expert_job_record *job, uint32_t runs,
					 unsigned char *dynamic_shared, exl3_product_shared *shared, uint32_t *flag,
					 uint32_t *, const struct moe_item &item, uint64_t products_offset)
{
	const struct exl3_expert_record &record = moe.base;
	const uint32_t lane = threadIdx.x % EXL3_WARP;
	const uint32_t H = record.input_size, I = record.inner_size, pairs = record.pair_count;
	const uint32_t groups = H / EXL3_TRANSFORM;
	const uint32_t group = item.group, run = item.run;
	const uint32_t steps = I / EXL3_TILE / runs;
	const uint32_t fed_column = lane / 4u < job->row_count ? lane / 4u : 0u;
	const __half *const operands =
		reinterpret_cast<const __half *>(arena + record.operands_offset) + (uint64_t)EXL3_PROJECTIONS * pairs * H;
	float sums[2][4];
	if (!exl3_product_core<BX2>(arena + job->down_offset, H, group, run * steps, steps,
				    operands + (uint64_t)job->pair_index[fed_column] * I, dynamic_shared, shared, sums))
		return;
	/* partial sums: FP32 [run][pair][H] at products_offset; run 0's rows are also where the pair outputs go */
	float *const partials = reinterpret_cast<float *>(arena + products_offset);
	const uint64_t run_stride = (uint64_t)pairs * H;
	float *rows[LINEAR_MAXIMUM_ROWS];
#pragma unroll
	for (uint32_t column = 0; column < LINEAR_MAXIMUM_ROWS; column++)
		rows[column] = partials + run * run_stride +
			       (uint64_t)job->pair_index[column < job->row_count ? column : 0u] * H + group * EXL3_TRANSFORM;
	store_partial(sums, rows, job->row_count);
	uint32_t *const counter = reinterpret_cast<uint32_t *>(arena + moe.counters_offset) +
				  (uint64_t)record.job_count * (I / EXL3_TRANSFORM) + item.job * groups + group;
	if (!last_of(counter, runs, flag))
		return;
	exl3_down_epilogue<BX2>(moe, arena, job, group, partials, run_stride, runs, products_offset);
}

#define EXL3_FUSED_WIDTH_SWITCH(function)                                                      \
	switch (exl3_job_bits_x2(record.base, job, moe_widths(record, arena))) {               \
	case EXL3_BITS_X2_K2:                                                                  \
		function<EXL3_BITS_X2_K2>(record, arena, job, runs, dynamic_shared, shared, flag, ready, item, products_offset);   \
		break;                                                                         \
	case EXL3_BITS_X2_K2_5:                                                                \
		function<EXL3_BITS_X2_K2_5>(record, arena, job, runs, dynamic_shared, shared, flag, ready, item, products_offset); \
		break;                                                                         \
	case EXL3_BITS_X2_K3:                                                                  \
		function<EXL3_BITS_X2_K3>(record, arena, job, runs, dynamic_shared, shared, flag, ready, item, products_offset);   \
		break;                                                                         \
	case EXL3_BITS_X2_K4:                                                                  \
		function<EXL3_BITS_X2_K4>(record, arena, job, runs, dynamic_shared, shared, flag, ready, item, products_offset);   \
		break;                                                                         \
	default:                                                                               \
		break;                                                                         \
	}

/* one item of either kind, for an entry that walks a list of items (job: the item's) */
__device__ __forceinline__ void exl3_moe_gate_up_item(const struct exl3_moe_record &record, unsigned char *arena,
						      const struct moe_item &item, uint32_t runs,
						      unsigned char *dynamic_shared, exl3_product_shared *shared,
						      uint32_t *flag, uint32_t *ready)
{
	const uint64_t products_offset = 0;
	const struct expert_job_record *const job = exl3_job(record.base, arena, item.job);
	EXL3_FUSED_WIDTH_SWITCH(moe_gate_up)
}

__device__ __forceinline__ void exl3_moe_down_item(const struct exl3_moe_record &record, unsigned char *arena,
						   const struct moe_item &item, uint32_t runs,
						   unsigned char *dynamic_shared, exl3_product_shared *shared, uint32_t *flag,
						   uint64_t products_offset)
{
	uint32_t *const ready = nullptr;
	const struct expert_job_record *const job = exl3_job(record.base, arena, item.job);
	EXL3_FUSED_WIDTH_SWITCH(moe_down)
}

/* the bodies of the two product kernels of the fixed cut, for any entry that holds a struct exl3_moe_record */
__device__ __forceinline__ void exl3_moe_gate_up_block(const struct exl3_moe_record &record, unsigned char *arena,
						       uint32_t runs, unsigned char *dynamic_shared,
						       exl3_product_shared *shared, uint32_t *flag,
						       uint32_t *ready = nullptr)
{
	const uint64_t products_offset = 0;
	const struct moe_item item = { blockIdx.y, blockIdx.x / runs, blockIdx.x % runs, blockIdx.z };
	const struct expert_job_record *const job = exl3_job(record.base, arena, blockIdx.y);
	if (job->row_count == 0)
		return;
	EXL3_FUSED_WIDTH_SWITCH(moe_gate_up)
}

__device__ __forceinline__ void exl3_moe_down_block(const struct exl3_moe_record &record, unsigned char *arena,
						    uint32_t runs, unsigned char *dynamic_shared,
						    exl3_product_shared *shared, uint32_t *flag)
{
	uint32_t *const ready = nullptr;
	const uint64_t products_offset = record.base.products_offset;
	const struct moe_item item = { blockIdx.y, blockIdx.x / runs, blockIdx.x % runs, 0u };
	const struct expert_job_record *const job = exl3_job(record.base, arena, blockIdx.y);
	if (job->row_count == 0)
		return;
	EXL3_FUSED_WIDTH_SWITCH(moe_down)
}

#endif
