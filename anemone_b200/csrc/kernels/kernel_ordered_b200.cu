/*
 * kernel_ordered_b200.cu: the production reduction of expert partial sums on NVLink (no counterpart file in the
 * reference; the arithmetic is its owner sums', source/kernel_tp_exchange.cu:190-247: FP32 adds in ascending rank
 * order from +0, ONE rounding to bfloat16).
 *
 *   ordered_row_sum_publish  grid (ceil(width / 512), up to 128 row blocks) x 128: waits until every rank has finished
 *       reading this slot's previous use (their DONE lines), writes this rank's FP32 row sums (slots added from +0 in
 *       ascending order) straight into its input array of the slot, and the last block to finish publishes READY.
 *   ordered_reduce_bf16      grid (up to 64 blocks, or up to 592 for many rows) x 256: waits for every rank's READY,
 *       pulls every rank's rows by 128-bit peer loads, adds them in rank order, rounds once, stores bfloat16
 *       [rows][width] at the arena offset output_offset; the last block to finish publishes DONE. With owner runs
 *       (mode 1) a rank adds only its run of the vectors and stores the result into every rank's memory.
 *   ordered_rows_push        the two above as ONE launch for decode steps, by stores instead of loads: row sums into
 *       every rank's inbox, READY, the adds in rank order, one rounding, bfloat16 kept locally (ordered_push_device.cuh).
 * All read the live row count and the sequence from the step block. The read-complete barrier of the FP32
 * collectives is moved from the end of a step to the next refill of the same slot (two steps later), where it costs
 * nothing; the slot's input must therefore only ever be written by ordered_row_sum_publish.
 */
#include "ordered_push_device.cuh"

/* true for exactly one block: the last of the grid to arrive. The counter is the owner's own, at `line` + 64. Every
 * block orders its stores at device scope before it counts itself; the block that sees the count complete then
 * publishes with a system-scope release, which is cumulative over the stores it has observed that way. */
__device__ __forceinline__ bool last_block_of_grid(unsigned char *line, uint32_t *shared_flag)
{
	__threadfence();
	__syncthreads();
	if (threadIdx.x == 0) {
		unsigned int *const counter = reinterpret_cast<unsigned int *>(line + ORDERED_LOCAL_COUNTER_OFFSET);
		const unsigned int blocks = gridDim.x * gridDim.y * gridDim.z;
		const unsigned int arrived = atomicAdd(counter, 1u) + 1u;
		*shared_flag = arrived == blocks ? 1u : 0u;
		if (arrived == blocks) {
			*counter = 0u; /* ready for the slot's next use */
			__threadfence();
		}
	}
	__syncthreads();
	return *shared_flag != 0;
}

extern "C" __global__ void __launch_bounds__(128)
	ordered_row_sum_publish(struct ordered_row_sum_publish_arguments arguments, unsigned char *arena)
{
	__shared__ uint32_t verdict, last;
	const struct ordered_collective_arguments &collective = arguments.collective;
	const struct step_block step = *reinterpret_cast<const struct step_block *>(arena + collective.step_offset);
	const uint64_t sequence = step.sequence;
	if (sequence == 0)
		return;
	unsigned char *const mine = ordered_slot(collective, arena, collective.rank, sequence);
	unsigned char *const ready_line = mine + ORDERED_READY_PHASE * ORDERED_COLLECTIVE_LINE_BYTES;
	/* the slot's previous use must have been read by everyone before it is overwritten */
	const uint64_t previous = *reinterpret_cast<const uint64_t *>(ready_line + ORDERED_LOCAL_PREVIOUS_OFFSET);
	bool alive = true;
	if (previous != 0 && previous < sequence)
		alive = ordered_wait_all(collective, arena, ORDERED_DONE_PHASE, sequence, previous, false,
					 arena + arguments.status_offset, &verdict);
	/* a block whose wait ran out writes no rows: the grid must then not publish them */
	unsigned int *const gave_up = reinterpret_cast<unsigned int *>(ready_line + ORDERED_LOCAL_GAVE_UP_OFFSET);
	if (!alive && threadIdx.x == 0)
		atomicExch(gave_up, 1u);
	/* a block takes rows blockIdx.y, blockIdx.y + gridDim.y, ...: the grid stays small for many rows, because every
	 * block counts itself on one counter at the end */
	const uint32_t live_rows = min(step.row_count, collective.element_count / arguments.width);
	const uint32_t vectors = arguments.width / 4u;
	const uint32_t vector = blockIdx.x * blockDim.x + threadIdx.x;
	if (alive && vector < vectors) {
		const float4 *const pairs = reinterpret_cast<const float4 *>(arena + arguments.pair_output_offset);
		float4 *const out = reinterpret_cast<float4 *>(mine + collective.input_offset);
		for (uint32_t row = blockIdx.y; row < live_rows; row += gridDim.y) {
			float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
			for (uint32_t slot = 0; slot < arguments.pairs_per_row; slot++) {
				const float4 value = pairs[((uint64_t)row * arguments.pairs_per_row + slot) * vectors + vector];
				sum.x = __fadd_rn(sum.x, value.x);
				sum.y = __fadd_rn(sum.y, value.y);
				sum.z = __fadd_rn(sum.z, value.z);
				sum.w = __fadd_rn(sum.w, value.w);
			}
			out[(uint64_t)row * vectors + vector] = sum;
		}
	}
	if (last_block_of_grid(ready_line, &last) && threadIdx.x == 0) {
		/* some block gave up: READY stays unpublished, the peers' own READY waits run out and say so */
		if (atomicExch(gave_up, 0u) != 0u)
			return;
		*reinterpret_cast<uint64_t *>(ready_line + ORDERED_LOCAL_PREVIOUS_OFFSET) = sequence;
		__threadfence_system();
		signal_store(ready_line, sequence);
	}
}

extern "C" __global__ void __launch_bounds__(ORDERED_COLLECTIVE_THREADS)
	ordered_reduce_bf16(struct ordered_reduce_bf16_arguments arguments, unsigned char *arena)
{
	__shared__ uint32_t verdict, last;
	const struct ordered_collective_arguments &collective = arguments.collective;
	const struct step_block step = *reinterpret_cast<const struct step_block *>(arena + collective.step_offset);
	const uint64_t sequence = step.sequence;
	if (sequence == 0 || collective.rank_count == 0 || collective.rank_count > ORDERED_COLLECTIVE_MAXIMUM_RANKS)
		return;
	unsigned char *const status = arena + arguments.status_offset;
	unsigned char *const mine = ordered_slot(collective, arena, collective.rank, sequence);
	const bool alive = ordered_wait_all(collective, arena, ORDERED_READY_PHASE, sequence, sequence, true, status, &verdict);
	const bool owner_runs = arguments.mode == ORDERED_REDUCE_OWNER_RUNS;
	if (alive) {
		const uint32_t live = min(step.row_count * arguments.width, collective.element_count);
		const uint32_t vectors = live / 4u;
		const float *inputs[ORDERED_COLLECTIVE_MAXIMUM_RANKS];
		uint2 *outputs[ORDERED_COLLECTIVE_MAXIMUM_RANKS];
#pragma unroll
		for (uint32_t rank = 0; rank < ORDERED_COLLECTIVE_MAXIMUM_RANKS; rank++) {
			inputs[rank] = rank < collective.rank_count ?
					       reinterpret_cast<const float *>(ordered_slot(collective, arena, rank, sequence) +
									       collective.input_offset) :
					       nullptr;
			/* every rank keeps its result at the same arena offset */
			outputs[rank] = rank == collective.rank ? reinterpret_cast<uint2 *>(arena + collective.output_offset) :
					rank < collective.rank_count ?
								  reinterpret_cast<uint2 *>(
									  reinterpret_cast<unsigned char *>(
										  ordered_peers(collective, arena)[rank].arena_address) +
									  collective.output_offset) :
								  nullptr;
		}
		uint2 *const own = reinterpret_cast<uint2 *>(arena + collective.output_offset);
		/* this rank's run of vectors */
		uint32_t first = 0, end = vectors;
		if (owner_runs) {
			const uint32_t share = vectors / collective.rank_count, longer = vectors % collective.rank_count;
			first = collective.rank * share + min(collective.rank, longer);
			end = first + share + (collective.rank < longer ? 1u : 0u);
		}
		for (uint32_t vector = first + blockIdx.x * blockDim.x + threadIdx.x; vector < end;
		     vector += gridDim.x * blockDim.x) {
			float4 values[ORDERED_COLLECTIVE_MAXIMUM_RANKS];
#pragma unroll
			for (uint32_t rank = 0; rank < ORDERED_COLLECTIVE_MAXIMUM_RANKS; rank++)
				if (rank < collective.rank_count)
					values[rank] = ordered_load4(inputs[rank] + 4u * (uint64_t)vector);
			float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
			for (uint32_t rank = 0; rank < ORDERED_COLLECTIVE_MAXIMUM_RANKS; rank++)
				if (rank < collective.rank_count) {
					sum.x = __fadd_rn(sum.x, values[rank].x);
					sum.y = __fadd_rn(sum.y, values[rank].y);
					sum.z = __fadd_rn(sum.z, values[rank].z);
					sum.w = __fadd_rn(sum.w, values[rank].w);
				}
			const uint2 rounded = make_uint2(bfloat16_bits(sum.x) | bfloat16_bits(sum.y) << 16,
							 bfloat16_bits(sum.z) | bfloat16_bits(sum.w) << 16);
			if (owner_runs) {
#pragma unroll
				for (uint32_t rank = 0; rank < ORDERED_COLLECTIVE_MAXIMUM_RANKS; rank++)
					if (rank < collective.rank_count)
						outputs[rank][vector] = rounded;
			} else {
				own[vector] = rounded;
			}
		}
	}
	if (owner_runs)
		__threadfence_system(); /* this block's peer stores, before it counts itself */
	/* this rank has read (or given up on) every peer's slot: say so, whatever happened. With owner runs the last
	 * block first publishes that this rank's run of the result is in every rank's memory, and waits for every
	 * rank's run to be in this rank's. */
	unsigned char *const done_line = mine + ORDERED_DONE_PHASE * ORDERED_COLLECTIVE_LINE_BYTES;
	unsigned int *const gave_up = reinterpret_cast<unsigned int *>(done_line + ORDERED_LOCAL_GAVE_UP_OFFSET);
	if (owner_runs && !alive && threadIdx.x == 0)
		atomicExch(gave_up, 1u); /* this block stored nothing of the rank's run */
	if (last_block_of_grid(done_line, &last)) {
		if (owner_runs) {
			/* REDUCED says the rank's WHOLE run is in every rank's result: only if every block of the grid was
			 * alive */
			if (threadIdx.x == 0)
				verdict = atomicExch(gave_up, 0u) == 0u ? 1u : 0u;
			__syncthreads();
			const bool whole = verdict != 0u;
			__syncthreads();
			if (whole && threadIdx.x == 0) { /* a rank that gave up leaves its peers to their own deadlines */
				__threadfence_system();
				signal_store(mine + ORDERED_REDUCED_PHASE * ORDERED_COLLECTIVE_LINE_BYTES, sequence);
			}
			if (whole)
				(void)ordered_wait_all(collective, arena, ORDERED_REDUCED_PHASE, sequence, sequence, true, status,
						       &verdict);
		}
		if (threadIdx.x == 0)
			signal_store(done_line, sequence);
	}
}

/* The reduction of the decode step's four launches as ONE launch (struct exl3_layer_route_record explains the slot):
 *   - wait until every rank has said it is done with the slot's previous use (their DONE words arrive in this rank's
 *     own memory, so the wait is local and normally over at once);
 *   - this rank's FP32 row sums (a row's pairs added from +0 in ascending slot order) straight into its rows of the
 *     slot; the last block to finish stores this rank's READY word into EVERY rank's slot (plain peer stores);
 *   - wait for all ranks' READY words, again in this rank's own memory: one trip over NVLink remains, the peer loads
 *     of the rows; the adds in rank order from +0, one rounding to bfloat16;
 *   - the last block stores this rank's DONE word into every rank's slot, whatever happened, so that no peer is held.
 * The blocks wait for a word their own grid's last block stores: the grid is at most ORDERED_B200_MAXIMUM_BLOCKS blocks
 * of 256 threads, which a card always holds at once. Every wait is bounded; one that runs out sets the status block
 * and, before READY, leaves READY unpublished (the peers' own waits then say so). */
template <bool BF16_PAIRS>
__device__ __forceinline__ void publish_reduce_flags(const struct ordered_publish_reduce_arguments &arguments,
						     uint64_t addend_offset, uint64_t row_output_offset,
						     unsigned char *arena)
{
	__shared__ uint32_t verdict, last;
	const struct ordered_collective_arguments &collective = arguments.collective;
	/* the launch may have been given its place on the card while the down products still run: all of them first */
	asm volatile("griddepcontrol.wait;" ::: "memory");
	const struct step_block step = *reinterpret_cast<const struct step_block *>(arena + collective.step_offset);
	const uint64_t sequence = step.sequence;
	if (sequence == 0 || collective.rank_count == 0 || collective.rank_count > ORDERED_COLLECTIVE_MAXIMUM_RANKS)
		return;
	unsigned char *const status = arena + arguments.status_offset;
	unsigned char *const mine = ordered_slot(collective, arena, collective.rank, sequence);
	unsigned char *const local = mine + EXL3_LAYER_LOCAL_LINE * ORDERED_COLLECTIVE_LINE_BYTES;
	unsigned int *const gave_up = reinterpret_cast<unsigned int *>(local + ORDERED_FLAGS_GAVE_UP_OFFSET);
	const uint32_t live_rows = min(step.row_count, collective.element_count / arguments.width);
	const uint32_t row_vectors = arguments.width / 4u, vectors = live_rows * row_vectors;
	/* the slot's previous use */
	const uint64_t previous = *reinterpret_cast<const volatile uint64_t *>(local + ORDERED_LOCAL_PREVIOUS_OFFSET);
	if (threadIdx.x == 0)
		verdict = 1u;
	__syncthreads();
	if (previous >= sequence) {
		if (threadIdx.x == 0) {
			ordered_status_set(status, ORDERED_STATUS_BAD_SEQUENCE, ORDERED_READY_PHASE, collective.rank);
			verdict = 0u;
		}
	} else if (previous != 0 && threadIdx.x < collective.rank_count) {
		const unsigned char *const line = mine + (EXL3_LAYER_DONE_LINE + threadIdx.x) * ORDERED_COLLECTIVE_LINE_BYTES;
		const long long begin = clock64();
		while (signal_load(line) < previous) {
			if ((uint64_t)(clock64() - begin) > collective.deadline_cycles) {
				ordered_status_set(status, ORDERED_STATUS_TIMED_OUT, ORDERED_DONE_PHASE, threadIdx.x);
				atomicExch(&verdict, 0u);
				break;
			}
			__nanosleep(40);
		}
	}
	__syncthreads();
	if (verdict != 0u) {
		float4 *const rows = reinterpret_cast<float4 *>(mine + collective.input_offset);
		for (uint32_t vector = blockIdx.x * blockDim.x + threadIdx.x; vector < vectors; vector += gridDim.x * blockDim.x) {
			const uint32_t row = vector / row_vectors, column = vector % row_vectors;
			float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
			if (BF16_PAIRS) {
				const uint2 *const pairs = reinterpret_cast<const uint2 *>(arena + arguments.pair_output_offset);
				for (uint32_t slot = 0; slot < arguments.pairs_per_row; slot++) {
					const uint2 value = __ldcg(pairs + ((uint64_t)row * arguments.pairs_per_row + slot) * row_vectors + column);
					sum.x = __fadd_rn(sum.x, __uint_as_float(value.x << 16));
					sum.y = __fadd_rn(sum.y, __uint_as_float(value.x & 0xFFFF0000u));
					sum.z = __fadd_rn(sum.z, __uint_as_float(value.y << 16));
					sum.w = __fadd_rn(sum.w, __uint_as_float(value.y & 0xFFFF0000u));
				}
				if (addend_offset != 0) {
					const uint2 value = __ldcg(reinterpret_cast<const uint2 *>(arena + addend_offset) + vector);
					sum.x = __fadd_rn(sum.x, __uint_as_float(value.x << 16));
					sum.y = __fadd_rn(sum.y, __uint_as_float(value.x & 0xFFFF0000u));
					sum.z = __fadd_rn(sum.z, __uint_as_float(value.y << 16));
					sum.w = __fadd_rn(sum.w, __uint_as_float(value.y & 0xFFFF0000u));
				}
				if (row_output_offset != 0)
					reinterpret_cast<float4 *>(arena + row_output_offset)[vector] = sum;
				/* as the publish launch of one "pair" a row enters it: onto +0 */
				sum = make_float4(__fadd_rn(0.0f, sum.x), __fadd_rn(0.0f, sum.y), __fadd_rn(0.0f, sum.z),
						  __fadd_rn(0.0f, sum.w));
			} else {
				const float4 *const pairs = reinterpret_cast<const float4 *>(arena + arguments.pair_output_offset);
				for (uint32_t slot = 0; slot < arguments.pairs_per_row; slot++) {
					const float4 value =
						__ldcg(pairs + ((uint64_t)row * arguments.pairs_per_row + slot) * row_vectors + column);
					sum.x = __fadd_rn(sum.x, value.x);
					sum.y = __fadd_rn(sum.y, value.y);
					sum.z = __fadd_rn(sum.z, value.z);
					sum.w = __fadd_rn(sum.w, value.w);
				}
			}
			rows[vector] = sum;
		}
	} else if (threadIdx.x == 0) {
		atomicExch(gave_up, 1u);
	}
	if (last_block_of_grid(local, &last)) {
		if (threadIdx.x == 0)
			verdict = atomicExch(gave_up, 0u) == 0u ? 1u : 0u;
		__syncthreads();
		if (verdict != 0u) {
			if (threadIdx.x == 0)
				*reinterpret_cast<volatile uint64_t *>(local + ORDERED_LOCAL_PREVIOUS_OFFSET) = sequence;
			if (threadIdx.x < collective.rank_count) {
				__threadfence_system();
				signal_store(ordered_slot(collective, arena, threadIdx.x, sequence) +
						     (EXL3_LAYER_READY_LINE + collective.rank) * ORDERED_COLLECTIVE_LINE_BYTES,
					     sequence);
			}
		}
	}
	/* every rank's READY word, in this rank's own memory */
	__syncthreads();
	if (threadIdx.x == 0)
		verdict = 1u;
	__syncthreads();
	if (threadIdx.x < collective.rank_count) {
		const unsigned char *const line = mine + (EXL3_LAYER_READY_LINE + threadIdx.x) * ORDERED_COLLECTIVE_LINE_BYTES;
		const long long begin = clock64();
		for (;;) {
			const uint64_t seen = signal_load(line);
			if (seen == sequence)
				break;
			if (seen > sequence) {
				ordered_status_set(status, ORDERED_STATUS_BAD_SEQUENCE, ORDERED_READY_PHASE, threadIdx.x);
				atomicExch(&verdict, 0u);
				break;
			}
			if ((uint64_t)(clock64() - begin) > collective.deadline_cycles) {
				ordered_status_set(status, ORDERED_STATUS_TIMED_OUT, ORDERED_READY_PHASE, threadIdx.x);
				atomicExch(&verdict, 0u);
				break;
			}
			__nanosleep(40);
		}
	}
	__syncthreads();
	if (verdict != 0u) {
		const float *inputs[ORDERED_COLLECTIVE_MAXIMUM_RANKS];
#pragma unroll
		for (uint32_t rank = 0; rank < ORDERED_COLLECTIVE_MAXIMUM_RANKS; rank++)
			inputs[rank] = rank < collective.rank_count ?
					       reinterpret_cast<const float *>(ordered_slot(collective, arena, rank, sequence) +
									       collective.input_offset) :
					       nullptr;
		uint2 *const own = reinterpret_cast<uint2 *>(arena + collective.output_offset);
		for (uint32_t vector = blockIdx.x * blockDim.x + threadIdx.x; vector < vectors;
		     vector += gridDim.x * blockDim.x) {
			float4 values[ORDERED_COLLECTIVE_MAXIMUM_RANKS];
#pragma unroll
			for (uint32_t rank = 0; rank < ORDERED_COLLECTIVE_MAXIMUM_RANKS; rank++)
				if (rank < collective.rank_count)
					values[rank] = ordered_load4(inputs[rank] + 4u * (uint64_t)vector);
			float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
			for (uint32_t rank = 0; rank < ORDERED_COLLECTIVE_MAXIMUM_RANKS; rank++)
				if (rank < collective.rank_count) {
					sum.x = __fadd_rn(sum.x, values[rank].x);
					sum.y = __fadd_rn(sum.y, values[rank].y);
					sum.z = __fadd_rn(sum.z, values[rank].z);
					sum.w = __fadd_rn(sum.w, values[rank].w);
				}
			own[vector] = make_uint2(bfloat16_bits(sum.x) | bfloat16_bits(sum.y) << 16,
						 bfloat16_bits(sum.z) | bfloat16_bits(sum.w) << 16);
		}
	}
	/* this rank has read (or given up on) every rank's rows of this step: a second counter of the local line */
	if (last_block_of_grid(local + ORDERED_FLAGS_SECOND_COUNTER_SHIFT, &last) && threadIdx.x < collective.rank_count)
		signal_store(ordered_slot(collective, arena, threadIdx.x, sequence) +
				     (EXL3_LAYER_DONE_LINE + collective.rank) * ORDERED_COLLECTIVE_LINE_BYTES,
			     sequence);
}

extern "C" __global__ void __launch_bounds__(ORDERED_COLLECTIVE_THREADS)
	ordered_publish_reduce_flags(struct ordered_publish_reduce_arguments arguments, unsigned char *arena)
{
	publish_reduce_flags<false>(arguments, 0, 0, arena);
}

extern "C" __global__ void __launch_bounds__(ORDERED_COLLECTIVE_THREADS)
	ordered_publish_reduce_flags_bf16(struct ordered_publish_reduce_bf16_arguments arguments, unsigned char *arena)
{
	publish_reduce_flags<true>(arguments.base, arguments.addend_offset, arguments.row_output_offset, arena);
}

extern "C" __global__ void __launch_bounds__(ORDERED_COLLECTIVE_THREADS)
	ordered_rows_push(struct ordered_rows_push_arguments arguments, unsigned char *arena)
{
	const struct step_block step = *reinterpret_cast<const struct step_block *>(arena + arguments.push.step_offset);
	if (step.sequence == 0 || arguments.width == 0 || arguments.width % 4u != 0 || arguments.pairs_per_row == 0)
		return;
	if (step.row_count > arguments.push.element_count / arguments.width) {
		if (threadIdx.x == 0)
			atomicOr(&exl3_wait_expired, PUSH_EXPIRED_ROWS);
		return;
	}
	struct push_call call;
	call.a = arguments.push;
	call.sequence = step.sequence;
	call.live = step.row_count * arguments.width;
	call.row_width = 0;
	call.pairs = reinterpret_cast<const float4 *>(arena + arguments.pair_output_offset);
	call.result = reinterpret_cast<uint2 *>(arena + arguments.push.output_offset);
	call.pairs_per_row = arguments.pairs_per_row;
	call.row_vectors = arguments.width / 4u;
	push_run(call, arena);
}
