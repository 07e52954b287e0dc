/*
 * kernel_ordered_collective.cu: the four FP32 collectives under the reference's names (kernel file
 * "kernel_ordered_collective": source/kernel_ordered_collective.cu:5-31, .cuh:152-288), one block of 256 threads, the
 * reference's record. Every rank launches the same kernel with the same sequence (read from the step block); a rank's
 * input is in its slot before the launch. Sums are ((+0 + rank 0) + rank 1) + ... with one rounded add per rank,
 * loads first, then adds. The closing DONE phase is an all-rank read-complete barrier, so a slot may be refilled as
 * soon as the kernel has returned on the refilling rank.
 * Remote data is read by peer loads over NVLink; host-mirror routes of the reference's PCIe cards are not offered.
 * Waits are bounded (ordered_device.cuh); these entries have no status block: a failed wait skips the data phase.
 */
#include "ordered_device.cuh"

__device__ __forceinline__ float ordered_rank_sum(const struct ordered_collective_arguments &arguments,
						  unsigned char *arena, uint64_t sequence, uint64_t array_offset,
						  uint32_t element)
{
	float values[ORDERED_COLLECTIVE_MAXIMUM_RANKS];
#pragma unroll
	for (uint32_t rank = 0; rank < ORDERED_COLLECTIVE_MAXIMUM_RANKS; rank++)
		if (rank < arguments.rank_count)
			values[rank] = __ldcg(reinterpret_cast<const float *>(ordered_slot(arguments, arena, rank, sequence) +
									      array_offset) +
					      element);
	float sum = 0.0f;
#pragma unroll
	for (uint32_t rank = 0; rank < ORDERED_COLLECTIVE_MAXIMUM_RANKS; rank++)
		if (rank < arguments.rank_count)
			sum = __fadd_rn(sum, values[rank]);
	return sum;
}

__device__ static void ordered_run(struct ordered_collective_arguments arguments, unsigned char *arena,
				   enum ordered_collective_operation operation)
{
	__shared__ uint32_t verdict;
	const uint64_t sequence = reinterpret_cast<const struct step_block *>(arena + arguments.step_offset)->sequence;
	if (sequence == 0 || arguments.rank_count == 0 || arguments.rank_count > ORDERED_COLLECTIVE_MAXIMUM_RANKS)
		return;
	const uint32_t count = arguments.element_count;
	const uint32_t slice = (count + arguments.rank_count - 1u) / arguments.rank_count;
	unsigned char *const mine = ordered_slot(arguments, arena, arguments.rank, sequence);
	float *const output = reinterpret_cast<float *>(mine + arguments.output_offset);

	ordered_publish(arguments, arena, ORDERED_READY_PHASE, sequence);
	bool alive = ordered_wait_all(arguments, arena, ORDERED_READY_PHASE, sequence, sequence, true, nullptr, &verdict);
	if (alive && operation == ORDERED_ALL_REDUCE) {
		for (uint32_t element = threadIdx.x; element < count; element += blockDim.x)
			output[element] = ordered_rank_sum(arguments, arena, sequence, arguments.input_offset, element);
	} else if (alive && operation == ORDERED_REDUCE_SCATTER) {
		const uint32_t end = min(count, (arguments.rank + 1u) * slice);
		for (uint32_t element = arguments.rank * slice + threadIdx.x; element < end; element += blockDim.x)
			output[element] = ordered_rank_sum(arguments, arena, sequence, arguments.input_offset, element);
	} else if (alive && operation == ORDERED_GATHER) {
		for (uint32_t element = threadIdx.x; element < count; element += blockDim.x)
			output[element] = __ldcg(reinterpret_cast<const float *>(
							 ordered_slot(arguments, arena, element / slice, sequence) +
							 arguments.input_offset) +
						 element);
	} else if (alive) { /* two-shot: reduce the own slice into scratch, publish, gather every slice */
		float *const scratch = reinterpret_cast<float *>(mine + arguments.scratch_offset);
		const uint32_t end = min(count, (arguments.rank + 1u) * slice);
		for (uint32_t element = arguments.rank * slice + threadIdx.x; element < end; element += blockDim.x)
			scratch[element] = ordered_rank_sum(arguments, arena, sequence, arguments.input_offset, element);
		ordered_publish(arguments, arena, ORDERED_REDUCED_PHASE, sequence);
		alive = ordered_wait_all(arguments, arena, ORDERED_REDUCED_PHASE, sequence, sequence, true, nullptr, &verdict);
		if (alive)
			for (uint32_t element = threadIdx.x; element < count; element += blockDim.x)
				output[element] = __ldcg(reinterpret_cast<const float *>(
								 ordered_slot(arguments, arena, element / slice, sequence) +
								 arguments.scratch_offset) +
							 element);
	}
	/* read-complete barrier: nobody returns while a peer may still read this rank's slot */
	ordered_publish(arguments, arena, ORDERED_DONE_PHASE, sequence);
	(void)ordered_wait_all(arguments, arena, ORDERED_DONE_PHASE, sequence, sequence, true, nullptr, &verdict);
}

extern "C" __global__ void __launch_bounds__(ORDERED_COLLECTIVE_THREADS)
	ordered_all_reduce(struct ordered_collective_arguments arguments, unsigned char *arena)
{
	ordered_run(arguments, arena, ORDERED_ALL_REDUCE);
}

extern "C" __global__ void __launch_bounds__(ORDERED_COLLECTIVE_THREADS)
	ordered_two_shot(struct ordered_collective_arguments arguments, unsigned char *arena)
{
	ordered_run(arguments, arena, ORDERED_TWO_SHOT);
}

extern "C" __global__ void __launch_bounds__(ORDERED_COLLECTIVE_THREADS)
	ordered_reduce_scatter(struct ordered_collective_arguments arguments, unsigned char *arena)
{
	ordered_run(arguments, arena, ORDERED_REDUCE_SCATTER);
}

extern "C" __global__ void __launch_bounds__(ORDERED_COLLECTIVE_THREADS)
	ordered_gather(struct ordered_collective_arguments arguments, unsigned char *arena)
{
	ordered_run(arguments, arena, ORDERED_GATHER);
}
