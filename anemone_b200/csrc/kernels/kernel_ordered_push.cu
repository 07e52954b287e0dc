/*
 * kernel_ordered_push.cu: the one-shot push all-reduce under the reference's name (kernel file "kernel_ordered_push",
 * entry "ordered_push": source/kernel_ordered_push.cu:5-13), its record, its arithmetic; the launch is this library's
 * (groups x blocks CTAs, see ordered_push_device.cuh). Every rank launches it with the same sequence, read from the
 * step block; all element_count elements are exchanged.
 */
#include "ordered_push_device.cuh"

/* the plain push: no live-row count, no owner shards, no row sums, FP32 sums kept in the slot */
__device__ __forceinline__ void plain_push_describe(const struct ordered_push_arguments &record,
						    const unsigned char *arena, struct push_call *call)
{
	const struct step_block *const step = reinterpret_cast<const struct step_block *>(arena + record.step_offset);
	call->a = record;
	call->live = record.element_count;
	call->sequence = step->sequence;
	call->row_width = call->pairs_per_row = call->row_vectors = 0;
	call->pairs = nullptr;
	call->result = nullptr;
}

extern "C" __global__ void __launch_bounds__(ORDERED_COLLECTIVE_THREADS)
	ordered_push(struct ordered_push_arguments arguments, unsigned char *arena)
{
	struct push_call call;
	plain_push_describe(arguments, arena, &call);
	push_run(call, arena);
}
