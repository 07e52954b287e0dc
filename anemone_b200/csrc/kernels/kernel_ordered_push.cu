/*
 * kernel_ordered_push.cu: the one-shot push all-reduce under the reference's name (kernel file "kernel_ordered_push",
 * entry "ordered_push": source/kernel_ordered_push.cu:5-13), its record, its arithmetic; the launch is this library's
 * (groups x blocks CTAs, see ordered_push_device.cuh). Every rank launches it with the same sequence, read from the
 * step block; all element_count elements are exchanged.
 */
#include "ordered_push_device.cuh"

extern "C" __global__ void __launch_bounds__(ORDERED_COLLECTIVE_THREADS)
	ordered_push(struct ordered_push_arguments arguments, unsigned char *arena)
{
	struct push_call call;
	call.a = arguments;
	call.sequence = reinterpret_cast<const struct step_block *>(arena + arguments.step_offset)->sequence;
	call.live = arguments.element_count;
	call.row_width = 0;
	call.pairs = nullptr;
	call.result = nullptr;
	call.pairs_per_row = call.row_vectors = 0;
	push_run(call, arena);
}
