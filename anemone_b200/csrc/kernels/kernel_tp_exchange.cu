/*
 * kernel_tp_exchange.cu: the exchange of a tensor-parallel layer site (kernel file "kernel_tp_exchange";
 * source/kernel_tp_exchange.cu:25-46 for the layer's sequence and live rows, :62-128 for the push forms, :130-249 for
 * the owner sums).
 *   tp_exchange          the push: every rank gets the FP32 sums of the step's live rows
 *   tp_exchange_owner    the owner sums: FP32 adds in rank order on the rows' owner, ONE rounding to bfloat16, the
 *                        bfloat16 rows stored into every rank's output array
 *   tp_exchange_settled  nothing: fills the places of the reference's READY / SUM / DONE launches in a caller's table
 *                        of four, the whole exchange being the first launch here
 * A step's sequence s becomes 2 (s layer_count + layer) + (s & 1): increasing over the layers of a step and over
 * steps, with the step's parity, which selects the slot.
 */
#include "ordered_push_device.cuh"

__device__ __forceinline__ bool exchange_call(const struct tp_exchange_arguments &arguments, const unsigned char *arena,
					      bool owner, struct push_call *call)
{
	const struct step_block step = *reinterpret_cast<const struct step_block *>(arena + arguments.collective.step_offset);
	if (step.sequence == 0 || arguments.layer_count == 0 || arguments.layer >= arguments.layer_count ||
	    arguments.row_width == 0 || arguments.row_width % 4u != 0 || arguments.reserved_zero != 0 ||
	    step.sequence > (UINT64_MAX / 2u - arguments.layer) / arguments.layer_count)
		return false;
	if (step.row_count > arguments.collective.element_count / arguments.row_width) {
		if (threadIdx.x == 0)
			atomicOr(&exl3_wait_expired, PUSH_EXPIRED_ROWS);
		return false;
	}
	call->a = arguments.collective;
	call->sequence = (step.sequence * arguments.layer_count + arguments.layer) * 2u + (step.sequence & 1u);
	call->live = step.row_count * arguments.row_width;
	call->row_width = owner ? arguments.row_width : 0u;
	call->pairs = nullptr;
	call->result = nullptr;
	call->pairs_per_row = call->row_vectors = 0;
	return true;
}

extern "C" __global__ void __launch_bounds__(ORDERED_COLLECTIVE_THREADS)
	tp_exchange(struct tp_exchange_arguments arguments, unsigned char *arena)
{
	struct push_call call;
	if (exchange_call(arguments, arena, false, &call))
		push_run(call, arena);
}

extern "C" __global__ void __launch_bounds__(ORDERED_COLLECTIVE_THREADS)
	tp_exchange_owner(struct tp_exchange_arguments arguments, unsigned char *arena)
{
	struct push_call call;
	if (exchange_call(arguments, arena, true, &call))
		push_run(call, arena);
}

extern "C" __global__ void tp_exchange_settled(struct tp_exchange_arguments arguments, unsigned char *arena)
{
	(void)arguments;
	(void)arena;
}
