/*
 * kernel_bf16_round_once_ring.cu: the reference's entry ("kernel_bf16_round_once_ring", "bf16_round_once_ring") over struct exact_ring_arguments, as a direct
 * exchange over NVLink (ring_exchange_device.cuh says what each of the three entries computes and how).
 */
#include "ring_exchange_device.cuh"

extern "C" __global__ void __launch_bounds__(EXACT_RING_THREADS)
	bf16_round_once_ring(struct exact_ring_arguments arguments, unsigned char *arena)
{
	ring_exchange<RING_KIND_ROUND_ONCE>(arguments, arena);
}
