/*
 * kernel_exact_ring.cu: the reference's entry ("kernel_exact_ring", "exact_ring") over struct exact_ring_arguments, as a direct
 * exchange over NVLink (ring_exchange_device.cuh says what each of the three entries computes and how).
 */
#include "ring_exchange_device.cuh"

extern "C" __global__ void __launch_bounds__(EXACT_RING_THREADS)
	exact_ring(struct exact_ring_arguments arguments, unsigned char *arena)
{
	ring_exchange<RING_KIND_EXACT>(arguments, arena);
}
