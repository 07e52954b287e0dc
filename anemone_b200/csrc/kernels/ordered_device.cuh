/*
 * ordered_device.cuh: signals and bounded waits of the fixed-order reduction kernels.
 *
 * A signal line is 128 bytes, written only by the rank that owns it. Its first 8 bytes hold the step sequence of the
 * owner's last completed phase on this slot; a line is published with a system-scope release store after the
 * payload stores, and polled by the other ranks over NVLink with a system-scope acquire load. Sequences are
 * positive and strictly increasing, so "line == my sequence" means the owner reached this phase of this step, and
 * "line > my sequence" that the slot was overwritten (reported, never consumed).
 * Every wait is bounded by the record's deadline in device clock cycles; a wait that runs out writes the status block
 * and the kernel skips every further remote access. Nothing traps.
 */
#ifndef AB_ORDERED_DEVICE_CUH
#define AB_ORDERED_DEVICE_CUH

#include <stdint.h>

#include "anemone_b200_records.h"

#define ORDERED_READY_PHASE 0u
#define ORDERED_REDUCED_PHASE 1u
#define ORDERED_DONE_PHASE 2u
#define ORDERED_LOCAL_COUNTER_OFFSET 64u /* inside a line: a counter only the owner's own CTAs touch */
#define ORDERED_LOCAL_PREVIOUS_OFFSET 72u /* inside the READY line: the sequence of the slot's previous use */
#define ORDERED_LOCAL_GAVE_UP_OFFSET 80u /* inside a line: set by a block of the owner's grid whose wait ran out */
/* the local line of the flags form (ordered_publish_reduce_flags): a counter at 64, the previous sequence at 72, a
 * second counter at 64 + 16, the gave-up word at 88 */
#define ORDERED_FLAGS_SECOND_COUNTER_SHIFT 16u
#define ORDERED_FLAGS_GAVE_UP_OFFSET 88u

__device__ __forceinline__ void signal_store(unsigned char *line, uint64_t sequence)
{
	asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(line), "l"(sequence) : "memory");
}

__device__ __forceinline__ uint64_t signal_load(const unsigned char *line)
{
	uint64_t value;
	asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(value) : "l"(line) : "memory");
	return value;
}

__device__ __forceinline__ const struct ordered_collective_peer *
ordered_peers(const struct ordered_collective_arguments &arguments, const unsigned char *arena)
{
	return reinterpret_cast<const struct ordered_collective_peer *>(arena + arguments.peer_table_offset);
}

/* the slot of `rank` for this sequence, as this card reaches it */
__device__ __forceinline__ unsigned char *ordered_slot(const struct ordered_collective_arguments &arguments,
						       unsigned char *arena, uint32_t rank, uint64_t sequence)
{
	unsigned char *region;
	if (rank == arguments.rank) {
		region = arena + arguments.region_offset;
	} else {
		const struct ordered_collective_peer *const peers = ordered_peers(arguments, arena);
		region = reinterpret_cast<unsigned char *>(peers[rank].arena_address) + peers[rank].region_offset;
	}
	return region + (sequence & 1u) * arguments.parity_stride;
}

__device__ __forceinline__ void ordered_status_set(unsigned char *status, uint32_t code, uint32_t phase, uint32_t rank)
{
	if (status == nullptr)
		return;
	uint32_t *const words = reinterpret_cast<uint32_t *>(status);
	if (atomicCAS(&words[0], ORDERED_STATUS_OK, code) == ORDERED_STATUS_OK) {
		words[1] = phase;
		words[2] = rank;
	}
}

/* Wait until rank's line of `phase` holds at least `sequence` (exactly it, for a phase of this step). true: it does.
 * false: the deadline passed or the slot was overwritten; the status block says which. One thread calls this. */
__device__ __forceinline__ bool ordered_wait_line(const struct ordered_collective_arguments &arguments,
						  unsigned char *arena, uint32_t rank, uint32_t phase,
						  uint64_t slot_sequence, uint64_t wanted, bool exact, unsigned char *status)
{
	const unsigned char *const line =
		ordered_slot(arguments, arena, rank, slot_sequence) + phase * ORDERED_COLLECTIVE_LINE_BYTES;
	const long long begin = clock64();
	for (;;) {
		const uint64_t seen = signal_load(line);
		if (exact ? seen == wanted : seen >= wanted)
			return true;
		if (exact && seen > wanted) {
			ordered_status_set(status, ORDERED_STATUS_BAD_SEQUENCE, phase, rank);
			return false;
		}
		if ((uint64_t)(clock64() - begin) > arguments.deadline_cycles) {
			ordered_status_set(status, ORDERED_STATUS_TIMED_OUT, phase, rank);
			return false;
		}
		__nanosleep(100);
	}
}

/* Lanes 0 .. rank_count - 1 of warp 0 each wait for one rank; the block learns the verdict. All threads call. */
__device__ __forceinline__ bool ordered_wait_all(const struct ordered_collective_arguments &arguments,
						 unsigned char *arena, uint32_t phase, uint64_t slot_sequence,
						 uint64_t wanted, bool exact, unsigned char *status, uint32_t *verdict)
{
	if (threadIdx.x == 0)
		*verdict = 1;
	__syncthreads();
	if (threadIdx.x < arguments.rank_count &&
	    !ordered_wait_line(arguments, arena, threadIdx.x, phase, slot_sequence, wanted, exact, status))
		atomicExch(verdict, 0u);
	__syncthreads();
	return *verdict != 0;
}

/* Publish this rank's line of `phase` once the whole block's payload stores are visible system-wide. */
__device__ __forceinline__ void ordered_publish(const struct ordered_collective_arguments &arguments,
						unsigned char *arena, uint32_t phase, uint64_t sequence)
{
	__threadfence_system();
	__syncthreads();
	if (threadIdx.x == 0)
		signal_store(ordered_slot(arguments, arena, arguments.rank, sequence) + phase * ORDERED_COLLECTIVE_LINE_BYTES,
			     sequence);
}

/* A peer's published FP32 payload: never through L1 */
__device__ __forceinline__ float4 ordered_load4(const float *pointer)
{
	return __ldcg(reinterpret_cast<const float4 *>(pointer));
}

/* source/kernel_linear_common.cuh:186-191: nearest-even, a not-a-number to 0x7FC0 */
__device__ __forceinline__ uint32_t bfloat16_bits(float value)
{
	const uint32_t bits = __float_as_uint(value);
	return (bits & 0x7FFFFFFFu) > 0x7F800000u ? 0x7FC0u : (bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16;
}

#endif
