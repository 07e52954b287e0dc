/*
 * ordered_push_device.cuh: the one-shot push all-reduce and the owner sums, as one launch of groups x blocks CTAs
 * (reference: source/kernel_ordered_push.cuh:68-372 for the push, source/kernel_tp_exchange.cu:130-249 for the owner
 * sums; there one CTA, or four launches of 64 and 1 CTAs).
 *
 * Group g (blockIdx.x) owns the g-th part of the payload and the g-th 8-byte word of every signal line; its CTAs
 * (blockIdx.y) stride over that part. A CTA stores its share into the inboxes, orders the stores at system scope and
 * counts itself on the group's counter; the last to arrive stores the sequence into word g of this rank's READY line
 * in every rank's slot. Every CTA of the group then waits (on local memory) for word g of every source's READY line,
 * adds its share in ascending rank order from +0, and the group's last CTA to finish publishes DONE the same way and
 * waits for every source's DONE: no rank returns while a peer may still read an inbox or write an output.
 * Arithmetic: one rounded FP32 add a rank; the bfloat16 wire rounds every rank's value (its own too) to nearest even
 * before the adds (cvt.rn.bf16.f32); the owner sums round the FP32 sum ONCE (a not-a-number to 0x7FC0).
 * Every wait is bounded by the record's deadline; a wait that runs out, a sequence not above the slot's last one or
 * a row count beyond the prepared rows sets the kernel file's exl3_wait_expired word (1, 2, 4) and the CTA moves and
 * adds nothing more, yet still counts itself so the counters stay whole. Nothing traps.
 */
#ifndef AB_ORDERED_PUSH_DEVICE_CUH
#define AB_ORDERED_PUSH_DEVICE_CUH

#include "ordered_device.cuh"

#define PUSH_EXPIRED_WAIT 1u
#define PUSH_EXPIRED_SEQUENCE 2u
#define PUSH_EXPIRED_ROWS 4u
#define PUSH_WORD_BYTES 8u
#define PUSH_COUNTER_OFFSET 64u /* inside this rank's own READY and DONE lines: a 32-bit counter a group */

/* read by the host after a queue has drained (backend_b200_waits_expired); sticky */
__device__ unsigned int exl3_wait_expired;

struct push_call {
	struct ordered_push_arguments a;
	uint64_t sequence;
	uint32_t live; /* elements exchanged by this launch */
	uint32_t row_width; /* the owner sums: elements of a row; 0: the push */
	/* the expert layer's form (push_rows): the values are row sums of pair outputs, added here from +0 in ascending
	 * slot order; the sums over the ranks are rounded once to bfloat16 and kept by every rank at `result`; the DONE
	 * barrier moves from the end of this use of the slot to the beginning of the next */
	const float4 *pairs; /* FP32 [rows * pairs_per_row][row_vectors * 4], or NULL */
	uint2 *result; /* bfloat16 [rows][row_vectors * 4] in this rank's memory, or NULL */
	uint32_t pairs_per_row;
	uint32_t row_vectors;
};

__device__ __forceinline__ unsigned char *push_slot(const struct ordered_push_arguments &a, unsigned char *arena,
						    uint32_t rank, uint64_t sequence)
{
	unsigned char *region;
	if (rank == a.rank) {
		region = arena + a.region_offset;
	} else {
		const struct ordered_collective_peer *const peers =
			reinterpret_cast<const struct ordered_collective_peer *>(arena + a.peer_table_offset);
		region = reinterpret_cast<unsigned char *>(peers[rank].arena_address) + peers[rank].region_offset;
	}
	return region + (sequence & 1u) * a.parity_stride;
}

__device__ __forceinline__ unsigned char *push_line(const struct ordered_push_arguments &a, unsigned char *slot,
						    uint32_t phase, uint32_t source)
{
	return slot + ((uint64_t)phase * a.rank_count + source) * ORDERED_COLLECTIVE_LINE_BYTES;
}

/* cvt.rn.bf16x2.f32 d, a, b: a in the upper half, b in the lower */
__device__ __forceinline__ uint32_t push_bfloat16_pair(float low, float high)
{
	uint32_t pair;
	asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(pair) : "f"(high), "f"(low));
	return pair;
}

__device__ __forceinline__ void push_store4(unsigned char *inbox, uint32_t format, uint32_t vector, float4 value)
{
	if (format == ORDERED_PUSH_FP32)
		reinterpret_cast<float4 *>(inbox)[vector] = value;
	else
		reinterpret_cast<uint2 *>(inbox)[vector] =
			make_uint2(push_bfloat16_pair(value.x, value.y), push_bfloat16_pair(value.z, value.w));
}

__device__ __forceinline__ void push_store1(unsigned char *inbox, uint32_t format, uint32_t element, float value)
{
	if (format == ORDERED_PUSH_FP32)
		reinterpret_cast<float *>(inbox)[element] = value;
	else
		reinterpret_cast<uint16_t *>(inbox)[element] = (uint16_t)push_bfloat16_pair(value, 0.0f);
}

__device__ __forceinline__ float4 push_load4(const unsigned char *inbox, uint32_t format, uint32_t vector)
{
	if (format == ORDERED_PUSH_FP32)
		return __ldcg(reinterpret_cast<const float4 *>(inbox) + vector);
	const uint2 pairs = __ldcg(reinterpret_cast<const uint2 *>(inbox) + vector);
	return make_float4(__uint_as_float(pairs.x << 16), __uint_as_float(pairs.x & 0xFFFF0000u),
			   __uint_as_float(pairs.y << 16), __uint_as_float(pairs.y & 0xFFFF0000u));
}

__device__ __forceinline__ float push_load1(const unsigned char *inbox, uint32_t format, uint32_t element)
{
	if (format == ORDERED_PUSH_FP32)
		return __ldcg(reinterpret_cast<const float *>(inbox) + element);
	return __uint_as_float((uint32_t)__ldcg(reinterpret_cast<const uint16_t *>(inbox) + element) << 16);
}

/* The group's last CTA to arrive here learns so (every thread of it). The CTA's peer stores are ordered first. */
__device__ __forceinline__ bool push_group_last(unsigned char *own_line, uint32_t *shared_flag)
{
	__threadfence_system();
	__syncthreads();
	if (threadIdx.x == 0) {
		unsigned int *const counter = reinterpret_cast<unsigned int *>(own_line + PUSH_COUNTER_OFFSET) + blockIdx.x;
		const unsigned int arrived = atomicAdd(counter, 1u) + 1u;
		*shared_flag = arrived == gridDim.y ? 1u : 0u;
		if (arrived == gridDim.y) {
			*counter = 0u; /* for the slot's next use */
			__threadfence();
		}
	}
	__syncthreads();
	return *shared_flag != 0;
}

/* threads 0 .. rank_count - 1: word `group` of this rank's line of `phase`, in every rank's slot */
__device__ __forceinline__ void push_signal_all(const struct push_call &call, unsigned char *arena, uint32_t phase)
{
	if (threadIdx.x < call.a.rank_count) {
		__threadfence_system();
		signal_store(push_line(call.a, push_slot(call.a, arena, threadIdx.x, call.sequence), phase, call.a.rank) +
				     PUSH_WORD_BYTES * blockIdx.x,
			     call.sequence);
	}
}

/* every thread calls; true when word `group` of every source's line of `phase` in this rank's slot holds `wanted`
 * (exact: a phase of this use of the slot) or at least `wanted` (the DONE of the slot's previous use) */
__device__ __forceinline__ bool push_wait_all(const struct push_call &call, unsigned char *arena, uint32_t phase,
					      uint64_t wanted, bool exact, uint32_t *verdict)
{
	if (threadIdx.x == 0)
		*verdict = 1;
	__syncthreads();
	if (threadIdx.x < call.a.rank_count) {
		const unsigned char *const word =
			push_line(call.a, push_slot(call.a, arena, call.a.rank, call.sequence), phase, threadIdx.x) +
			PUSH_WORD_BYTES * blockIdx.x;
		const long long begin = clock64();
		for (;;) {
			const uint64_t seen = signal_load(word);
			if (exact ? seen == wanted : seen >= wanted)
				break;
			if (seen > wanted) {
				atomicOr(&exl3_wait_expired, PUSH_EXPIRED_SEQUENCE);
				atomicExch(verdict, 0u);
				break;
			}
			if ((uint64_t)(clock64() - begin) > call.a.deadline_cycles) {
				atomicOr(&exl3_wait_expired, PUSH_EXPIRED_WAIT);
				atomicExch(verdict, 0u);
				break;
			}
		}
	}
	__syncthreads();
	return *verdict != 0;
}

/* The vectors [begin, end) of part `group` of `groups` of the vectors [first, last) */
__device__ __forceinline__ void push_part(uint32_t first, uint32_t last, uint32_t &begin, uint32_t &end)
{
	const uint64_t length = last - first;
	begin = first + (uint32_t)(length * blockIdx.x / gridDim.x);
	end = first + (uint32_t)(length * (blockIdx.x + 1u) / gridDim.x);
}

/* the owner sums: the first vector of the rows rank `shard` owns (source/kernel_tp_exchange.cu:122-128) */
__device__ __forceinline__ uint32_t push_owner_first(const struct push_call &call, uint32_t shard)
{
	const uint32_t rows = call.live / call.row_width;
	return (uint32_t)((uint64_t)rows * shard / call.a.rank_count) * (call.row_width / 4u);
}

__device__ static void push_run(const struct push_call &call, unsigned char *arena)
{
	__shared__ uint32_t verdict, last;
	const struct ordered_push_arguments &a = call.a;
	if (call.sequence == 0 || a.rank_count == 0 || a.rank_count > ORDERED_COLLECTIVE_MAXIMUM_RANKS ||
	    a.rank >= a.rank_count || blockDim.x != ORDERED_COLLECTIVE_THREADS || gridDim.x > ORDERED_PUSH_GROUPS)
		return;
	unsigned char *const mine = push_slot(a, arena, a.rank, call.sequence);
	unsigned char *const ready_line = push_line(a, mine, ORDERED_PUSH_READY, a.rank);
	unsigned char *const done_line = push_line(a, mine, ORDERED_PUSH_DONE, a.rank);
	/* a sequence must be above the last one this slot carried: the group's own word is only written once every CTA
	 * of the group has passed this check */
	bool alive = *reinterpret_cast<const volatile uint64_t *>(ready_line + PUSH_WORD_BYTES * blockIdx.x) <
		     call.sequence;
	if (!alive && threadIdx.x == 0)
		atomicOr(&exl3_wait_expired, PUSH_EXPIRED_SEQUENCE);
	const bool owner = call.row_width != 0;
	const bool rows_form = call.pairs != nullptr;
	const bool aligned = ((a.input_offset | a.output_offset | a.inbox_offset | a.inbox_rank_stride) % 16u) == 0;
	const uint32_t vectors = aligned ? call.live / 4u : 0u;
	const float *const input = reinterpret_cast<const float *>(mine + a.input_offset);
	const uint32_t lane = blockIdx.y * blockDim.x + threadIdx.x, lanes = gridDim.y * blockDim.x;
	if (rows_form && alive) {
		/* the slot's previous use: every rank must have read its inboxes of it before they are written again */
		const uint64_t previous = *reinterpret_cast<const volatile uint64_t *>(ready_line + PUSH_WORD_BYTES * blockIdx.x);
		if (previous != 0)
			alive = push_wait_all(call, arena, ORDERED_PUSH_DONE, previous, false, &verdict);
	}

	/* ---- this rank's values into the inboxes, from the next rank on ---- */
	if (alive && owner) {
		for (uint32_t step = 1; step <= a.rank_count; step++) {
			const uint32_t destination = (a.rank + step) % a.rank_count;
			unsigned char *const inbox = push_slot(a, arena, destination, call.sequence) + a.inbox_offset +
						     (uint64_t)a.rank * a.inbox_rank_stride;
			uint32_t begin, end;
			push_part(push_owner_first(call, destination), push_owner_first(call, destination + 1u), begin, end);
			for (uint32_t vector = begin + lane; vector < end; vector += lanes)
				push_store4(inbox, a.payload_format, vector,
					    __ldg(reinterpret_cast<const float4 *>(input) + vector));
		}
	} else if (alive) {
		unsigned char *inboxes[ORDERED_COLLECTIVE_MAXIMUM_RANKS];
#pragma unroll
		for (uint32_t step = 0; step < ORDERED_COLLECTIVE_MAXIMUM_RANKS; step++)
			inboxes[step] = step < a.rank_count ?
						push_slot(a, arena, (a.rank + 1u + step) % a.rank_count, call.sequence) +
							a.inbox_offset + (uint64_t)a.rank * a.inbox_rank_stride :
						nullptr;
		uint32_t begin, end;
		push_part(0, vectors, begin, end);
		for (uint32_t vector = begin + lane; vector < end; vector += lanes) {
			float4 value;
			if (rows_form) {
				const uint32_t row = vector / call.row_vectors, column = vector % call.row_vectors;
				value = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
				for (uint32_t slot = 0; slot < call.pairs_per_row; slot++) {
					const float4 pair =
						call.pairs[((uint64_t)row * call.pairs_per_row + slot) * call.row_vectors + column];
					value.x = __fadd_rn(value.x, pair.x);
					value.y = __fadd_rn(value.y, pair.y);
					value.z = __fadd_rn(value.z, pair.z);
					value.w = __fadd_rn(value.w, pair.w);
				}
			} else {
				value = __ldg(reinterpret_cast<const float4 *>(input) + vector);
			}
#pragma unroll
			for (uint32_t step = 0; step < ORDERED_COLLECTIVE_MAXIMUM_RANKS; step++)
				if (step < a.rank_count)
					push_store4(inboxes[step], a.payload_format, vector, value);
		}
		if (blockIdx.x == 0 && !rows_form) /* what no vector covers: group 0's */
			for (uint32_t element = vectors * 4u + lane; element < call.live; element += lanes)
				for (uint32_t step = 0; step < a.rank_count; step++)
					push_store1(inboxes[step], a.payload_format, element, input[element]);
	}
	/* a group that moved nothing publishes nothing: its peers' waits run out and report, rather than add stale bytes */
	if (push_group_last(ready_line, &last) && alive)
		push_signal_all(call, arena, ORDERED_PUSH_READY);
	alive = alive && push_wait_all(call, arena, ORDERED_PUSH_READY, call.sequence, true, &verdict);

	/* ---- the adds, ascending ranks from +0 ---- */
	if (alive) {
		const unsigned char *const inboxes = mine + a.inbox_offset;
		uint32_t begin, end;
		if (owner)
			push_part(push_owner_first(call, a.rank), push_owner_first(call, a.rank + 1u), begin, end);
		else
			push_part(0, vectors, begin, end);
		for (uint32_t vector = begin + lane; vector < end; vector += lanes) {
			float4 values[ORDERED_COLLECTIVE_MAXIMUM_RANKS];
#pragma unroll
			for (uint32_t source = 0; source < ORDERED_COLLECTIVE_MAXIMUM_RANKS; source++)
				if (source < a.rank_count)
					values[source] = push_load4(inboxes + (uint64_t)source * a.inbox_rank_stride,
								    a.payload_format, vector);
			float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
			for (uint32_t source = 0; source < ORDERED_COLLECTIVE_MAXIMUM_RANKS; source++)
				if (source < a.rank_count) {
					sum.x = __fadd_rn(sum.x, values[source].x);
					sum.y = __fadd_rn(sum.y, values[source].y);
					sum.z = __fadd_rn(sum.z, values[source].z);
					sum.w = __fadd_rn(sum.w, values[source].w);
				}
			if (!owner && !rows_form) {
				reinterpret_cast<float4 *>(mine + a.output_offset)[vector] = sum;
				continue;
			}
			const uint2 rounded = make_uint2(bfloat16_bits(sum.x) | bfloat16_bits(sum.y) << 16,
							 bfloat16_bits(sum.z) | bfloat16_bits(sum.w) << 16);
			if (rows_form)
				call.result[vector] = rounded;
			else
				for (uint32_t step = 1; step <= a.rank_count; step++)
					reinterpret_cast<uint2 *>(push_slot(a, arena, (a.rank + step) % a.rank_count, call.sequence) +
								  a.output_offset)[vector] = rounded;
		}
		if (!owner && !rows_form && blockIdx.x == 0)
			for (uint32_t element = vectors * 4u + lane; element < call.live; element += lanes) {
				float sum = 0.0f;
				for (uint32_t source = 0; source < a.rank_count; source++)
					sum = __fadd_rn(sum, push_load1(inboxes + (uint64_t)source * a.inbox_rank_stride,
									a.payload_format, element));
				reinterpret_cast<float *>(mine + a.output_offset)[element] = sum;
			}
	}
	/* ---- every rank has read its inboxes (and stored its sums) before any returns; the expert layer's form only
	 * says so, and looks at the others' word before the slot's next use ---- */
	if (push_group_last(done_line, &last)) {
		push_signal_all(call, arena, ORDERED_PUSH_DONE);
		if (alive && !rows_form)
			(void)push_wait_all(call, arena, ORDERED_PUSH_DONE, call.sequence, true, &verdict);
	}
}

#endif
