/*
 * ring_exchange_device.cuh: the reference's three output-axis exchanges between the ranks of a tensor-parallel group
 * (struct exact_ring_arguments, include/anemone/exact_ring_records.h) as DIRECT exchanges over NVLink / NVSwitch:
 *   exact_ring            mode 0: a lossless gather of every owner's packs (source/kernel_exact_ring.cu);
 *                         modes 1, 2: the BF16 sum whose additions round to bfloat16 one after the other in the order
 *                         the reference's ring visits the ranks (source/kernel_cut_through.cuh:368-431)
 *   bf16_compressed_ring  the same sum with every pack on the wire in the lossless exponent-delta code
 *                         (source/kernel_bf16_compressed_ring.cu, source/bf16_wire_codec.h)
 *   bf16_round_once_ring  the owners' FP32 sums in rank order from +0, rounded ONCE to bfloat16
 *                         (source/kernel_bf16_round_once_ring.cu:70-195)
 * The reference passes a pack from neighbour to neighbour of a ring of four PCIe cards. On NVSwitch every peer is as
 * near as a neighbour, so here a rank stores its packs of owner o's part straight into o's bank, o computes what the
 * ring's hops would have computed, in their order, and stores the result straight into every rank's bank: two trips
 * instead of 2 (R - 1) hops, the same bits. Record, entry names, bank sizes, the grid (at most 16 blocks of 256
 * threads, block b owning the same packs on every rank, so that no block waits for another block of its own grid),
 * generations in the bank's first 128 bytes: the reference's. Differences: 2, 4 or 8 ranks (reserved_words[0], 0
 * meaning the reference's 4); a deadline or a bad record sets the bank's status word and the kernel returns, nothing
 * traps.
 */
#ifndef AB_RING_EXCHANGE_DEVICE_CUH
#define AB_RING_EXCHANGE_DEVICE_CUH

#include <stdint.h>

#include "anemone_b200_records.h"
#include "anemone_b200_wire_codec.h"

#define RING_KIND_EXACT 0u
#define RING_KIND_COMPRESSED 1u
#define RING_KIND_ROUND_ONCE 2u

struct ring_world {
	struct exact_ring_arguments arguments;
	unsigned char *arena;
	const struct ordered_collective_peer *peers;
	uint32_t ranks, generation;
	long long start;
	unsigned int *status;
};

__device__ __forceinline__ unsigned char *ring_bank(const struct ring_world &w, uint32_t rank)
{
	if (rank == w.arguments.rank)
		return w.arena + w.arguments.bank_offset;
	return reinterpret_cast<unsigned char *>(w.peers[rank].arena_address + w.peers[rank].region_offset +
						 w.arguments.peer_bank_delta);
}

__device__ __forceinline__ void ring_release(uint32_t *address, uint32_t value)
{
	asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(address), "r"(value) : "memory");
}

__device__ __forceinline__ uint32_t ring_acquire(const uint32_t *address)
{
	uint32_t value;
	asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(value) : "l"(address) : "memory");
	return value;
}

__device__ __forceinline__ uint4 ring_load(const uint4 *address)
{
	uint4 value;
	asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
		     : "=r"(value.x), "=r"(value.y), "=r"(value.z), "=r"(value.w)
		     : "l"(address)
		     : "memory");
	return value;
}

__device__ __forceinline__ void ring_store(uint4 *address, uint4 value)
{
	asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(address), "r"(value.x), "r"(value.y),
		     "r"(value.z), "r"(value.w)
		     : "memory");
}

/* true while the wait may go on; false once the deadline has passed (the status word then says so) */
__device__ __forceinline__ bool ring_in_time(const struct ring_world &w)
{
	if ((uint64_t)(clock64() - w.start) < w.arguments.deadline_cycles)
		return true;
	atomicExch(w.status, EXACT_RING_STATUS_DEADLINE);
	return false;
}

/* where owner `owner`'s pack `pack` lies in the input and the output of the sums: owner-major, or with column owners
 * [row][owner][the row's packs] (source/kernel_cut_through.cuh:299-307, for any rank count) */
__device__ __forceinline__ uint64_t ring_place(const struct ring_world &w, uint32_t row_packs, uint32_t owner,
					       uint32_t pack)
{
	if (row_packs == 0)
		return (uint64_t)owner * w.arguments.packs_per_owner + pack;
	const uint32_t row = pack / row_packs;
	return ((uint64_t)row * w.ranks + owner) * row_packs + (pack - row * row_packs);
}

/* the gather's place of owner's pack in the output: owner-major, or [vector][all owners' channels] */
__device__ __forceinline__ uint64_t ring_gather_place(const struct ring_world &w, uint32_t owner, uint32_t pack)
{
	const uint32_t packs = w.arguments.packs_per_owner, vectors = w.arguments.vectors;
	if (vectors == 0)
		return (uint64_t)owner * packs + pack;
	const uint32_t row_packs = packs / vectors, row = pack / row_packs;
	return ((uint64_t)row * w.ranks + owner) * row_packs + (pack - row * row_packs);
}

/* the reference's transport sends a +0 half as -0 (its zero word means "nothing arrived yet"): the sums see that */
__device__ __forceinline__ uint32_t ring_nonzero_halves(uint32_t word)
{
	const uint32_t low = word & 0xFFFFu, high = word >> 16;
	return (low == 0 ? 0x8000u : low) | ((high == 0 ? 0x8000u : high) << 16);
}

__device__ __forceinline__ uint4 ring_nonzero(uint4 v)
{
	return make_uint4(ring_nonzero_halves(v.x), ring_nonzero_halves(v.y), ring_nonzero_halves(v.z),
			  ring_nonzero_halves(v.w));
}

/* two bfloat16 additions, each one rounding (the reference: fma.rn.bf16x2 with ones, kernel_cut_through.cuh:277-285) */
__device__ __forceinline__ uint32_t ring_add_pair(uint32_t left, uint32_t right)
{
	uint32_t result;
	asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(result) : "r"(left), "r"(0x3F803F80u), "r"(right));
	return result;
}

__device__ __forceinline__ uint4 ring_add(uint4 a, uint4 b)
{
	return make_uint4(ring_add_pair(a.x, b.x), ring_add_pair(a.y, b.y), ring_add_pair(a.z, b.z),
			  ring_add_pair(a.w, b.w));
}

__device__ __forceinline__ uint32_t ring_bfloat16_bits(float value)
{
	const uint32_t bits = __float_as_uint(value);
	return (bits & 0x7FFFFFFFu) > 0x7F800000u ? 0x7FC0u : (bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16;
}

/* ---- the uncompressed kinds: planes of uint4 [rank][pack] behind the metadata, then flags [phase][rank][block] ---- */

__device__ __forceinline__ uint4 *ring_plane(unsigned char *bank, const struct ring_world &w, uint32_t plane)
{
	return reinterpret_cast<uint4 *>(bank + EXACT_RING_METADATA_BYTES) +
	       (uint64_t)plane * w.ranks * w.arguments.packs_per_owner;
}

__device__ __forceinline__ uint32_t *ring_flag(unsigned char *bank, const struct ring_world &w, uint32_t planes,
					       uint32_t phase, uint32_t rank)
{
	uint32_t *const flags = reinterpret_cast<uint32_t *>(ring_plane(bank, w, planes));
	return flags + (phase * w.ranks + rank) * EXACT_RING_BLOCKS + blockIdx.x;
}

/* Every thread's stores are ordered system-wide, then this block's flag of `phase` goes to every rank, then the block
 * waits for every rank's flag of the same block. All threads call; false after a deadline. */
__device__ __forceinline__ bool ring_phase(const struct ring_world &w, uint32_t planes, uint32_t phase)
{
	__shared__ uint32_t good;
	__threadfence_system();
	if (threadIdx.x == 0)
		good = 1u;
	__syncthreads();
	if (threadIdx.x < w.ranks) {
		ring_release(ring_flag(ring_bank(w, threadIdx.x), w, planes, phase, w.arguments.rank), w.generation);
		const uint32_t *const mine = ring_flag(ring_bank(w, w.arguments.rank), w, planes, phase, threadIdx.x);
		while (ring_acquire(mine) != w.generation)
			if (!ring_in_time(w)) {
				atomicExch(&good, 0u);
				break;
			}
	}
	__syncthreads();
	return good != 0u;
}

/* the sum of owner `owner`'s pack from the ranks' packs (values[rank]) */
template <uint32_t KIND>
__device__ __forceinline__ uint4 ring_owner_sum(const uint4 *values, uint32_t ranks, uint32_t owner)
{
	if (KIND == RING_KIND_ROUND_ONCE) {
		uint32_t out[4];
#pragma unroll
		for (uint32_t word = 0; word < 4; word++) {
			float low = 0.0f, high = 0.0f;
			for (uint32_t rank = 0; rank < ranks; rank++) {
				const uint32_t bits = word == 0 ? values[rank].x : word == 1 ? values[rank].y :
						      word == 2 ? values[rank].z : values[rank].w;
				low = __fadd_rn(low, __uint_as_float(bits << 16));
				high = __fadd_rn(high, __uint_as_float(bits & 0xFFFF0000u));
			}
			out[word] = ring_bfloat16_bits(low) | ring_bfloat16_bits(high) << 16;
		}
		return make_uint4(out[0], out[1], out[2], out[3]);
	}
	/* the ring's hops: from the rank behind the owner round to the owner; what travels has no +0 half */
	uint4 sum = ring_nonzero(values[(owner + 1u) % ranks]);
	for (uint32_t hop = 2; hop < ranks; hop++)
		sum = ring_nonzero(ring_add(sum, values[(owner + hop) % ranks]));
	return ring_add(sum, values[owner]);
}

template <uint32_t KIND> __device__ __forceinline__ void ring_plain(const struct ring_world &w)
{
	const struct exact_ring_arguments &a = w.arguments;
	const uint32_t packs = a.packs_per_owner, rank = a.rank, ranks = w.ranks;
	const uint32_t first = blockIdx.x * blockDim.x + threadIdx.x, stride = gridDim.x * blockDim.x;
	const uint4 *const input = reinterpret_cast<const uint4 *>(w.arena + a.input_offset);
	uint4 *const output = reinterpret_cast<uint4 *>(w.arena + a.output_offset);
	unsigned char *const local = ring_bank(w, rank);
	if (KIND == RING_KIND_EXACT && a.mode == EXACT_RING_GATHER) {
		/* every rank's packs to every rank, then everyone copies; a second meeting keeps the next call's packs off
		 * a bank that is still being read */
		for (uint32_t peer = 0; peer < ranks; peer++) {
			uint4 *const incoming = ring_plane(ring_bank(w, peer), w, 0) + (uint64_t)rank * packs;
			for (uint32_t pack = first; pack < packs; pack += stride)
				ring_store(incoming + pack, input[(uint64_t)rank * packs + pack]);
		}
		if (!ring_phase(w, 1, 0))
			return;
		for (uint32_t owner = 0; owner < ranks; owner++)
			for (uint32_t pack = first; pack < packs; pack += stride)
				output[ring_gather_place(w, owner, pack)] = ring_load(ring_plane(local, w, 0) + (uint64_t)owner * packs + pack);
		(void)ring_phase(w, 1, 1);
		return;
	}
	const uint32_t row_packs = a.mode == EXACT_RING_BF16_SUM_COLUMNS ? packs / a.vectors : 0u;
	for (uint32_t owner = 0; owner < ranks; owner++) {
		uint4 *const incoming = ring_plane(ring_bank(w, owner), w, 0) + (uint64_t)rank * packs;
		for (uint32_t pack = first; pack < packs; pack += stride)
			ring_store(incoming + pack, input[ring_place(w, row_packs, owner, pack)]);
	}
	if (!ring_phase(w, 2, 0))
		return;
	for (uint32_t pack = first; pack < packs; pack += stride) {
		uint4 values[ORDERED_COLLECTIVE_MAXIMUM_RANKS];
		for (uint32_t source = 0; source < ranks; source++)
			values[source] = ring_load(ring_plane(local, w, 0) + (uint64_t)source * packs + pack);
		const uint4 sum = ring_owner_sum<KIND>(values, ranks, rank);
		/* the ring's other ranks receive the owner's sum over its transport: no +0 half (round once: as it is) */
		const uint4 sent = KIND == RING_KIND_ROUND_ONCE ? sum : ring_nonzero(sum);
		for (uint32_t peer = 0; peer < ranks; peer++)
			ring_store(ring_plane(ring_bank(w, peer), w, 1) + (uint64_t)rank * packs + pack, peer == rank ? sum : sent);
	}
	if (!ring_phase(w, 2, 1))
		return;
	for (uint32_t owner = 0; owner < ranks; owner++)
		for (uint32_t pack = first; pack < packs; pack += stride)
			output[ring_place(w, row_packs, owner, pack)] = ring_load(ring_plane(local, w, 1) + (uint64_t)owner * packs + pack);
}

/* ---- the compressed kind: packets of COMPRESSED_RING_PACKET_WORDS words, [slot][group of 32 packs] ---- */

__device__ __forceinline__ uint32_t *ring_packet(unsigned char *bank, uint32_t groups, uint32_t slot, uint32_t group)
{
	return reinterpret_cast<uint32_t *>(bank + EXACT_RING_METADATA_BYTES) +
	       ((uint64_t)slot * groups + group) * COMPRESSED_RING_PACKET_WORDS;
}

/* one warp: lane 0 waits until *address == wanted; every lane learns the verdict */
__device__ __forceinline__ bool ring_warp_wait(const struct ring_world &w, const uint32_t *address, uint32_t wanted)
{
	uint32_t good = 1u;
	if (threadIdx.x % 32u == 0)
		while (ring_acquire(address) != wanted)
			if (!ring_in_time(w)) {
				good = 0u;
				break;
			}
	good = __shfl_sync(0xFFFFFFFFu, good, 0);
	__syncwarp();
	return good != 0u;
}

/* A warp sends its 32 packs (one a lane) of a group to rank `to` on slot `slot`. The lanes' exponents are coded against
 * the warp's largest: a lane whose eight exponents lie within 15 of it sends three words, any other lane its four. */
__device__ __forceinline__ bool ring_send_coded(const struct ring_world &w, uint32_t groups, uint32_t to, uint32_t slot,
						uint32_t group, uint4 value)
{
	const uint32_t lane = threadIdx.x % 32u;
	uint32_t *const mine = ring_packet(ring_bank(w, w.arguments.rank), groups, slot, group);
	/* the receiver has taken this slot's packet of the call before */
	if (!ring_warp_wait(w, mine + COMPRESSED_RING_ACK_WORD, w.generation - 1u))
		return false;
	const uint32_t words[4] = { value.x, value.y, value.z, value.w };
	uint32_t top = 0u, bottom = 255u;
#pragma unroll
	for (uint32_t word = 0; word < 4; word++) {
		const uint32_t low = bf16_wire_low_exponent(words[word]), high = bf16_wire_high_exponent(words[word]);
		top = max(top, max(low, high));
		bottom = min(bottom, min(low, high));
	}
	top = __reduce_max_sync(0xFFFFFFFFu, top);
	const bool raw = top - bottom > BF16_WIRE_DELTA_MASK;
	const uint32_t mask = __ballot_sync(0xFFFFFFFFu, raw);
	uint32_t *const target = ring_packet(ring_bank(w, to), groups, slot, group);
	volatile uint32_t *const payload = target + COMPRESSED_RING_PAYLOAD_WORD + lane * COMPRESSED_RING_COMPRESSED_WORDS +
					   (uint32_t)__popc(mask & ((1u << lane) - 1u));
	if (raw) {
		payload[0] = value.x, payload[1] = value.y, payload[2] = value.z, payload[3] = value.w;
	} else {
		const uint32_t a = bf16_wire_pair_pack(value.x, top), b = bf16_wire_pair_pack(value.y, top);
		const uint32_t c = bf16_wire_pair_pack(value.z, top), d = bf16_wire_pair_pack(value.w, top);
		payload[0] = (a & 0xFFFFu) | (b << 16);
		payload[1] = (c & 0xFFFFu) | (d << 16);
		payload[2] = (a >> 16) | ((b >> 16) << 8) | ((c >> 16) << 16) | ((d >> 16) << 24);
	}
	if (lane == 0) {
		*reinterpret_cast<volatile uint32_t *>(target) = top;
		*reinterpret_cast<volatile uint32_t *>(target + COMPRESSED_RING_RAW_MASK_WORD) = mask;
	}
	__threadfence_system();
	__syncwarp();
	if (lane == 0)
		ring_release(target + COMPRESSED_RING_READY_WORD, w.generation);
	return true;
}

/* the counterpart: the warp takes the group's packet of slot `slot` from its own bank and tells the sender */
__device__ __forceinline__ bool ring_receive_coded(const struct ring_world &w, uint32_t groups, uint32_t slot,
						   uint32_t group, uint4 *value)
{
	const uint32_t lane = threadIdx.x % 32u, ranks = w.ranks, rank = w.arguments.rank;
	uint32_t *const mine = ring_packet(ring_bank(w, rank), groups, slot, group);
	if (!ring_warp_wait(w, mine + COMPRESSED_RING_READY_WORD, w.generation))
		return false;
	const uint32_t top = *reinterpret_cast<volatile uint32_t *>(mine);
	const uint32_t mask = *reinterpret_cast<volatile uint32_t *>(mine + COMPRESSED_RING_RAW_MASK_WORD);
	const volatile uint32_t *const payload = mine + COMPRESSED_RING_PAYLOAD_WORD +
						 lane * COMPRESSED_RING_COMPRESSED_WORDS +
						 (uint32_t)__popc(mask & ((1u << lane) - 1u));
	if ((mask >> lane) & 1u) {
		*value = make_uint4(payload[0], payload[1], payload[2], payload[3]);
	} else {
		const uint32_t first = payload[0], second = payload[1], deltas = payload[2];
		*value = make_uint4(bf16_wire_pair_unpack(first & 0xFFFFu, deltas & 0xFFu, top),
				    bf16_wire_pair_unpack(first >> 16, (deltas >> 8) & 0xFFu, top),
				    bf16_wire_pair_unpack(second & 0xFFFFu, (deltas >> 16) & 0xFFu, top),
				    bf16_wire_pair_unpack(second >> 16, deltas >> 24, top));
	}
	__syncwarp();
	/* the sender of a slot: incoming slots 0 .. R-2 and result slots R-1 .. 2R-3 alike */
	const uint32_t sender = (rank + 1u + slot % (ranks - 1u)) % ranks;
	if (lane == 0)
		ring_release(ring_packet(ring_bank(w, sender), groups, slot, group) + COMPRESSED_RING_ACK_WORD, w.generation);
	return true;
}

__device__ __forceinline__ void ring_compressed(const struct ring_world &w)
{
	const struct exact_ring_arguments &a = w.arguments;
	const uint32_t packs = a.packs_per_owner, rank = a.rank, ranks = w.ranks, lane = threadIdx.x % 32u;
	const uint32_t groups = packs / COMPRESSED_RING_PACKS;
	const uint32_t row_packs = a.mode == EXACT_RING_BF16_SUM_COLUMNS ? packs / a.vectors : 0u;
	const uint32_t warps = gridDim.x * (blockDim.x / 32u), warp = blockIdx.x * (blockDim.x / 32u) + threadIdx.x / 32u;
	const uint4 *const input = reinterpret_cast<const uint4 *>(w.arena + a.input_offset);
	uint4 *const output = reinterpret_cast<uint4 *>(w.arena + a.output_offset);
	for (uint32_t group = warp; group < groups; group += warps) {
		const uint32_t pack = group * COMPRESSED_RING_PACKS + lane;
		/* this rank's packs of the other owners' parts, to the owners */
		for (uint32_t away = 1; away < ranks; away++) {
			const uint32_t owner = (rank + ranks - away) % ranks; /* slot away - 1 of the owner comes from here */
			if (!ring_send_coded(w, groups, owner, away - 1u, group, input[ring_place(w, row_packs, owner, pack)]))
				return;
		}
		/* this rank's part: the ranks behind it in the ring's order, then itself */
		uint4 sum;
		if (!ring_receive_coded(w, groups, 0u, group, &sum))
			return;
		sum = ring_nonzero(sum);
		for (uint32_t hop = 2; hop < ranks; hop++) {
			uint4 next;
			if (!ring_receive_coded(w, groups, hop - 1u, group, &next))
				return;
			sum = ring_nonzero(ring_add(sum, next));
		}
		sum = ring_add(sum, input[ring_place(w, row_packs, rank, pack)]);
		output[ring_place(w, row_packs, rank, pack)] = sum;
		const uint4 sent = ring_nonzero(sum);
		for (uint32_t away = 1; away < ranks; away++) {
			const uint32_t peer = (rank + ranks - away) % ranks;
			if (!ring_send_coded(w, groups, peer, ranks - 1u + (away - 1u), group, sent))
				return;
		}
		for (uint32_t ahead = 1; ahead < ranks; ahead++) {
			const uint32_t owner = (rank + ahead) % ranks; /* result slot R - 1 + ahead - 1 comes from that owner */
			uint4 result;
			if (!ring_receive_coded(w, groups, ranks - 1u + (ahead - 1u), group, &result))
				return;
			output[ring_place(w, row_packs, owner, pack)] = result;
		}
	}
}

/* ---- the entry's body ---- */

template <uint32_t KIND>
__device__ __forceinline__ void ring_exchange(const struct exact_ring_arguments &arguments, unsigned char *arena)
{
	__shared__ uint32_t generation;
	struct ring_world w;
	w.arguments = arguments;
	w.arena = arena;
	w.peers = reinterpret_cast<const struct ordered_collective_peer *>(arena + arguments.peer_table_offset);
	w.ranks = arguments.reserved_words[0] == 0 ? EXACT_RING_RANKS : (uint32_t)arguments.reserved_words[0];
	w.start = clock64();
	w.status = reinterpret_cast<unsigned int *>(arena + arguments.bank_offset + EXACT_RING_STATUS_OFFSET);
	const bool sums = arguments.mode == EXACT_RING_BF16_SUM || arguments.mode == EXACT_RING_BF16_SUM_COLUMNS;
	const bool columns = arguments.mode == EXACT_RING_BF16_SUM_COLUMNS;
	if ((w.ranks != 2u && w.ranks != 4u && w.ranks != 8u) || arguments.rank >= w.ranks ||
	    arguments.packs_per_owner == 0 || arguments.packs_per_owner % COMPRESSED_RING_PACKS != 0 ||
	    (!sums && !(KIND == RING_KIND_EXACT && arguments.mode == EXACT_RING_GATHER)) ||
	    (columns && (arguments.vectors == 0 || arguments.packs_per_owner % arguments.vectors != 0)) ||
	    (arguments.mode == EXACT_RING_GATHER && arguments.vectors != 0 &&
	     arguments.packs_per_owner % arguments.vectors != 0) ||
	    arguments.reserved_words[1] != 0 || gridDim.x > EXACT_RING_BLOCKS || blockDim.x != EXACT_RING_THREADS) {
		if (threadIdx.x == 0)
			atomicExch(w.status, EXACT_RING_STATUS_ARGUMENTS);
		return;
	}
	if (*reinterpret_cast<const volatile unsigned int *>(w.status) != 0u)
		return; /* a bank that failed is not used again */
	if (threadIdx.x == 0) {
		uint32_t *const counter = reinterpret_cast<uint32_t *>(arena + arguments.bank_offset) + blockIdx.x;
		generation = *counter + 1u;
		*counter = generation;
		if (generation == 0)
			atomicExch(w.status, EXACT_RING_STATUS_GENERATION);
	}
	__syncthreads();
	w.generation = generation;
	if (generation == 0)
		return;
	if (KIND == RING_KIND_COMPRESSED)
		ring_compressed(w);
	else
		ring_plain<KIND>(w);
}

#endif
