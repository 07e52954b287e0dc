/*
 * kernel_exl3_prefill.cu: the routed-expert layer for many rows (struct exl3_prefill_record): rows are grouped per
 * expert into tiles of 128 and every (row tile, 128 outputs) is one dense contraction on the fifth-generation tensor
 * cores. The reference's counterpart is its tensor-core prefill family (source/kernel_exl3_tcp.cuh), fixed to its
 * model's shapes and to mma.sync; here a CTA
 *   - streams the row tile's FP16 operand blocks (pre-tiled in the tensor cores' no-swizzle K-major layout) into a ring
 *     of shared-memory stages by bulk asynchronous copies (one warp),
 *   - streams the trellis words of its outputs into a second ring by bulk copies a whole turn of the ring ahead,
 *     decodes them in registers into FP16 and stores them as the B operand block of the stage (sixteen warps in four
 *     teams, a team a stage; the decode's fragment order makes every store a contiguous 128 bytes of the block); two
 *     row tiles of one expert share one decode,
 *   - multiplies with tcgen05.mma (one thread), FP32 accumulators in tensor memory, the stage released by
 *     tcgen05.commit,
 *   - reads the accumulators back with tcgen05.ld and applies the chain's FP32 epilogue (exl3_passes.cuh: Hadamard,
 *     scales, SwiGLU, down-side transform / route weight) a warp a row.
 * Arithmetic per value is the retained chain's; only the association of the FP32 sums over K is the tensor cores'.
 * Every wait is bounded: one that runs out raises exl3_wait_expired, the CTA stores nothing, waits (bounded) for what
 * it has in flight, frees its tensor memory and returns.
 */
#include "exl3_passes.cuh"
#include "router_device.cuh"

#define PREFILL_FIRST_DECODE_WARP 2u /* behind the copy warp and the issuing warp */
#define PREFILL_DECODE_WARPS 16u
#define PREFILL_GROUPS 2u /* groups of 128 outputs of one product CTA */
#define PREFILL_DECODE_THREADS (PREFILL_DECODE_WARPS * EXL3_WARP)
#define PREFILL_COLUMNS 128u /* tensor-memory columns of one accumulator tile */
#define PREFILL_GROUP_THREADS 256u

struct prefill_shared {
	uint64_t a_full[EXL3_PREFILL_A_STAGES]; /* the stage's operand blocks have landed */
	uint64_t a_free[EXL3_PREFILL_A_STAGES]; /* the products that read them are done */
	uint64_t b_full[EXL3_PREFILL_B_STAGES]; /* the stage's decoded weights are written */
	uint64_t b_free[EXL3_PREFILL_B_STAGES]; /* the products that read them are done */
	uint64_t w_full[EXL3_PREFILL_B_STAGES]; /* the stage's trellis words have landed */
	uint64_t done; /* every product of the CTA is done */
	uint32_t tensor_memory;
	volatile uint32_t failed;
	uint32_t armed_a; /* K blocks whose operand copies were started */
	uint32_t armed_w[EXL3_PREFILL_B_STAGES]; /* a team's stages whose trellis copies were started */
	uint32_t issued; /* 1: products were issued and `done` will complete */
};

struct prefill_view {
	const struct exl3_prefill_parts parts;
	unsigned char *workspace;
	uint32_t experts; /* held here: routed + always-on */
	uint32_t pairs_per_row;
	uint32_t live;
	uint32_t widest; /* the larger intermediate width */
};

__device__ __forceinline__ prefill_view prefill_view_of(const struct exl3_prefill_record &record, unsigned char *arena)
{
	const struct step_block step = *reinterpret_cast<const struct step_block *>(arena + record.step_offset);
	const uint32_t widest = max(record.inner_size, record.shared_inner_size);
	prefill_view view = { exl3_prefill_parts_of(record.row_capacity, record.picks, record.shared_count,
						    record.local_count, record.input_size, widest),
			      arena + record.workspace_offset, record.local_count + record.shared_count,
			      record.picks + record.shared_count, min(step.row_count, record.row_capacity), widest };
	return view;
}

/* ------------------------------------------------------------------ routing */

extern "C" __global__ void __launch_bounds__(ROUTER_B200_THREADS)
	exl3_prefill_picks(struct exl3_prefill_record record, unsigned char *arena)
{
	__shared__ uint32_t chosen[ROUTER_B200_THREADS / WARP][ROUTER_B200_MAXIMUM_PICKS];
	__shared__ float weight[ROUTER_B200_THREADS / WARP][ROUTER_B200_MAXIMUM_PICKS];
	const struct step_block step = *reinterpret_cast<const struct step_block *>(arena + record.step_offset);
	const uint32_t live = min(step.row_count, record.row_capacity);
	const uint32_t warp = threadIdx.x / WARP, lane = threadIdx.x % WARP;
	const uint32_t row = blockIdx.x * (ROUTER_B200_THREADS / WARP) + warp;
	if (row >= live)
		return;
	router_row(reinterpret_cast<const float *>(arena + record.scores_offset) + (uint64_t)row * record.expert_count,
		   record.bias_offset != 0 ? reinterpret_cast<const float *>(arena + record.bias_offset) : nullptr,
		   record.expert_count, record.picks, record.scoring, record.route_scale, lane, chosen[warp], weight[warp],
		   reinterpret_cast<uint32_t *>(arena + record.picks_offset) + (uint64_t)row * record.picks,
		   reinterpret_cast<float *>(arena + record.weights_offset) + (uint64_t)row * record.picks);
}

/* A block an expert: its entries in ascending row order (a row holds an expert at most once) and their count. */
extern "C" __global__ void __launch_bounds__(PREFILL_GROUP_THREADS)
	exl3_prefill_group(struct exl3_prefill_record record, unsigned char *arena)
{
	__shared__ uint32_t warp_total[PREFILL_GROUP_THREADS / WARP];
	const prefill_view view = prefill_view_of(record, arena);
	const uint32_t expert = blockIdx.x, lane = threadIdx.x % WARP, warp = threadIdx.x / WARP;
	const uint32_t *const picked = reinterpret_cast<const uint32_t *>(arena + record.picks_offset);
	const float *const weights = reinterpret_cast<const float *>(arena + record.weights_offset);
	struct exl3_prefill_entry *const entries =
		reinterpret_cast<struct exl3_prefill_entry *>(view.workspace + view.parts.entries) +
		(uint64_t)expert * record.row_capacity;
	uint32_t base = 0;
	for (uint32_t first = 0; first < view.live; first += PREFILL_GROUP_THREADS) {
		const uint32_t row = first + threadIdx.x;
		bool found = false;
		uint32_t slot = 0;
		float route_weight = 1.0f;
		if (row < view.live) {
			if (expert >= record.local_count) {
				found = true;
				slot = record.picks + (expert - record.local_count);
			} else {
				for (uint32_t place = 0; place < record.picks; place++)
					if (picked[(uint64_t)row * record.picks + place] == record.local_first + expert) {
						found = true;
						slot = place;
						route_weight = weights[(uint64_t)row * record.picks + place];
					}
			}
		}
		const uint32_t ballot = __ballot_sync(0xFFFFFFFFu, found);
		if (lane == 0)
			warp_total[warp] = (uint32_t)__popc(ballot);
		__syncthreads();
		uint32_t before = 0, total = 0;
		for (uint32_t other = 0; other < PREFILL_GROUP_THREADS / WARP; other++) {
			before += other < warp ? warp_total[other] : 0u;
			total += warp_total[other];
		}
		if (found) {
			struct exl3_prefill_entry entry;
			entry.pair = row * view.pairs_per_row + slot;
			entry.route_weight = route_weight;
			entries[base + before + (uint32_t)__popc(ballot & ((1u << lane) - 1u))] = entry;
		}
		base += total;
		__syncthreads();
	}
	if (threadIdx.x == 0)
		reinterpret_cast<uint32_t *>(view.workspace + view.parts.counts)[expert] = base;
}

/* One block: the tile table in ascending expert order and the tile count. */
extern "C" __global__ void __launch_bounds__(ROUTER_B200_THREADS)
	exl3_prefill_tiles(struct exl3_prefill_record record, unsigned char *arena)
{
	__shared__ uint32_t warp_total[ROUTER_B200_THREADS / WARP];
	const prefill_view view = prefill_view_of(record, arena);
	uint32_t *const counts = reinterpret_cast<uint32_t *>(view.workspace + view.parts.counts);
	struct exl3_prefill_tile *const tiles =
		reinterpret_cast<struct exl3_prefill_tile *>(view.workspace + view.parts.tiles);
	const uint32_t expert = threadIdx.x, lane = threadIdx.x % WARP, warp = threadIdx.x / WARP;
	const uint32_t rows = expert < view.experts ? counts[expert] : 0u;
	const uint32_t mine = (rows + EXL3_PREFILL_TILE_ROWS - 1u) / EXL3_PREFILL_TILE_ROWS;
	uint32_t inclusive = mine;
	for (uint32_t distance = 1; distance < WARP; distance <<= 1) {
		const uint32_t other = __shfl_up_sync(0xFFFFFFFFu, inclusive, distance);
		if (lane >= distance)
			inclusive += other;
	}
	if (lane == WARP - 1u)
		warp_total[warp] = inclusive;
	__syncthreads();
	uint32_t before = 0, total = 0;
	for (uint32_t other = 0; other < ROUTER_B200_THREADS / WARP; other++) {
		before += other < warp ? warp_total[other] : 0u;
		total += warp_total[other];
	}
	const uint32_t first_tile = before + inclusive - mine;
	for (uint32_t index = 0; index < mine; index++) {
		struct exl3_prefill_tile tile;
		tile.expert = expert;
		tile.first_entry = index * EXL3_PREFILL_TILE_ROWS;
		tile.row_count = min(rows - tile.first_entry, EXL3_PREFILL_TILE_ROWS);
		tile.reserved_zero = 0;
		if (first_tile + index < view.parts.tile_capacity)
			tiles[first_tile + index] = tile;
	}
	if (threadIdx.x == 0)
		counts[view.experts] = min(total, view.parts.tile_capacity);
}

/* the intermediate width of a local expert's matrices */
__device__ __forceinline__ uint32_t prefill_inner_of(const struct exl3_prefill_record &record, uint32_t expert)
{
	return expert < record.local_count ? record.inner_size : record.shared_inner_size;
}

/* byte of (row, input) inside an operand block of 128 rows x 64 inputs: 16-byte pieces of eight inputs, the pieces of
 * eight rows adjacent, the 16 row groups adjacent, then the next eight inputs */
__device__ __forceinline__ uint32_t prefill_block_byte(uint32_t row, uint32_t input)
{
	return (input / 8u) * 2048u + (row / 8u) * 128u + (row % 8u) * 16u + (input % 8u) * 2u;
}

/* grid (tile capacity, ceil(H / 128 / 4) x EXL3_PREFILL_OPERAND_PARTS, 2) x 128: x . suh, Hadamard, FP16 operands of
 * gate (z = 0) and up (z = 1). A warp takes one 128-channel block of a quarter of the tile's rows, eight rows at a time:
 * the eight transforms are independent, and their FP16 rows go through shared memory so that every store to the
 * operand blocks is a whole 128-byte piece (eight rows x eight inputs). Rows beyond the tile's count are written as
 * zeros. */
#define OPERAND_ROW_BYTES 272u /* 128 FP16 and a pad that spreads eight rows over the banks */
extern "C" __global__ void __launch_bounds__(EXL3_TRANSFORM_THREADS)
	exl3_prefill_operands(struct exl3_prefill_record record, unsigned char *arena)
{
	__shared__ __align__(16) unsigned char staged[EXL3_TRANSFORM_WARPS][8u * OPERAND_ROW_BYTES];
	const prefill_view view = prefill_view_of(record, arena);
	const uint32_t tile_index = blockIdx.x;
	if (tile_index >= reinterpret_cast<const uint32_t *>(view.workspace + view.parts.counts)[view.experts])
		return;
	const struct exl3_prefill_tile tile =
		reinterpret_cast<const struct exl3_prefill_tile *>(view.workspace + view.parts.tiles)[tile_index];
	const uint32_t lane = threadIdx.x % EXL3_WARP, warp = threadIdx.x / EXL3_WARP;
	const uint32_t part = blockIdx.y % EXL3_PREFILL_OPERAND_PARTS;
	const uint32_t block = blockIdx.y / EXL3_PREFILL_OPERAND_PARTS * EXL3_TRANSFORM_WARPS + warp;
	const uint32_t H = record.input_size;
	constexpr uint32_t part_rows = EXL3_PREFILL_TILE_ROWS / EXL3_PREFILL_OPERAND_PARTS;
	if (block >= H / EXL3_TRANSFORM || part * part_rows >= tile.row_count)
		return;
	const uint32_t channel = block * EXL3_TRANSFORM + lane * 4u;
	const uint32_t bits_x2 = exl3_bits_x2(reinterpret_cast<const uint32_t *>(arena + record.widths_offset)[tile.expert]);
	const uint64_t matrix =
		reinterpret_cast<const uint64_t *>(arena + record.expert_table_offset)[3u * tile.expert + blockIdx.z];
	float scale[4];
	load_half4(reinterpret_cast<const __half *>(arena + matrix +
						    exl3_code_bytes(H, prefill_inner_of(record, tile.expert), bits_x2)) +
			   channel,
		   scale);
	const struct exl3_prefill_entry *const entries =
		reinterpret_cast<const struct exl3_prefill_entry *>(view.workspace + view.parts.entries) +
		(uint64_t)tile.expert * record.row_capacity + tile.first_entry;
	const __nv_bfloat16 *const input = reinterpret_cast<const __nv_bfloat16 *>(arena + record.input_offset);
	/* the two operand blocks (64 inputs each) this warp's 128 channels fall in */
	unsigned char *const blocks = view.workspace + view.parts.gate_up_operands +
				      (((uint64_t)blockIdx.z * view.parts.tile_capacity + tile_index) *
					       (H / EXL3_PREFILL_BLOCK_INPUTS) +
				       2u * block) *
					      EXL3_PREFILL_BLOCK_BYTES;
	unsigned char *const mine = staged[warp];
	for (uint32_t first = part * part_rows; first < (part + 1u) * part_rows && first < tile.row_count; first += 8u) {
		uint2 raw[8];
#pragma unroll
		for (uint32_t r = 0; r < 8; r++) {
			raw[r] = make_uint2(0u, 0u);
			if (first + r < tile.row_count) {
				const uint32_t source_row = entries[first + r].pair / view.pairs_per_row;
				raw[r] = *reinterpret_cast<const uint2 *>(input + (uint64_t)source_row * H + channel);
			}
		}
#pragma unroll
		for (uint32_t r = 0; r < 8; r++) {
			float v[4] = { __uint_as_float(raw[r].x << 16), __uint_as_float(raw[r].x & 0xFFFF0000u),
				       __uint_as_float(raw[r].y << 16), __uint_as_float(raw[r].y & 0xFFFF0000u) };
#pragma unroll
			for (uint32_t i = 0; i < 4; i++)
				v[i] = __fmul_rn(v[i], scale[i]);
			hadamard128_warp(v, lane);
#pragma unroll
			for (uint32_t i = 0; i < 4; i++)
				v[i] = __fmul_rn(v[i], EXL3_NORMALIZATION);
			store_half4(reinterpret_cast<__half *>(mine + r * OPERAND_ROW_BYTES + lane * 8u), v);
		}
		__syncwarp();
		/* piece p (eight inputs) of the eight rows: 128 contiguous bytes of the block; lane = 8 (p % 4) + row */
#pragma unroll
		for (uint32_t turn = 0; turn < 4; turn++) {
			const uint32_t piece = turn * 4u + lane / 8u, row = lane % 8u;
			const uint4 value = *reinterpret_cast<const uint4 *>(mine + row * OPERAND_ROW_BYTES + piece * 16u);
			*reinterpret_cast<uint4 *>(blocks + (piece / 8u) * EXL3_PREFILL_BLOCK_BYTES + (piece % 8u) * 2048u +
						   (first / 8u) * 128u + row * 16u) = value;
		}
		__syncwarp();
	}
}

/* ------------------------------------------------------------------ tensor-core products */

/* shared-memory matrix descriptor of an operand block at a 16-byte aligned address: no swizzle, K-major;
 * piece_bytes between the two 16-byte K pieces of a K = 16 step (128 bytes a group of eight rows: 2048 for 128 rows,
 * 4096 for 256), 128 bytes between groups of eight rows */
__device__ __forceinline__ uint64_t prefill_descriptor(uint32_t shared_address, uint32_t piece_bytes)
{
	return (uint64_t)((shared_address >> 4) & 0x3FFFu) | (uint64_t)(piece_bytes >> 4) << 16 |
	       (uint64_t)(128u >> 4) << 32 | (uint64_t)1 << 46;
}

/* FP16 A and B, both K-major, FP32 accumulators, M = 128, N = 128 x groups */
__device__ __forceinline__ uint32_t prefill_instruction(uint32_t groups)
{
	return (1u << 4) | ((groups * 128u >> 3) << 17) | ((128u >> 4) << 24);
}

__device__ __forceinline__ void tensor_fence_before()
{
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tensor_fence_after()
{
	asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tensor_commit(uint64_t *barrier)
{
	asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
			     smem_address(barrier))
		     : "memory");
}

__device__ __forceinline__ void decode_sync()
{
	asm volatile("bar.sync 1, %0;" ::"n"(PREFILL_DECODE_THREADS) : "memory");
}

/* Dynamic shared memory of a product CTA, for TILES row tiles of one expert, MATRICES matrices, GROUPS groups of 128
 * outputs and stages of KSTEPS steps of 16 inputs. Three rings:
 *   A ring        EXL3_PREFILL_A_STAGES x [tile][matrix] operand blocks (128 rows x 16 KSTEPS FP16 in the tensor cores'
 *                 layout, KSTEPS x 4096 bytes): bulk copies, mostly from L2
 *   B ring        EXL3_PREFILL_B_STAGES x [matrix] blocks of decoded weights, 128 GROUPS outputs x 16 KSTEPS FP16 in
 *                 the same layout (one instruction multiplies all groups and reads the operand rows once): written by
 *                 the decode warps, read by the products of EVERY row tile
 *   W ring        EXL3_PREFILL_B_STAGES x EXL3_PREFILL_W_STAGE bytes: the stage's trellis words as they lie in the
 *                 matrix, one run of GROUPS x 8 tiles for every (matrix, step): bulk copies by the copy warp, read by the
 *                 decode warps with shared-memory loads. The team that owns a stage starts the copies of its next use
 *                 as soon as its four warps have read this one, a whole turn of the ring before it needs them. */
template <uint32_t MATRICES, uint32_t KSTEPS, uint32_t TILES, uint32_t GROUPS> struct prefill_rings {
	static constexpr uint32_t block_bytes = KSTEPS * 4096u;
	static constexpr uint32_t a_stage = TILES * MATRICES * block_bytes;
	static constexpr uint32_t b_piece = GROUPS * 2048u; /* eight inputs of 128 GROUPS outputs */
	static constexpr uint32_t b_block = GROUPS * block_bytes; /* of one matrix */
	static constexpr uint32_t b_stage = MATRICES * b_block;
	static constexpr uint32_t b_at = EXL3_PREFILL_A_STAGES * a_stage;
	static constexpr uint32_t w_at = b_at + EXL3_PREFILL_B_STAGES * b_stage;
	static constexpr uint32_t bytes = w_at + EXL3_PREFILL_B_STAGES * EXL3_PREFILL_W_STAGE;
	static constexpr uint32_t columns = TILES * MATRICES * GROUPS * PREFILL_COLUMNS; /* of tensor memory */
	static_assert(bytes <= EXL3_PREFILL_DYNAMIC_BYTES, "the host sizes the rings");
	static_assert(columns <= 512u, "tensor memory has 512 columns");
	/* first column of the accumulator of (row tile, matrix, group) */
	__device__ static constexpr uint32_t column(uint32_t tile, uint32_t m, uint32_t g)
	{
		return ((tile * MATRICES + m) * GROUPS + g) * PREFILL_COLUMNS;
	}
};

/* The K loop of one CTA. matrices[m]: the codes of matrix m (`outputs` outputs), of which the CTA takes the `groups`
 * (1 .. GROUPS) groups of 128 outputs from group `first_group`; operand_blocks[tile * MATRICES + m]: row tile `tile`'s
 * operand blocks for matrix m; `blocks` stages of 16 KSTEPS inputs. Warp 0 copies operand blocks, one thread of warp 1
 * issues the products, warps 2 .. copy trellis words and decode. On return the decode warps know whether the
 * accumulators (prefill_rings::column from shared->tensor_memory) are complete; the other warps return false.
 * All threads call. */
template <uint32_t BX2, uint32_t MATRICES, uint32_t KSTEPS, uint32_t TILES, uint32_t GROUPS>
__device__ __forceinline__ bool prefill_products(const unsigned char *const (&matrices)[MATRICES], uint32_t outputs,
						 uint32_t first_group, uint32_t groups,
						 const unsigned char *const (&operand_blocks)[TILES * MATRICES],
						 uint32_t blocks, unsigned char *dynamic_shared, prefill_shared *shared)
{
	typedef exl3_ring<BX2> ring;
	typedef prefill_rings<MATRICES, KSTEPS, TILES, GROUPS> rings;
	constexpr uint32_t AS = EXL3_PREFILL_A_STAGES, BS = EXL3_PREFILL_B_STAGES;
	/* the trellis words of one (matrix, step) of a stage: GROUPS groups of eight tiles, adjacent in the matrix */
	constexpr uint32_t w_chunk = GROUPS * EXL3_GROUP_TILES * ring::words * 4u;
	static_assert(MATRICES * KSTEPS * w_chunk <= EXL3_PREFILL_W_STAGE, "the W ring holds a stage");
	static_assert(MATRICES <= 2u && MATRICES * KSTEPS <= EXL3_WARP && w_chunk % 16u == 0u, "a lane a copy, whole 16 bytes");
	const uint32_t lane = threadIdx.x % EXL3_WARP, warp = threadIdx.x / EXL3_WARP;
	const uint64_t step_words = (uint64_t)(outputs / EXL3_TILE) * ring::words; /* of one step of 16 inputs */

	if (threadIdx.x == 0) {
		for (uint32_t stage = 0; stage < AS; stage++) {
			barrier_init(&shared->a_full[stage], 1);
			barrier_init(&shared->a_free[stage], 1);
		}
		for (uint32_t stage = 0; stage < BS; stage++) {
			barrier_init(&shared->b_full[stage], 4u); /* the four warps of the team that decodes the stage */
			barrier_init(&shared->b_free[stage], 1);
			barrier_init(&shared->w_full[stage], 1);
		}
		barrier_init(&shared->done, 1);
		shared->failed = 0;
		shared->armed_a = 0;
		for (uint32_t stage = 0; stage < BS; stage++)
			shared->armed_w[stage] = 0;
		shared->issued = 0;
		asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
	}
	if (warp == 1) {
		asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
				     smem_address(&shared->tensor_memory)),
			     "r"(rings::columns)
			     : "memory");
		asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
	}
	tensor_fence_before();
	__syncthreads();
	tensor_fence_after();
	const uint32_t accumulators = shared->tensor_memory;

	if (warp == 0) {
		/* operand copies: lane (tile, m) copies that block */
		uint32_t block = 0;
		for (; block < blocks; block++) {
			const uint32_t stage = block % AS, use = block / AS;
			uint32_t good = 1;
			if (lane == 0) {
				if (use > 0 && !barrier_wait(&shared->a_free[stage], (use - 1u) & 1u))
					good = 0;
				else
					barrier_expect(&shared->a_full[stage], rings::a_stage);
			}
			good = __shfl_sync(0xFFFFFFFFu, good, 0);
			if (good == 0)
				break;
			if (lane < TILES * MATRICES)
				bulk_load(dynamic_shared + stage * rings::a_stage + lane * rings::block_bytes,
					  operand_blocks[lane] + (uint64_t)block * rings::block_bytes, rings::block_bytes,
					  &shared->a_full[stage]);
		}
		if (lane == 0) {
			shared->armed_a = block;
			if (block < blocks)
				shared->failed = 1;
		}
		return false;
	}
	if (warp == 1) {
		/* products: one thread; every row tile's products read the same decoded weights */
		if (lane == 0) {
			bool good = true;
			const uint32_t instruction = prefill_instruction(groups);
			for (uint32_t block = 0; block < blocks && good; block++) {
				const uint32_t sa = block % AS, sb = block % BS;
				good = barrier_wait(&shared->a_full[sa], (block / AS) & 1u) &&
				       barrier_wait(&shared->b_full[sb], (block / BS) & 1u);
				if (!good)
					break;
				tensor_fence_after();
				/* the stage's first descriptors; every other one lies a constant number of 16-byte units behind */
				const uint64_t a_first =
					prefill_descriptor(smem_address(dynamic_shared + sa * rings::a_stage), 2048u);
				const uint64_t b_first = prefill_descriptor(
					smem_address(dynamic_shared + rings::b_at + sb * rings::b_stage), rings::b_piece);
#pragma unroll
				for (uint32_t tile = 0; tile < TILES; tile++)
#pragma unroll
					for (uint32_t m = 0; m < MATRICES; m++)
#pragma unroll
						for (uint32_t step = 0; step < KSTEPS; step++) {
							const uint64_t a =
								a_first + (((tile * MATRICES + m) * rings::block_bytes + step * 2u * 2048u) >> 4);
							const uint64_t b = b_first + ((m * rings::b_block + step * 2u * rings::b_piece) >> 4);
							const uint32_t accumulate = block > 0 || step > 0 ? 1u : 0u;
							asm volatile("{\n\t.reg .pred p;\n\t"
								     "setp.ne.b32 p, %4, 0;\n\t"
								     "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(
									     accumulators + rings::column(tile, m, 0)),
								     "l"(a), "l"(b), "r"(instruction), "r"(accumulate)
								     : "memory");
						}
				tensor_commit(&shared->a_free[sa]);
				tensor_commit(&shared->b_free[sb]);
				shared->issued = 1;
			}
			if (!good) {
				shared->failed = 1;
				__threadfence_block();
			}
			if (shared->issued != 0) /* the decode warps and the release wait on this */
				tensor_commit(&shared->done);
		}
		return false;
	}

	/* decode: the sixteen warps are four teams of four; team q decodes the WHOLE stages q, q + 4, ... (with four
	 * decoded-weights stages in the ring a team owns one of them, and the W stage of the same number), so that the
	 * teams work on four different stages at once and a warp crosses a barrier and a proxy fence once per stage of 8
	 * or 16 tiles, not once per 2 or 4. Warp r of a team takes the stage's units r * units_a_warp .. : a unit is the
	 * eight adjacent tiles of one (matrix, group, step), whose ring words the lane reads from the W ring. */
	{
		static_assert(EXL3_PREFILL_B_STAGES == 4u && PREFILL_DECODE_WARPS == 16u, "a team of four warps a stage");
		constexpr uint32_t units = MATRICES * GROUPS * KSTEPS, units_a_warp = units / 4u;
		static_assert(units % 4u == 0u, "whole units a warp");
		const uint32_t decoder = warp - PREFILL_FIRST_DECODE_WARP, team = decoder / 4u, member = decoder % 4u;
		const uint32_t begin = ring::begin(lane);
		const uint32_t word_index = begin / 32u, shift = begin % 32u, next_index = (word_index + 1u) % ring::words;
		const uint32_t *const words_at =
			reinterpret_cast<const uint32_t *>(dynamic_shared + rings::w_at + team * EXL3_PREFILL_W_STAGE);
		unsigned char *const b_at = dynamic_shared + rings::b_at + team * rings::b_stage + lane * 4u;
		/* the team's first warp copies the stage's trellis words: lane (m, step) the run of that matrix and step */
		const uint32_t w_bytes = groups * EXL3_GROUP_TILES * ring::words * 4u;
		const unsigned char *const w_from =
			(MATRICES > 1u && lane >= KSTEPS ? matrices[MATRICES - 1u] : matrices[0]) +
			((uint64_t)(lane % KSTEPS) * step_words + (uint64_t)first_group * EXL3_GROUP_TILES * ring::words) * 4u;
		unsigned char *const w_to = dynamic_shared + rings::w_at + team * EXL3_PREFILL_W_STAGE + lane * w_chunk;
#define PREFILL_WORDS_COPY(block)                                                                             \
	do {                                                                                                  \
		if (lane == 0) {                                                                              \
			barrier_expect(&shared->w_full[team], MATRICES * KSTEPS * w_bytes);                   \
			shared->armed_w[team] = (block) / BS + 1u;                                            \
		}                                                                                             \
		__syncwarp();                                                                                 \
		if (lane < MATRICES * KSTEPS)                                                                 \
			bulk_load(w_to, w_from + (uint64_t)(block) * KSTEPS * step_words * 4u, w_bytes,      \
				  &shared->w_full[team]);                                                     \
	} while (0)
		bool good = true;
		if (member == 0u && team < blocks)
			PREFILL_WORDS_COPY(team);
		for (uint32_t block = team; block < blocks; block += 4u) {
			const uint32_t use = block / BS;
			if (use > 0u)
				good = barrier_wait(&shared->b_free[team], (use - 1u) & 1u);
			if (good)
				good = barrier_wait(&shared->w_full[team], use & 1u);
			if (!good)
				break;
#pragma unroll
			for (uint32_t turn = 0; turn < units_a_warp; turn++) {
				/* unit = (matrix m, group g, step) in that order of significance */
				const uint32_t unit = member * units_a_warp + turn;
				const uint32_t step = unit % KSTEPS, g = unit / KSTEPS % GROUPS, m = unit / (KSTEPS * GROUPS);
				if (g >= groups)
					continue;
				const uint32_t *const from =
					words_at + (m * KSTEPS + step) * (w_chunk / 4u) + g * EXL3_GROUP_TILES * ring::words;
				unsigned char *const to_unit = b_at + m * rings::b_block + step * 2u * rings::b_piece +
							       g * EXL3_GROUP_TILES * 2u * 128u;
#pragma unroll
				for (uint32_t tile = 0; tile < EXL3_GROUP_TILES; tile++) {
					uint32_t fragment[4];
					exl3_decode_fragment<BX2>(from[tile * ring::words + word_index],
								  from[tile * ring::words + next_index], shift, fragment);
					/* fragment f: outputs 16 tile + g + 8 (f % 2), inputs 16 step + 2 t + 8 (f / 2): the warp's 32
					 * words are the 128 bytes of one K piece of one group of eight outputs */
					uint32_t *const to = reinterpret_cast<uint32_t *>(to_unit + tile * 2u * 128u);
					to[0] = fragment[0];
					to[128u / 4u] = fragment[1];
					to[rings::b_piece / 4u] = fragment[2];
					to[(rings::b_piece + 128u) / 4u] = fragment[3];
				}
			}
			asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
			__syncwarp();
			if (lane == 0)
				barrier_arrive(&shared->b_full[team]);
			/* the stage's next use: its words may be overwritten once all four warps have read these */
			if (member == 0u && block + 4u < blocks) {
				good = barrier_wait(&shared->b_full[team], use & 1u);
				if (!good)
					break;
				PREFILL_WORDS_COPY(block + 4u);
			}
		}
#undef PREFILL_WORDS_COPY
		if (good)
			good = barrier_wait(&shared->done, 0u);
		if (!good)
			shared->failed = 1;
		tensor_fence_after();
		decode_sync(); /* every decode warp has its verdict in */
		return shared->failed == 0;
	}
}

/* `matrices` accumulator tiles (first columns first_column, first_column + column_stride, ...) into shared memory,
 * FP32 [matrix][128 rows][EXL3_PREFILL_STAGING_ROW]. A warp reads the 32 tensor-memory lanes of its quarter (warp % 4)
 * and one quarter of the columns. Decode warps only; ends with their barrier. */
__device__ __forceinline__ void prefill_stage_out(uint32_t accumulators, uint32_t matrices, uint32_t first_column,
						  uint32_t column_stride, float *staging)
{
	const uint32_t lane = threadIdx.x % EXL3_WARP, warp = threadIdx.x / EXL3_WARP;
	const uint32_t quarter = warp % 4u, column = (warp - PREFILL_FIRST_DECODE_WARP) / 4u * 32u;
	__syncwarp();
	for (uint32_t m = 0; m < matrices; m++) {
		uint32_t r[32];
		asm volatile(
			"tcgen05.ld.sync.aligned.32x32b.x32.b32 "
			"{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,"
			"%26,%27,%28,%29,%30,%31}, [%32];"
			: "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
			  "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
			  "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
			  "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
			  "=r"(r[30]), "=r"(r[31])
			: "r"(accumulators + ((quarter * 32u) << 16) + first_column + m * column_stride + column)
			: "memory");
		asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
		uint4 *const to = reinterpret_cast<uint4 *>(
			staging + ((uint64_t)m * EXL3_PREFILL_TILE_ROWS + quarter * 32u + lane) * EXL3_PREFILL_STAGING_ROW +
			column);
#pragma unroll
		for (uint32_t index = 0; index < 8; index++)
			to[index] = make_uint4(r[4 * index], r[4 * index + 1], r[4 * index + 2], r[4 * index + 3]);
	}
	tensor_fence_before();
	decode_sync();
}

/* All threads, at the end of a product CTA: wait (bounded) for what a failed CTA still has in flight, then free the
 * tensor memory. */
template <uint32_t COLUMNS> __device__ __forceinline__ void prefill_release(prefill_shared *shared)
{
	tensor_fence_before();
	__syncthreads();
	if (shared->failed != 0 && threadIdx.x == 0) {
		for (uint32_t back = 0; back < EXL3_PREFILL_A_STAGES && back < shared->armed_a; back++) {
			const uint32_t block = shared->armed_a - 1u - back;
			(void)barrier_wait(&shared->a_full[block % EXL3_PREFILL_A_STAGES], (block / EXL3_PREFILL_A_STAGES) & 1u);
		}
		for (uint32_t team = 0; team < EXL3_PREFILL_B_STAGES; team++)
			if (shared->armed_w[team] != 0)
				(void)barrier_wait(&shared->w_full[team], (shared->armed_w[team] - 1u) & 1u);
		if (shared->issued != 0)
			(void)barrier_wait(&shared->done, 0u);
	}
	__syncthreads();
	if (threadIdx.x / EXL3_WARP == 1u) {
		tensor_fence_after();
		__syncwarp();
		asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(shared->tensor_memory),
			     "r"(COLUMNS)
			     : "memory");
	}
}

struct prefill_tile_view {
	struct exl3_prefill_tile tile;
	const struct exl3_prefill_entry *entries; /* of the tile's rows */
	uint64_t gate, up, down; /* matrix offsets */
};

__device__ __forceinline__ prefill_tile_view prefill_tile_of(const struct exl3_prefill_record &record,
							     const unsigned char *arena, const prefill_view &view,
							     uint32_t tile_index)
{
	prefill_tile_view out;
	out.tile = reinterpret_cast<const struct exl3_prefill_tile *>(view.workspace + view.parts.tiles)[tile_index];
	out.entries = reinterpret_cast<const struct exl3_prefill_entry *>(view.workspace + view.parts.entries) +
		      (uint64_t)out.tile.expert * record.row_capacity + out.tile.first_entry;
	const uint64_t *const table = reinterpret_cast<const uint64_t *>(arena + record.expert_table_offset);
	out.gate = table[3u * out.tile.expert];
	out.up = table[3u * out.tile.expert + 1u];
	out.down = table[3u * out.tile.expert + 2u];
	return out;
}

/* An expert's row tiles are taken two at a time: the CTAs of an even-numbered tile that has a successor also take the
 * successor's rows, so that every decoded weight is multiplied with 256 rows; the CTAs of an odd-numbered tile return. */
#define PREFILL_SINGLE 0u
#define PREFILL_FIRST_OF_TWO 1u
#define PREFILL_SECOND_OF_TWO 2u
__device__ __forceinline__ uint32_t prefill_pairing(const prefill_view &view, const struct exl3_prefill_tile &tile,
						    uint32_t tile_index, uint32_t tile_count)
{
	if ((tile.first_entry / EXL3_PREFILL_TILE_ROWS) % 2u != 0u)
		return PREFILL_SECOND_OF_TWO;
	const struct exl3_prefill_tile *const tiles =
		reinterpret_cast<const struct exl3_prefill_tile *>(view.workspace + view.parts.tiles);
	return tile_index + 1u < tile_count && tiles[tile_index + 1u].expert == tile.expert ? PREFILL_FIRST_OF_TWO :
											       PREFILL_SINGLE;
}

/* The gate/up epilogue of one row tile and one group of 128 outputs, from the staged accumulators (gate rows, then up
 * rows): Hadamard, scales, SwiGLU, down-side transform, FP16 down operand blocks. Decode warps; a warp a row. */
template <uint32_t BX2>
__device__ __forceinline__ void prefill_gate_up_rows(const struct exl3_prefill_record &record, unsigned char *arena,
						     const prefill_view &view, const prefill_tile_view &tile,
						     uint32_t tile_index, uint32_t group, const float *staging)
{
	const uint32_t H = record.input_size, I = prefill_inner_of(record, tile.tile.expert);
	const uint32_t lane = threadIdx.x % EXL3_WARP, warp = threadIdx.x / EXL3_WARP;
	const uint32_t channel = group * EXL3_TRANSFORM + lane * 4u;
	const uint64_t codes = exl3_code_bytes(H, I, BX2);
	float gate_scale[4], up_scale[4], down_scale[4];
	load_half4(reinterpret_cast<const __half *>(arena + tile.gate + codes) + H + channel, gate_scale);
	load_half4(reinterpret_cast<const __half *>(arena + tile.up + codes) + H + channel, up_scale);
	load_half4(reinterpret_cast<const __half *>(arena + tile.down + exl3_code_bytes(I, H, BX2)) + channel, down_scale);
	unsigned char *const blocks = view.workspace + view.parts.down_operands +
				      ((uint64_t)tile_index * (view.widest / EXL3_PREFILL_BLOCK_INPUTS) +
				       channel / EXL3_PREFILL_BLOCK_INPUTS) *
					      EXL3_PREFILL_BLOCK_BYTES;
	for (uint32_t row = warp - PREFILL_FIRST_DECODE_WARP; row < tile.tile.row_count; row += PREFILL_DECODE_WARPS) {
		const float4 gate_raw = *reinterpret_cast<const float4 *>(staging + row * EXL3_PREFILL_STAGING_ROW + lane * 4u);
		const float4 up_raw = *reinterpret_cast<const float4 *>(
			staging + (EXL3_PREFILL_TILE_ROWS + row) * EXL3_PREFILL_STAGING_ROW + lane * 4u);
		float gate[4] = { gate_raw.x, gate_raw.y, gate_raw.z, gate_raw.w };
		float up[4] = { up_raw.x, up_raw.y, up_raw.z, up_raw.w };
		hadamard128_warp(gate, lane);
		hadamard128_warp(up, lane);
		float hidden[4], fed[4];
		exl3_swiglu4(gate, up, gate_scale, up_scale, record.activation_limit, hidden);
#pragma unroll
		for (uint32_t i = 0; i < 4; i++)
			fed[i] = __fmul_rn(hidden[i], down_scale[i]);
		hadamard128_warp(fed, lane);
#pragma unroll
		for (uint32_t i = 0; i < 4; i++)
			fed[i] = __fmul_rn(fed[i], EXL3_NORMALIZATION);
		store_half4(reinterpret_cast<__half *>(blocks + prefill_block_byte(row, channel % EXL3_PREFILL_BLOCK_INPUTS)),
			    fed);
	}
}

/* TILES row tiles (tile_index, tile_index + 1) of one expert by GROUPS groups of 128 outputs from first_group */
template <uint32_t BX2, uint32_t TILES, uint32_t GROUPS>
__device__ __forceinline__ void prefill_gate_up(const struct exl3_prefill_record &record, unsigned char *arena,
						const prefill_view &view, uint32_t tile_index, uint32_t first_group,
						unsigned char *dynamic_shared, prefill_shared *shared)
{
	typedef prefill_rings<2, EXL3_PREFILL_GATE_UP_STEPS, TILES, GROUPS> rings;
	prefill_tile_view tiles[TILES];
#pragma unroll
	for (uint32_t tile = 0; tile < TILES; tile++)
		tiles[tile] = prefill_tile_of(record, arena, view, tile_index + tile);
	const uint32_t H = record.input_size, I = prefill_inner_of(record, tiles[0].tile.expert);
	const uint32_t groups = min(GROUPS, I / EXL3_TRANSFORM - first_group);
	const uint32_t warp = threadIdx.x / EXL3_WARP;
	const unsigned char *const matrices[2] = { arena + tiles[0].gate, arena + tiles[0].up };
	const uint64_t tile_bytes = (uint64_t)(H / EXL3_PREFILL_BLOCK_INPUTS) * EXL3_PREFILL_BLOCK_BYTES;
	const unsigned char *operands[TILES * 2];
#pragma unroll
	for (uint32_t tile = 0; tile < TILES; tile++) {
		operands[tile * 2u] = view.workspace + view.parts.gate_up_operands + (tile_index + tile) * tile_bytes;
		operands[tile * 2u + 1u] = view.workspace + view.parts.gate_up_operands +
					   ((uint64_t)view.parts.tile_capacity + tile_index + tile) * tile_bytes;
	}
	const bool complete = prefill_products<BX2, 2, EXL3_PREFILL_GATE_UP_STEPS, TILES, GROUPS>(
		matrices, I, first_group, groups, operands, H / (EXL3_PREFILL_GATE_UP_STEPS * EXL3_TILE), dynamic_shared,
		shared);
	if (warp >= PREFILL_FIRST_DECODE_WARP && complete) {
		float *const staging = reinterpret_cast<float *>(dynamic_shared);
		for (uint32_t tile = 0; tile < TILES; tile++)
			for (uint32_t g = 0; g < groups; g++) {
				prefill_stage_out(shared->tensor_memory, 2, rings::column(tile, 0, g), rings::column(0, 1, 0),
						  staging);
				prefill_gate_up_rows<BX2>(record, arena, view, tiles[tile], tile_index + tile, first_group + g,
							  staging);
				decode_sync(); /* the staging rows are read: the next tile may overwrite them */
			}
	}
	prefill_release<rings::columns>(shared);
}

template <uint32_t BX2, uint32_t TILES, uint32_t KSTEPS>
__device__ __forceinline__ void prefill_down(const struct exl3_prefill_record &record, unsigned char *arena,
					     const prefill_view &view, uint32_t tile_index, uint32_t first_group,
					     unsigned char *dynamic_shared, prefill_shared *shared)
{
	typedef prefill_rings<1, KSTEPS, TILES, PREFILL_GROUPS> rings;
	prefill_tile_view tiles[TILES];
#pragma unroll
	for (uint32_t tile = 0; tile < TILES; tile++)
		tiles[tile] = prefill_tile_of(record, arena, view, tile_index + tile);
	const uint32_t H = record.input_size, I = prefill_inner_of(record, tiles[0].tile.expert);
	const uint32_t groups = min(PREFILL_GROUPS, H / EXL3_TRANSFORM - first_group);
	const uint32_t lane = threadIdx.x % EXL3_WARP, warp = threadIdx.x / EXL3_WARP;
	const unsigned char *const matrices[1] = { arena + tiles[0].down };
	const unsigned char *operands[TILES];
#pragma unroll
	for (uint32_t tile = 0; tile < TILES; tile++)
		operands[tile] = view.workspace + view.parts.down_operands +
				 (uint64_t)(tile_index + tile) * (view.widest / EXL3_PREFILL_BLOCK_INPUTS) *
					 EXL3_PREFILL_BLOCK_BYTES;
	const bool complete = prefill_products<BX2, 1, KSTEPS, TILES, PREFILL_GROUPS>(
		matrices, H, first_group, groups, operands, I / (KSTEPS * EXL3_TILE), dynamic_shared, shared);
	if (warp >= PREFILL_FIRST_DECODE_WARP && complete) {
		float *const staging = reinterpret_cast<float *>(dynamic_shared);
		float *const outputs = reinterpret_cast<float *>(arena + record.pair_output_offset);
		for (uint32_t tile = 0; tile < TILES; tile++)
			for (uint32_t g = 0; g < groups; g++) {
				prefill_stage_out(shared->tensor_memory, 1, rings::column(tile, 0, g), 0, staging);
				const uint32_t channel = (first_group + g) * EXL3_TRANSFORM + lane * 4u;
				float scale[4];
				load_half4(reinterpret_cast<const __half *>(arena + tiles[tile].down + exl3_code_bytes(I, H, BX2)) +
						   I + channel,
					   scale);
				for (uint32_t row = warp - PREFILL_FIRST_DECODE_WARP; row < tiles[tile].tile.row_count;
				     row += PREFILL_DECODE_WARPS) {
					const struct exl3_prefill_entry entry = tiles[tile].entries[row];
					const float4 raw = *reinterpret_cast<const float4 *>(
						staging + row * EXL3_PREFILL_STAGING_ROW + lane * 4u);
					float v[4] = { raw.x, raw.y, raw.z, raw.w };
					hadamard128_warp(v, lane);
#pragma unroll
					for (uint32_t i = 0; i < 4; i++)
						v[i] = __fmul_rn(__fmul_rn(__fmul_rn(v[i], EXL3_NORMALIZATION), scale[i]),
								 entry.route_weight);
					*reinterpret_cast<float4 *>(outputs + (uint64_t)entry.pair * H + channel) =
						make_float4(v[0], v[1], v[2], v[3]);
				}
				decode_sync();
			}
	}
	prefill_release<rings::columns>(shared);
}

#define PREFILL_WIDTH_SWITCH(call)                                                                     \
	switch (exl3_bits_x2(reinterpret_cast<const uint32_t *>(arena + record.widths_offset)[tile.expert])) { \
	case EXL3_BITS_X2_K2: {                                                                        \
		constexpr uint32_t BX2 = EXL3_BITS_X2_K2;                                              \
		call;                                                                                  \
	} break;                                                                                       \
	case EXL3_BITS_X2_K2_5: {                                                                      \
		constexpr uint32_t BX2 = EXL3_BITS_X2_K2_5;                                            \
		call;                                                                                  \
	} break;                                                                                       \
	case EXL3_BITS_X2_K3: {                                                                        \
		constexpr uint32_t BX2 = EXL3_BITS_X2_K3;                                              \
		call;                                                                                  \
	} break;                                                                                       \
	case EXL3_BITS_X2_K4: {                                                                        \
		constexpr uint32_t BX2 = EXL3_BITS_X2_K4;                                              \
		call;                                                                                  \
	} break;                                                                                       \
	default:                                                                                       \
		break;                                                                                 \
	}

/* grid (widest I / 128, tile capacity) x 576: a single row tile is taken by the CTAs of even x with two groups of 128
 * outputs each; two row tiles of one expert by every x with one group each (tensor memory holds 512 columns) */
extern "C" __global__ void __launch_bounds__(EXL3_PREFILL_GEMM_THREADS, 1)
	exl3_prefill_gate_up(struct exl3_prefill_record record, unsigned char *arena)
{
	extern __shared__ __align__(1024) unsigned char dynamic_shared[];
	__shared__ prefill_shared shared;
	const prefill_view view = prefill_view_of(record, arena);
	const uint32_t tile_count = reinterpret_cast<const uint32_t *>(view.workspace + view.parts.counts)[view.experts];
	/* once a wait has run out (the flag is never cleared while the kernel file stays loaded), later CTAs do not
	 * queue up behind the same fault: the host reads the flag and rejects the result */
	if (*reinterpret_cast<volatile unsigned int *>(&exl3_wait_expired) != 0u || blockIdx.y >= tile_count)
		return;
	const struct exl3_prefill_tile tile =
		reinterpret_cast<const struct exl3_prefill_tile *>(view.workspace + view.parts.tiles)[blockIdx.y];
	const uint32_t pairing = prefill_pairing(view, tile, blockIdx.y, tile_count);
	const uint32_t group_count = prefill_inner_of(record, tile.expert) / EXL3_TRANSFORM;
	if (pairing == PREFILL_SECOND_OF_TWO || blockIdx.x >= group_count ||
	    (pairing == PREFILL_SINGLE && blockIdx.x % PREFILL_GROUPS != 0u))
		return;
	if (pairing == PREFILL_FIRST_OF_TWO) {
		PREFILL_WIDTH_SWITCH((prefill_gate_up<BX2, 2, 1>(record, arena, view, blockIdx.y, blockIdx.x, dynamic_shared,
								 &shared)))
	} else {
		PREFILL_WIDTH_SWITCH((prefill_gate_up<BX2, 1, PREFILL_GROUPS>(record, arena, view, blockIdx.y, blockIdx.x,
									      dynamic_shared, &shared)))
	}
}

/* grid (ceil(H / 256), tile capacity) x 576: two groups of 128 outputs a CTA, for one row tile or for two of one expert */
extern "C" __global__ void __launch_bounds__(EXL3_PREFILL_GEMM_THREADS, 1)
	exl3_prefill_down(struct exl3_prefill_record record, unsigned char *arena)
{
	extern __shared__ __align__(1024) unsigned char dynamic_shared[];
	__shared__ prefill_shared shared;
	const prefill_view view = prefill_view_of(record, arena);
	const uint32_t tile_count = reinterpret_cast<const uint32_t *>(view.workspace + view.parts.counts)[view.experts];
	if (*reinterpret_cast<volatile unsigned int *>(&exl3_wait_expired) != 0u || blockIdx.y >= tile_count)
		return;
	const struct exl3_prefill_tile tile =
		reinterpret_cast<const struct exl3_prefill_tile *>(view.workspace + view.parts.tiles)[blockIdx.y];
	const uint32_t pairing = prefill_pairing(view, tile, blockIdx.y, tile_count);
	if (pairing == PREFILL_SECOND_OF_TWO)
		return;
	if (pairing == PREFILL_FIRST_OF_TWO) {
		PREFILL_WIDTH_SWITCH((prefill_down<BX2, 2, EXL3_PREFILL_GATE_UP_STEPS>(
			record, arena, view, blockIdx.y, blockIdx.x * PREFILL_GROUPS, dynamic_shared, &shared)))
	} else {
		PREFILL_WIDTH_SWITCH((prefill_down<BX2, 1, EXL3_PREFILL_DOWN_STEPS>(
			record, arena, view, blockIdx.y, blockIdx.x * PREFILL_GROUPS, dynamic_shared, &shared)))
	}
}

/* grid (ceil(H / 512), row capacity) x 128: FP32 row sums over the row's local pairs from +0 in ascending slot order,
 * four channels a thread */
extern "C" __global__ void __launch_bounds__(EXL3_ROW_SUM_THREADS)
	exl3_prefill_row_sum(struct exl3_prefill_record record, unsigned char *arena)
{
	const struct step_block step = *reinterpret_cast<const struct step_block *>(arena + record.step_offset);
	const uint32_t channel = (blockIdx.x * blockDim.x + threadIdx.x) * 4u;
	const uint64_t row = blockIdx.y;
	if (channel >= record.input_size || row >= min(step.row_count, record.row_capacity))
		return;
	const uint32_t width = record.input_size, slots = record.picks + record.shared_count;
	const float *const pairs = reinterpret_cast<const float *>(arena + record.pair_output_offset);
	const uint32_t *const picked = reinterpret_cast<const uint32_t *>(arena + record.picks_offset) + row * record.picks;
	float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
	for (uint32_t slot = 0; slot < slots; slot++) {
		/* a routed pair counts where its expert is held; an always-on pair everywhere it exists */
		if (slot < record.picks && picked[slot] - record.local_first >= record.local_count)
			continue;
		const float4 value = *reinterpret_cast<const float4 *>(pairs + (row * slots + slot) * width + channel);
		sum.x = __fadd_rn(sum.x, value.x);
		sum.y = __fadd_rn(sum.y, value.y);
		sum.z = __fadd_rn(sum.z, value.z);
		sum.w = __fadd_rn(sum.w, value.w);
	}
	*reinterpret_cast<float4 *>(reinterpret_cast<float *>(arena + record.row_output_offset) + row * width + channel) = sum;
}
