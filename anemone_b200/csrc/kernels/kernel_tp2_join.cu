/*
 * kernel_tp2_join.cu: the local completion around the exchange (kernel file "kernel_tp2_join", entry "tp2_join":
 * source/kernel_tp2_join.cu:43-108): element-wise, no signals. grid (ceil(width / 256), rows) x 256, a thread an
 * element; rows beyond row_count and columns beyond width are not touched, nor the gaps between strided rows.
 */
#include "ordered_device.cuh"

/* The place of element (row, column) in the owner-major order of the reference's four-rank ring
 * (source/kernel_tp2_join.cu:6-41): a slab is 8 rows (the last one what is left); owner o holds quarter o of a slab's
 * elements, counted row by row; an owner's quarters follow slab after slab, the owners one another. */
__device__ __forceinline__ uint64_t join_ring_place(uint32_t row, uint32_t column, uint32_t rows, uint32_t width)
{
	const uint32_t slab = row / TP2_JOIN_RING_SLAB_ROWS, row_in_slab = row % TP2_JOIN_RING_SLAB_ROWS;
	const uint32_t slab_rows = min(rows - slab * TP2_JOIN_RING_SLAB_ROWS, TP2_JOIN_RING_SLAB_ROWS);
	const uint32_t quarter = slab_rows * width / TP2_JOIN_RING_OWNERS; /* width is a multiple of the owners */
	const uint32_t in_slab = row_in_slab * width + column;
	const uint32_t owner = in_slab / quarter;
	return (uint64_t)owner * ((uint64_t)rows * width / TP2_JOIN_RING_OWNERS) +
	       (uint64_t)slab * (TP2_JOIN_RING_SLAB_ROWS * width / TP2_JOIN_RING_OWNERS) + (in_slab - owner * quarter);
}

__device__ __forceinline__ float join_bfloat16_value(uint16_t bits)
{
	return __uint_as_float((uint32_t)bits << 16);
}

extern "C" __global__ void __launch_bounds__(TP2_JOIN_THREADS)
	tp2_join(struct tp2_join_arguments arguments, unsigned char *arena)
{
	const uint32_t column = blockIdx.x * blockDim.x + threadIdx.x, row = blockIdx.y;
	if (column >= arguments.width || row >= arguments.row_count)
		return;
	const uint64_t parity = arguments.source_slot_stride != 0 || arguments.output_slot_stride != 0 ?
					reinterpret_cast<const struct step_block *>(arena + arguments.step_offset)->sequence & 1u :
					0u;
	const unsigned char *const source = arena + arguments.source_offset + parity * arguments.source_slot_stride;
	unsigned char *const output = arena + arguments.output_offset + parity * arguments.output_slot_stride;
	const uint64_t from = (uint64_t)row * arguments.source_row_stride + column;
	const uint64_t to = (uint64_t)row * arguments.output_row_stride + column;
	const uint32_t operation = arguments.operation;
	if (operation == TP2_JOIN_BFLOAT16_COPY) {
		reinterpret_cast<uint16_t *>(output)[to] = reinterpret_cast<const uint16_t *>(source)[from];
		return;
	}
	if (operation == TP2_JOIN_FLOAT32_COPY) {
		reinterpret_cast<uint32_t *>(output)[to] = reinterpret_cast<const uint32_t *>(source)[from];
		return;
	}
	if (operation == TP2_JOIN_RING_UNPACK) {
		reinterpret_cast<uint16_t *>(output)[to] = reinterpret_cast<const uint16_t *>(
			source)[join_ring_place(row, column, arguments.row_count, arguments.width)];
		return;
	}
	if (operation == TP2_JOIN_FLOAT32_TO_BFLOAT16) {
		reinterpret_cast<uint16_t *>(output)[to] =
			(uint16_t)bfloat16_bits(reinterpret_cast<const float *>(source)[from]);
		return;
	}
	/* the three that take a bfloat16 value and may add the routed FP32 sum in front of it */
	float value = join_bfloat16_value(reinterpret_cast<const uint16_t *>(source)[from]);
	if (arguments.has_routed_sums != 0)
		value = __fadd_rn(reinterpret_cast<const float *>(
					  arena + arguments.routed_sums_offset)[(uint64_t)row * arguments.routed_row_stride + column],
				  value);
	if (operation == TP2_JOIN_BFLOAT16_TO_FLOAT32)
		reinterpret_cast<float *>(output)[to] = value;
	else if (operation == TP2_JOIN_BFLOAT16_SUM_TO_BFLOAT16)
		reinterpret_cast<uint16_t *>(output)[to] = (uint16_t)bfloat16_bits(value);
	else
		reinterpret_cast<uint16_t *>(output)[join_ring_place(row, column, arguments.row_count, arguments.width)] =
			(uint16_t)bfloat16_bits(value);
}
