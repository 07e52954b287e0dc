/*
 * anemone_b200_noalloc.h: the one entry point of this library that needs no scratch memory from its caller.
 */
#ifndef ANEMONE_B200_NOALLOC_H
#define ANEMONE_B200_NOALLOC_H

#include <stdint.h>

#include "anemone_b200_status.h"

#ifdef __cplusplus
extern "C" {
#endif

#define EXL3_NOALLOC_MOST_ROWS 8u
#define EXL3_NOALLOC_MOST_HIDDEN 8192u
#define EXL3_NOALLOC_MOST_INNER 8192u
/* job record 256 + FP16 operands 262144 + FP32 products 524288 + bfloat16 hidden 131072 bytes, held in the library
 * image by every GPU that loads it */
#define EXL3_NOALLOC_SCRATCH_BYTES 917760u

/* This entry point has no counterpart in the reference, whose every launch works on ranges its caller reserved in the
 * card's arena. It exists for callers that cannot allocate device memory at the moment of the call (a serving loop
 * that must not stall the GPU with cudaMalloc between tokens, a plug-in that only receives device pointers, a process
 * with a memory budget fixed at start-up): the chain's scratch is a fixed array inside the library instead.
 *
 * One EXL3 expert block on the current CUDA device: output[row] = route_weights[row] * down(SwiGLU(gate(x), up(x)))
 * for rows 0 .. rows - 1, FP32 [rows][hidden], with the arithmetic of exl3_experts_prepare's five launches.
 *   gate, up     device pointers to stored matrices of hidden inputs x inner outputs; down: inner x hidden;
 *   tokens       device pointer, bfloat16 [rows][hidden]; output: device pointer, FP32 [rows][hidden];
 *   route_weights  HOST pointer to `rows` floats, or NULL for all ones;  every device pointer 16-byte aligned;
 *   stream       a cudaStream_t of the current device (NULL: the default stream);
 *   wait_for_result  non-zero: return only when the output is complete.
 * Limits: rows <= EXL3_NOALLOC_MOST_ROWS, hidden <= EXL3_NOALLOC_MOST_HIDDEN, inner <= EXL3_NOALLOC_MOST_INNER and
 * inner <= hidden, both multiples of 128, a stored width of 2, 40 (2.5 bits), 3 or 4; anything else is
 * STATUS_INVALID_ARGUMENT (sizes beyond the limits also print one line on stderr). It allocates nothing.
 * All calls on one GPU share the fixed scratch: calls that overlap in time on the same GPU race and must be serialised
 * by the caller. Every call looks up the scratch's device address for the current device (no allocation, no state
 * kept between calls); the first call on a device makes the CUDA runtime load the library's device code there and
 * should come before any stream capture is begun. The scratch lives in the context the CUDA runtime uses for the
 * calling thread (the device's primary context unless the caller made another current) and does not outlive a
 * cudaDeviceReset (the next call finds the new one). */
MUST_CHECK result_status exl3_expert_block_noalloc(const void *gate, const void *up, const void *down,
						   const void *tokens, const float *route_weights, void *output,
						   uint32_t rows, uint32_t hidden, uint32_t inner, uint32_t stored_width,
						   float activation_limit, void *stream, uint32_t wait_for_result);

#ifdef __cplusplus
}
#endif
#endif
