/*
 * exl3_expert_noalloc.cu: one EXL3 expert block (gate, up, SwiGLU, down for up to eight token rows) for callers that
 * cannot allocate device memory.
 *
 * Who that is: code that runs where an allocation is forbidden or would stall everything else on the GPU - a serving
 * loop that must not call cudaMalloc between tokens (it synchronises the whole device), a plug-in that is handed
 * device pointers by its host application and has no allocator of its own, or a process whose memory budget was fixed
 * at start-up. The card interface of this library asks its caller to reserve scratch ranges in the arena; here the
 * scratch (FP16 operands, FP32 products, the job record) lives instead in a file-scope device array of fixed size, so
 * the caller passes only the expert's matrices, the tokens and the output.
 *
 * The price, all of it to be known by the caller:
 *   - the array (EXL3_NOALLOC_SCRATCH_BYTES) is part of the library image: every GPU that loads the library holds it
 *     until the process exits, whether or not this entry point is ever called;
 *   - sizes beyond EXL3_NOALLOC_MOST_ROWS / _MOST_HIDDEN / _MOST_INNER are refused with STATUS_INVALID_ARGUMENT and one
 *     line on stderr;
 *   - every call on a device shares the one array and finds the previous call's contents in it. Each call rewrites
 *     everything it later reads, and nothing in it needs to start at zero, but two calls that overlap on the same GPU
 *     (different streams, different threads) race on it: serialise them;
 *   - every call looks up the array's device address for the device that is current (cudaGetSymbolAddress, which
 *     allocates nothing and keeps no state here: nothing goes stale when a context is reset, and two host threads
 *     share no variable of this file). The first call on a device makes the CUDA runtime load this library's device
 *     code there; that first call should come before any stream capture begins. The address is that of the context
 *     the CUDA runtime uses for the calling thread (the device's primary context unless the caller made another one
 *     current); asking on every call is what keeps it right.
 * It calls no cudaMalloc, cudaFree or any allocating routine. The arithmetic is the five-pass chain's
 * (exl3_passes.cuh), so its results equal exl3_experts_prepare's launches on the same inputs.
 */
#include <cuda_runtime.h>
#include <stdio.h>

#include "exl3_passes.cuh"

extern "C" {
#include "anemone_b200_noalloc.h"
}

/* the scratch, in the order the chain uses it; every part a multiple of 256 bytes */
#define NOALLOC_JOB_BYTES 256u
#define NOALLOC_OPERAND_BYTES (2u * EXL3_NOALLOC_MOST_ROWS * EXL3_NOALLOC_MOST_HIDDEN * 2u)
#define NOALLOC_PRODUCT_BYTES (2u * EXL3_NOALLOC_MOST_ROWS * EXL3_NOALLOC_MOST_HIDDEN * 4u)
#define NOALLOC_HIDDEN_BYTES (EXL3_NOALLOC_MOST_ROWS * EXL3_NOALLOC_MOST_INNER * 2u)
static_assert(NOALLOC_JOB_BYTES + NOALLOC_OPERAND_BYTES + NOALLOC_PRODUCT_BYTES + NOALLOC_HIDDEN_BYTES ==
		      EXL3_NOALLOC_SCRATCH_BYTES,
	      "the stated scratch size is the sum of its parts");

/* In host code this name is only a stand-in for the symbol: it is not a device address. Host code gets the address
 * from cudaGetSymbolAddress, with the device current, and hands it to the kernels as their arena. */
static __device__ __align__(256) unsigned char noalloc_scratch[EXL3_NOALLOC_SCRATCH_BYTES];
static_assert(EXL3_PRODUCT_PARTIAL_BYTES <= 48u * 1024u,
	      "the product kernels' dynamic shared memory needs no opt-in attribute (no per-device set-up to keep)");

/* The chain's records name memory by offset from an arena. Here the arena is the scratch array and a caller's pointer
 * becomes the (wrapping) 64-bit distance from it, so the shared device functions run unchanged. */
static uint64_t distance_from(const unsigned char *arena, const void *pointer)
{
	return (uint64_t)(uintptr_t)pointer - (uint64_t)(uintptr_t)arena;
}

static __global__ void noalloc_job(struct expert_job_record job, unsigned char *arena)
{
	if (threadIdx.x == 0)
		*reinterpret_cast<struct expert_job_record *>(arena) = job;
}

static __global__ void __launch_bounds__(EXL3_TRANSFORM_THREADS)
	noalloc_input(struct exl3_expert_record record, unsigned char *arena)
{
	exl3_input_pass(record, arena, nullptr);
}

static __global__ void __launch_bounds__(EXL3_TRANSFORM_THREADS)
	noalloc_activate(struct exl3_expert_record record, unsigned char *arena)
{
	exl3_activate_pass(record, arena, nullptr, record.inner_size, record.input_size, 0u);
}

static __global__ void __launch_bounds__(EXL3_TRANSFORM_THREADS)
	noalloc_finish(struct exl3_expert_record record, unsigned char *arena)
{
	exl3_finish_pass(record, arena, nullptr);
}

template <bool DOWN>
static __global__ void __launch_bounds__(EXL3_PRODUCT_THREADS)
	noalloc_product(struct exl3_expert_record record, unsigned char *arena)
{
	extern __shared__ __align__(128) unsigned char dynamic_shared[];
	__shared__ exl3_product_shared shared;
	exl3_product_any_width<DOWN>(record, arena, nullptr, dynamic_shared, &shared);
}

static result_status runtime_failure(const char *what, cudaError_t error)
{
	(void)fprintf(stderr, "anemone_b200: exl3_expert_block_noalloc: %s failed: %s\n", what, cudaGetErrorString(error));
	return STATUS_DEVICE_ERROR;
}

extern "C" result_status exl3_expert_block_noalloc(const void *gate, const void *up, const void *down,
						   const void *tokens, const float *route_weights, void *output,
						   uint32_t rows, uint32_t hidden, uint32_t inner, uint32_t stored_width,
						   float activation_limit, void *stream, uint32_t wait_for_result)
{
	if (gate == NULL || up == NULL || down == NULL || tokens == NULL || output == NULL || rows == 0 ||
	    hidden == 0 || inner == 0 || hidden % EXL3_TRANSFORM != 0 || inner % EXL3_TRANSFORM != 0 || inner > hidden ||
	    !exl3_width_supported(stored_width) || !(activation_limit > 0.0f) ||
	    ((uintptr_t)gate | (uintptr_t)up | (uintptr_t)down | (uintptr_t)tokens | (uintptr_t)output) % 16u != 0)
		return STATUS_INVALID_ARGUMENT;
	if (rows > EXL3_NOALLOC_MOST_ROWS || hidden > EXL3_NOALLOC_MOST_HIDDEN || inner > EXL3_NOALLOC_MOST_INNER) {
		(void)fprintf(stderr,
			      "anemone_b200: exl3_expert_block_noalloc: %u rows x hidden %u x inner %u is beyond the fixed "
			      "scratch (at most %u rows, hidden %u, inner %u)\n",
			      rows, hidden, inner, EXL3_NOALLOC_MOST_ROWS, EXL3_NOALLOC_MOST_HIDDEN, EXL3_NOALLOC_MOST_INNER);
		return STATUS_INVALID_ARGUMENT;
	}
	/* the scratch's address on the device that is current: asked for on every call (it allocates nothing) */
	unsigned char *arena = NULL;
	cudaError_t error = cudaGetSymbolAddress((void **)&arena, noalloc_scratch);
	if (error != cudaSuccess || arena == NULL)
		return runtime_failure("cudaGetSymbolAddress", error);
	struct expert_job_record job;
	memset(&job, 0, sizeof(job));
	job.gate_offset = distance_from(arena, gate);
	job.up_offset = distance_from(arena, up);
	job.down_offset = distance_from(arena, down);
	job.row_count = rows;
	for (uint32_t row = 0; row < rows; row++) {
		job.pair_index[row] = row;
		job.route_weight[row] = route_weights != NULL ? route_weights[row] : 1.0f;
	}
	struct exl3_expert_record record;
	memset(&record, 0, sizeof(record));
	record.jobs_offset = 0;
	record.input_offset = distance_from(arena, tokens);
	record.operands_offset = NOALLOC_JOB_BYTES;
	record.products_offset = NOALLOC_JOB_BYTES + NOALLOC_OPERAND_BYTES;
	record.hidden_offset = record.products_offset + NOALLOC_PRODUCT_BYTES;
	record.output_offset = distance_from(arena, output); /* the finish pass reads products, writes here */
	record.input_size = hidden;
	record.inner_size = inner;
	record.pair_count = rows;
	record.pairs_per_row = 1;
	record.job_count = 1;
	record.bits_per_weight = stored_width;
	record.activation_limit = activation_limit;
	const cudaStream_t queue = (cudaStream_t)stream;
	const uint32_t bits_x2 = exl3_bits_x2(stored_width);
	const uint32_t shared_bytes = exl3_product_dynamic_bytes(bits_x2);
	const uint32_t outer_blocks = (hidden / EXL3_TRANSFORM + EXL3_TRANSFORM_WARPS - 1u) / EXL3_TRANSFORM_WARPS;
	const uint32_t inner_blocks = (inner / EXL3_TRANSFORM + EXL3_TRANSFORM_WARPS - 1u) / EXL3_TRANSFORM_WARPS;
	noalloc_job<<<1, 32, 0, queue>>>(job, arena);
	noalloc_input<<<dim3(outer_blocks, 1, EXL3_PROJECTIONS), EXL3_TRANSFORM_THREADS, 0, queue>>>(record, arena);
	noalloc_product<false><<<dim3(inner / EXL3_TRANSFORM, 1, EXL3_PROJECTIONS), EXL3_PRODUCT_THREADS, shared_bytes,
				 queue>>>(record, arena);
	noalloc_activate<<<dim3(inner_blocks, 1, 1), EXL3_TRANSFORM_THREADS, 0, queue>>>(record, arena);
	noalloc_product<true><<<dim3(hidden / EXL3_TRANSFORM, 1, 1), EXL3_PRODUCT_THREADS, shared_bytes, queue>>>(record,
													  arena);
	noalloc_finish<<<dim3(outer_blocks, 1, 1), EXL3_TRANSFORM_THREADS, 0, queue>>>(record, arena);
	error = cudaGetLastError();
	if (error != cudaSuccess)
		return runtime_failure("a launch", error);
	if (wait_for_result != 0) {
		error = cudaStreamSynchronize(queue);
		if (error != cudaSuccess)
			return runtime_failure("waiting for the result", error);
	}
	return STATUS_OK;
}
