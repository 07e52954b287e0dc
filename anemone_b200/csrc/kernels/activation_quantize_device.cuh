/*
 * activation_quantize_device.cuh: one warp's task of the activation quantizer: a load of 64 bfloat16 values of one
 * vector to E4M3 codes, the two E8M0 exponents of its blocks of 32 and the operands (the arithmetic is stated at
 * kernel_activation_quantize.cu). All 32 lanes call.
 */
#ifndef AB_ACTIVATION_QUANTIZE_DEVICE_CUH
#define AB_ACTIVATION_QUANTIZE_DEVICE_CUH

#include <cuda_fp8.h>
#include <stdint.h>

#include "anemone_b200_records.h"

__device__ __forceinline__ void activation_quantize_load(const struct activation_quantize_arguments &arguments,
							  unsigned char *arena, uint32_t vector, uint32_t load,
							  uint32_t lane)
{
	const uint32_t width = arguments.width;
	const uint32_t raw = reinterpret_cast<const uint32_t *>(arena + arguments.values_offset)[((uint64_t)vector * width +
												 64u * load) / 2u + lane];
	const float low = __uint_as_float(raw << 16), high = __uint_as_float(raw & 0xFFFF0000u);
	float largest = fmaxf(fabsf(low), fabsf(high));
	for (uint32_t distance = 1; distance < 16u; distance <<= 1)
		largest = fmaxf(largest, __shfl_xor_sync(0xFFFFFFFFu, largest, distance));
	const float ratio = __fmul_rn(fmaxf(largest, 1.0e-4f), 1.0f / 448.0f);
	const uint32_t bits = __float_as_uint(ratio);
	const uint32_t code = (bits >> 23) + ((bits & 0x007FFFFFu) != 0 ? 1u : 0u); /* E8M0 has float32's bias */
	const float inverse = __uint_as_float((254u - code) << 23);
	const float2 scaled = make_float2(__fmul_rn(low, inverse), __fmul_rn(high, inverse));
	uint32_t pair = __nv_cvt_float2_to_fp8x2(scaled, __NV_SATFINITE, __NV_E4M3); /* byte 0: low, byte 1: high */
	/* the conversion drops the sign of a zero on some inputs' paths: restore it from the source bits */
	pair = (pair & 0x7F7Fu) | ((raw >> 8) & 0x80u) | ((raw >> 16) & 0x8000u);
	const uint32_t code_low = pair & 0xFFu, code_high = (pair >> 8) & 0xFFu;
	/* value v = 2 lane + h of the load: step s = v / 16, k = v % 16, lane place t = (k % 8) / 2, register r = k / 8 */
	const uint32_t k = (2u * lane) % 16u, s = (2u * lane) / 16u, t = (k % 8u) / 2u, r = k / 8u;
	unsigned char *const codes = arena + arguments.codes_offset + (uint64_t)vector * width + 64u * load;
	codes[(t * 4u + s) * 4u + r] = (unsigned char)code_low; /* j = 2 (k % 2) + k / 8: h = 0 */
	codes[(t * 4u + s) * 4u + 2u + r] = (unsigned char)code_high; /* h = 1 */
	const uint32_t placed_low = ((code_low & 0x80u) << 8) | ((code_low & 0x7Fu) << 7);
	const uint32_t placed_high = ((code_high & 0x80u) << 8) | ((code_high & 0x7Fu) << 7);
	reinterpret_cast<uint32_t *>(arena + arguments.operands_offset)[((uint64_t)vector * width + 64u * load) / 2u +
									(t * 4u + s) * 2u + r] = placed_low | placed_high << 16;
	if (lane % 16u == 0)
		(arena + arguments.exponents_offset)[(uint64_t)vector * (width / 32u) + 2u * load + lane / 16u] =
			(unsigned char)code;
}

#endif
