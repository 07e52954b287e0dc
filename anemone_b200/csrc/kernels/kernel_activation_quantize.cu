/*
 * kernel_activation_quantize.cu: bfloat16 vectors to E4M3 codes with one E8M0 exponent per 32 values, for the
 * original-weights experts (reference: source/kernel_activation_quantize.cu, contract include/anemone/
 * linear_records.h:36-44 and 222-235). grid (width / 64, vectors), block 32: a warp a load of 64 values, lane i holds
 * values 2 i and 2 i + 1, lanes 0-15 are one block of 32 and lanes 16-31 the other.
 * Per block, in FP32: m = max(largest magnitude, 1e-4f) * (1 / 448.0f); the code c of the smallest power of two not
 * below m is read from the bits of m; magnitudes are divided by 2^(c - 127) (exact), limited to 448 and converted to
 * E4M3 to nearest, a tie to the even code (the hardware conversion cvt.rn.satfinite.e4m3x2.f32 rounds so). The sign is
 * kept, also of a zero. Writes the codes in lane order, the exponents, and the operands of this arithmetic class: the
 * code placed as an FP16 (value times 2^-8) in operand order.
 */
#include "activation_quantize_device.cuh"

extern "C" __global__ void __launch_bounds__(32)
	activation_quantize_entry(struct activation_quantize_arguments arguments, unsigned char *arena)
{
	activation_quantize_load(arguments, arena, blockIdx.y, blockIdx.x, threadIdx.x);
}
