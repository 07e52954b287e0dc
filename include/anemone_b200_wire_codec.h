/*
 * anemone_b200_wire_codec.h: the lossless exponent-delta code of eight bfloat16 values (two to a word) against a shared
 * top exponent: eight sign-and-mantissa bytes and eight exponent nibbles, three words instead of four (reference:
 * source/bf16_wire_codec.h:38-70). Integer leaves only: every bfloat16 bit survives, signed zeros and not-a-number
 * payloads included; the caller proves top >= every exponent and top - exponent <= 15 before packing and unpacks with
 * the same top. C11 and CUDA.
 */
#ifndef ANEMONE_B200_WIRE_CODEC_H
#define ANEMONE_B200_WIRE_CODEC_H

#include <stdint.h>

#if defined(__CUDACC__)
#define AB_WIRE_INLINE static __host__ __device__ __forceinline__
#else
#define AB_WIRE_INLINE static inline
#endif

#define BF16_WIRE_DELTA_MASK 15u /* the largest exponent difference a packed value may have */

/* the exponent field of the low and of the high bfloat16 of a word */
AB_WIRE_INLINE uint32_t bf16_wire_low_exponent(uint32_t word)
{
	return (word >> 7) & 255u;
}

AB_WIRE_INLINE uint32_t bf16_wire_high_exponent(uint32_t word)
{
	return (word >> 23) & 255u;
}

/* sign and mantissa of a bfloat16 as one byte: the mantissa's seven bits, the sign on top */
AB_WIRE_INLINE uint32_t bf16_wire_byte(uint32_t half)
{
	return (half & 127u) | ((half >> 8) & 128u);
}

/* a word's two values: their bytes in bits 0..15, their exponent distances from top in bits 16..19 and 20..23 */
AB_WIRE_INLINE uint32_t bf16_wire_pair_pack(uint32_t word, uint32_t top)
{
	const uint32_t bytes = bf16_wire_byte(word & 0xFFFFu) | bf16_wire_byte(word >> 16) << 8;
	const uint32_t deltas = (top - bf16_wire_low_exponent(word)) | (top - bf16_wire_high_exponent(word)) << 4;
	return bytes | deltas << 16;
}

AB_WIRE_INLINE uint32_t bf16_wire_half(uint32_t byte, uint32_t delta, uint32_t top)
{
	return (byte & 127u) | ((byte & 128u) << 8) | ((top - (delta & BF16_WIRE_DELTA_MASK)) << 7);
}

/* the word back from its two bytes (bits 0..15 of `bytes`) and its two distances (bits 0..7 of `deltas`) */
AB_WIRE_INLINE uint32_t bf16_wire_pair_unpack(uint32_t bytes, uint32_t deltas, uint32_t top)
{
	return bf16_wire_half(bytes, deltas, top) | bf16_wire_half(bytes >> 8, deltas >> 4, top) << 16;
}

#undef AB_WIRE_INLINE
#endif
