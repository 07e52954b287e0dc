/*
 * ref_shims.c: exports of static inline functions of the REFERENCE's headers, so that the tests can compare this
 * library's restated formulas with them. TEST INFRASTRUCTURE: compiled only into oracle/_ref/libanemone_ref.so, where
 * the reference tree is present; it holds no reference code, only calls into its headers.
 */
#include <stdint.h>

#include "anemone/exl3_tc_records.h"
#include "bf16_wire_codec.h"

uint64_t ref_exl3_tc_workspace_bytes(uint64_t pair_count, uint64_t intermediate)
{
	return exl3_tc_workspace_bytes(pair_count, intermediate);
}

uint64_t ref_exl3_tcp_workspace_bytes(uint64_t rows, uint64_t intermediate)
{
	return exl3_tcp_workspace_bytes(rows, intermediate);
}

uint64_t ref_exl3_tc_record_bytes(void)
{
	return sizeof(struct exl3_tc_record);
}

uint64_t ref_exl3_tcp_record_bytes(void)
{
	return sizeof(struct exl3_tcp_record);
}

uint32_t ref_bf16_wire_pair_pack(uint32_t word, uint32_t top)
{
	return bf16_wire_pair_pack(word, top);
}

uint32_t ref_bf16_wire_pair_unpack(uint32_t mantissas, uint32_t deltas, uint32_t top)
{
	return bf16_wire_pair_unpack(mantissas, deltas, top);
}

/* a digest of the reference's packed words over every bfloat16 value doubled into a word, at every shared exponent it
 * admits (the sweep of the reference's tests/bf16_wire_codec_test.c:39-47) */
uint64_t ref_bf16_wire_digest(void)
{
	uint64_t digest = 0xCBF29CE484222325ull;
	for (uint32_t value = 0; value < 65536u; value++) {
		const uint32_t word = value | value << 16, exponent = bf16_wire_low_exponent(word);
		for (uint32_t delta = 0; delta <= 15u && exponent + delta <= 255u; delta++)
			digest = (digest ^ bf16_wire_pair_pack(word, exponent + delta)) * 0x100000001B3ull;
	}
	return digest;
}
