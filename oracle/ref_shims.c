/*
 * ref_shims.c: exports of static inline functions of the REFERENCE's headers, so that the tests can compare this
 * library's restated formulas with them. TEST INFRASTRUCTURE: compiled only into oracle/_ref/libanemone_ref.so, where
 * the reference tree is present; it holds no reference code, only calls into its headers.
 */
#include <stdint.h>

#include "anemone/exl3_tc_records.h"

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
