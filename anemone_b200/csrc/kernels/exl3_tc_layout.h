/*
 * exl3_tc_layout.h: how the entry points of anemone_b200_exl3_tc.h lay this library's scratch out inside the
 * workspace a caller sized with the reference's formulas, and the struct exl3_moe_record their kernels work on.
 * C11 and CUDA: the host preparer checks that the layout fits, the kernels derive the same record from the caller's.
 */
#ifndef AB_EXL3_TC_LAYOUT_H
#define AB_EXL3_TC_LAYOUT_H

#include "anemone_b200_exl3_tc.h"
#include "exl3_geometry.h"

struct exl3_tc_layout {
	uint64_t operands, products, counters, hidden, routed, jobs, total; /* byte offsets inside the workspace */
	uint32_t gate_up_runs, down_runs, job_capacity, reserved_zero;
};

/* pairs, intermediate: the call's; own_jobs: the job table lies in the workspace (the prefill entry points build it
 * there) for this many jobs, else 0. Products are cut as exl3_moe_splits cuts them while that fits the workspace the
 * caller reserved; a call of many pairs has enough work items uncut. */
AB_INLINE struct exl3_tc_layout exl3_tc_layout_of(uint64_t pairs, uint32_t job_capacity, uint32_t intermediate,
						   uint32_t own_jobs, uint64_t workspace_bytes)
{
	struct exl3_tc_layout layout;
	const uint64_t H = EXL3_TC_HIDDEN, I = intermediate;
	layout.job_capacity = own_jobs != 0 ? own_jobs : job_capacity;
	layout.reserved_zero = 0;
	layout.gate_up_runs = exl3_moe_splits(EXL3_TC_HIDDEN, intermediate);
	layout.down_runs = exl3_moe_splits(intermediate, EXL3_TC_HIDDEN);
	for (;;) {
		const uint64_t gate_up = 2u * layout.gate_up_runs * pairs * I * 4u, down = layout.down_runs * pairs * H * 4u;
		uint64_t cursor = 0;
		layout.operands = cursor;
		cursor += exl3_tc_aligned(pairs * H * 4u + pairs * I * 2u);
		layout.products = cursor;
		cursor += exl3_tc_aligned(gate_up > down ? gate_up : down);
		layout.counters = cursor;
		cursor += exl3_tc_aligned((uint64_t)layout.job_capacity * (I / EXL3_TRANSFORM + H / EXL3_TRANSFORM) * 4u);
		layout.hidden = cursor;
		cursor += exl3_tc_aligned(pairs * I * 2u);
		layout.routed = cursor;
		cursor += exl3_tc_aligned(pairs * 4u);
		layout.jobs = cursor;
		cursor += exl3_tc_aligned((uint64_t)own_jobs * sizeof(struct expert_job_record));
		layout.total = cursor;
		if (cursor <= workspace_bytes || (layout.gate_up_runs == 1u && layout.down_runs == 1u))
			return layout;
		if (layout.gate_up_runs > 1u)
			layout.gate_up_runs /= 2u;
		else
			layout.down_runs /= 2u;
	}
}

/* jobs the route launch of the prefill entry points may write: an expert's pairs in jobs of eight, the last ragged */
AB_INLINE uint32_t exl3_tcp_job_capacity(uint64_t pairs)
{
	const uint64_t most = pairs / LINEAR_MAXIMUM_ROWS + EXL3_TCP_EXPERTS;
	return (uint32_t)(most < pairs ? most : pairs);
}

AB_INLINE uint32_t exl3_tc_stored_width(uint32_t bits_x2)
{
	return (bits_x2 & 1u) != 0 ? 8u * bits_x2 : bits_x2 / 2u;
}

/* The record the fused kernels work on, from a decode record (rotation 0). */
AB_INLINE struct exl3_moe_record exl3_tc_moe_record(uint64_t jobs_offset, uint64_t hidden_offset,
						    uint64_t workspace_offset, uint64_t output_offset,
						    uint32_t row_count, uint32_t intermediate, uint32_t bits_x2,
						    float activation_limit, const struct exl3_tc_layout *layout)
{
	struct exl3_moe_record moe;
	moe.base.jobs_offset = jobs_offset;
	moe.base.input_offset = hidden_offset;
	moe.base.operands_offset = workspace_offset + layout->operands;
	moe.base.products_offset = workspace_offset + layout->products;
	moe.base.hidden_offset = workspace_offset + layout->hidden;
	moe.base.output_offset = moe.base.products_offset;
	moe.base.input_size = EXL3_TC_HIDDEN;
	moe.base.inner_size = intermediate;
	moe.base.pair_count = row_count * EXL3_TC_PAIRS_PER_ROW;
	moe.base.pairs_per_row = EXL3_TC_PAIRS_PER_ROW;
	moe.base.job_count = layout->job_capacity;
	moe.base.bits_per_weight = exl3_tc_stored_width(bits_x2);
	/* no limit: one no finite value reaches */
	moe.base.activation_limit = activation_limit > 0.0f ? activation_limit : 3.0e38f;
	moe.base.reserved_zero = 0;
	moe.widths_offset = 0;
	moe.row_output_offset = output_offset;
	moe.counters_offset = workspace_offset + layout->counters;
	moe.expert_count = EXL3_TCP_EXPERTS;
	moe.reserved_zero = 0;
	return moe;
}

#endif
