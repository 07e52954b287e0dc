/*
 * anemone_b200_router.h: load-time preparation of the router select that feeds the expert launches their job table.
 * Host C11. A refusal leaves the launch unchanged.
 */
#ifndef ANEMONE_B200_ROUTER_H
#define ANEMONE_B200_ROUTER_H

#include "anemone_b200_backend.h"
#include "anemone_b200_records.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Worst-case jobs of `rows` live rows: every pick its own job, plus the shared experts' jobs of eight rows. */
uint32_t router_b200_job_capacity(uint32_t rows, uint32_t picks, uint32_t shared_count);

/* Takes the place of router_select_prepare for this path (include/anemone/router.h; the reference's record is fixed
 * to its model's 384 experts and 6 picks, this one carries them). Checks counts against the kernel's limits
 * (ROUTER_B200_MAXIMUM_*), that job_capacity covers the worst case of row_capacity rows, the scoring code, a finite
 * positive route scale, and that the six ranges lie inside the arena, 16-byte aligned and disjoint. One launch:
 * ("kernel_router_b200", "router_select_b200"), one block of ROUTER_B200_THREADS threads. */
MUST_CHECK result_status router_select_b200_prepare(const struct router_select_b200_arguments *arguments,
						    uint64_t arena_byte_count,
						    const struct backend_operations *backend, struct device_card *card,
						    struct kernel_launch *launch_out);

/* B200 extension: router_select_b200 and the activation quantizer of the step's rows in ONE launch
 * ("router_select_quantize", struct router_select_quantize_arguments): the first launch of an original-weights decode
 * step. router: as router_select_b200_prepare takes it; quantize_launch: the launch linear_quantize_prepare wrote for
 * the rows (its record and row count are taken over). The results are the two launches'. */
MUST_CHECK result_status router_select_quantize_prepare(const struct router_select_b200_arguments *router,
							const struct kernel_launch *quantize_launch,
							uint64_t arena_byte_count,
							const struct backend_operations *backend, struct device_card *card,
							struct kernel_launch *launch_out);

/* B200 extension: the job table of many rows (struct router_wide_arguments): ROUTER_WIDE_LAUNCHES launches. Checks
 * the counts against the kernels' limits, routing.local_first == 0, local_count == expert_count, shared_count == 0,
 * job_capacity >= row_capacity * picks / 8 + expert_count, and the ranges (scores, bias, expert table, picks, weights,
 * the workspace up to its operand blocks, jobs, step block): inside the arena, aligned, disjoint. */
MUST_CHECK result_status router_wide_prepare(const struct router_wide_arguments *arguments, uint64_t arena_byte_count,
					     const struct backend_operations *backend, struct device_card *card,
					     struct kernel_launch *launches_out);

/* No reference counterpart (its step driver uploads every step block from the host). Checks the pool, the destination
 * and the cursor ranges (16-byte aligned, inside the arena, disjoint), pool_count >= 1, byte_count a positive multiple
 * of 16 not above pool_stride. One launch: ("kernel_router_b200", "step_input_select"), one block. */
MUST_CHECK result_status step_input_select_prepare(const struct step_input_select_arguments *arguments,
						   uint64_t arena_byte_count,
						   const struct backend_operations *backend, struct device_card *card,
						   struct kernel_launch *launch_out);

#ifdef __cplusplus
}
#endif
#endif
