/*
 * linear.c: preparation of the original-weights routed experts (anemone_b200_linear.h). Takes the place of the part of
 * the reference's source/linear.c that prepares activation_quantize_entry, expert_gate_up_<S>, expert_down_<S> and
 * expert_row_sum_entry.
 */
#include "anemone_b200_linear.h"

#include <math.h>
#include <stddef.h>
#include <stdio.h>
#include <string.h>

#include "prepare_common.h"

static const uint32_t slice_counts[LINEAR_SLICE_INSTANCES] = { 1, 2, 4, 8, 16 };

static result_status e2m1_stored_byte_count(const struct matrix_shape_record *shape, uint64_t *byte_count_out)
{
	if (shape == NULL || byte_count_out == NULL || shape->reserved_must_be_zero != 0 || shape->output_size == 0 ||
	    shape->input_size == 0 || shape->output_size % LINEAR_OUTPUTS_PER_TILE != 0 ||
	    shape->input_size % LINEAR_VALUES_PER_LOAD != 0 || shape->bits_per_weight != 4)
		return STATUS_INVALID_ARGUMENT;
	const uint64_t weights = (uint64_t)shape->output_size * shape->input_size;
	*byte_count_out = weights / 2u + weights / LINEAR_VALUES_PER_BLOCK;
	return STATUS_OK;
}

const struct weight_format_operations e2m1_scaled_weight_operations = { .name = "e2m1_scaled",
									 .stored_byte_count = e2m1_stored_byte_count };

uint64_t linear_values_byte_count(uint64_t vector_count, uint32_t width)
{
	return vector_count > UINT64_MAX / 2u / (width ? width : 1u) ? UINT64_MAX : vector_count * width * 2u;
}

uint64_t linear_codes_byte_count(uint64_t vector_count, uint32_t width)
{
	return vector_count > UINT64_MAX / (width ? width : 1u) ? UINT64_MAX : vector_count * width;
}

uint64_t linear_exponents_byte_count(uint64_t vector_count, uint32_t width)
{
	return linear_codes_byte_count(vector_count, width / LINEAR_VALUES_PER_BLOCK);
}

uint64_t linear_sums_byte_count(uint64_t row_count, uint32_t width)
{
	return row_count > UINT64_MAX / 4u / (width ? width : 1u) ? UINT64_MAX : row_count * width * 4u;
}

uint64_t linear_jobs_byte_count(uint64_t job_count)
{
	return job_count > UINT64_MAX / sizeof(struct expert_job_record) ? UINT64_MAX :
									   job_count * sizeof(struct expert_job_record);
}

result_status linear_kernels_prepare(const struct backend_operations *backend, struct device_card *card,
				     uint32_t arithmetic_class, struct linear_kernels_record *kernels_out)
{
	if (backend == NULL || backend->kernel_prepare == NULL || card == NULL || kernels_out == NULL)
		return STATUS_INVALID_ARGUMENT;
	if (arithmetic_class == ARITHMETIC_CLASS_SM_80 || arithmetic_class == ARITHMETIC_CLASS_SM_120 ||
	    arithmetic_class == ARITHMETIC_CLASS_SM_120_NATIVE)
		return STATUS_UNSUPPORTED;
	if (arithmetic_class != ARITHMETIC_CLASS_SM_100)
		return STATUS_INVALID_ARGUMENT;
	struct linear_kernels_record kernels;
	memset(&kernels, 0xFF, sizeof(kernels)); /* every member BACKEND_NO_KERNEL */
	result_status status = backend->kernel_prepare(card, KERNEL_FILE_ACTIVATION_QUANTIZE, KERNEL_ACTIVATION_QUANTIZE,
						       sizeof(struct activation_quantize_arguments),
						       &kernels.activation_quantize);
	for (uint32_t instance = 0; status == STATUS_OK && instance < LINEAR_SLICE_INSTANCES; instance++) {
		char name[48];
		(void)snprintf(name, sizeof(name), KERNEL_EXPERT_GATE_UP_STEM "%u", slice_counts[instance]);
		status = backend->kernel_prepare(card, KERNEL_FILE_EXPERT_LINEAR, name,
						 sizeof(struct expert_gate_up_arguments), &kernels.expert_gate_up[instance]);
		if (status != STATUS_OK)
			break;
		(void)snprintf(name, sizeof(name), KERNEL_EXPERT_DOWN_STEM "%u", slice_counts[instance]);
		status = backend->kernel_prepare(card, KERNEL_FILE_EXPERT_LINEAR, name, sizeof(struct expert_down_arguments),
						 &kernels.expert_down[instance]);
	}
	if (status == STATUS_OK)
		status = backend->kernel_prepare(card, KERNEL_FILE_EXPERT_LINEAR, KERNEL_EXPERT_ROW_SUM,
						 sizeof(struct expert_row_sum_arguments), &kernels.expert_row_sum);
	for (uint32_t instance = 0; status == STATUS_OK && instance < LINEAR_SLICE_INSTANCES; instance++) {
		char name[48];
		(void)snprintf(name, sizeof(name), KERNEL_TRUNK_LINEAR_QUANTIZED_STEM "%u", slice_counts[instance]);
		status = backend->kernel_prepare(card, KERNEL_FILE_TRUNK_LINEAR, name,
						 sizeof(struct trunk_linear_quantized_arguments),
						 &kernels.trunk_linear_quantized[instance]);
	}
	if (status == STATUS_OK)
		status = backend->kernel_prepare(card, KERNEL_FILE_TRUNK_LINEAR, KERNEL_TRUNK_HIDDEN_VALUE,
						 sizeof(struct trunk_hidden_arguments), &kernels.trunk_hidden);
	if (status != STATUS_OK) {
		(void)fprintf(stderr, "linear kernels: a kernel could not be prepared (%s)\n", status_text(status));
		return status;
	}
	*kernels_out = kernels;
	return STATUS_OK;
}

static bool range_holds(const struct linear_range *range, uint64_t needed)
{
	return needed != UINT64_MAX && range->byte_count >= needed;
}

result_status linear_quantize_prepare(const struct linear_quantize_description *description, uint64_t arena_byte_count,
				      const struct linear_kernels_record *kernels, struct kernel_launch *launch_out)
{
	if (description == NULL || kernels == NULL || launch_out == NULL ||
	    kernels->activation_quantize == BACKEND_NO_KERNEL || description->width == 0 ||
	    description->width % LINEAR_VALUES_PER_LOAD != 0 || description->row_count == 0 ||
	    description->row_count > 65535u ||
	    !range_holds(&description->values, linear_values_byte_count(description->row_count, description->width)) ||
	    !range_holds(&description->codes, linear_codes_byte_count(description->row_count, description->width)) ||
	    !range_holds(&description->exponents, linear_exponents_byte_count(description->row_count, description->width)) ||
	    !range_holds(&description->operands, linear_values_byte_count(description->row_count, description->width)))
		return STATUS_INVALID_ARGUMENT;
	const struct checked_range ranges[4] = {
		{ "values", description->values.byte_offset, description->values.byte_count },
		{ "codes", description->codes.byte_offset, description->codes.byte_count },
		{ "exponents", description->exponents.byte_offset, description->exponents.byte_count },
		{ "operands", description->operands.byte_offset, description->operands.byte_count }
	};
	if (!prepare_ranges_are_valid("activation quantize", ranges, 4, arena_byte_count))
		return STATUS_INVALID_ARGUMENT;
	const struct activation_quantize_arguments arguments = { description->values.byte_offset,
								  description->codes.byte_offset,
								  description->exponents.byte_offset,
								  description->operands.byte_offset, description->width, 0 };
	prepare_launch_fill(launch_out, kernels->activation_quantize, description->width / LINEAR_VALUES_PER_LOAD,
			    description->row_count, 1, 32, 0, &arguments, sizeof(arguments));
	return STATUS_OK;
}

/* the instance of a slice count, or LINEAR_SLICE_INSTANCES */
static uint32_t slice_instance(uint32_t slice_count, uint32_t input_size)
{
	for (uint32_t instance = 0; instance < LINEAR_SLICE_INSTANCES; instance++)
		if (slice_counts[instance] == slice_count && slice_count <= input_size / LINEAR_VALUES_PER_LOAD)
			return instance;
	return LINEAR_SLICE_INSTANCES;
}

result_status linear_routed_experts_prepare(const struct linear_routed_experts_description *description,
					    uint64_t arena_byte_count, const struct linear_kernels_record *kernels,
					    struct kernel_launch *launches_out)
{
	if (description == NULL || kernels == NULL || launches_out == NULL || description->reserved_zero != 0 ||
	    description->weight_format != WEIGHT_FORMAT_E2M1_SCALED || description->job_count == 0 ||
	    description->job_count > 65535u || description->row_count == 0 || description->pairs_per_row == 0 ||
	    !isfinite(description->activation_limit) || description->activation_limit <= 0)
		return STATUS_INVALID_ARGUMENT;
	uint64_t gate_up_bytes = 0, down_bytes = 0;
	const struct matrix_shape_record *const gate_up = &description->gate_up_shape, *const down = &description->down_shape;
	if (e2m1_stored_byte_count(gate_up, &gate_up_bytes) != STATUS_OK ||
	    e2m1_stored_byte_count(down, &down_bytes) != STATUS_OK || down->input_size != gate_up->output_size ||
	    down->output_size != gate_up->input_size)
		return STATUS_INVALID_ARGUMENT;
	const uint32_t gate_up_instance = slice_instance(description->gate_up_slice_count, gate_up->input_size);
	const uint32_t down_instance = slice_instance(description->down_slice_count, down->input_size);
	if (gate_up_instance == LINEAR_SLICE_INSTANCES || down_instance == LINEAR_SLICE_INSTANCES ||
	    kernels->expert_gate_up[gate_up_instance] == BACKEND_NO_KERNEL ||
	    kernels->expert_down[down_instance] == BACKEND_NO_KERNEL || kernels->activation_quantize == BACKEND_NO_KERNEL ||
	    kernels->expert_row_sum == BACKEND_NO_KERNEL)
		return STATUS_INVALID_ARGUMENT;
	const uint64_t rows = description->row_count, pairs = rows * description->pairs_per_row;
	const uint32_t H = gate_up->input_size, I = gate_up->output_size;
	if (pairs > UINT32_MAX || pairs > 65535u * 64u ||
	    !range_holds(&description->jobs, linear_jobs_byte_count(description->job_count)) ||
	    !range_holds(&description->expert_weights, gate_up_bytes > down_bytes ? gate_up_bytes : down_bytes) ||
	    !range_holds(&description->codes, linear_codes_byte_count(rows, H)) ||
	    !range_holds(&description->exponents, linear_exponents_byte_count(rows, H)) ||
	    !range_holds(&description->operands, linear_values_byte_count(rows, H)) ||
	    !range_holds(&description->hidden, linear_values_byte_count(pairs, I)) ||
	    !range_holds(&description->hidden_codes, linear_codes_byte_count(pairs, I)) ||
	    !range_holds(&description->hidden_exponents, linear_exponents_byte_count(pairs, I)) ||
	    !range_holds(&description->hidden_operands, linear_values_byte_count(pairs, I)) ||
	    !range_holds(&description->pair_output, linear_values_byte_count(pairs, H)) ||
	    !range_holds(&description->row_output, linear_sums_byte_count(rows, H)))
		return STATUS_INVALID_ARGUMENT;
	const struct linear_range *const all[11] = { &description->jobs, &description->expert_weights,
						     &description->codes, &description->exponents,
						     &description->operands, &description->hidden,
						     &description->hidden_codes, &description->hidden_exponents,
						     &description->hidden_operands, &description->pair_output,
						     &description->row_output };
	static const char *const names[11] = { "jobs", "expert weights", "codes", "exponents", "operands", "hidden",
					       "hidden codes", "hidden exponents", "hidden operands", "pair output",
					       "row output" };
	struct checked_range ranges[11];
	for (uint32_t index = 0; index < 11; index++)
		ranges[index] = (struct checked_range){ names[index], all[index]->byte_offset, all[index]->byte_count };
	if (!prepare_ranges_are_valid("routed experts", ranges, 11, arena_byte_count))
		return STATUS_INVALID_ARGUMENT;
	const struct expert_gate_up_arguments gate_up_arguments = { description->jobs.byte_offset,
								    description->codes.byte_offset,
								    description->exponents.byte_offset,
								    description->operands.byte_offset,
								    description->hidden.byte_offset, I, H, (uint32_t)pairs,
								    description->pairs_per_row,
								    description->activation_limit, 0 };
	const struct activation_quantize_arguments quantize_arguments = { description->hidden.byte_offset,
									   description->hidden_codes.byte_offset,
									   description->hidden_exponents.byte_offset,
									   description->hidden_operands.byte_offset, I, 0 };
	const struct expert_down_arguments down_arguments = { description->jobs.byte_offset,
							      description->hidden_codes.byte_offset,
							      description->hidden_exponents.byte_offset,
							      description->hidden_operands.byte_offset,
							      description->pair_output.byte_offset, H, I, (uint32_t)pairs, 0 };
	const struct expert_row_sum_arguments sum_arguments = { description->pair_output.byte_offset,
								description->row_output.byte_offset, H,
								description->pairs_per_row };
	struct kernel_launch launches[LINEAR_ROUTED_EXPERTS_LAUNCH_COUNT];
	prepare_launch_fill(&launches[LINEAR_ROUTED_EXPERTS_GATE_UP], kernels->expert_gate_up[gate_up_instance],
			    I / LINEAR_OUTPUTS_PER_TILE, description->job_count, 1, 64u * description->gate_up_slice_count, 0,
			    &gate_up_arguments, sizeof(gate_up_arguments));
	/* pairs can exceed a grid's second dimension only beyond 65 535: the quantizer takes them in its second dimension */
	prepare_launch_fill(&launches[LINEAR_ROUTED_EXPERTS_QUANTIZE], kernels->activation_quantize,
			    I / LINEAR_VALUES_PER_LOAD, (uint32_t)(pairs > 65535u ? 65535u : pairs), 1, 32, 0,
			    &quantize_arguments, sizeof(quantize_arguments));
	if (pairs > 65535u)
		return STATUS_INVALID_ARGUMENT;
	prepare_launch_fill(&launches[LINEAR_ROUTED_EXPERTS_DOWN], kernels->expert_down[down_instance],
			    H / LINEAR_OUTPUTS_PER_TILE, description->job_count, 1, 32u * description->down_slice_count, 0,
			    &down_arguments, sizeof(down_arguments));
	prepare_launch_fill(&launches[LINEAR_ROUTED_EXPERTS_ROW_SUM], kernels->expert_row_sum,
			    (H + LINEAR_ELEMENT_THREADS - 1u) / LINEAR_ELEMENT_THREADS, description->row_count, 1,
			    LINEAR_ELEMENT_THREADS, 0, &sum_arguments, sizeof(sum_arguments));
	memcpy(launches_out, launches, sizeof(launches));
	return STATUS_OK;
}

/* The routed experts for a job table of MANY rows: linear_routed_experts_prepare's four launches with the two product
 * launches given to expert_gate_up_many and expert_down_many (a group of LINEAR_MANY_JOBS jobs and several tiles a
 * block; the slice counts travel in the argument records, so every slice count the thin instances have is accepted). */
result_status linear_routed_experts_wide_prepare(const struct linear_routed_experts_description *description,
						 uint64_t arena_byte_count, const struct linear_kernels_record *kernels,
						 const struct backend_operations *backend, struct device_card *card,
						 struct kernel_launch *launches_out)
{
	if (backend == NULL || backend->kernel_prepare == NULL || card == NULL)
		return STATUS_INVALID_ARGUMENT;
	struct kernel_launch launches[LINEAR_ROUTED_EXPERTS_LAUNCH_COUNT];
	result_status status = linear_routed_experts_prepare(description, arena_byte_count, kernels, launches);
	if (status != STATUS_OK)
		return status;
	const uint32_t H = description->gate_up_shape.input_size, I = description->gate_up_shape.output_size;
	/* whole blocks of four tiles of gate and up, of eight tiles of down */
	if (I % (4u * LINEAR_OUTPUTS_PER_TILE) != 0 || H % (8u * LINEAR_OUTPUTS_PER_TILE) != 0)
		return STATUS_INVALID_ARGUMENT;
	uint32_t gate_up = BACKEND_NO_KERNEL, down = BACKEND_NO_KERNEL;
	status = backend->kernel_prepare(card, KERNEL_FILE_EXPERT_LINEAR, KERNEL_EXPERT_GATE_UP_MANY,
					 sizeof(struct expert_gate_up_many_arguments), &gate_up);
	if (status == STATUS_OK)
		status = backend->kernel_prepare(card, KERNEL_FILE_EXPERT_LINEAR, KERNEL_EXPERT_DOWN_MANY,
						 sizeof(struct expert_down_many_arguments), &down);
	if (status != STATUS_OK)
		return status;
	if (gate_up == BACKEND_NO_KERNEL || down == BACKEND_NO_KERNEL)
		return STATUS_UNSUPPORTED;
	struct expert_gate_up_many_arguments gate_up_arguments;
	struct expert_down_many_arguments down_arguments;
	memcpy(&gate_up_arguments.base, launches[LINEAR_ROUTED_EXPERTS_GATE_UP].argument, sizeof(gate_up_arguments.base));
	memcpy(&down_arguments.base, launches[LINEAR_ROUTED_EXPERTS_DOWN].argument, sizeof(down_arguments.base));
	gate_up_arguments.slice_count = description->gate_up_slice_count;
	gate_up_arguments.job_count = description->job_count;
	down_arguments.slice_count = description->down_slice_count;
	down_arguments.job_count = description->job_count;
	const uint32_t groups = (description->job_count + LINEAR_MANY_JOBS - 1u) / LINEAR_MANY_JOBS;
	prepare_launch_fill(&launches[LINEAR_ROUTED_EXPERTS_GATE_UP], gate_up, I / (4u * LINEAR_OUTPUTS_PER_TILE), groups, 1,
			    256, 0, &gate_up_arguments, sizeof(gate_up_arguments));
	prepare_launch_fill(&launches[LINEAR_ROUTED_EXPERTS_DOWN], down, H / (8u * LINEAR_OUTPUTS_PER_TILE), groups, 1, 256,
			    0, &down_arguments, sizeof(down_arguments));
	memcpy(launches_out, launches, sizeof(launches));
	return STATUS_OK;
}

static result_status e4m3_stored_byte_count(const struct matrix_shape_record *shape, uint64_t *byte_count_out)
{
	if (shape == NULL || byte_count_out == NULL || shape->reserved_must_be_zero != 0 || shape->bits_per_weight != 8 ||
	    shape->output_size == 0 || shape->input_size == 0 || shape->output_size % LINEAR_OUTPUTS_PER_TILE != 0 ||
	    shape->input_size % LINEAR_VALUES_PER_BLOCK != 0)
		return STATUS_INVALID_ARGUMENT;
	*byte_count_out = e4m3_scaled_byte_count(shape->output_size, shape->input_size);
	return STATUS_OK;
}

const struct weight_format_operations e4m3_scaled_weight_operations = { .name = "e4m3_scaled",
									 .stored_byte_count = e4m3_stored_byte_count };

#define E4M3_BLOCK128 128u
static result_status e4m3_block128_stored_byte_count(const struct matrix_shape_record *shape, uint64_t *byte_count_out)
{
	if (shape == NULL || byte_count_out == NULL || shape->reserved_must_be_zero != 0 || shape->bits_per_weight != 8 ||
	    shape->output_size == 0 || shape->input_size == 0 || shape->output_size % LINEAR_OUTPUTS_PER_TILE != 0 ||
	    shape->input_size % E4M3_BLOCK128 != 0)
		return STATUS_INVALID_ARGUMENT;
	*byte_count_out = (uint64_t)shape->output_size * shape->input_size +
			  (uint64_t)((shape->output_size + E4M3_BLOCK128 - 1u) / E4M3_BLOCK128) *
				  (shape->input_size / E4M3_BLOCK128) * 4u;
	return STATUS_OK;
}

const struct weight_format_operations e4m3_block128_weight_operations = {
	.name = "e4m3_block128", .stored_byte_count = e4m3_block128_stored_byte_count
};

/* a stored E4M3 matrix the trunk kernels can take: its exact bytes, whole loads of 64 inputs, a slice count on offer.
 * handles: the kernels of the matrix's format, by slice instance. */
static uint32_t trunk_matrix_instance(const struct linear_matrix *matrix, enum weight_format_code format,
				      const uint32_t *handles)
{
	uint64_t bytes = 0;
	const result_status sized = format == WEIGHT_FORMAT_E4M3_BLOCK128 ?
					    e4m3_block128_stored_byte_count(&matrix->shape, &bytes) :
					    e4m3_stored_byte_count(&matrix->shape, &bytes);
	if (matrix->weight_format != format || matrix->reserved_zero != 0 || matrix->wide_form != 0 || sized != STATUS_OK ||
	    matrix->stored.byte_count != bytes || matrix->shape.input_size % LINEAR_VALUES_PER_LOAD != 0 ||
	    matrix->stored.byte_offset % WEIGHT_FORMAT_MATRIX_ALIGNMENT_BYTES != 0)
		return LINEAR_SLICE_INSTANCES;
	const uint32_t instance = slice_instance(matrix->slice_count, matrix->shape.input_size);
	return instance < LINEAR_SLICE_INSTANCES && handles[instance] != BACKEND_NO_KERNEL ? instance :
											       LINEAR_SLICE_INSTANCES;
}

static result_status shared_expert_prepare(const struct linear_shared_expert_description *description,
					   uint64_t arena_byte_count, const struct linear_kernels_record *kernels,
					   enum weight_format_code format, const uint32_t *handles, uint32_t row_limit,
					   struct kernel_launch *launches_out);

#define SHARED_EXPERT_WIDE_ROWS 65535u

result_status linear_shared_expert_prepare(const struct linear_shared_expert_description *description,
					   uint64_t arena_byte_count, const struct linear_kernels_record *kernels,
					   struct kernel_launch *launches_out)
{
	if (kernels == NULL)
		return STATUS_INVALID_ARGUMENT;
	return shared_expert_prepare(description, arena_byte_count, kernels, WEIGHT_FORMAT_E4M3_SCALED,
				     kernels->trunk_linear_quantized, LINEAR_MAXIMUM_ROWS, launches_out);
}

static result_status block128_handles(const struct backend_operations *backend, struct device_card *card,
				      uint32_t handles[LINEAR_SLICE_INSTANCES])
{
	for (uint32_t instance = 0; instance < LINEAR_SLICE_INSTANCES; instance++) {
		char name[48];
		(void)snprintf(name, sizeof(name), "trunk_linear_block128_%u", slice_counts[instance]);
		handles[instance] = BACKEND_NO_KERNEL;
		const result_status status = backend->kernel_prepare(card, KERNEL_FILE_TRUNK_LINEAR, name,
								     sizeof(struct trunk_linear_quantized_arguments),
								     &handles[instance]);
		if (status != STATUS_OK)
			return status;
	}
	return STATUS_OK;
}

result_status linear_shared_expert_wide_prepare(const struct linear_shared_expert_description *description,
						uint64_t arena_byte_count, const struct linear_kernels_record *kernels,
						const struct backend_operations *backend, struct device_card *card,
						struct kernel_launch *launches_out)
{
	if (description == NULL || kernels == NULL || backend == NULL || backend->kernel_prepare == NULL || card == NULL)
		return STATUS_INVALID_ARGUMENT;
	if (description->gate.weight_format != WEIGHT_FORMAT_E4M3_BLOCK128)
		return shared_expert_prepare(description, arena_byte_count, kernels, WEIGHT_FORMAT_E4M3_SCALED,
					     kernels->trunk_linear_quantized, SHARED_EXPERT_WIDE_ROWS, launches_out);
	uint32_t handles[LINEAR_SLICE_INSTANCES];
	const result_status status = block128_handles(backend, card, handles);
	if (status != STATUS_OK)
		return status;
	return shared_expert_prepare(description, arena_byte_count, kernels, WEIGHT_FORMAT_E4M3_BLOCK128, handles,
				     SHARED_EXPERT_WIDE_ROWS, launches_out);
}

result_status linear_shared_expert_block128_prepare(const struct linear_shared_expert_description *description,
						    uint64_t arena_byte_count,
						    const struct linear_kernels_record *kernels,
						    const struct backend_operations *backend, struct device_card *card,
						    struct kernel_launch *launches_out)
{
	if (kernels == NULL || backend == NULL || backend->kernel_prepare == NULL || card == NULL)
		return STATUS_INVALID_ARGUMENT;
	uint32_t handles[LINEAR_SLICE_INSTANCES];
	const result_status status = block128_handles(backend, card, handles);
	if (status != STATUS_OK)
		return status;
	return shared_expert_prepare(description, arena_byte_count, kernels, WEIGHT_FORMAT_E4M3_BLOCK128, handles,
				     LINEAR_MAXIMUM_ROWS, launches_out);
}

static result_status shared_expert_prepare(const struct linear_shared_expert_description *description,
					   uint64_t arena_byte_count, const struct linear_kernels_record *kernels,
					   enum weight_format_code format, const uint32_t *handles, uint32_t row_limit,
					   struct kernel_launch *launches_out)
{
	if (description == NULL || kernels == NULL || launches_out == NULL || description->row_count == 0 ||
	    description->row_count > row_limit || !isfinite(description->activation_limit) ||
	    description->activation_limit <= 0 || kernels->trunk_hidden == BACKEND_NO_KERNEL ||
	    kernels->activation_quantize == BACKEND_NO_KERNEL)
		return STATUS_INVALID_ARGUMENT;
	const struct linear_matrix *const gate = &description->gate, *const up = &description->up,
				   *const down = &description->down;
	const uint32_t gate_instance = trunk_matrix_instance(gate, format, handles);
	const uint32_t up_instance = trunk_matrix_instance(up, format, handles);
	const uint32_t down_instance = trunk_matrix_instance(down, format, handles);
	if (gate_instance == LINEAR_SLICE_INSTANCES || up_instance != gate_instance ||
	    down_instance == LINEAR_SLICE_INSTANCES || gate->shape.input_size != up->shape.input_size ||
	    gate->shape.output_size != up->shape.output_size || down->shape.input_size != gate->shape.output_size)
		return STATUS_INVALID_ARGUMENT;
	const uint64_t rows = description->row_count;
	const uint32_t H = gate->shape.input_size, I = gate->shape.output_size, O = down->shape.output_size;
	if (!range_holds(&description->codes, linear_codes_byte_count(rows, H)) ||
	    !range_holds(&description->exponents, linear_exponents_byte_count(rows, H)) ||
	    !range_holds(&description->operands, linear_values_byte_count(rows, H)) ||
	    !range_holds(&description->gate_output, linear_values_byte_count(rows, I)) ||
	    !range_holds(&description->up_output, linear_values_byte_count(rows, I)) ||
	    !range_holds(&description->hidden, linear_values_byte_count(rows, I)) ||
	    !range_holds(&description->hidden_codes, linear_codes_byte_count(rows, I)) ||
	    !range_holds(&description->hidden_exponents, linear_exponents_byte_count(rows, I)) ||
	    !range_holds(&description->hidden_operands, linear_values_byte_count(rows, I)) ||
	    !range_holds(&description->output, linear_values_byte_count(rows, O)))
		return STATUS_INVALID_ARGUMENT;
	const struct linear_range *const all[13] = { &gate->stored, &up->stored, &down->stored, &description->codes,
						     &description->exponents, &description->operands,
						     &description->gate_output, &description->up_output,
						     &description->hidden, &description->hidden_codes,
						     &description->hidden_exponents, &description->hidden_operands,
						     &description->output };
	static const char *const names[13] = { "gate", "up", "down", "codes", "exponents", "operands", "gate output",
					       "up output", "hidden", "hidden codes", "hidden exponents",
					       "hidden operands", "output" };
	struct checked_range ranges[13];
	for (uint32_t index = 0; index < 13; index++)
		ranges[index] = (struct checked_range){ names[index], all[index]->byte_offset, all[index]->byte_count };
	if (!prepare_ranges_are_valid("shared expert", ranges, 13, arena_byte_count))
		return STATUS_INVALID_ARGUMENT;
	const struct trunk_linear_quantized_arguments gate_up_arguments = {
		{ gate->stored.byte_offset, up->stored.byte_offset },
		{ description->gate_output.byte_offset, description->up_output.byte_offset },
		description->codes.byte_offset,
		description->exponents.byte_offset,
		description->operands.byte_offset,
		{ I, I },
		H,
		description->row_count
	};
	const struct trunk_hidden_arguments hidden_arguments = { description->gate_output.byte_offset,
								 description->up_output.byte_offset,
								 description->hidden.byte_offset, I,
								 description->activation_limit };
	const struct activation_quantize_arguments quantize_arguments = { description->hidden.byte_offset,
									   description->hidden_codes.byte_offset,
									   description->hidden_exponents.byte_offset,
									   description->hidden_operands.byte_offset, I, 0 };
	const struct trunk_linear_quantized_arguments down_arguments = { { down->stored.byte_offset, 0 },
									 { description->output.byte_offset, 0 },
									 description->hidden_codes.byte_offset,
									 description->hidden_exponents.byte_offset,
									 description->hidden_operands.byte_offset,
									 { O, 0 },
									 I,
									 description->row_count };
	struct kernel_launch launches[LINEAR_SHARED_EXPERT_LAUNCH_COUNT];
	/* eight rows a block column of the two product launches */
	const uint32_t row_groups = (description->row_count + LINEAR_MAXIMUM_ROWS - 1u) / LINEAR_MAXIMUM_ROWS;
	prepare_launch_fill(&launches[LINEAR_SHARED_EXPERT_GATE_UP], handles[gate_instance],
			    2u * I / LINEAR_OUTPUTS_PER_TILE, row_groups, 1, 32u * gate->slice_count, 0, &gate_up_arguments,
			    sizeof(gate_up_arguments));
	prepare_launch_fill(&launches[LINEAR_SHARED_EXPERT_HIDDEN], kernels->trunk_hidden,
			    (I + LINEAR_ELEMENT_THREADS - 1u) / LINEAR_ELEMENT_THREADS, description->row_count, 1,
			    LINEAR_ELEMENT_THREADS, 0, &hidden_arguments, sizeof(hidden_arguments));
	prepare_launch_fill(&launches[LINEAR_SHARED_EXPERT_QUANTIZE], kernels->activation_quantize,
			    I / LINEAR_VALUES_PER_LOAD, description->row_count, 1, 32, 0, &quantize_arguments,
			    sizeof(quantize_arguments));
	prepare_launch_fill(&launches[LINEAR_SHARED_EXPERT_DOWN], handles[down_instance],
			    O / LINEAR_OUTPUTS_PER_TILE, row_groups, 1, 32u * down->slice_count, 0, &down_arguments,
			    sizeof(down_arguments));
	memcpy(launches_out, launches, sizeof(launches));
	return STATUS_OK;
}

result_status linear_rows_add_prepare(const struct linear_range *sums, const struct linear_range *values,
				      uint32_t width, uint32_t row_count, uint64_t arena_byte_count,
				      const struct backend_operations *backend, struct device_card *card,
				      struct kernel_launch *launch_out)
{
	if (sums == NULL || values == NULL || backend == NULL || backend->kernel_prepare == NULL || card == NULL ||
	    launch_out == NULL || width == 0 || row_count == 0 || row_count > 65535u ||
	    !range_holds(sums, linear_sums_byte_count(row_count, width)) ||
	    !range_holds(values, linear_values_byte_count(row_count, width)))
		return STATUS_INVALID_ARGUMENT;
	const struct checked_range ranges[2] = { { "sums", sums->byte_offset, sums->byte_count },
						 { "values", values->byte_offset, values->byte_count } };
	if (!prepare_ranges_are_valid("rows add", ranges, 2, arena_byte_count))
		return STATUS_INVALID_ARGUMENT;
	uint32_t kernel = BACKEND_NO_KERNEL;
	const result_status status = backend->kernel_prepare(card, KERNEL_FILE_TRUNK_LINEAR, KERNEL_TRUNK_ROWS_ADD,
							     sizeof(struct trunk_rows_add_arguments), &kernel);
	if (status != STATUS_OK)
		return status;
	if (kernel == BACKEND_NO_KERNEL)
		return STATUS_UNSUPPORTED;
	const struct trunk_rows_add_arguments arguments = { sums->byte_offset, values->byte_offset, width, 0 };
	prepare_launch_fill(launch_out, kernel, (width + LINEAR_ELEMENT_THREADS - 1u) / LINEAR_ELEMENT_THREADS, row_count,
			    1, LINEAR_ELEMENT_THREADS, 0, &arguments, sizeof(arguments));
	return STATUS_OK;
}
