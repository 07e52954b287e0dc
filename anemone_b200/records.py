"""ctypes mirrors of the C records of include/anemone_b200_records.h and include/anemone_b200_backend.h.

Field order and sizes follow the C headers exactly; sizes are asserted at import.
"""
import ctypes as C

LINEAR_MAXIMUM_ROWS = 8
LAUNCH_ARGUMENT_BYTES = 192
EXL3_WIDTH_PER_EXPERT = 0xFFFF
BACKEND_NO_KERNEL = 0xFFFFFFFF

STATUS_NAMES = ["OK", "INVALID_ARGUMENT", "OUT_OF_MEMORY", "INPUT_OUTPUT_ERROR", "CORRUPT_PACK", "DEVICE_ERROR",
                "TIMED_OUT", "UNSUPPORTED", "BUSY_VALUE", "INJECTED_FAULT"]
STATUS_OK, STATUS_INVALID_ARGUMENT, STATUS_OUT_OF_MEMORY = 0, 1, 2
STATUS_DEVICE_ERROR, STATUS_TIMED_OUT, STATUS_UNSUPPORTED, STATUS_BUSY_VALUE = 5, 6, 7, 8


class Exl3Reconstruct(C.Structure):
    _fields_ = [("matrix_offset", C.c_uint64), ("output_offset", C.c_uint64), ("input_size", C.c_uint32),
                ("output_size", C.c_uint32), ("bits_per_weight", C.c_uint32), ("reserved_zero", C.c_uint32)]


class Exl3Expert(C.Structure):
    _fields_ = [("jobs_offset", C.c_uint64), ("input_offset", C.c_uint64), ("operands_offset", C.c_uint64),
                ("products_offset", C.c_uint64), ("hidden_offset", C.c_uint64), ("output_offset", C.c_uint64),
                ("input_size", C.c_uint32), ("inner_size", C.c_uint32), ("pair_count", C.c_uint32),
                ("pairs_per_row", C.c_uint32), ("job_count", C.c_uint32), ("bits_per_weight", C.c_uint32),
                ("activation_limit", C.c_float), ("reserved_zero", C.c_uint32)]


class ExpertJob(C.Structure):
    _fields_ = [("gate_offset", C.c_uint64), ("up_offset", C.c_uint64), ("down_offset", C.c_uint64),
                ("row_count", C.c_uint32), ("expert", C.c_uint32), ("pair_index", C.c_uint32 * LINEAR_MAXIMUM_ROWS),
                ("route_weight", C.c_float * LINEAR_MAXIMUM_ROWS)]


class ExpertRowSum(C.Structure):
    _fields_ = [("pair_output_offset", C.c_uint64), ("row_output_offset", C.c_uint64), ("width", C.c_uint32),
                ("pairs_per_row", C.c_uint32)]


class Exl3ShardActivation(C.Structure):
    _fields_ = [("base", Exl3Expert), ("down_input_size", C.c_uint32), ("down_output_size", C.c_uint32),
                ("down_input_begin", C.c_uint32), ("reserved_zero", C.c_uint32)]


class Exl3Moe(C.Structure):
    _fields_ = [("base", Exl3Expert), ("widths_offset", C.c_uint64), ("row_output_offset", C.c_uint64),
                ("counters_offset", C.c_uint64), ("expert_count", C.c_uint32), ("reserved_zero", C.c_uint32)]


class Exl3LayerRoute(C.Structure):
    _fields_ = [("moe", Exl3Moe), ("scores_offset", C.c_uint64), ("expert_table_offset", C.c_uint64),
                ("picks_offset", C.c_uint64), ("weights_offset", C.c_uint64), ("bias_offset", C.c_uint64),
                ("step_offset", C.c_uint64), ("routed_count", C.c_uint32), ("shared_count", C.c_uint32),
                ("picks", C.c_uint32), ("row_capacity", C.c_uint32), ("scoring", C.c_uint32),
                ("route_scale", C.c_float)]


class Exl3LayerPublish(C.Structure):
    _fields_ = [("peer_table_offset", C.c_uint64), ("region_offset", C.c_uint64), ("input_offset", C.c_uint64),
                ("status_offset", C.c_uint64), ("step_offset", C.c_uint64), ("parity_stride", C.c_uint64),
                ("deadline_cycles", C.c_uint64), ("rank_count", C.c_uint32), ("rank", C.c_uint32),
                ("row_capacity", C.c_uint32), ("reserved_zero", C.c_uint32)]


class Exl3LayerDescription(C.Structure):
    _fields_ = [("route", Exl3LayerRoute), ("publish", Exl3LayerPublish), ("result_offset", C.c_uint64),
                ("arena_byte_count", C.c_uint64), ("gate_up_runs", C.c_uint32), ("down_runs", C.c_uint32)]


EXL3_LAYER_SIGNAL_BYTES = 33 * 128
ORDERED_COLLECTIVE_MAXIMUM_ELEMENTS = 262144
EXL3_LAYER_LAUNCHES = 3
EXL3_LAYER_READY_LINE, EXL3_LAYER_DONE_LINE, EXL3_LAYER_LOCAL_LINE = 0, 16, 32


class Exl3Tc(C.Structure):
    _fields_ = [("jobs_offset", C.c_uint64), ("hidden_offset", C.c_uint64), ("workspace_offset", C.c_uint64),
                ("output_offset", C.c_uint64), ("row_count", C.c_uint32), ("job_capacity", C.c_uint32),
                ("intermediate", C.c_uint32), ("bits_x2", C.c_uint32), ("activation_limit", C.c_float),
                ("pass_", C.c_uint32), ("rotation", C.c_uint32), ("shared_sum", C.c_uint32),
                ("shared_offset", C.c_uint64)]


class RouterPick(C.Structure):
    _fields_ = [("expert", C.c_uint32), ("route_weight", C.c_float)]


class Exl3Tcp(C.Structure):
    _fields_ = [("picks_offset", C.c_uint64), ("expert_offsets_offset", C.c_uint64), ("hidden_offset", C.c_uint64),
                ("workspace_offset", C.c_uint64), ("output_offset", C.c_uint64), ("row_count", C.c_uint32),
                ("intermediate", C.c_uint32), ("bits_x2", C.c_uint32), ("pass_", C.c_uint32),
                ("activation_limit", C.c_float), ("rotation", C.c_uint32), ("half_rows", C.c_uint32),
                ("part", C.c_uint32), ("step_offset", C.c_uint64), ("cone_layer", C.c_uint32),
                ("two_blocks", C.c_uint32)]


class Exl3MoeSizes(C.Structure):
    _fields_ = [("operand_bytes", C.c_uint64), ("product_bytes", C.c_uint64), ("counter_bytes", C.c_uint64),
                ("gate_up_splits", C.c_uint32), ("down_splits", C.c_uint32)]


class Exl3Prefill(C.Structure):
    _fields_ = [("scores_offset", C.c_uint64), ("input_offset", C.c_uint64), ("expert_table_offset", C.c_uint64),
                ("widths_offset", C.c_uint64), ("picks_offset", C.c_uint64), ("weights_offset", C.c_uint64),
                ("workspace_offset", C.c_uint64), ("pair_output_offset", C.c_uint64),
                ("row_output_offset", C.c_uint64), ("step_offset", C.c_uint64), ("input_size", C.c_uint32),
                ("inner_size", C.c_uint32), ("shared_inner_size", C.c_uint32), ("expert_count", C.c_uint32),
                ("local_first", C.c_uint32), ("local_count", C.c_uint32), ("shared_count", C.c_uint32),
                ("picks", C.c_uint32), ("row_capacity", C.c_uint32), ("scoring", C.c_uint32),
                ("route_scale", C.c_float), ("activation_limit", C.c_float), ("bias_offset", C.c_uint64)]


class RouterWide(C.Structure):
    _fields_ = [("routing", Exl3Prefill), ("jobs_offset", C.c_uint64), ("job_capacity", C.c_uint32),
                ("reserved_zero", C.c_uint32)]


ROUTER_WIDE_LAUNCHES = 3


class Exl3PrefillTile(C.Structure):
    _fields_ = [("expert", C.c_uint32), ("first_entry", C.c_uint32), ("row_count", C.c_uint32),
                ("reserved_zero", C.c_uint32)]


class Exl3PrefillEntry(C.Structure):
    _fields_ = [("pair", C.c_uint32), ("route_weight", C.c_float)]


class Exl3PrefillParts(C.Structure):
    _fields_ = [("counts", C.c_uint64), ("tiles", C.c_uint64), ("entries", C.c_uint64),
                ("gate_up_operands", C.c_uint64), ("down_operands", C.c_uint64), ("total", C.c_uint64),
                ("tile_capacity", C.c_uint32), ("reserved_zero", C.c_uint32)]


class StepBlock(C.Structure):
    _fields_ = [("sequence", C.c_uint64), ("row_count", C.c_uint32), ("flags", C.c_uint32)]


class OrderedPeer(C.Structure):
    _fields_ = [("arena_address", C.c_uint64), ("region_offset", C.c_uint64), ("host_address", C.c_uint64),
                ("route", C.c_uint32), ("reserved_zero", C.c_uint32)]


class OrderedCollective(C.Structure):
    _fields_ = [("peer_table_offset", C.c_uint64), ("region_offset", C.c_uint64), ("input_offset", C.c_uint64),
                ("output_offset", C.c_uint64), ("scratch_offset", C.c_uint64), ("step_offset", C.c_uint64),
                ("parity_stride", C.c_uint64), ("deadline_cycles", C.c_uint64), ("element_count", C.c_uint32),
                ("rank_count", C.c_uint32), ("rank", C.c_uint32), ("reserved_zero", C.c_uint32)]


ORDERED_REDUCE_EVERY_RANK, ORDERED_REDUCE_OWNER_RUNS = 0, 1


class OrderedReduceBf16(C.Structure):
    _fields_ = [("collective", OrderedCollective), ("status_offset", C.c_uint64), ("width", C.c_uint32),
                ("mode", C.c_uint32)]


class OrderedPublishReduce(C.Structure):
    _fields_ = [("collective", OrderedCollective), ("status_offset", C.c_uint64), ("pair_output_offset", C.c_uint64),
                ("width", C.c_uint32), ("pairs_per_row", C.c_uint32)]


class OrderedPublishReduceBf16(C.Structure):
    _fields_ = [("base", OrderedPublishReduce), ("addend_offset", C.c_uint64), ("row_output_offset", C.c_uint64)]


class OrderedRowSumPublish(C.Structure):
    _fields_ = [("collective", OrderedCollective), ("pair_output_offset", C.c_uint64), ("width", C.c_uint32),
                ("pairs_per_row", C.c_uint32), ("status_offset", C.c_uint64)]


class Exl3LayerProducts(C.Structure):
    _fields_ = [("moe", Exl3Moe), ("down_products_offset", C.c_uint64), ("gate_up_runs", C.c_uint32),
                ("down_runs", C.c_uint32)]


class ExactRing(C.Structure):
    _fields_ = [("input_offset", C.c_uint64), ("output_offset", C.c_uint64), ("bank_offset", C.c_uint64),
                ("peer_table_offset", C.c_uint64), ("peer_bank_delta", C.c_uint64), ("deadline_cycles", C.c_uint64),
                ("packs_per_owner", C.c_uint32), ("vectors", C.c_uint32), ("rank", C.c_uint32), ("mode", C.c_uint32),
                ("reserved_words", C.c_uint64 * 2)]


class RingExchangeDescription(C.Structure):
    _fields_ = [("arguments", ExactRing), ("arena_byte_count", C.c_uint64), ("kind", C.c_uint32),
                ("blocks", C.c_uint32)]


RING_EXCHANGE_EXACT, RING_EXCHANGE_COMPRESSED, RING_EXCHANGE_ROUND_ONCE = 0, 1, 2
EXACT_RING_GATHER, EXACT_RING_BF16_SUM, EXACT_RING_BF16_SUM_COLUMNS = 0, 1, 2
EXACT_RING_PACK_BYTES, EXACT_RING_BLOCKS, EXACT_RING_METADATA_BYTES, EXACT_RING_STATUS_OFFSET = 16, 16, 128, 64
COMPRESSED_RING_PACKS, COMPRESSED_RING_PACKET_WORDS = 32, 136
COMPRESSED_RING_READY_WORD, COMPRESSED_RING_ACK_WORD = 132, 133

ORDERED_PUSH_FP32, ORDERED_PUSH_BF16 = 0, 1
TP_EXCHANGE_FORM_PUSH, TP_EXCHANGE_FORM_OWNER_SUMS = 0, 1


class OrderedPush(C.Structure):
    _fields_ = [("peer_table_offset", C.c_uint64), ("region_offset", C.c_uint64), ("input_offset", C.c_uint64),
                ("output_offset", C.c_uint64), ("inbox_offset", C.c_uint64), ("step_offset", C.c_uint64),
                ("parity_stride", C.c_uint64), ("deadline_cycles", C.c_uint64), ("inbox_rank_stride", C.c_uint64),
                ("element_count", C.c_uint32), ("rank_count", C.c_uint32), ("rank", C.c_uint32),
                ("payload_format", C.c_uint32), ("incoming_host_mask", C.c_uint32), ("reserved_zero", C.c_uint32)]


class TpExchange(C.Structure):
    _fields_ = [("collective", OrderedPush), ("layer", C.c_uint32), ("layer_count", C.c_uint32),
                ("row_width", C.c_uint32), ("reserved_zero", C.c_uint32)]


class Tp2Join(C.Structure):
    _fields_ = [("source_offset", C.c_uint64), ("routed_sums_offset", C.c_uint64), ("output_offset", C.c_uint64),
                ("step_offset", C.c_uint64), ("source_slot_stride", C.c_uint64), ("output_slot_stride", C.c_uint64),
                ("width", C.c_uint32), ("row_count", C.c_uint32), ("source_row_stride", C.c_uint32),
                ("routed_row_stride", C.c_uint32), ("output_row_stride", C.c_uint32), ("operation", C.c_uint32),
                ("has_routed_sums", C.c_uint32), ("reserved_zero", C.c_uint32)]


class Tp2JoinRange(C.Structure):
    _fields_ = [("byte_offset", C.c_uint64), ("byte_count", C.c_uint64)]


class Tp2JoinDescription(C.Structure):
    _fields_ = [("source", Tp2JoinRange), ("routed_sums", Tp2JoinRange), ("output", Tp2JoinRange),
                ("step", Tp2JoinRange), ("source_slot_stride", C.c_uint64), ("output_slot_stride", C.c_uint64),
                ("width", C.c_uint32), ("row_count", C.c_uint32), ("source_row_stride", C.c_uint32),
                ("routed_row_stride", C.c_uint32), ("output_row_stride", C.c_uint32), ("operation", C.c_uint32),
                ("reserved_zero", C.c_uint32)]


class OrderedRowsPush(C.Structure):
    _fields_ = [("push", OrderedPush), ("pair_output_offset", C.c_uint64), ("width", C.c_uint32),
                ("pairs_per_row", C.c_uint32)]


class OrderedRowsPushDescription(C.Structure):
    _fields_ = [("arguments", OrderedRowsPush), ("arena_byte_count", C.c_uint64)]


class OrderedPushDescription(C.Structure):
    _fields_ = [("arguments", OrderedPush), ("arena_byte_count", C.c_uint64)]


class RouterSelectB200(C.Structure):
    _fields_ = [("scores_offset", C.c_uint64), ("expert_table_offset", C.c_uint64), ("picks_offset", C.c_uint64),
                ("weights_offset", C.c_uint64), ("jobs_offset", C.c_uint64), ("step_offset", C.c_uint64),
                ("expert_count", C.c_uint32), ("shared_count", C.c_uint32), ("picks", C.c_uint32),
                ("row_capacity", C.c_uint32), ("job_capacity", C.c_uint32), ("scoring", C.c_uint32),
                ("route_scale", C.c_float), ("reserved_zero", C.c_uint32), ("bias_offset", C.c_uint64)]


class StepInputSelect(C.Structure):
    _fields_ = [("pool_offset", C.c_uint64), ("pool_stride", C.c_uint64), ("destination_offset", C.c_uint64),
                ("cursor_offset", C.c_uint64), ("pool_count", C.c_uint32), ("byte_count", C.c_uint32)]


class ActivationQuantize(C.Structure):
    _fields_ = [("values_offset", C.c_uint64), ("codes_offset", C.c_uint64), ("exponents_offset", C.c_uint64),
                ("operands_offset", C.c_uint64), ("width", C.c_uint32), ("reserved_zero", C.c_uint32)]


class RouterSelectQuantize(C.Structure):
    _fields_ = [("router", RouterSelectB200), ("quantize", ActivationQuantize), ("vector_count", C.c_uint32),
                ("reserved_zero", C.c_uint32)]


class ExpertGateUp(C.Structure):
    _fields_ = [("jobs_offset", C.c_uint64), ("codes_offset", C.c_uint64), ("exponents_offset", C.c_uint64),
                ("operands_offset", C.c_uint64), ("hidden_offset", C.c_uint64), ("output_size", C.c_uint32),
                ("input_size", C.c_uint32), ("pair_count", C.c_uint32), ("pairs_per_row", C.c_uint32),
                ("activation_limit", C.c_float), ("reserved_zero", C.c_uint32)]


class ExpertDown(C.Structure):
    _fields_ = [("jobs_offset", C.c_uint64), ("codes_offset", C.c_uint64), ("exponents_offset", C.c_uint64),
                ("operands_offset", C.c_uint64), ("output_offset", C.c_uint64), ("output_size", C.c_uint32),
                ("input_size", C.c_uint32), ("pair_count", C.c_uint32), ("reserved_zero", C.c_uint32)]


LINEAR_MANY_JOBS = 2


class ExpertGateUpMany(C.Structure):
    _fields_ = [("base", ExpertGateUp), ("slice_count", C.c_uint32), ("job_count", C.c_uint32)]


class ExpertDownMany(C.Structure):
    _fields_ = [("base", ExpertDown), ("slice_count", C.c_uint32), ("job_count", C.c_uint32)]


class LinearRange(C.Structure):
    _fields_ = [("byte_offset", C.c_uint64), ("byte_count", C.c_uint64)]


class MatrixShape(C.Structure):
    _fields_ = [("output_size", C.c_uint32), ("input_size", C.c_uint32), ("bits_per_weight", C.c_uint32),
                ("reserved_must_be_zero", C.c_uint32)]


class LinearKernels(C.Structure):
    _fields_ = [("activation_quantize", C.c_uint32), ("expert_gate_up", C.c_uint32 * 5),
                ("expert_down", C.c_uint32 * 5), ("expert_row_sum", C.c_uint32),
                ("trunk_linear_quantized", C.c_uint32 * 5), ("trunk_linear_bfloat16", C.c_uint32 * 5),
                ("trunk_hidden", C.c_uint32), ("trunk_linear_quantized_wide", C.c_uint32 * 5),
                ("trunk_linear_bfloat16_wide", C.c_uint32 * 5), ("trunk_linear_quantized_interleaved", C.c_uint32)]


class LinearQuantizeDescription(C.Structure):
    _fields_ = [("values", LinearRange), ("codes", LinearRange), ("exponents", LinearRange),
                ("operands", LinearRange), ("width", C.c_uint32), ("row_count", C.c_uint32)]


class LinearRoutedExpertsDescription(C.Structure):
    _fields_ = [(name, LinearRange) for name in ("jobs", "expert_weights", "codes", "exponents", "operands", "hidden",
                                                 "hidden_codes", "hidden_exponents", "hidden_operands", "pair_output",
                                                 "row_output")] + \
               [("gate_up_shape", MatrixShape), ("down_shape", MatrixShape), ("weight_format", C.c_int),
                ("job_count", C.c_uint32), ("row_count", C.c_uint32), ("pairs_per_row", C.c_uint32),
                ("gate_up_slice_count", C.c_uint32), ("down_slice_count", C.c_uint32),
                ("activation_limit", C.c_float), ("reserved_zero", C.c_uint32)]


class TrunkLinearQuantized(C.Structure):
    _fields_ = [("weights_offset", C.c_uint64 * 2), ("output_offset", C.c_uint64 * 2), ("codes_offset", C.c_uint64),
                ("exponents_offset", C.c_uint64), ("operands_offset", C.c_uint64), ("output_size", C.c_uint32 * 2),
                ("input_size", C.c_uint32), ("row_count", C.c_uint32)]


class TrunkHidden(C.Structure):
    _fields_ = [("gate_offset", C.c_uint64), ("up_offset", C.c_uint64), ("hidden_offset", C.c_uint64),
                ("width", C.c_uint32), ("activation_limit", C.c_float)]


class TrunkRowsAdd(C.Structure):
    _fields_ = [("sums_offset", C.c_uint64), ("values_offset", C.c_uint64), ("width", C.c_uint32),
                ("reserved_zero", C.c_uint32)]


class LinearMatrix(C.Structure):
    _fields_ = [("stored", LinearRange), ("shape", MatrixShape), ("weight_format", C.c_int),
                ("slice_count", C.c_uint32), ("wide_form", C.c_uint32), ("reserved_zero", C.c_uint32)]


class LinearSharedExpertDescription(C.Structure):
    _fields_ = [("gate", LinearMatrix), ("up", LinearMatrix), ("down", LinearMatrix)] + \
               [(name, LinearRange) for name in ("codes", "exponents", "operands", "gate_output", "up_output", "hidden",
                                                 "hidden_codes", "hidden_exponents", "hidden_operands", "output")] + \
               [("row_count", C.c_uint32), ("activation_limit", C.c_float)]


class KernelLaunch(C.Structure):
    _fields_ = [("kernel", C.c_uint32), ("grid", C.c_uint32 * 3), ("block", C.c_uint32 * 3),
                ("dynamic_shared_byte_count", C.c_uint32), ("argument_byte_count", C.c_uint32),
                ("branch", C.c_uint32), ("argument", C.c_ubyte * LAUNCH_ARGUMENT_BYTES)]


LAUNCH_CHAIN, LAUNCH_SIDE, LAUNCH_RESUME, LAUNCH_JOIN, LAUNCH_SIDE_MORE = range(5)
BACKEND_COPY, EXCHANGE_OWN_ARENA = 0xFFFFFFFE, 0xFFFFFFFFFFFFFFFF


class ExchangePlace(C.Structure):
    _fields_ = [("address_word_offset", C.c_uint64), ("offset", C.c_uint64)]


class ExchangeCopy(C.Structure):
    _fields_ = [("source", ExchangePlace), ("destination", ExchangePlace), ("byte_count", C.c_uint64)]


class LaunchOrder(C.Structure):
    _fields_ = [("behind_count", C.c_uint32), ("behind", C.c_uint32 * 5)]


def copy_launch(source_offset, destination_offset, byte_count, branch=LAUNCH_CHAIN, source_word=EXCHANGE_OWN_ARENA,
                destination_word=EXCHANGE_OWN_ARENA):
    """A launch of BACKEND_COPY: byte_count bytes between two places (own arena, or behind an address word)."""
    launch = KernelLaunch()
    launch.kernel, launch.branch, launch.argument_byte_count = BACKEND_COPY, branch, C.sizeof(ExchangeCopy)
    record = ExchangeCopy(ExchangePlace(source_word, source_offset), ExchangePlace(destination_word, destination_offset),
                          byte_count)
    C.memmove(launch.argument, C.byref(record), C.sizeof(record))
    return launch


class CardDescription(C.Structure):
    _fields_ = [("name", C.c_char * 96), ("bus_address", C.c_char * 32), ("arithmetic_class", C.c_uint32),
                ("link_generation", C.c_uint32), ("link_lane_count", C.c_uint32), ("reserved_zero", C.c_uint32),
                ("memory_total_bytes", C.c_uint64), ("memory_free_bytes", C.c_uint64),
                ("memory_reserved_bytes", C.c_uint64)]


class OrderedCollectiveDescription(C.Structure):
    _fields_ = [("arguments", OrderedCollective), ("arena_byte_count", C.c_uint64), ("operation", C.c_int)]


class OrderedReduceBf16Description(C.Structure):
    _fields_ = [("reduce", OrderedReduceBf16), ("pair_output_offset", C.c_uint64), ("arena_byte_count", C.c_uint64),
                ("pairs_per_row", C.c_uint32), ("row_capacity", C.c_uint32)]


class OrderedCollectiveKernels(C.Structure):
    _fields_ = [("handles", C.c_uint32 * 4)]


for _record, _bytes in ((Exl3Reconstruct, 32), (Exl3Expert, 80), (ExpertJob, 96), (ExpertRowSum, 24),
                        (Exl3ShardActivation, 96), (Exl3Moe, 112), (Exl3Tc, 72), (Exl3Tcp, 88), (RouterPick, 8), (Exl3LayerRoute, 184), (Exl3LayerPublish, 72), (TrunkLinearQuantized, 72), (TrunkHidden, 32), (TrunkRowsAdd, 24), (Exl3Prefill, 136), (Exl3PrefillTile, 16), (Exl3PrefillEntry, 8), (Exl3PrefillParts, 56), (StepBlock, 16), (OrderedPeer, 32),
                        (OrderedCollective, 80), (OrderedReduceBf16, 96), (OrderedRowSumPublish, 104), (OrderedPublishReduce, 104), (OrderedPush, 96), (ExactRing, 80),
                        (TpExchange, 112), (OrderedRowsPush, 112), (Tp2Join, 80),
                        (RouterSelectB200, 88), (StepInputSelect, 40), (ActivationQuantize, 40), (ExpertGateUp, 64), (ExpertDown, 56),
                        (KernelLaunch, 232), (CardDescription, 168)):
    assert C.sizeof(_record) == _bytes, (_record.__name__, C.sizeof(_record), _bytes)
