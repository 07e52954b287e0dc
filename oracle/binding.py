"""ctypes bindings of the CPU oracle (oracle/liboracle.so) and of the reference's own host code (oracle/_ref).

TEST INFRASTRUCTURE: only tests, the smoke check and the benchmark's CPU-baseline legs import this module; the
product package (anemone_b200/) never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

ORACLE_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(ORACLE_DIR)
ORACLE_SO = os.path.join(ORACLE_DIR, "liboracle.so")
REFERENCE_SO = os.path.join(ORACLE_DIR, "_ref", "libanemone_ref.so")

u8p = C.POINTER(C.c_ubyte)
u16p = C.POINTER(C.c_uint16)
u32p = C.POINTER(C.c_uint32)
u64p = C.POINTER(C.c_uint64)
f32p = C.POINTER(C.c_float)


def ptr(array, kind):
    return array.ctypes.data_as(kind)


def build_oracle():
    subprocess.run(["make", "-C", ORACLE_DIR, "all"], check=True, capture_output=True)


def load_oracle():
    if not os.path.exists(ORACLE_SO):
        build_oracle()
    lib = C.CDLL(ORACLE_SO)
    lib.orc_half_value.restype = C.c_float
    lib.orc_half_value.argtypes = [C.c_uint16]
    lib.orc_half_nearest.restype = C.c_uint16
    lib.orc_half_nearest.argtypes = [C.c_double]
    lib.orc_bfloat16_bits.restype = C.c_uint16
    lib.orc_bfloat16_bits.argtypes = [C.c_float]
    lib.orc_exl3_codebook.restype = C.c_uint16
    lib.orc_exl3_codebook.argtypes = [C.c_uint32]
    lib.orc_exl3_state.restype = C.c_uint16
    lib.orc_exl3_state.argtypes = [u8p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]
    for name in ("orc_exl3_states", "orc_exl3_decode"):
        getattr(lib, name).restype = None
        getattr(lib, name).argtypes = [u8p, C.c_uint32, C.c_uint32, C.c_uint32, u16p]
    lib.orc_exl3_states_digest.restype = C.c_uint64
    lib.orc_exl3_states_digest.argtypes = [u8p, C.c_uint32, C.c_uint32, C.c_uint32]
    lib.orc_exl3_slice.restype = C.c_uint64
    lib.orc_exl3_slice.argtypes = [u8p] + [C.c_uint32] * 7 + [u8p]
    lib.orc_hadamard128.restype = None
    lib.orc_hadamard128.argtypes = [f32p]
    lib.orc_exl3_experts.restype = None
    lib.orc_exl3_experts.argtypes = [C.c_void_p, u8p, u32p, C.c_uint32]
    lib.orc_exl3_row_sum.restype = None
    lib.orc_exl3_row_sum.argtypes = [C.c_void_p, C.c_uint32, u8p]
    lib.orc_ordered_sum.restype = None
    lib.orc_ordered_sum.argtypes = [C.POINTER(f32p), C.c_uint32, C.c_uint32, f32p]
    lib.orc_ordered_reduce_bf16.restype = None
    lib.orc_ordered_reduce_bf16.argtypes = [C.POINTER(f32p), C.c_uint32, C.c_uint32, u16p]
    lib.orc_ordered_push.restype = None
    lib.orc_ordered_push.argtypes = [C.POINTER(f32p), C.c_uint32, C.c_uint32, C.c_uint32, f32p]
    lib.orc_owner_sums.restype = None
    lib.orc_owner_sums.argtypes = [C.POINTER(f32p), C.c_uint32, C.c_uint32, C.c_uint32, u16p]
    lib.orc_tp2_join.restype = None
    lib.orc_tp2_join.argtypes = [C.c_void_p, C.c_void_p]
    lib.orc_ordered_collective.restype = C.c_int
    lib.orc_ordered_collective.argtypes = [C.POINTER(f32p), C.POINTER(f32p), C.c_uint32, C.c_uint32, C.c_int]
    lib.orc_router_row.restype = None
    lib.orc_router_row.argtypes = [f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float, u32p, f32p]
    lib.orc_router_row_biased.restype = None
    lib.orc_router_row_biased.argtypes = [f32p, f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float, u32p, f32p]
    lib.orc_router_affinity.restype = C.c_float
    lib.orc_router_affinity.argtypes = [C.c_float, C.c_uint32]
    lib.orc_router_jobs.restype = C.c_uint32
    lib.orc_router_jobs.argtypes = [u32p, f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, u64p, C.c_uint32,
                                    C.c_void_p]
    u8 = u8p
    lib.orc_e2m1_value.restype = lib.orc_e4m3_value.restype = lib.orc_e8m0_value.restype = C.c_double
    lib.orc_e2m1_value.argtypes = lib.orc_e4m3_value.argtypes = lib.orc_e8m0_value.argtypes = [C.c_uint32]
    lib.orc_mx_quantize.restype = None
    lib.orc_mx_quantize.argtypes = [u16p, C.c_uint32, u8, u8]
    lib.orc_mx_codes_lay_out.restype = None
    lib.orc_mx_codes_lay_out.argtypes = [u8, C.c_uint32, u8]
    lib.orc_mx_operands_lay_out.restype = None
    lib.orc_mx_operands_lay_out.argtypes = [u8, C.c_uint32, u16p]
    lib.orc_mx_weights_lay_out.restype = None
    lib.orc_mx_weights_lay_out.argtypes = [u8, u8, C.c_uint32, C.c_uint32, u8]
    lib.orc_mx_output.restype = C.c_uint16
    lib.orc_mx_output.argtypes = [u8, C.c_uint32, C.c_uint32, C.c_uint32, u8, u8, C.c_uint32]
    lib.orc_mx_hidden.restype = C.c_uint16
    lib.orc_mx_hidden.argtypes = [C.c_uint16, C.c_uint16, C.c_float, C.c_float]
    lib.orc_e4m3_weights_lay_out.restype = None
    lib.orc_e4m3_weights_lay_out.argtypes = [u8, u8, C.c_uint32, C.c_uint32, u8]
    lib.orc_trunk_output.restype = C.c_uint16
    lib.orc_trunk_output.argtypes = [u8, C.c_uint32, C.c_uint32, C.c_uint32, u8, u8, C.c_uint32]
    lib.orc_shared_expert.restype = None
    lib.orc_shared_expert.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, u8]
    lib.orc_shared_expert_block128.restype = None
    lib.orc_shared_expert_block128.argtypes = lib.orc_shared_expert.argtypes
    lib.orc_trunk_output_block128.restype = C.c_uint16
    lib.orc_trunk_output_block128.argtypes = lib.orc_trunk_output.argtypes
    lib.orc_e4m3_block128_lay_out.restype = None
    lib.orc_e4m3_block128_lay_out.argtypes = [u8, f32p, C.c_uint32, C.c_uint32, u8]
    lib.orc_mx_experts.restype = None
    lib.orc_mx_experts.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint64,
                                   C.c_uint64, C.c_uint64, u8]
    lib.orc_mx_row_sum.restype = None
    lib.orc_mx_row_sum.argtypes = [C.c_void_p, C.c_uint32, u8]
    lib.orc_ring_bf16_add.restype = C.c_uint16
    lib.orc_ring_bf16_add.argtypes = [C.c_uint16, C.c_uint16]
    lib.orc_ring_bf16_sum.restype = None
    lib.orc_ring_bf16_sum.argtypes = [C.POINTER(u16p), C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(u16p)]
    lib.orc_ring_round_once.restype = None
    lib.orc_ring_round_once.argtypes = [C.POINTER(u16p), C.c_uint32, C.c_uint64, u16p]
    lib.orc_ring_gather.restype = None
    lib.orc_ring_gather.argtypes = [C.POINTER(u16p), C.c_uint32, C.c_uint32, C.c_uint32, u16p]
    lib.orc_ring_packet_encode.restype = None
    lib.orc_ring_packet_encode.argtypes = [u16p, u32p]
    lib.orc_ring_packet_decode.restype = None
    lib.orc_ring_packet_decode.argtypes = [u32p, u16p]
    return lib


def load_reference():
    if not os.path.exists(REFERENCE_SO):
        return None
    lib = C.CDLL(REFERENCE_SO)
    lib.test_exl3_codebook.restype = C.c_uint16
    lib.test_exl3_codebook.argtypes = [C.c_uint32]
    lib.test_exl3_position.restype = C.c_uint32
    lib.test_exl3_position.argtypes = [C.c_uint32, C.c_uint32]
    lib.test_exl3_state.restype = C.c_uint16
    lib.test_exl3_state.argtypes = [u8p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]
    lib.test_exl3_reconstruct.restype = C.c_uint16
    lib.test_exl3_reconstruct.argtypes = [u8p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]
    for name in ("test_weight_format_e2m1_value", "test_weight_format_e4m3_value", "test_weight_format_e8m0_value"):
        getattr(lib, name).restype = C.c_double
        getattr(lib, name).argtypes = [C.c_uint32]
    lib.test_linear_quantize.argtypes = [u16p, C.c_uint32, u8p, u8p]
    lib.test_linear_codes_lay_out.argtypes = [u8p, C.c_uint32, u8p]
    lib.test_weight_format_lay_out.argtypes = [C.c_int, C.c_void_p, u8p, C.c_uint64, u8p, C.c_uint64, u8p, C.c_uint64]
    lib.test_linear_bfloat16_nearest.restype = C.c_uint16
    lib.test_linear_bfloat16_nearest.argtypes = [C.c_double]
    lib.test_linear_hidden_value.restype = C.c_double
    lib.test_linear_hidden_value.argtypes = [C.c_double] * 4
    lib.test_linear_fed_values_of_codes.argtypes = [u8p, C.c_uint32, C.POINTER(C.c_double)]
    lib.test_linear_output_is_within_tolerance.restype = C.c_bool
    lib.ordered_collective_host.restype = C.c_int
    lib.ordered_collective_host.argtypes = [C.POINTER(f32p), C.POINTER(f32p), C.c_uint32, C.c_uint32, C.c_int]
    if hasattr(lib, "ref_bf16_wire_pair_pack"):
        lib.ref_bf16_wire_pair_pack.restype = lib.ref_bf16_wire_pair_unpack.restype = C.c_uint32
        lib.ref_bf16_wire_pair_pack.argtypes = [C.c_uint32, C.c_uint32]
        lib.ref_bf16_wire_pair_unpack.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32]
        lib.ref_bf16_wire_digest.restype = C.c_uint64
        lib.ref_bf16_wire_digest.argtypes = []
    return lib


def pointer_array(arrays, kind=f32p):
    """A C array of pointers to the rows of `arrays` (numpy arrays kept alive by the caller)."""
    holder = (kind * len(arrays))()
    for index, array in enumerate(arrays):
        holder[index] = ptr(array, kind)
    return holder


def splitmix_words(seed, count):
    """The 32-bit words of the splitmix64 stream the reference's known-answer test draws its tiles from."""
    mask = (1 << 64) - 1
    state = seed & mask
    out = np.empty(count, dtype=np.uint32)
    for index in range(count):
        state = (state + 0x9E3779B97F4A7C15) & mask
        mixed = state
        mixed = ((mixed ^ (mixed >> 30)) * 0xBF58476D1CE4E5B9) & mask
        mixed = ((mixed ^ (mixed >> 27)) * 0x94D049BB133111EB) & mask
        out[index] = (mixed ^ (mixed >> 31)) & 0xFFFFFFFF
    return out
