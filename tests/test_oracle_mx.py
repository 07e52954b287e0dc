"""The original-weights (MXFP4 by E4M3) oracle against the reference's own test references compiled from its sources
(oracle/_ref): code values, activation quantization, both layouts, the product tolerance and the hidden step."""
import ctypes as C

import numpy as np
import pytest

from anemone_b200 import synthetic
from oracle.binding import ptr, u16p, u8p


class Shape(C.Structure):
    _fields_ = [("output_size", C.c_uint32), ("input_size", C.c_uint32), ("bits_per_weight", C.c_uint32),
                ("reserved", C.c_uint32)]


class Product(C.Structure):
    _fields_ = [("sum", C.c_double), ("magnitude_sum", C.c_double)]


def test_code_values_equal_reference(oracle, reference):
    for code in range(16):
        assert oracle.orc_e2m1_value(code) == reference.test_weight_format_e2m1_value(code)
    for code in range(256):
        if code & 0x7F != 0x7F:
            assert oracle.orc_e4m3_value(code) == reference.test_weight_format_e4m3_value(code)
        if code != 255:
            assert oracle.orc_e8m0_value(code) == reference.test_weight_format_e8m0_value(code)


def vectors(rng, width):
    out = [synthetic.to_bfloat16(rng.normal(0, scale, width).astype(np.float32)) for scale in (1.0, 1e-3, 300.0, 1e-6)]
    special = synthetic.to_bfloat16(rng.normal(0, 1, width).astype(np.float32))
    special[:40] = 0
    special[5] = 0x8000  # minus zero keeps its sign
    special[64:96] = synthetic.to_bfloat16(np.full(32, 0.4375, dtype=np.float32))  # ties between codes
    special[96] = synthetic.to_bfloat16(np.array([448.0], dtype=np.float32))[0]
    out.append(special)
    return out


def test_quantize_equals_reference(oracle, reference):
    rng = np.random.default_rng(21)
    for width in (128, 512):
        for values in vectors(rng, width):
            ours_codes, ours_exp = np.zeros(width, np.uint8), np.zeros(width // 32, np.uint8)
            ref_codes, ref_exp = np.zeros(width, np.uint8), np.zeros(width // 32, np.uint8)
            oracle.orc_mx_quantize(ptr(values, u16p), width, ptr(ours_codes, u8p), ptr(ours_exp, u8p))
            assert reference.test_linear_quantize(ptr(values, u16p), width, ptr(ref_codes, u8p), ptr(ref_exp, u8p)) == 0
            assert np.array_equal(ours_codes, ref_codes) and np.array_equal(ours_exp, ref_exp)
            a, b = np.zeros(width, np.uint8), np.zeros(width, np.uint8)
            oracle.orc_mx_codes_lay_out(ptr(ours_codes, u8p), width, ptr(a, u8p))
            assert reference.test_linear_codes_lay_out(ptr(ref_codes, u8p), width, ptr(b, u8p)) == 0
            assert np.array_equal(a, b)


def test_weight_layout_equals_reference(oracle, reference):
    rng = np.random.default_rng(22)
    outputs, inputs = 48, 192
    codes = rng.integers(0, 16, size=outputs * inputs, dtype=np.uint8)
    scales = rng.integers(119, 124, size=outputs * inputs // 32, dtype=np.uint8)
    size = outputs * inputs // 2 + outputs * inputs // 32
    ours, theirs = np.zeros(size, np.uint8), np.zeros(size, np.uint8)
    oracle.orc_mx_weights_lay_out(ptr(codes, u8p), ptr(scales, u8p), outputs, inputs, ptr(ours, u8p))
    shape = Shape(outputs, inputs, 4, 0)
    assert reference.test_weight_format_lay_out(3, C.byref(shape), ptr(codes, u8p), codes.size, ptr(scales, u8p),
                                                scales.size, ptr(theirs, u8p), size) == 0
    assert np.array_equal(ours, theirs)


def test_outputs_within_reference_tolerance(oracle, reference):
    rng = np.random.default_rng(23)
    outputs, inputs = 32, 512
    codes = rng.integers(0, 16, size=outputs * inputs, dtype=np.uint8)
    scales = rng.integers(119, 124, size=outputs * inputs // 32, dtype=np.uint8)
    stored = np.zeros(outputs * inputs // 2 + outputs * inputs // 32, np.uint8)
    oracle.orc_mx_weights_lay_out(ptr(codes, u8p), ptr(scales, u8p), outputs, inputs, ptr(stored, u8p))
    values = synthetic.to_bfloat16(rng.normal(0, 1, inputs).astype(np.float32))
    fed_codes, fed_exp = np.zeros(inputs, np.uint8), np.zeros(inputs // 32, np.uint8)
    oracle.orc_mx_quantize(ptr(values, u16p), inputs, ptr(fed_codes, u8p), ptr(fed_exp, u8p))
    fed_values = np.zeros(inputs, np.float64)
    assert reference.test_linear_fed_values_of_codes(ptr(fed_codes, u8p), inputs,
                                                     fed_values.ctypes.data_as(C.POINTER(C.c_double))) == 0
    products = (Product * outputs)()
    shape = Shape(outputs, inputs, 4, 0)
    reference.test_linear_products.argtypes = [C.c_int, C.c_void_p, u8p, C.c_uint64, C.c_uint32, C.c_uint32,
                                               C.POINTER(C.c_double), u8p, C.c_uint32, C.c_uint32, C.c_void_p]
    assert reference.test_linear_products(3, C.byref(shape), ptr(stored, u8p), stored.size, 0, outputs,
                                          fed_values.ctypes.data_as(C.POINTER(C.c_double)), ptr(fed_exp, u8p), 1, 1,
                                          C.byref(products)) == 0
    reference.test_linear_output_is_within_tolerance.argtypes = [C.c_uint16, C.c_void_p, C.c_uint32, C.c_uint32]
    for slices in (1, 4, 8):
        for output in range(outputs):
            bits = oracle.orc_mx_output(ptr(stored, u8p), outputs, inputs, output, ptr(fed_codes, u8p), ptr(fed_exp, u8p),
                                        slices)
            assert reference.test_linear_output_is_within_tolerance(bits, C.byref(products[output]), inputs, slices)
            exact = synthetic.from_bfloat16(np.array([reference.test_linear_bfloat16_nearest(products[output].sum)],
                                                     dtype=np.uint16))[0]
            assert abs(synthetic.from_bfloat16(np.array([bits], dtype=np.uint16))[0] - exact) <= abs(exact) * 2 ** -7


def test_hidden_equals_reference(oracle, reference):
    rng = np.random.default_rng(24)
    gates = synthetic.to_bfloat16(rng.normal(0, 4, 2000).astype(np.float32))
    ups = synthetic.to_bfloat16(rng.normal(0, 4, 2000).astype(np.float32))
    differing = 0
    for gate, up in zip(gates.tolist(), ups.tolist()):
        for weight in (1.0, 0.37):
            ours = oracle.orc_mx_hidden(gate, up, 7.0, weight)
            g = float(synthetic.from_bfloat16(np.array([gate], np.uint16))[0])
            u = float(synthetic.from_bfloat16(np.array([up], np.uint16))[0])
            theirs = reference.test_linear_bfloat16_nearest(reference.test_linear_hidden_value(g, u, 7.0,
                                                                                               float(np.float32(weight))))
            differing += abs(int(ours & 0x7FFF) - int(theirs & 0x7FFF)) > 1 or (ours ^ theirs) & 0x8000 and ours & 0x7FFF > 1
    assert differing == 0  # float32 steps against the double reference: never more than one last place apart


def e4m3_codes(rng, count):
    """E4M3 bytes that are numbers (no 0x7F, no 0xFF), both signs, subnormals included."""
    codes = rng.integers(0, 127, size=count, dtype=np.uint8)
    return (codes | (rng.integers(0, 2, size=count, dtype=np.uint8) << 7)).astype(np.uint8)


def test_e4m3_weight_layout_equals_reference(oracle, reference):
    rng = np.random.default_rng(25)
    for outputs, inputs in ((48, 192), (64, 128)):  # the first: a last block of 16 outputs
        codes = e4m3_codes(rng, outputs * inputs)
        scales = rng.integers(110, 130, size=(outputs + 31) // 32 * (inputs // 32), dtype=np.uint8)
        size = outputs * inputs + scales.size
        ours, theirs = np.zeros(size, np.uint8), np.zeros(size, np.uint8)
        oracle.orc_e4m3_weights_lay_out(ptr(codes, u8p), ptr(scales, u8p), outputs, inputs, ptr(ours, u8p))
        shape = Shape(outputs, inputs, 8, 0)
        assert reference.test_weight_format_lay_out(5, C.byref(shape), ptr(codes, u8p), codes.size, ptr(scales, u8p),
                                                    scales.size, ptr(theirs, u8p), size) == 0
        assert np.array_equal(ours, theirs)


def test_trunk_outputs_within_reference_tolerance(oracle, reference):
    rng = np.random.default_rng(26)
    outputs, inputs = 48, 512
    codes = e4m3_codes(rng, outputs * inputs)
    scales = rng.integers(115, 125, size=(outputs + 31) // 32 * (inputs // 32), dtype=np.uint8)
    stored = np.zeros(outputs * inputs + scales.size, np.uint8)
    oracle.orc_e4m3_weights_lay_out(ptr(codes, u8p), ptr(scales, u8p), outputs, inputs, ptr(stored, u8p))
    values = synthetic.to_bfloat16(rng.normal(0, 1, inputs).astype(np.float32))
    fed_codes, fed_exp = np.zeros(inputs, np.uint8), np.zeros(inputs // 32, np.uint8)
    oracle.orc_mx_quantize(ptr(values, u16p), inputs, ptr(fed_codes, u8p), ptr(fed_exp, u8p))
    fed_values = np.zeros(inputs, np.float64)
    assert reference.test_linear_fed_values_of_codes(ptr(fed_codes, u8p), inputs,
                                                     fed_values.ctypes.data_as(C.POINTER(C.c_double))) == 0
    products = (Product * outputs)()
    shape = Shape(outputs, inputs, 8, 0)
    reference.test_linear_products.argtypes = [C.c_int, C.c_void_p, u8p, C.c_uint64, C.c_uint32, C.c_uint32,
                                               C.POINTER(C.c_double), u8p, C.c_uint32, C.c_uint32, C.c_void_p]
    assert reference.test_linear_products(5, C.byref(shape), ptr(stored, u8p), stored.size, 0, outputs,
                                          fed_values.ctypes.data_as(C.POINTER(C.c_double)), ptr(fed_exp, u8p), 1, 1,
                                          C.byref(products)) == 0
    reference.test_linear_output_is_within_tolerance.argtypes = [C.c_uint16, C.c_void_p, C.c_uint32, C.c_uint32]
    for slices in (1, 2, 8):
        for output in range(outputs):
            bits = oracle.orc_trunk_output(ptr(stored, u8p), outputs, inputs, output, ptr(fed_codes, u8p),
                                           ptr(fed_exp, u8p), slices)
            assert reference.test_linear_output_is_within_tolerance(bits, C.byref(products[output]), inputs, slices)


def test_block128_outputs_follow_the_same_chain(oracle):
    """WEIGHT_FORMAT_E4M3_BLOCK128 is not a format of the reference (parity unpinned for it): its oracle is the pinned
    chain with the FP32 scale of the 128 by 128 block in the place of 2^(weight code - 127). Where every FP32 scale IS
    such a power of two, the outputs equal the pinned format's bit for bit."""
    rng = np.random.default_rng(27)
    outputs, inputs = 256, 512
    codes = e4m3_codes(rng, outputs * inputs)
    exponent_codes = rng.integers(115, 125, size=(outputs // 128, inputs // 128), dtype=np.uint8)
    scales32 = np.ldexp(np.float32(1.0), exponent_codes.astype(np.int32) - 127).astype(np.float32)
    scales8 = np.repeat(np.repeat(exponent_codes, 4, axis=0), 4, axis=1)  # one code per 32 by 32
    block128 = np.zeros(outputs * inputs + scales32.size * 4, np.uint8)
    scaled = np.zeros(outputs * inputs + scales8.size, np.uint8)
    oracle.orc_e4m3_block128_lay_out(ptr(codes, u8p), scales32.ctypes.data_as(C.POINTER(C.c_float)), outputs, inputs,
                                     ptr(block128, u8p))
    oracle.orc_e4m3_weights_lay_out(ptr(codes, u8p), ptr(np.ascontiguousarray(scales8).reshape(-1), u8p), outputs,
                                    inputs, ptr(scaled, u8p))
    assert np.array_equal(block128[:outputs * inputs], scaled[:outputs * inputs])
    values = synthetic.to_bfloat16(rng.normal(0, 1, inputs).astype(np.float32))
    fed_codes, fed_exp = np.zeros(inputs, np.uint8), np.zeros(inputs // 32, np.uint8)
    oracle.orc_mx_quantize(ptr(values, u16p), inputs, ptr(fed_codes, u8p), ptr(fed_exp, u8p))
    for slices in (1, 4):
        for output in range(0, outputs, 7):
            assert oracle.orc_trunk_output_block128(ptr(block128, u8p), outputs, inputs, output, ptr(fed_codes, u8p),
                                                    ptr(fed_exp, u8p), slices) == \
                oracle.orc_trunk_output(ptr(scaled, u8p), outputs, inputs, output, ptr(fed_codes, u8p),
                                        ptr(fed_exp, u8p), slices)
