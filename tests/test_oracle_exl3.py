"""The CPU oracle against the reference's known-answer vectors and against the reference's own compiled host code.

Mirrors tests/exl3_test.c, tests/exl3_widths_test.c and tests/exl3_sm120_reference_test.c of the reference.
"""
import ctypes as C
import json
import os

import numpy as np
import pytest

from oracle.binding import ptr, splitmix_words, u8p, u16p, f32p

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
WIDTHS = [2, 40, 3, 4]


def kat():
    with open(os.path.join(GOLDEN, "exl3_kat.json")) as handle:
        return json.load(handle)


def bits_x2(stored):
    return 2 * stored if stored <= 8 else stored // 8


def random_codes(rng, inputs, outputs, stored):
    count = inputs * outputs // 16 * bits_x2(stored)
    return rng.integers(0, 256, size=count, dtype=np.uint8)


def test_known_answer_states(oracle):
    golden = kat()
    for case in golden["widths"]:
        tile_words = 256 * case["bits_x2"] // 2 // 32
        words = splitmix_words(golden["seed_base"] + case["stored"], 4 * tile_words)
        codes = words.view(np.uint8)
        first = [oracle.orc_exl3_state(ptr(codes, u8p), 32, 32, case["stored"], 0, output) for output in range(8)]
        assert first == [int(value, 16) for value in case["first"]]
        assert oracle.orc_exl3_states_digest(ptr(codes, u8p), 32, 32, case["stored"]) == int(case["digest"], 16)
        # the sliding-window path sees the same states as the bit walk
        states = np.zeros((32, 32), dtype=np.uint16)
        oracle.orc_exl3_states(ptr(codes, u8p), 32, 32, case["stored"], ptr(states, u16p))
        walked = [[oracle.orc_exl3_state(ptr(codes, u8p), 32, 32, case["stored"], i, o) for o in range(32)]
                  for i in range(32)]
        assert np.array_equal(states, np.array(walked, dtype=np.uint16))


def test_expert_byte_counts():
    golden = kat()
    for case in golden["widths"]:
        inputs, outputs = golden["expert_inputs"], golden["expert_outputs"]
        assert inputs * outputs // 16 * case["bits_x2"] + 2 * (inputs + outputs) == case["expert_bytes"]


def test_zero_trellis_and_codebook_range(oracle):
    golden = kat()
    assert oracle.orc_exl3_codebook(0) == int(golden["zero_trellis_weight"], 16)
    assert oracle.orc_half_value(oracle.orc_exl3_codebook(0)) == -3.453125
    for stored in WIDTHS:
        codes = np.zeros(32 * 32 // 16 * bits_x2(stored), dtype=np.uint8)
        weights = np.zeros((32, 32), dtype=np.uint16)
        oracle.orc_exl3_decode(ptr(codes, u8p), 32, 32, stored, ptr(weights, u16p))
        assert (weights == 0xC2E8).all()
    values = np.array([oracle.orc_half_value(oracle.orc_exl3_codebook(state)) for state in range(0, 65536, 7)])
    # every state is a finite number of the codebook's span (1774 b - 905216) / 2^18, b = 0 .. 1020
    assert np.isfinite(values).all() and values.min() >= -3.453125 and values.max() <= 3.45


def test_codebook_is_the_affine_form(oracle):
    for state in range(0, 65536, 11):
        hashed = (state * 0x83DCD12D) & 0xFFFFFFFF
        byte_sum = sum((hashed >> shift) & 255 for shift in (0, 8, 16, 24))
        exact = (1774 * byte_sum - 905216) / 2.0 ** 18
        assert oracle.orc_exl3_codebook(state) == int(np.float16(exact).view(np.uint16))


def test_tile_permutation_is_a_bijection(oracle):
    # tests/exl3_test.c:95-108: 256 (input, output) places <-> 256 stream positions
    places = {}
    for i in range(16):
        for o in range(16):
            lane = ((o & 7) << 2) | ((i & 7) >> 1)
            element = (i & 1) | ((i >> 3) << 1) | ((o >> 3) << 2)
            places[(i, o)] = lane * 8 + element
    assert sorted(places.values()) == list(range(256))


def test_half_rounding_matches_numpy(oracle):
    rng = np.random.default_rng(5)
    samples = np.concatenate([rng.normal(0, 1, 4000), rng.normal(0, 1e-5, 2000), rng.normal(0, 3e4, 2000),
                              [0.0, -0.0, 65504.0, 65519.9, 65520.0, 2.0 ** -24, 2.0 ** -25, 3 * 2.0 ** -25]])
    for value in samples:
        assert oracle.orc_half_nearest(float(value)) == int(np.float64(value).astype(np.float16).view(np.uint16)), value
    for bits in range(0, 65536, 3):
        value = np.uint16(bits).view(np.float16)
        if np.isnan(value):
            continue
        assert oracle.orc_half_value(bits) == np.float32(value)


def test_bfloat16_rounding(oracle):
    assert oracle.orc_bfloat16_bits(1.0) == 0x3F80
    assert oracle.orc_bfloat16_bits(float(np.uint32(0x3F808000).view(np.float32))) == 0x3F80  # tie to even (down)
    assert oracle.orc_bfloat16_bits(float(np.uint32(0x3F818000).view(np.float32))) == 0x3F82  # tie to even (up)
    assert oracle.orc_bfloat16_bits(float("nan")) == 0x7FC0
    assert oracle.orc_bfloat16_bits(float("inf")) == 0x7F80
    assert oracle.orc_bfloat16_bits(-0.0) == 0x8000


def test_hadamard_is_the_scaled_involution(oracle):
    rng = np.random.default_rng(11)
    values = rng.normal(0, 1, 128).astype(np.float32)
    work = values.copy()
    oracle.orc_hadamard128(ptr(work, f32p))
    # Sylvester matrix by definition, in double
    h = np.array([[1.0]])
    for _ in range(7):
        h = np.block([[h, h], [h, -h]])
    assert np.allclose(work, h @ values.astype(np.float64), rtol=0, atol=1e-4)
    oracle.orc_hadamard128(ptr(work, f32p))
    assert np.allclose(work / 128.0, values, atol=1e-5)


# ---- against the reference's own host code compiled from its sources (oracle/_ref) ----

def test_codebook_equals_reference(oracle, reference):
    for state in range(65536):
        assert oracle.orc_exl3_codebook(state) == reference.test_exl3_codebook(state)


def test_positions_equal_reference(reference):
    for i in range(16):
        for o in range(16):
            lane = ((o & 7) << 2) | ((i & 7) >> 1)
            element = (i & 1) | ((i >> 3) << 1) | ((o >> 3) << 2)
            assert reference.test_exl3_position(i, o) == lane * 8 + element


@pytest.mark.parametrize("stored", WIDTHS)
def test_decode_equals_reference(oracle, reference, stored):
    rng = np.random.default_rng(100 + stored)
    inputs, outputs = 48, 64
    codes = random_codes(rng, inputs, outputs, stored)
    weights = np.zeros((inputs, outputs), dtype=np.uint16)
    oracle.orc_exl3_decode(ptr(codes, u8p), inputs, outputs, stored, ptr(weights, u16p))
    for i in range(inputs):
        for o in range(outputs):
            assert weights[i, o] == reference.test_exl3_reconstruct(ptr(codes, u8p), inputs, outputs, stored, i, o)
