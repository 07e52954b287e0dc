"""The CPU oracle of the output-axis exchanges against the reference's own vectors: the round-once model against the
known answers of tests/compressed_ring_card_test.c:500-520, the wire code against the reference's header (exhaustively,
where it was compiled) and its round-trip sweep (tests/bf16_wire_codec_test.c:37-55), this library's codec header
against both, and the properties of the sums."""
import ctypes as C
import os
import subprocess
import tempfile

import numpy as np
import pytest

from oracle.binding import pointer_array, ptr, u16p, u32p

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ONE, HALF_ULP, TIE_EPSILON, LARGE = 0x3F80, 0x3B80, 0x3780, 0x4780


def round_once(oracle, inputs):
    inputs = [np.ascontiguousarray(x, dtype=np.uint16) for x in inputs]
    out = np.zeros(inputs[0].size, dtype=np.uint16)
    oracle.orc_ring_round_once(pointer_array(inputs, u16p), len(inputs), out.size, ptr(out, u16p))
    return out


def test_round_once_known_answers(oracle):
    # values 0..3 of the reference's special pattern on ranks 0..3: zeros, negative zeros, a tie with a small excess,
    # a large term that cancels
    ranks = [[0, 0x8000, ONE, LARGE], [0, 0x8000, HALF_ULP, ONE], [0, 0x8000, TIE_EPSILON, LARGE | 0x8000],
             [0, 0x8000, 0, ONE]]
    first = round_once(oracle, ranks)
    assert first.tolist() == [0, 0, 0x3F81, 0x4000]
    # in place: every rank feeds the previous result
    assert round_once(oracle, [first] * 4).tolist()[2:] == [0x4081, 0x4100]


def test_bf16_addition_rounds_once(oracle):
    add = oracle.orc_ring_bf16_add
    assert add(ONE, HALF_ULP) == ONE            # a tie goes to the even fraction
    assert add(0x3F81, HALF_ULP) == 0x3F82
    assert add(0, 0x8000) == 0 and add(0x8000, 0x8000) == 0x8000
    assert add(0x7F7F, 0x7F7F) == 0x7F80       # overflow to infinity
    assert add(0x7F80, 0xFF80) == 0x7FFF       # the canonical not-a-number
    assert add(0x0001, 0x0001) == 0x0002       # subnormals stay
    rng = np.random.default_rng(5)
    for a, b in rng.integers(0, 0x7F80, size=(2000, 2)):
        a, b = int(a) | int(rng.integers(0, 2)) << 15, int(b) | int(rng.integers(0, 2)) << 15
        exact = float(np.array([a << 16], dtype=np.uint32).view(np.float32)[0]) + \
            float(np.array([b << 16], dtype=np.uint32).view(np.float32)[0])
        got = float(np.array([add(a, b) << 16], dtype=np.uint32).view(np.float32)[0])
        if np.isinf(got):
            assert abs(exact) >= 2.0 ** 127 * (2 - 2 ** -8)
        else:
            ulp = max(abs(exact) * 2.0 ** -7, 2.0 ** -133)
            assert abs(got - exact) <= ulp / 2 * 1.0000001 + 0.0


@pytest.mark.parametrize("ranks,vectors", [(2, 0), (4, 0), (4, 4), (8, 2)])
def test_bf16_sum_properties(oracle, ranks, vectors):
    packs = 64
    rng = np.random.default_rng(ranks * 10 + vectors)
    inputs = [((rng.integers(0, 128, ranks * packs * 8) | rng.integers(0, 2, ranks * packs * 8) << 15 |
                rng.integers(110, 125, ranks * packs * 8) << 7)).astype(np.uint16) for _ in range(ranks)]
    for x in inputs:
        x[::17] = 0
        x[1::17] = 0x8000
    outputs = [np.zeros_like(inputs[0]) for _ in range(ranks)]
    oracle.orc_ring_bf16_sum(pointer_array(inputs, u16p), ranks, packs, vectors, pointer_array(outputs, u16p))
    row_packs = packs // vectors if vectors else 0
    for rank in range(ranks):
        for other in range(ranks):
            differs = np.flatnonzero(outputs[rank] != outputs[other])
            # ranks differ only where the owner holds a +0 that travelled as -0
            assert all({int(outputs[rank][i]), int(outputs[other][i])} == {0, 0x8000} for i in differs)
    # a rank holds +0 only inside its own part
    for rank in range(ranks):
        zeros = np.flatnonzero(outputs[rank] == 0) // 8
        owner = zeros // packs if not vectors else (zeros // row_packs) % ranks
        assert (owner == rank).all()
    # two ranks: one addition, whatever the order
    if ranks == 2:
        for i in range(0, inputs[0].size, 37):
            want = oracle.orc_ring_bf16_add(int(inputs[0][i]), int(inputs[1][i]))
            assert {int(outputs[0][i]), int(outputs[1][i])} <= {want, 0x8000 if want == 0 else want}


def test_gather_orders(oracle):
    ranks, packs, vectors = 4, 32, 4
    inputs = [np.zeros(ranks * packs * 8, dtype=np.uint16) for _ in range(ranks)]
    for rank in range(ranks):
        inputs[rank][rank * packs * 8:(rank + 1) * packs * 8] = rank * 1000 + np.arange(packs * 8)
    out = np.zeros(ranks * packs * 8, dtype=np.uint16)
    oracle.orc_ring_gather(pointer_array(inputs, u16p), ranks, packs, 0, ptr(out, u16p))
    assert all((out[r * packs * 8:(r + 1) * packs * 8] == r * 1000 + np.arange(packs * 8)).all() for r in range(ranks))
    oracle.orc_ring_gather(pointer_array(inputs, u16p), ranks, packs, vectors, ptr(out, u16p))
    rows = out.reshape(vectors, ranks, packs // vectors * 8)
    for rank in range(ranks):
        assert (rows[:, rank, :].reshape(-1) == rank * 1000 + np.arange(packs * 8)).all()


def packet_round_trip(oracle, values):
    packet, back = np.zeros(136, dtype=np.uint32), np.zeros(256, dtype=np.uint16)
    oracle.orc_ring_packet_encode(ptr(values, u16p), ptr(packet, u32p))
    oracle.orc_ring_packet_decode(ptr(packet, u32p), ptr(back, u16p))
    return packet, back


def test_packets_keep_every_bit(oracle):
    rng = np.random.default_rng(11)
    near = (rng.integers(0, 128, 256) | rng.integers(0, 2, 256) << 15 | rng.integers(112, 121, 256) << 7).astype(np.uint16)
    packet, back = packet_round_trip(oracle, near)
    assert np.array_equal(back, near) and packet[1] == 0 and packet[0] == 120
    assert not packet[4 + 96:132].any()  # 32 coded lanes: 96 words
    wide = near.copy()
    wide[8 * 5:8 * 5 + 8] = [0, 0x8000, 0x7F80, 0x7FC5, 0x0001, 0xFFFF, 0x3F80, 0x0080]  # lane 5: specials
    wide[8 * 31 + 3] = 0x0100                                                            # lane 31: one far value
    packet, back = packet_round_trip(oracle, wide)
    assert np.array_equal(back, wide) and packet[0] == 255 and packet[1] == 0xFFFFFFFF  # a 255 exponent: all lanes raw
    wide[8 * 5 + 2:8 * 5 + 4] = 0x3F80
    wide[8 * 5 + 5] = 0x3F80
    packet, back = packet_round_trip(oracle, wide)
    assert np.array_equal(back, wide) and packet[1] == (1 << 5 | 1 << 31)
    for _ in range(50):  # any bits at all
        values = rng.integers(0, 65536, 256).astype(np.uint16)
        assert np.array_equal(packet_round_trip(oracle, values)[1], values)


def library_codec():
    """This library's codec header compiled for the host, as a small shared object of its four functions."""
    folder = tempfile.mkdtemp()
    source, target = os.path.join(folder, "codec.c"), os.path.join(folder, "codec.so")
    with open(source, "w") as file:
        file.write('#include "anemone_b200_wire_codec.h"\n'
                   "uint32_t pack(uint32_t w, uint32_t t) { return bf16_wire_pair_pack(w, t); }\n"
                   "uint32_t unpack(uint32_t b, uint32_t d, uint32_t t) { return bf16_wire_pair_unpack(b, d, t); }\n"
                   "uint64_t digest(void) { uint64_t h = 0xCBF29CE484222325ull;\n"
                   "  for (uint32_t v = 0; v < 65536u; v++) { uint32_t w = v | v << 16, e = bf16_wire_low_exponent(w);\n"
                   "    for (uint32_t d = 0; d <= 15u && e + d <= 255u; d++) {\n"
                   "      uint32_t p = bf16_wire_pair_pack(w, e + d);\n"
                   "      if (bf16_wire_pair_unpack(p & 65535u, p >> 16, e + d) != w) return 0;\n"
                   "      h = (h ^ p) * 0x100000001B3ull; } }\n"
                   "  return h; }\n")
    subprocess.run(["gcc", "-std=c11", "-O2", "-shared", "-fPIC", "-I", os.path.join(ROOT, "include"), "-o", target,
                    source], check=True)
    lib = C.CDLL(target)
    lib.pack.restype = lib.unpack.restype = C.c_uint32
    lib.pack.argtypes = [C.c_uint32] * 2
    lib.unpack.argtypes = [C.c_uint32] * 3
    lib.digest.restype = C.c_uint64
    return lib


# FNV-1a over the reference's packed words on its own exhaustive sweep (oracle/ref_shims.c: ref_bf16_wire_digest),
# recorded from its header source/bf16_wire_codec.h
REFERENCE_WIRE_DIGEST = 0x97937948C839F325


def test_codec_header_round_trips_on_the_reference_sweep():
    digest = library_codec().digest()
    assert digest != 0  # every bfloat16 value, every admitted shared exponent, comes back
    assert digest == REFERENCE_WIRE_DIGEST


def test_codec_header_matches_the_reference(reference):
    codec = library_codec()
    assert reference.ref_bf16_wire_digest() == REFERENCE_WIRE_DIGEST
    mixed = 1013904223
    for _ in range(20000):  # mixed pairs, the reference's generator
        mixed = (mixed * 2654435761 + 1013904223) & 0xFFFFFFFF
        low, high = (mixed >> 7) & 255, (mixed >> 23) & 255
        top = max(low, high)
        if top - min(low, high) <= 15:
            packed = codec.pack(mixed, top)
            assert packed == reference.ref_bf16_wire_pair_pack(mixed, top)
            assert codec.unpack(packed & 0xFFFF, packed >> 16, top) == mixed


def test_oracle_packets_use_the_codec_words(oracle):
    """A coded lane's three words are the codec's four packed words regrouped (bytes, bytes, distances)."""
    codec = library_codec()
    rng = np.random.default_rng(3)
    values = (rng.integers(0, 128, 256) | rng.integers(0, 2, 256) << 15 | rng.integers(100, 116, 256) << 7).astype(np.uint16)
    packet, _ = packet_round_trip(oracle, values)
    top = int(packet[0])
    words = values.view(np.uint32).reshape(32, 4)
    for lane in range(32):
        packed = [codec.pack(int(w), top) for w in words[lane]]
        assert int(packet[4 + 3 * lane]) == (packed[0] & 0xFFFF) | (packed[1] & 0xFFFF) << 16
        assert int(packet[5 + 3 * lane]) == (packed[2] & 0xFFFF) | (packed[3] & 0xFFFF) << 16
        assert int(packet[6 + 3 * lane]) == sum((packed[i] >> 16) << (8 * i) for i in range(4))
