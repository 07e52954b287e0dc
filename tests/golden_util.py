"""Helpers shared by the tests that read the committed golden fixtures."""
import json
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    with open(os.path.join(GOLDEN, name)) as handle:
        return json.load(handle)


def fnv64(values):
    digest = 0xCBF29CE484222325
    for byte in np.ascontiguousarray(values).reshape(-1).view(np.uint8).tolist():
        digest = ((digest ^ byte) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return digest


def bits_x2(stored):
    return 2 * stored if stored <= 8 else stored // 8


def golden_decode_case(case):
    """The seeded code bytes of one decode fixture (the generator's draw)."""
    rng = np.random.default_rng(case["seed"])
    return rng.integers(0, 256, size=case["inputs"] * case["outputs"] // 16 * bits_x2(case["stored"]), dtype=np.uint8)


def golden_reduce_case(case):
    rng = np.random.default_rng(case["seed"])
    count = case["rows"] * 4096
    return [rng.normal(0.0, 0.05, count).astype(np.float32) for _ in range(case["ranks"])]
