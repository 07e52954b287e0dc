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


def router_case_inputs(seed):
    """Scores [rows][384], bias [384] and an expert table of one router fixture (the generator's draw): N(0, 2) scores
    with ties, not-a-numbers, infinities, -0 and saturated rows; a small bias with ties of its own."""
    rng = np.random.default_rng(seed)
    rows = 1 + seed % 8
    scores = rng.normal(0.0, 2.0, size=(rows, 384)).astype(np.float32)
    bias = rng.normal(0.0, 0.05, size=384).astype(np.float32)
    scores[0, [5, 300]] = 7.5  # equal scores: with equal bias the lower expert first
    bias[[5, 300]] = 0.25
    scores[rows - 1, 17] = np.float32("nan")
    scores[rows - 1, 18] = np.float32("inf")
    scores[rows - 1, 19] = np.float32("-inf")
    scores[rows // 2, 100:110] = 30.0  # above the softplus threshold
    scores[rows // 2, 200:204] = [-0.0, 0.0, -90.0, -120.0]
    if seed & 1:
        bias[:] = 0.0
    table = (np.arange(384 * 3, dtype=np.uint64) * 4096 + 64).reshape(384, 3)
    return scores, bias, table
