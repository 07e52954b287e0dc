"""The router's CPU oracle pinned to the reference's own router reference (tests/router_reference.c, compiled unchanged
into oracle/_ref) at the reference's geometry: 384 experts, 6 picks, route scale 1.5, sqrt(softplus) affinities, a
per-expert selection bias. Affinities: inside the reference's tolerance for a card's affinity; choice, slot order,
weights and job table: bit for bit given the affinities. The committed fixtures carry the reference's answers to
machines without the reference tree."""
import ctypes as C

import numpy as np
import pytest

from anemone_b200 import records as R
from oracle.binding import f32p, ptr, u32p, u64p
from tests import golden_util

EXPERTS, PICKS, SCALE, SOFTPLUS = 384, 6, 1.5, 1


def oracle_rows(oracle, scores, bias):
    rows = scores.shape[0]
    experts = np.zeros((rows, PICKS), dtype=np.uint32)
    weights = np.zeros((rows, PICKS), dtype=np.float32)
    for row in range(rows):
        oracle.orc_router_row_biased(ptr(scores[row], f32p), ptr(bias, f32p) if bias is not None else None, EXPERTS,
                                     PICKS, SOFTPLUS, SCALE, ptr(experts[row], u32p), ptr(weights[row], f32p))
    return experts, weights


def oracle_jobs(oracle, experts, weights, table, capacity):
    jobs = (R.ExpertJob * capacity)()
    count = oracle.orc_router_jobs(ptr(experts, u32p), ptr(weights, f32p), experts.shape[0], PICKS, EXPERTS, 0,
                                   ptr(table, u64p), capacity, C.byref(jobs))
    return np.frombuffer(bytes(jobs), dtype=np.uint8), count


def test_affinity_is_inside_the_reference_tolerance(oracle, reference):
    reference.test_router_affinity_holds.restype = C.c_bool
    reference.test_router_affinity_holds.argtypes = [C.c_float, C.c_float]
    rng = np.random.default_rng(0)
    scores = np.concatenate([rng.normal(0, 1, 20000), rng.uniform(-110, 25, 20000), rng.uniform(-0.01, 0.01, 2000),
                             [0.0, -0.0, 20.0, 20.000002, 19.999998, -87.3, -88, -95, -103.9, -104, -120, np.inf,
                              -np.inf, 1e-30, -1e-30, np.nan]]).astype(np.float32)
    for score in scores:
        assert reference.test_router_affinity_holds(float(score), oracle.orc_router_affinity(float(score), SOFTPLUS)), score


def test_sigmoid_affinity_is_accurate(oracle):
    rng = np.random.default_rng(1)
    scores = np.concatenate([rng.normal(0, 2, 20000), rng.uniform(-100, 100, 5000)]).astype(np.float32)
    for score in scores:
        exact = 1.0 / (1.0 + np.exp(-np.float64(score)))
        got = oracle.orc_router_affinity(float(score), 0)
        if exact > 1e-37:
            assert abs(got - exact) <= 2.5 * np.spacing(np.float32(exact)), score
    assert oracle.orc_router_affinity(float("inf"), 0) == 1.0 and oracle.orc_router_affinity(float("-inf"), 0) == 0.0


def test_select_and_jobs_equal_the_reference(oracle, reference):
    reference.test_router_select.argtypes = [f32p, f32p, C.c_bool, u32p, f32p]
    rng = np.random.default_rng(11)
    for trial in range(40):
        rows = int(rng.integers(1, 9))
        scores = rng.normal(0.0, 2.0, size=(rows, EXPERTS)).astype(np.float32)
        bias = rng.normal(0.0, 0.1, size=EXPERTS).astype(np.float32)
        if trial % 4 == 0:  # many equal keys: quantized scores and bias
            scores = np.round(scores).astype(np.float32)
            bias = (np.round(bias * 4) / 4).astype(np.float32)
        if trial % 5 == 1:
            scores[0, rng.integers(0, EXPERTS, 3)] = [np.nan, np.inf, -np.inf]
            bias[rng.integers(0, EXPERTS)] = np.float32("nan")
        if trial % 7 == 2:
            bias[:] = 0.0
        affinities = np.array([[oracle.orc_router_affinity(float(s), SOFTPLUS) for s in row] for row in scores],
                              dtype=np.float32)
        want_experts = np.zeros((rows, PICKS), dtype=np.uint32)
        want_weights = np.zeros((rows, PICKS), dtype=np.float32)
        for row in range(rows):
            reference.test_router_select(ptr(affinities[row], f32p), ptr(bias, f32p), False,
                                         ptr(want_experts[row], u32p), ptr(want_weights[row], f32p))
        experts, weights = oracle_rows(oracle, scores, bias)
        assert np.array_equal(experts, want_experts), trial
        assert np.array_equal(weights.view(np.uint32), want_weights.view(np.uint32)), trial
        table = (np.arange(EXPERTS * 3, dtype=np.uint64) * 4096 + 64).reshape(EXPERTS, 3)
        want_jobs = np.zeros(8 * PICKS * 96, dtype=np.uint8)
        reference.test_router_jobs(ptr(want_experts, u32p), ptr(want_weights, f32p), rows, 8, ptr(table, u64p),
                                   want_jobs.ctypes.data_as(C.c_void_p))
        jobs, count = oracle_jobs(oracle, experts, weights, table, 8 * PICKS)
        if np.isnan(weights).any():  # a not-a-number's payload is not compared
            assert np.array_equal(jobs.reshape(-1, 96)[:, :64], want_jobs.reshape(-1, 96)[:, :64])
        else:
            assert np.array_equal(jobs, want_jobs), trial
        assert count == len(set(experts.reshape(-1).tolist()))


def test_golden_router_fixtures(oracle):
    for case in golden_util.load("reference_vectors.json")["router_select"]:
        scores, bias, table = golden_util.router_case_inputs(case["seed"])
        experts, weights = oracle_rows(oracle, scores, bias)
        assert experts.tolist() == case["experts"]
        assert [[hex(v) for v in row] for row in weights.view(np.uint32).tolist()] == case["weights"]
        jobs, _ = oracle_jobs(oracle, experts, weights, table, case["rows"] * PICKS)
        assert hex(golden_util.fnv64(jobs)) == case["jobs_fnv64"]


def test_no_bias_means_a_zero_bias(oracle):
    rng = np.random.default_rng(5)
    scores = rng.normal(0.0, 2.0, size=(4, EXPERTS)).astype(np.float32)
    with_zero = oracle_rows(oracle, scores, np.zeros(EXPERTS, dtype=np.float32))
    without = oracle_rows(oracle, scores, None)
    assert np.array_equal(with_zero[0], without[0])
    assert np.array_equal(with_zero[1].view(np.uint32), without[1].view(np.uint32))
