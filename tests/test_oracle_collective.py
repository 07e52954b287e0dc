"""The ordered-reduction and router oracles: the reference's cancellation vectors (tests/ordered_collective_test.c:
190-272), the committed fixtures generated from the reference's own host code, and that code itself where built."""
import ctypes as C

import numpy as np
import pytest

from tests import golden_util
from oracle.binding import f32p, pointer_array, ptr, u16p, u32p, u64p, u8p

RANKS, ELEMENTS, BIG = 5, 7, 16777216.0


def cancellation_inputs():
    order = [BIG, 1.0, -BIG, 1.0, 1.0]
    return [np.full(ELEMENTS, value, dtype=np.float32) for value in order]


def test_cancellation_sensitive_order(oracle):
    inputs = cancellation_inputs()
    out = np.full(ELEMENTS, -99.0, dtype=np.float32)
    oracle.orc_ordered_sum(pointer_array(inputs), RANKS, ELEMENTS, ptr(out, f32p))
    assert (out == 2.0).all()  # ((((0 + 2^24) + 1) - 2^24) + 1) + 1 with one rounding per add
    swapped = inputs[::-1]
    oracle.orc_ordered_sum(pointer_array(swapped), RANKS, ELEMENTS, ptr(out, f32p))
    assert (out != 2.0).all()  # a changed order must change the bits


def test_scatter_then_gather_is_all_reduce(oracle):
    inputs = cancellation_inputs()
    outputs = [np.full(ELEMENTS, -99.0, dtype=np.float32) for _ in range(RANKS)]
    assert oracle.orc_ordered_collective(pointer_array(inputs), pointer_array(outputs), RANKS, ELEMENTS, 2) == 0
    piece = (ELEMENTS + RANKS - 1) // RANKS
    for rank in range(RANKS):
        for element in range(ELEMENTS):
            assert outputs[rank][element] == (2.0 if element // piece == rank else -99.0)
    gathered = [np.zeros(ELEMENTS, dtype=np.float32) for _ in range(RANKS)]
    assert oracle.orc_ordered_collective(pointer_array(outputs), pointer_array(gathered), RANKS, ELEMENTS, 3) == 0
    for rank in range(RANKS):
        assert (gathered[rank] == 2.0).all()
    assert oracle.orc_ordered_collective(pointer_array(inputs), pointer_array(outputs), 0, ELEMENTS, 0) == 1
    assert oracle.orc_ordered_collective(pointer_array(inputs), pointer_array(outputs), RANKS, 0, 0) == 1


def test_golden_all_reduce(oracle):
    golden = golden_util.load("reference_vectors.json")
    for case in golden["ordered_all_reduce"]:
        inputs = golden_util.golden_reduce_case(case)
        out = np.zeros(case["rows"] * 4096, dtype=np.float32)
        oracle.orc_ordered_sum(pointer_array(inputs), case["ranks"], out.size, ptr(out, f32p))
        assert hex(golden_util.fnv64(out)) == case["sum_fnv64"]
        assert [hex(v) for v in out[:8].view(np.uint32).tolist()] == case["first"]
        rounded = np.zeros(out.size, dtype=np.uint16)
        oracle.orc_ordered_reduce_bf16(pointer_array(inputs), case["ranks"], out.size, ptr(rounded, u16p))
        expected = np.array([oracle.orc_bfloat16_bits(float(v)) for v in out[:512]], dtype=np.uint16)
        assert np.array_equal(rounded[:512], expected)


def test_golden_decode(oracle):
    golden = golden_util.load("reference_vectors.json")
    table = np.array([oracle.orc_exl3_codebook(s) for s in range(65536)], dtype=np.uint16)
    assert hex(golden_util.fnv64(table)) == golden["codebook_fnv64"]
    for case in golden["decode"]:
        codes = golden_util.golden_decode_case(case)
        weights = np.zeros((case["inputs"], case["outputs"]), dtype=np.uint16)
        oracle.orc_exl3_decode(ptr(codes, u8p), case["inputs"], case["outputs"], case["stored"], ptr(weights, u16p))
        assert hex(golden_util.fnv64(weights)) == case["weights_fnv64"]
        assert [hex(v) for v in weights[0, :8].tolist()] == case["first_row"]


@pytest.mark.parametrize("operation", [0, 1, 2, 3])
def test_collective_equals_reference_host(oracle, reference, operation):
    rng = np.random.default_rng(77 + operation)
    for ranks, count in ((2, 13), (4, 4096), (8, 1000), (16, 33)):
        inputs = [rng.normal(0, 0.05, count).astype(np.float32) for _ in range(ranks)]
        inputs[0][:3] = [BIG, -BIG, np.float32(1e-30)]
        ours = [np.full(count, -99.0, dtype=np.float32) for _ in range(ranks)]
        theirs = [np.full(count, -99.0, dtype=np.float32) for _ in range(ranks)]
        assert oracle.orc_ordered_collective(pointer_array(inputs), pointer_array(ours), ranks, count, operation) == 0
        assert reference.ordered_collective_host(pointer_array(inputs), pointer_array(theirs), ranks, count,
                                                 operation) == 0
        for rank in range(ranks):
            assert np.array_equal(ours[rank].view(np.uint32), theirs[rank].view(np.uint32))


def test_router_row_conventions(oracle):
    scores = np.zeros(256, dtype=np.float32)
    scores[[200, 7, 31, 100]] = [3.0, 3.0, 2.0, np.float32("nan")]  # NaN above all; ties to the lower expert
    scores[50] = -0.0
    experts = np.zeros(8, dtype=np.uint32)
    weights = np.zeros(8, dtype=np.float32)
    oracle.orc_router_row(ptr(scores, f32p), 256, 8, 0, 1.0, ptr(experts, u32p), ptr(weights, f32p))
    # picks: 100 (NaN), 7 and 200 (3.0), 31 (2.0), then +0 scores from the lowest expert: 0, 1, 2, 3 (-0 at 50 loses)
    assert experts.tolist() == [0, 1, 2, 3, 7, 31, 100, 200]
    rng = np.random.default_rng(3)
    scores = rng.normal(0, 1, 256).astype(np.float32)
    oracle.orc_router_row(ptr(scores, f32p), 256, 8, 0, 1.0, ptr(experts, u32p), ptr(weights, f32p))
    assert sorted(experts.tolist()) == sorted(np.argsort(-scores, kind="stable")[:8].tolist())
    assert experts.tolist() == sorted(experts.tolist())
    affinity = 1.0 / (1.0 + np.exp(-scores[experts].astype(np.float64)))
    assert np.allclose(weights, affinity / affinity.sum(), rtol=1e-6)
    assert abs(float(weights.sum()) - 1.0) < 1e-6


def test_router_jobs(oracle):
    from anemone_b200.records import ExpertJob
    rows, picks, experts_n, shared = 11, 2, 6, 1
    experts = np.array([[0, 3]] * 9 + [[1, 3], [3, 5]], dtype=np.uint32)
    weights = np.full((rows, picks), 0.5, dtype=np.float32)
    table = np.arange(3 * (experts_n + shared), dtype=np.uint64) * 64
    jobs = (ExpertJob * 16)()
    count = oracle.orc_router_jobs(ptr(experts, u32p), ptr(weights, f32p), rows, picks, experts_n, shared,
                                   ptr(table, u64p), 16, C.byref(jobs))
    # expert 0: 9 rows -> 8 + 1; expert 1: 1; expert 3: 11 rows -> 8 + 3; expert 5: 1; shared: 11 rows -> 8 + 3
    assert count == 8
    assert [(j.expert, j.row_count) for j in jobs[:count]] == [(0, 8), (0, 1), (1, 1), (3, 8), (3, 3), (5, 1),
                                                               (6, 8), (6, 3)]
    assert jobs[3].pair_index[0] == 0 * 3 + 1 and jobs[2].pair_index[0] == 9 * 3 + 0
    assert jobs[6].pair_index[1] == 1 * 3 + 2 and jobs[6].route_weight[1] == 1.0
    assert jobs[0].gate_offset == 0 and jobs[3].down_offset == (3 * 3 + 2) * 64
    assert jobs[count].row_count == 0 and jobs[count].gate_offset == 0
