"""The whole layer call (router -> fused EXL3 experts -> ordered reduction -> bfloat16) on a CUDA device against the
CPU oracle, through the library's own public path: host arrays in, host array out."""
import ctypes as C

import numpy as np
import pytest

from anemone_b200 import records as R
from anemone_b200 import synthetic
from anemone_b200.moe import MoeConfig, MoeLayer, MoeLayout, local_matrices
from oracle import moe_reference

pytestmark = pytest.mark.gpu

MAX_ABS, COSINE = 2e-2, 0.9999  # the path's stated tolerance for layer outputs in bfloat16


@pytest.fixture(scope="module")
def api():
    from anemone_b200 import api as module
    assert module.card_count() >= 1, "no CUDA device: the CUDA path cannot run and there is no fallback"
    return module


def make_layer_inputs(seed, config, rows):
    rng = np.random.default_rng(seed)
    widths = np.concatenate([synthetic.expert_widths(rng, config.experts), [3] * config.shared]).astype(np.uint32)
    matrices = [(synthetic.exl3_matrix(rng, config.hidden, config.inner, int(w)),
                 synthetic.exl3_matrix(rng, config.hidden, config.inner, int(w)),
                 synthetic.exl3_matrix(rng, config.inner, config.hidden, int(w))) for w in widths]
    tokens = synthetic.tokens(rng, rows, config.hidden)
    scores = rng.normal(0, 1, size=(rows, config.experts)).astype(np.float32)
    return widths, matrices, tokens, scores


def cosine(a, b):
    a, b = a.astype(np.float64).reshape(-1), b.astype(np.float64).reshape(-1)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-300))


@pytest.mark.parametrize("form", ["push", "pull"])
@pytest.mark.parametrize("rows", [1, 4, 8, 32])
def test_layer_single_rank(api, oracle, rows, form):
    config = MoeConfig(hidden=512, inner=256, experts=32, shared=1, picks=4, row_capacity=rows)
    widths, matrices, tokens, scores = make_layer_inputs(10 + rows, config, rows)
    expected, _, experts, weights = moe_reference.layer(oracle, config, widths, matrices, tokens, scores, 1)
    layout = MoeLayout(config, widths, 1, 0, reduce_form=form)
    card = api.Card(0, layout.arena_bytes)
    try:
        layer = MoeLayer(card, config, widths, matrices, reduce_form=form)
        layer.connect_local([layer])
        for repeat in range(3):  # both parity slots and a reuse
            got = layer.step(tokens, scores)
            picks = card.download(layer.layout.picks, rows * config.picks * 4, np.uint32).reshape(rows, config.picks)
            assert np.array_equal(picks, experts)  # router indices: bit-exact
            a, b = synthetic.from_bfloat16(got), synthetic.from_bfloat16(expected)
            assert np.isfinite(a).all()
            assert np.abs(a - b).max() <= MAX_ABS and cosine(a, b) >= COSINE
        # the reduction is bit-exact given the rank's own FP32 rows: re-round what the rank published
        slot = layer.layout.region + (layer.sequence & 1) * layer.layout.parity_stride + layer.layout.slot_input
        published = card.download(slot, rows * config.hidden * 4, np.float32)
        assert np.array_equal(synthetic.to_bfloat16(np.float32(0.0) + published), got.reshape(-1))
    finally:
        card.close()


def test_router_job_table_matches_oracle(api, oracle):
    config = MoeConfig(hidden=512, inner=256, experts=256, shared=1, picks=8, row_capacity=32)
    rows = 29
    widths, matrices, tokens, scores = make_layer_inputs(5, MoeConfig(hidden=128, inner=128, experts=1, shared=0), 1)
    rng = np.random.default_rng(8)
    scores = rng.normal(0, 1, size=(rows, config.experts)).astype(np.float32)
    scores[3, 10] = scores[3, 200] = 9.0  # a tie: the lower expert first
    scores[5, 77] = np.float32("nan")  # above every number
    widths = np.full(config.total_experts, 2, dtype=np.uint32)
    tiny = [tuple(np.zeros(synthetic.matrix_bytes(i, o, 2), dtype=np.uint8) for i, o in
                  ((512, 256), (512, 256), (256, 512)))] * config.total_experts
    layout = MoeLayout(config, widths, 1, 0)
    card = api.Card(0, layout.arena_bytes)
    try:
        layer = MoeLayer(card, config, widths, tiny)
        layer.connect_local([layer])
        tokens = np.zeros((rows, config.hidden), dtype=np.uint16)
        layer.step(tokens, scores)
        L = layer.layout
        picks = card.download(L.picks, rows * config.picks * 4, np.uint32).reshape(rows, config.picks)
        weights = card.download(L.weights, rows * config.picks * 4, np.float32).reshape(rows, config.picks)
        jobs_bytes = card.download(L.jobs, L.job_capacity * 96)
        table = card.download(L.expert_table, config.total_experts * 24, np.uint64)
    finally:
        card.close()
    experts, want_weights = moe_reference.route(oracle, config, scores)
    assert np.array_equal(picks[:rows], experts)
    assert 10 in picks[3] and 200 in picks[3] and 77 in picks[5]
    assert np.allclose(weights[:rows], want_weights, rtol=2e-6, atol=0, equal_nan=True)
    from oracle.binding import f32p, ptr, u32p, u64p
    want_jobs = (R.ExpertJob * L.job_capacity)()
    count = oracle.orc_router_jobs(ptr(experts, u32p), ptr(want_weights, f32p), rows, config.picks, config.experts,
                                   config.shared, ptr(table, u64p), L.job_capacity, C.byref(want_jobs))
    got_jobs = (R.ExpertJob * L.job_capacity).from_buffer_copy(jobs_bytes.tobytes())
    for index in range(L.job_capacity):
        g, w = got_jobs[index], want_jobs[index]
        assert (g.gate_offset, g.up_offset, g.down_offset, g.row_count, g.expert) == \
               (w.gate_offset, w.up_offset, w.down_offset, w.row_count, w.expert), index
        assert list(g.pair_index) == list(w.pair_index)
        assert np.allclose(list(g.route_weight), list(w.route_weight), rtol=2e-6, atol=0, equal_nan=True)
    assert count > rows
