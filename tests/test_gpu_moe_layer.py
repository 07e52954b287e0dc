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


@pytest.mark.parametrize("form", ["fused", "push", "pull"])
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


@pytest.mark.parametrize("form", ["fused", "pull"])
def test_router_job_table_matches_oracle(api, oracle, form):
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
    layout = MoeLayout(config, widths, 1, 0, reduce_form=form)
    card = api.Card(0, layout.arena_bytes)
    try:
        layer = MoeLayer(card, config, widths, tiny, reduce_form=form)
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
    finite = ~np.isnan(want_weights)  # the affinity is a fixed FP32 sequence: the card's bits are the host's
    assert np.array_equal(np.isnan(weights[:rows]), ~finite)
    assert np.array_equal(weights[:rows][finite].view(np.uint32), want_weights[finite].view(np.uint32))
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
        got_w, want_w = np.array(list(g.route_weight), np.float32), np.array(list(w.route_weight), np.float32)
        assert np.array_equal(np.isnan(got_w), np.isnan(want_w))
        assert np.array_equal(got_w[~np.isnan(want_w)].view(np.uint32), want_w[~np.isnan(want_w)].view(np.uint32))
    assert count > rows


@pytest.mark.parametrize("form", ["fused", "pull"])
def test_router_at_the_reference_geometry(api, form):
    """384 experts, 6 picks, route scale 1.5, sqrt(softplus) affinities and a selection bias: picks, slot order,
    weights and job table equal the answers of the reference's own router reference (committed fixtures), bit for
    bit: ties, not-a-numbers, infinities, -0 and saturated scores among them."""
    from tests import golden_util
    config = MoeConfig(hidden=512, inner=256, experts=384, shared=0, picks=6, row_capacity=8, scoring=1,
                       route_scale=1.5, bias=True)
    widths = np.full(config.total_experts, 2, dtype=np.uint32)
    tiny = [tuple(np.zeros(synthetic.matrix_bytes(i, o, 2), dtype=np.uint8) for i, o in
                  ((512, 256), (512, 256), (256, 512)))] * config.total_experts
    for case in golden_util.load("reference_vectors.json")["router_select"]:
        scores, bias, table = golden_util.router_case_inputs(case["seed"])
        rows = case["rows"]
        card = api.Card(0, MoeLayout(config, widths, 1, 0, reduce_form=form).arena_bytes)
        try:
            layer = MoeLayer(card, config, widths, tiny, reduce_form=form, bias=bias)
            layer.connect_local([layer])
            L = layer.layout
            card.upload(L.expert_table, table)  # the fixture's offsets: the table is only copied into the jobs
            layer.sequence += 1
            layer.stage_step(0, layer.sequence, np.zeros((rows, config.hidden), dtype=np.uint16), scores)
            card.upload_async(L.step, 0, L.step_input_bytes)
            card.run(layer.launches[:1])  # the routing launch alone: the fixture's offsets name no matrices
            card.wait()
            picks = card.download(L.picks, rows * 6 * 4, np.uint32).reshape(rows, 6)
            weights = card.download(L.weights, rows * 6 * 4, np.uint32).reshape(rows, 6)
            jobs = card.download(L.jobs, rows * 6 * 96).reshape(-1, 96).copy()
        finally:
            card.close()
        assert picks.tolist() == case["experts"]
        want = np.array([[int(v, 16) for v in row] for row in case["weights"]], dtype=np.uint32)
        nan = (want & 0x7FFFFFFF) > 0x7F800000
        assert np.array_equal((weights & 0x7FFFFFFF) > 0x7F800000, nan)
        assert np.array_equal(weights[~nan], want[~nan])
        if not nan.any():
            assert hex(golden_util.fnv64(jobs)) == case["jobs_fnv64"]


def emulated_world(api, config, widths, ranks):
    """Rank 0 of `ranks` real; the other ranks' reduction regions are further ranges of the SAME arena, which the host
    fills before a step (kernels that wait on one another must not share a GPU). Returns the card, rank 0's layout
    and the peers' region offsets."""
    layout = MoeLayout(config, widths, ranks, 0)
    regions = [layout.region]
    cursor = layout.arena_bytes
    for _ in range(1, ranks):
        regions.append(cursor)
        cursor += 2 * layout.parity_stride
    return api.Card(0, cursor + 4096), layout, regions


def emulate_peers(card, layer, regions, sequence, partials):
    """What ranks 1 .. R-1 would have done by now: their FP32 rows in their slots, their READY words in rank 0's
    slot, and their DONE words for the slot's previous use."""
    L, parity = layer.layout, sequence & 1
    for rank in range(1, len(regions)):
        rows = np.ascontiguousarray(partials[rank], dtype=np.float32)
        card.upload(regions[rank] + parity * L.parity_stride + L.slot_input, rows)
        mine = L.region + parity * L.parity_stride
        card.upload(mine + (R.EXL3_LAYER_READY_LINE + rank) * 128, np.array([sequence], dtype=np.uint64))
        card.upload(mine + (R.EXL3_LAYER_DONE_LINE + rank) * 128, np.array([max(sequence - 2, 0)], dtype=np.uint64))


def connect_emulated(card, layer, regions):
    peers = (R.OrderedPeer * len(regions))()
    for rank, region in enumerate(regions):
        peers[rank].region_offset = region
    card.upload(layer.layout.peer_table, np.frombuffer(bytes(peers), dtype=np.uint8))
    layer.connect_local([layer] * len(regions))  # every rank's arena address: this arena
    for region in regions[1:]:
        card.fill(region, 0, 2 * layer.layout.parity_stride)


def full_shape_inputs(oracle, seed, rows, ranks):
    """Configuration 3's shapes: hidden 4096, intermediate 2048, 256 routed experts of widths {2, 3, 4} and one
    always-on expert, top-8 sigmoid routing. Matrices are drawn for the experts that stand in a job; the others
    share one filler per width (they are never read)."""
    config = MoeConfig(hidden=4096, inner=2048, experts=256, shared=1, picks=8, row_capacity=rows)
    rng = np.random.default_rng(seed)
    widths = np.concatenate([synthetic.expert_widths(rng, config.experts), [3]]).astype(np.uint32)
    tokens = synthetic.tokens(rng, rows, config.hidden)
    scores = rng.normal(0, 1, size=(rows, config.experts)).astype(np.float32)
    experts, _ = moe_reference.route(oracle, config, scores)
    active = set(experts.reshape(-1).tolist()) | {config.experts}
    filler = {int(w): (synthetic.exl3_matrix(rng, config.hidden, config.inner, int(w)),
                       synthetic.exl3_matrix(rng, config.hidden, config.inner, int(w)),
                       synthetic.exl3_matrix(rng, config.inner, config.hidden, int(w))) for w in (2, 3, 4)}
    matrices = [(synthetic.exl3_matrix(rng, config.hidden, config.inner, int(widths[e])),
                 synthetic.exl3_matrix(rng, config.hidden, config.inner, int(widths[e])),
                 synthetic.exl3_matrix(rng, config.inner, config.hidden, int(widths[e])))
                if e in active else filler[int(widths[e])] for e in range(config.total_experts)]
    return config, widths, matrices, tokens, scores


@pytest.mark.parametrize("rows", [1, 4, 8, 32])
def test_configuration_3_full_shapes_tp4(api, oracle, rows):
    """The MoE decode layer at the configured shapes on rank 0 of a four-way tensor-parallel group whose other three
    ranks are emulated from the CPU oracle's partial rows: rank 0's own FP32 rows and the layer's bfloat16 output
    within the stated tolerance of the oracle, the rank-ordered reduction bit for bit."""
    from oracle.binding import pointer_array, ptr, u16p
    ranks = 4
    config, widths, matrices, tokens, scores = full_shape_inputs(oracle, 4000 + rows, rows, ranks)
    expected, partials, experts, _ = moe_reference.layer(oracle, config, widths, matrices, tokens, scores, ranks)
    card, layout, regions = emulated_world(api, config, widths, ranks)
    try:
        local = [local_matrices(*matrices[e], config, int(widths[e]), ranks, 0) for e in range(config.total_experts)]
        layer = MoeLayer(card, config, widths, local, rank=0, rank_count=ranks)
        connect_emulated(card, layer, regions)
        for repeat in range(3):  # both parity slots and a reuse
            emulate_peers(card, layer, regions, layer.sequence + 1, partials)
            got = layer.step(tokens, scores)
            picks = card.download(layout.picks, rows * config.picks * 4, np.uint32).reshape(rows, config.picks)
            assert np.array_equal(picks, experts)
            slot = layout.region + (layer.sequence & 1) * layout.parity_stride + layout.slot_input
            mine = card.download(slot, rows * config.hidden * 4, np.float32)
            assert np.abs(mine - partials[0].reshape(-1)).max() <= MAX_ABS and cosine(mine, partials[0]) >= COSINE
            inputs = [mine] + [np.ascontiguousarray(partials[rank].reshape(-1)) for rank in range(1, ranks)]
            want = np.zeros(rows * config.hidden, dtype=np.uint16)
            oracle.orc_ordered_reduce_bf16(pointer_array(inputs), ranks, want.size, ptr(want, u16p))
            assert np.array_equal(got.reshape(-1), want)  # the ordered reduction: bit-exact
            a, b = synthetic.from_bfloat16(got), synthetic.from_bfloat16(expected)
            assert np.abs(a - b).max() <= MAX_ABS and cosine(a, b) >= COSINE
            # every rank was told that rank 0 has read the step
            for rank in range(ranks):
                region = regions[rank] + (layer.sequence & 1) * layout.parity_stride
                assert card.download(region + R.EXL3_LAYER_DONE_LINE * 128, 8, np.uint64)[0] == layer.sequence
                assert card.download(region + R.EXL3_LAYER_READY_LINE * 128, 8, np.uint64)[0] == layer.sequence
    finally:
        card.close()


def test_configuration_3_full_shapes_one_rank(api, oracle):
    rows = 8
    config, widths, matrices, tokens, scores = full_shape_inputs(oracle, 4100, rows, 1)
    expected, _, experts, _ = moe_reference.layer(oracle, config, widths, matrices, tokens, scores, 1)
    card = api.Card(0, MoeLayout(config, widths, 1, 0).arena_bytes)
    try:
        layer = MoeLayer(card, config, widths, matrices)
        layer.connect_local([layer])
        for repeat in range(2):
            got = layer.step(tokens, scores)
            a, b = synthetic.from_bfloat16(got), synthetic.from_bfloat16(expected)
            assert np.abs(a - b).max() <= MAX_ABS and cosine(a, b) >= COSINE
    finally:
        card.close()


def test_fused_step_reports_a_wait_that_runs_out(api, oracle):
    """A peer that never says it is done with a slot, and a peer that never publishes: the bounded waits end, the
    status block says which phase and rank, nothing stale is published, and the card stays usable."""
    ranks, rows = 2, 4
    config = MoeConfig(hidden=512, inner=256, experts=16, shared=1, picks=4, row_capacity=rows,
                       deadline_cycles=2_000_000)  # about a millisecond of device clock
    widths, matrices, tokens, scores = make_layer_inputs(77, config, rows)
    _, partials, _, _ = moe_reference.layer(oracle, config, widths, matrices, tokens, scores, ranks)
    card, layout, regions = emulated_world(api, config, widths, ranks)
    try:
        local = [local_matrices(*matrices[e], config, int(widths[e]), ranks, 0) for e in range(config.total_experts)]
        layer = MoeLayer(card, config, widths, local, rank=0, rank_count=ranks)
        connect_emulated(card, layer, regions)
        # step 1: rank 1 never publishes READY: the reduction's wait runs out
        with pytest.raises(RuntimeError):
            layer.step(tokens, scores)
        status = card.download(layout.status, 16, np.uint32)
        assert status[0] == 1 and status[1] == 0 and status[2] == 1  # timed out, READY phase, rank 1
        card.fill(layout.status, 0, 16)
        # step 2 (the other parity) goes through
        emulate_peers(card, layer, regions, layer.sequence + 1, partials)
        layer.step(tokens, scores)
        # step 3 refills step 1's slot, but rank 1 never said it was done with step 1: the publish gives up, READY
        # is NOT stored into rank 1's slot, and rank 0's own reduction then misses its own READY word
        ready_of_rank0_at_rank1 = regions[1] + (3 & 1) * layout.parity_stride + R.EXL3_LAYER_READY_LINE * 128
        before = card.download(ready_of_rank0_at_rank1, 8, np.uint64)[0]
        mine = layout.region + (3 & 1) * layout.parity_stride
        card.upload(mine + (R.EXL3_LAYER_READY_LINE + 1) * 128, np.array([3], dtype=np.uint64))
        with pytest.raises(RuntimeError):
            layer.step(tokens, scores)
        status = card.download(layout.status, 16, np.uint32)
        assert status[0] == 1 and status[1] == 2 and status[2] == 1  # timed out, DONE phase, rank 1
        assert card.download(ready_of_rank0_at_rank1, 8, np.uint64)[0] == before
        card.fill(layout.status, 0, 16)
        # the card is usable: the next steps (both parities) complete once the peer's words are there
        for _ in range(2):
            emulate_peers(card, layer, regions, layer.sequence + 1, partials)
            card.upload(layout.region + ((layer.sequence + 1) & 1) * layout.parity_stride +
                        (R.EXL3_LAYER_DONE_LINE + 1) * 128, np.array([layer.sequence], dtype=np.uint64))
            layer.step(tokens, scores)
    finally:
        card.close()


@pytest.mark.parametrize("form", ["fused", "pull"])
def test_step_as_one_graph_equals_the_three_calls(api, oracle, form):
    """MoeLayer.step's own graph (the copy in, the chain and the copy out captured together,
    backend_b200_step_capture + backend_b200_graph_run_wait) against backend_b200_step_run on the same steps: the
    same bits, for fewer live rows than the capacity too; a table with a side run is refused as unsupported."""
    config = MoeConfig(hidden=512, inner=256, experts=32, shared=1, picks=4, row_capacity=8)
    widths, matrices, tokens, scores = make_layer_inputs(77, config, 8)
    layout = MoeLayout(config, widths, 1, 0, reduce_form=form)
    card = api.Card(0, layout.arena_bytes)
    try:
        layer = MoeLayer(card, config, widths, matrices, reduce_form=form)
        layer.connect_local([layer])
        results = {}
        for one_graph in (True, False):
            layer.step_graph = None if one_graph else -1
            results[one_graph] = [layer.step(tokens[:rows], scores[:rows]).copy() for rows in (8, 3, 8, 5)]
            assert (layer.step_graph >= 0) == one_graph
        for a, b in zip(results[True], results[False]):
            assert a.shape == b.shape and np.array_equal(a, b) and np.any(a != 0)
        side = [R.KernelLaunch.from_buffer_copy(bytes(layer.launches[index])) for index in (0, 1, 1, 2)]
        side[1].branch, side[2].branch, side[3].branch = R.LAUNCH_SIDE, R.LAUNCH_RESUME, R.LAUNCH_JOIN
        assert card.step_capture(side, layout.step, 0, layout.step_input_bytes, layout.status, 1 << 20, 16) is None
    finally:
        card.close()
