"""The prefill launches (router -> grouping in row tiles -> operands -> tensor-core products -> row sums) on a CUDA
device against the CPU oracle, through the C-ABI preparer: picks bit-exact, FP32 row sums within the path's tolerance,
grouping tables checked for their invariants, and the decode launches on the same rows for consistency."""
import numpy as np
import pytest

from anemone_b200 import records as R
from anemone_b200 import synthetic
from anemone_b200.moe import MoeConfig, MoeLayer, MoeLayout
from anemone_b200.prefill import PrefillLayer, PrefillLayout, Share
from oracle import moe_reference

pytestmark = pytest.mark.gpu

MAX_ABS, COSINE = 2e-2, 0.9999  # the path's stated tolerance for layer outputs


@pytest.fixture(scope="module")
def api():
    from anemone_b200 import api as module
    assert module.card_count() >= 1, "no CUDA device: the CUDA path cannot run and there is no fallback"
    return module


def make_inputs(seed, config, rows, width=None):
    rng = np.random.default_rng(seed)
    if width is None:
        widths = np.concatenate([synthetic.expert_widths(rng, config.experts), [3] * config.shared])
    else:
        widths = np.full(config.total_experts, width)
    widths = widths.astype(np.uint32)
    matrices = [(synthetic.exl3_matrix(rng, config.hidden, config.inner, int(w)),
                 synthetic.exl3_matrix(rng, config.hidden, config.inner, int(w)),
                 synthetic.exl3_matrix(rng, config.inner, config.hidden, int(w))) for w in widths]
    tokens = synthetic.tokens(rng, rows, config.hidden)
    scores = rng.normal(0, 1, size=(rows, config.experts)).astype(np.float32)
    return widths, matrices, tokens, scores


def cosine(a, b):
    a, b = a.astype(np.float64).reshape(-1), b.astype(np.float64).reshape(-1)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-300))


def check_tables(card, layer, config, rows, experts):
    """The grouping the products ran on: every pair once, rows ascending inside an expert, tiles cover the entries."""
    L = layer.layout
    total = config.total_experts
    counts = card.download(L.workspace + L.parts.counts, (total + 1) * 4, np.uint32)
    want = np.bincount(experts.reshape(-1), minlength=total).astype(np.uint32)
    want[config.experts:] = rows
    assert np.array_equal(counts[:total], want)
    assert counts[total] == sum((int(c) + 127) // 128 for c in want)
    tiles = card.download(L.workspace + L.parts.tiles, int(counts[total]) * 16, np.uint32).reshape(-1, 4)
    seen = set()
    at = 0
    for expert in range(total):
        entries = card.download(L.workspace + L.parts.entries + expert * config.row_capacity * 8,
                                max(int(want[expert]), 1) * 8, np.uint32).reshape(-1, 2)[:want[expert]]
        pairs = entries[:, 0].astype(np.int64)
        assert np.all(np.diff(pairs // config.pairs_per_row) > 0)
        for pair in pairs:
            row, slot = divmod(int(pair), config.pairs_per_row)
            assert (experts[row, slot] if slot < config.picks else config.experts + slot - config.picks) == expert
            seen.add(int(pair))
        for first in range(0, int(want[expert]), 128):
            assert list(tiles[at]) == [expert, first, min(128, int(want[expert]) - first), 0]
            at += 1
    assert at == counts[total] and len(seen) == rows * config.pairs_per_row


@pytest.mark.parametrize("rows,capacity", [(1, 1), (37, 64), (300, 300), (129, 512)])
def test_prefill_rows_match_oracle(api, oracle, rows, capacity):
    config = MoeConfig(hidden=512, inner=256, experts=32, shared=1, picks=4, row_capacity=capacity)
    widths, matrices, tokens, scores = make_inputs(100 + rows, config, rows)
    experts, weights = moe_reference.route(oracle, config, scores)
    expected = moe_reference.rank_partial(oracle, config, widths, matrices, tokens, experts, weights, 1, 0)[0]
    layout = PrefillLayout(config, widths)
    card = api.Card(0, layout.arena_bytes)
    try:
        layer = PrefillLayer(card, config, widths, matrices)
        for repeat in range(2):  # the workspace needs no clearing between calls
            got = layer.step(tokens, scores)
            picks = card.download(layer.layout.picks, rows * config.picks * 4, np.uint32).reshape(rows, config.picks)
            assert np.array_equal(picks, experts)  # router indices: bit-exact
            assert np.isfinite(got).all()
            assert np.abs(got - expected).max() <= MAX_ABS and cosine(got, expected) >= COSINE
        # one rank: the reduction's result is the rank's own rows added to +0 and rounded once
        assert np.array_equal(layer.result(rows), synthetic.to_bfloat16(np.float32(0.0) + got))
        check_tables(card, layer, config, rows, experts)
        # fewer live rows than before: stale entries and tiles of the longer call must not be used
        fewer = max(1, rows // 3)
        got = layer.step(tokens[:fewer], scores[:fewer])
        assert np.abs(got - expected[:fewer]).max() <= MAX_ABS and cosine(got, expected[:fewer]) >= COSINE
    finally:
        card.close()


@pytest.mark.parametrize("width", [2, 40, 3, 4])
def test_prefill_every_width(api, oracle, width):
    # three and five groups of 128 outputs: the last product CTA of a row tile has one group, the others two
    config = MoeConfig(hidden=640, inner=384, experts=4, shared=0, picks=2, row_capacity=140)
    rows = 140
    widths, matrices, tokens, scores = make_inputs(width, config, rows, width)
    experts, weights = moe_reference.route(oracle, config, scores)
    expected = moe_reference.rank_partial(oracle, config, widths, matrices, tokens, experts, weights, 1, 0)[0]
    card = api.Card(0, PrefillLayout(config, widths).arena_bytes)
    try:
        got = PrefillLayer(card, config, widths, matrices).step(tokens, scores)
        assert np.abs(got - expected).max() <= MAX_ABS and cosine(got, expected) >= COSINE
    finally:
        card.close()


def test_prefill_agrees_with_decode_launches(api):
    """The same 64 rows through the decode launches and through the prefill launches: same picks, and row sums that
    differ only by the association of the FP32 products."""
    config = MoeConfig(hidden=1024, inner=512, experts=16, shared=1, picks=2, row_capacity=64)
    rows = 64
    widths, matrices, tokens, scores = make_inputs(7, config, rows)
    card = api.Card(0, MoeLayout(config, widths, 1, 0).arena_bytes)
    try:
        decode = MoeLayer(card, config, widths, matrices)
        decode.connect_local([decode])
        decode.step(tokens, scores)
        slot = decode.layout.region + (decode.sequence & 1) * decode.layout.parity_stride + decode.layout.slot_input
        decode_rows = card.download(slot, rows * config.hidden * 4, np.float32).reshape(rows, config.hidden)
        decode_picks = card.download(decode.layout.picks, rows * config.picks * 4, np.uint32)
    finally:
        card.close()
    card = api.Card(0, PrefillLayout(config, widths).arena_bytes)
    try:
        prefill = PrefillLayer(card, config, widths, matrices)
        prefill_rows = prefill.step(tokens, scores)
        prefill_picks = card.download(prefill.layout.picks, rows * config.picks * 4, np.uint32)
    finally:
        card.close()
    assert np.array_equal(decode_picks, prefill_picks)
    scale = np.abs(decode_rows).max()
    assert np.abs(prefill_rows - decode_rows).max() <= 2e-3 * max(scale, 1.0)
    assert cosine(prefill_rows, decode_rows) >= 0.99999


@pytest.mark.parametrize("kind,ranks", [("expert_parallel", 2), ("expert_parallel", 4), ("tensor_parallel", 2)])
def test_prefill_shares_add_up(api, oracle, kind, ranks):
    """Every rank of a group in turn on one card: each holds its share of the experts; the ranks' FP32 rows, added in
    rank order, are the whole layer's rows (the oracle's, which computes all experts in one place)."""
    config = MoeConfig(hidden=512, inner=512, experts=16, shared=1, picks=4, row_capacity=200)
    rows = 200
    widths, matrices, tokens, scores = make_inputs(31, config, rows)
    scores[:, :4] += 2.0  # skewed routing: the first rank of an expert-parallel group gets most pairs
    experts, weights = moe_reference.route(oracle, config, scores)
    expected = moe_reference.rank_partial(oracle, config, widths, matrices, tokens, experts, weights, 1, 0)[0]
    total = np.zeros_like(expected)
    for rank in range(ranks):
        share = getattr(Share, kind)(config, ranks, rank)
        held = share.experts(config)
        local_widths = widths[held]
        local_matrices = [share.matrices(config, e, int(widths[e]), *matrices[e]) for e in held]
        card = api.Card(0, PrefillLayout(config, local_widths, share).arena_bytes)
        try:
            layer = PrefillLayer(card, config, local_widths, local_matrices, share)
            total = total + layer.step(tokens, scores)
            picks = card.download(layer.layout.picks, rows * config.picks * 4, np.uint32).reshape(rows, config.picks)
            assert np.array_equal(picks, experts)
            counts = card.download(layer.layout.workspace, (len(held) + 1) * 4, np.uint32)
            want = [int((experts == e).sum()) if e < config.experts else rows for e in held]
            assert list(counts[:len(held)]) == want
        finally:
            card.close()
    assert np.abs(total - expected).max() <= MAX_ABS and cosine(total, expected) >= COSINE


def test_prefill_preparer_refusals(api):
    config = MoeConfig(hidden=256, inner=128, experts=4, shared=0, picks=2, row_capacity=16)
    widths = np.full(4, 3, dtype=np.uint32)
    layout = PrefillLayout(config, widths)
    card = api.Card(0, layout.arena_bytes)
    try:
        import ctypes as C
        good = R.Exl3Prefill(layout.scores, layout.tokens, layout.expert_table, layout.widths, layout.picks,
                             layout.weights, layout.workspace, layout.pair_outputs, layout.row_output, layout.step,
                             256, 128, 0, 4, 0, 4, 0, 2, 16, 0, 1.0, 10.0)
        launches = (R.KernelLaunch * 7)()
        lib = api.library()

        def status(**changes):
            record = R.Exl3Prefill.from_buffer_copy(bytes(good))
            for name, value in changes.items():
                setattr(record, name, value)
            before = bytes(launches)
            code = lib.exl3_prefill_prepare(C.byref(record), card.arena_bytes, card.ops_pointer, card.handle, launches)
            if code != 0:
                assert bytes(launches) == before  # a refusal leaves the launch table unchanged
            return code

        assert status() == 0
        assert launches[4].grid[0] == 1 and launches[4].block[0] == 576 and launches[5].grid[0] == 1
        assert status(local_first=2, local_count=2) == 0
        for changes in ({"input_size": 192}, {"inner_size": 64}, {"picks": 0}, {"picks": 5}, {"expert_count": 0},
                        {"bias_offset": 8}, {"bias_offset": card.arena_bytes}, {"workspace_offset": layout.workspace + 512},
                        {"row_output_offset": layout.pair_outputs}, {"activation_limit": 0.0},
                        {"row_capacity": 0}, {"scores_offset": card.arena_bytes}, {"local_first": 3},
                        {"local_count": 0}, {"shared_inner_size": 128}, {"shared_count": 1}):
            assert status(**changes) == 1, changes  # STATUS_INVALID_ARGUMENT
    finally:
        card.close()


def test_prefill_intermediate_wider_than_hidden(api, oracle):
    config = MoeConfig(hidden=256, inner=640, experts=6, shared=1, picks=2, row_capacity=200)
    rows = 200
    widths, matrices, tokens, scores = make_inputs(77, config, rows)
    experts, weights = moe_reference.route(oracle, config, scores)
    expected = moe_reference.rank_partial(oracle, config, widths, matrices, tokens, experts, weights, 1, 0)[0]
    card = api.Card(0, PrefillLayout(config, widths).arena_bytes)
    try:
        got = PrefillLayer(card, config, widths, matrices).step(tokens, scores)
        assert np.abs(got - expected).max() <= MAX_ABS and cosine(got, expected) >= COSINE
    finally:
        card.close()


def test_prefill_full_size_properties(api):
    """The benchmark's shapes (256 + 1 experts, hidden 4096, intermediate 2048, top-8, 4096 rows), where the oracle is
    too slow: size-independent properties instead. (1) A row's result does not depend on which other rows are in the
    call or where it stands in its row tile: permuting the rows permutes the results bit for bit. (2) The first eight
    rows through the decode launches agree with the same rows of the prefill call within the association of the FP32
    products. (3) Every pair is grouped exactly once."""
    config = MoeConfig(hidden=4096, inner=2048, experts=256, shared=1, picks=8, row_capacity=4096)
    rows = 4096
    rng = np.random.default_rng(2026)
    widths = np.concatenate([synthetic.expert_widths(rng, config.experts), [3]]).astype(np.uint32)
    matrices = [(synthetic.exl3_matrix(rng, config.hidden, config.inner, int(w)),
                 synthetic.exl3_matrix(rng, config.hidden, config.inner, int(w)),
                 synthetic.exl3_matrix(rng, config.inner, config.hidden, int(w))) for w in widths]
    tokens = synthetic.tokens(rng, rows, config.hidden)
    popularity = 1.0 / np.arange(1, config.experts + 1) ** 1.1
    scores = (rng.normal(0, 1, size=(rows, config.experts)) +
              np.log(popularity / popularity.mean())[rng.permutation(config.experts)]).astype(np.float32)
    order = rng.permutation(rows)
    card = api.Card(0, PrefillLayout(config, widths).arena_bytes)
    try:
        layer = PrefillLayer(card, config, widths, matrices)
        first = layer.step(tokens, scores)
        picks = card.download(layer.layout.picks, rows * config.picks * 4, np.uint32).reshape(rows, config.picks)
        total = config.total_experts
        counts = card.download(layer.layout.workspace, (total + 1) * 4, np.uint32)
        want = np.bincount(picks.reshape(-1), minlength=total)
        want[config.experts] = rows
        assert np.array_equal(counts[:total], want) and counts[total] == ((want + 127) // 128).sum()
        assert np.all(np.diff(picks.astype(np.int64), axis=1) > 0)  # slots in ascending expert order
        second = layer.step(tokens[order], scores[order])
        assert np.isfinite(first).all() and np.abs(first).max() > 0
        assert np.array_equal(second.view(np.uint32), first[order].view(np.uint32))
    finally:
        card.close()
    small = MoeConfig(hidden=4096, inner=2048, experts=256, shared=1, picks=8, row_capacity=8)
    card = api.Card(0, MoeLayout(small, widths, 1, 0).arena_bytes)
    try:
        decode = MoeLayer(card, small, widths, matrices)
        decode.connect_local([decode])
        decode.step(tokens[:8], scores[:8])
        slot = decode.layout.region + (decode.sequence & 1) * decode.layout.parity_stride + decode.layout.slot_input
        decode_rows = card.download(slot, 8 * config.hidden * 4, np.float32).reshape(8, config.hidden)
    finally:
        card.close()
    scale = max(float(np.abs(decode_rows).max()), 1.0)
    assert np.abs(first[:8] - decode_rows).max() <= 2e-3 * scale and cosine(first[:8], decode_rows) >= 0.99999
    # (4) the CPU oracle on a sample of the call's rows (a row's result does not depend on the others, (1)): the FP32
    # rows of the prefill launches at the configured shapes within the layer's tolerance
    sample = np.array([0, 1, 2, 1000, 2047, 2048, 4000, 4095])
    from oracle import binding
    wanted = moe_reference.layer(binding.load_oracle(), small, widths, matrices, tokens[sample], scores[sample], 1)[1][0]
    wanted = np.asarray(wanted, dtype=np.float32).reshape(len(sample), config.hidden)
    assert np.abs(first[sample] - wanted).max() <= 2e-2 and cosine(first[sample], wanted) >= 0.9999


def test_prefill_empty_and_full_calls(api, oracle):
    """A call with no live row writes nothing and the next call is unaffected; a call at the row capacity, where one
    expert takes every row (its tiles: one pair and none left over), matches the oracle."""
    config = MoeConfig(hidden=256, inner=256, experts=4, shared=0, picks=1, row_capacity=256)
    rows = 256
    widths, matrices, tokens, scores = make_inputs(5, config, rows, 3)
    scores[:, 2] += 100.0  # every row picks expert 2: 256 rows = exactly two full tiles, taken as one pair
    experts, weights = moe_reference.route(oracle, config, scores)
    assert (experts == 2).all()
    expected = moe_reference.rank_partial(oracle, config, widths, matrices, tokens, experts, weights, 1, 0)[0]
    card = api.Card(0, PrefillLayout(config, widths).arena_bytes)
    try:
        layer = PrefillLayer(card, config, widths, matrices)
        first = layer.step(tokens, scores)
        assert np.abs(first - expected).max() <= MAX_ABS and cosine(first, expected) >= COSINE
        counts = card.download(layer.layout.workspace, 5 * 4, np.uint32)
        assert list(counts) == [0, 0, 256, 0, 2]
        before = card.download(layer.layout.row_output, rows * config.hidden * 4)
        layer.load(tokens[:0], scores[:0])
        layer.run()
        assert layer.result(0).shape == (0, config.hidden)
        counts = card.download(layer.layout.workspace, 5 * 4, np.uint32)
        assert list(counts) == [0, 0, 0, 0, 0]
        assert np.array_equal(card.download(layer.layout.row_output, rows * config.hidden * 4), before)
        again = layer.step(tokens[:130], scores[:130])  # two tiles, the second with two rows
        assert np.array_equal(again.view(np.uint32), first[:130].view(np.uint32))
    finally:
        card.close()
