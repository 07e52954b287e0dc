"""Graphs with side runs and copy launches on a card (the reference's fork/join launch branches and BACKEND_COPY
nodes, source/backend_cuda_launch.c:486-632): the data that flows through copies on side runs into a kernel behind the
join, the same table run eagerly, and the refusals."""
import ctypes as C

import numpy as np
import pytest

from anemone_b200 import records as R

pytestmark = pytest.mark.gpu
WIDTH, SLOTS = 4096, 4


@pytest.fixture(scope="module")
def api():
    from anemone_b200 import api as module
    assert module.card_count() >= 1, "no CUDA device: the CUDA path cannot run and there is no fallback"
    return module


def row_sum_launch(api, card, pairs_offset, output_offset, arena_bytes, branch):
    record, launch = R.ExpertRowSum(pairs_offset, output_offset, WIDTH, SLOTS), R.KernelLaunch()
    api.check(api.library().bb_exl3_row_sum_prepare(C.byref(record), 1, arena_bytes, card.ops_pointer, card.handle,
                                                    C.byref(launch)), "bb_exl3_row_sum_prepare")
    launch.branch = branch
    return launch


def test_side_runs_and_copies(api):
    layout = api.Layout()
    row = WIDTH * 4
    sources = [layout.take(row) for _ in range(4)]
    pairs, other_pairs = layout.take(SLOTS * row), layout.take(SLOTS * row)
    output, other_output = layout.take(row), layout.take(row)
    arena_bytes = layout.take(0, 4096) + 4096
    card = api.Card(0, arena_bytes)
    try:
        rng = np.random.default_rng(12)
        values = [rng.normal(0, 1, WIDTH).astype(np.float32) for _ in range(4)]
        others = rng.normal(0, 1, (SLOTS, WIDTH)).astype(np.float32)
        table = [
            R.copy_launch(sources[0], pairs, row),                                  # 0 the main run
            R.copy_launch(sources[1], pairs + row, row, R.LAUNCH_SIDE),            # 1 a side run of two: behind 0
            R.copy_launch(pairs + row, pairs + 2 * row, row, R.LAUNCH_SIDE),       # 2 behind 1
            R.copy_launch(sources[3], pairs + 3 * row, row, R.LAUNCH_SIDE_MORE),   # 3 another side run: behind 0
            row_sum_launch(api, card, other_pairs, other_output, arena_bytes, R.LAUNCH_RESUME),  # 4 behind 0
            row_sum_launch(api, card, pairs, output, arena_bytes, R.LAUNCH_JOIN),  # 5 behind 2, 3 and 4
        ]
        want = np.zeros(WIDTH, dtype=np.float32)
        for term in (values[0], values[1], values[1], values[3]):
            want = want + term
        other_want = np.zeros(WIDTH, dtype=np.float32)
        for term in others:
            other_want = other_want + term
        graph = card.graph(table)
        for form in ("graph", "graph", "eager"):
            card.fill(0, 0, arena_bytes)
            for offset, value in zip(sources, values):
                card.upload(offset, value)
            card.upload(other_pairs, others)
            before = card.launch_count()
            if form == "graph":
                card.graph_run(graph)
            else:
                card.run(table)
            card.wait()
            assert card.launch_count() - before == 2  # the kernels; copies are no kernels
            assert np.array_equal(card.download(output, row, np.float32).view(np.uint32), want.view(np.uint32))
            assert np.array_equal(card.download(other_output, row, np.float32).view(np.uint32),
                                  other_want.view(np.uint32))
        # refusals: a table outside the grammar, a copy beyond the arena, a word nobody connected, an empty copy
        bad = list(table)
        bad[3] = R.copy_launch(sources[3], pairs + 3 * row, row, R.LAUNCH_RESUME)
        bad[4] = row_sum_launch(api, card, other_pairs, other_output, arena_bytes, R.LAUNCH_SIDE_MORE)
        graph_out = C.c_uint32(77)
        for broken in (bad, [R.copy_launch(sources[0], arena_bytes - 8, row)],
                       [R.copy_launch(sources[0], pairs, row, source_word=64)], [R.copy_launch(sources[0], pairs, 0)]):
            array = (R.KernelLaunch * len(broken))(*broken)
            assert card.ops.graph_capture(card.handle, array, len(array), C.byref(graph_out)) == R.STATUS_INVALID_ARGUMENT
            assert graph_out.value == 77
        for broken in ([R.copy_launch(sources[0], arena_bytes - 8, row)], [R.copy_launch(sources[0], pairs, 0)]):
            array = (R.KernelLaunch * len(broken))(*broken)
            assert card.ops.launch_run(card.handle, array, len(array)) == R.STATUS_INVALID_ARGUMENT
        # a copy through an address word: the card's own arena behind a word peer_connect wrote
        word = sources[2]
        card.peer_connect(card, pairs, word)
        card.upload(sources[0], values[2])
        card.run([R.copy_launch(sources[0], 2 * row, row, destination_word=word)])
        card.wait()
        assert np.array_equal(card.download(pairs + 2 * row, row, np.float32), values[2])
        beyond = (R.KernelLaunch * 1)(R.copy_launch(sources[0], arena_bytes - pairs - 8, row, destination_word=word))
        assert card.ops.launch_run(card.handle, beyond, 1) == R.STATUS_INVALID_ARGUMENT
    finally:
        card.close()
