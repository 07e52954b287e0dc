"""Expert matrices loaded through an EXL3 virtual pack (storage_exl3, exl3_map_upload) into a card's arena: the chain
on matrices that came through the map leaves the bits it leaves on matrices the host uploaded itself."""
import ctypes as C
import os

import numpy as np
import pytest

from anemone_b200 import records as R
from anemone_b200.exl3_map import BLOCK, MapReader, write_map
from tests.exl3_cases import ChainCase

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    from anemone_b200 import api as module
    assert module.card_count() >= 1, "no CUDA device: the CUDA path cannot run and there is no fallback"
    return module


def chain(api, card, case):
    launches = (R.KernelLaunch * 5)()
    api.check(api.library().exl3_experts_prepare(C.byref(case.record), case.arena_bytes, card.ops_pointer, card.handle,
                                                 100, launches), "exl3_experts_prepare")
    card.run(launches)
    card.wait()
    return card.download(0, case.arena_bytes)


def test_matrices_through_a_map(api, oracle, tmp_path):
    case = ChainCase(oracle, 912, hidden=1024, inner=512, rows=6, picks=2, expert_count=5, widths=[3, 4, 2, 40, 3])
    matrices = sorted((name, span) for name, span in case.ranges.items() if name.startswith("matrix_"))
    # two source files holding the matrices back to back, unaligned; the map puts each on a block of the pack
    sources = [str(tmp_path / "first.bin"), str(tmp_path / "second.bin")]
    segments, cursor, placed = [], [13, 4099], {}
    files = [open(path, "wb") for path in sources]
    for file, lead in zip(files, cursor):
        file.write(bytes(lead))
    logical = BLOCK  # the first block of the pack is a hole
    for index, (name, (offset, size)) in enumerate(matrices):
        which = index % 2
        files[which].write(case.image[offset:offset + size].tobytes())
        segments.append((logical, size, cursor[which], 1 + which))
        placed[name] = logical
        cursor[which] += size
        logical += (size + BLOCK - 1) // BLOCK * BLOCK + (BLOCK if index % 3 == 0 else 0)
    for file in files:
        file.close()
    path = str(tmp_path / "experts.exl3map")
    write_map(path, logical + BLOCK, sources, segments)
    card = api.Card(0, case.arena_bytes)
    try:
        card.upload(0, case.image)
        expected = chain(api, card, case)
        blank = case.image.copy()
        for _, (offset, size) in matrices:
            blank[offset:offset + size] = 0
        card.upload(0, blank)
        reader = MapReader(path)
        try:
            for name, (offset, size) in matrices:
                reader.upload(card, placed[name], size, offset, staging_bytes=64 * BLOCK)
        finally:
            reader.close()
        for _, (offset, size) in matrices:  # the matrices arrived, byte for byte
            assert np.array_equal(card.download(offset, size), case.image[offset:offset + size])
        received = chain(api, card, case)
        assert np.array_equal(received, expected)
        # a range beyond the arena is the backend's refusal, passed on; nothing is left in flight
        reader = MapReader(path)
        try:
            with pytest.raises(api.StatusError):
                reader.upload(card, BLOCK, 8 * BLOCK, case.arena_bytes - BLOCK, staging_bytes=4 * BLOCK)
            card.wait()
        finally:
            reader.close()
    finally:
        card.close()
