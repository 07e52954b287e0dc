"""The entry point that needs no scratch memory from its caller (exl3_expert_block_noalloc), through the C-ABI,
against the card interface's five-pass chain on the same inputs.

It is for callers that cannot allocate device memory when they call: its scratch is a fixed array inside the library.
This file is named so that pytest collects it last: if it fails, a run that stops at the first failure has already
run every other test. It passes alone in a fresh process and after the other tests.
"""
import ctypes as C

import numpy as np
import pytest

from anemone_b200 import records as R
from tests.exl3_cases import ChainCase

pytestmark = pytest.mark.gpu


def test_no_alloc_entry_matches_the_chain_twice(oracle):
    from anemone_b200 import api
    assert api.card_count() >= 1, "no CUDA device: the CUDA path cannot run and there is no fallback"
    lib = api.library()
    lib.exl3_expert_block_noalloc.argtypes = [C.c_void_p] * 4 + [C.POINTER(C.c_float), C.c_void_p] + \
        [C.c_uint32] * 4 + [C.c_float, C.c_void_p, C.c_uint32]
    # the last two cases fill parts of the fixed scratch exactly: hidden at its limit, and inner == hidden at 8 rows
    for seed, (hidden, inner, rows, stored) in enumerate([(512, 256, 3, 3), (1024, 512, 8, 4), (512, 384, 1, 40),
                                                          (8192, 256, 8, 2), (2048, 2048, 8, 3)]):
        case = ChainCase(oracle, 600 + seed, hidden=hidden, inner=inner, rows=rows, picks=1, expert_count=1,
                         widths=[stored])
        # one job holding every row, with distinct route weights
        job = case.jobs[0]
        job.row_count = rows
        weights = np.linspace(0.25, 1.0, rows).astype(np.float32)
        for row in range(rows):
            job.pair_index[row], job.route_weight[row] = row, float(weights[row])
        for index in range(1, case.job_capacity):
            case.jobs[index].row_count = 0
        offset = case.record.jobs_offset
        case.image[offset:offset + C.sizeof(case.jobs)] = np.frombuffer(bytes(case.jobs), dtype=np.uint8)
        card = api.Card(0, case.arena_bytes + rows * hidden * 4 + 4096)
        try:
            card.upload(0, case.image)
            launches = (R.KernelLaunch * 5)()
            api.check(lib.exl3_experts_prepare(C.byref(case.record), case.arena_bytes, card.ops_pointer, card.handle,
                                               100, launches), "exl3_experts_prepare")
            card.run(launches)
            card.wait()
            expected = card.download(case.record.output_offset, rows * hidden * 4, np.float32)
            assert np.isfinite(expected).all() and np.abs(expected).max() > 0
            # the chain itself against the CPU oracle, within the path's tolerance
            oracle_rows = case.run_oracle(False)[case.record.output_offset:
                                                 case.record.output_offset + rows * hidden * 4].view(np.float32)
            assert np.abs(expected - oracle_rows).max() <= 2e-2
            assert float(expected.astype(np.float64) @ oracle_rows.astype(np.float64) /
                         (np.linalg.norm(expected) * np.linalg.norm(oracle_rows))) >= 0.9999
            base = api.library().backend_b200_arena_address(card.handle)
            gate, up, down = (base + case.ranges["matrix_0_%d" % which][0] for which in range(3))
            tokens = base + case.record.input_offset
            output_offset = api.align(case.arena_bytes, 256)
            for call in range(2):  # two calls in a row share the library's fixed scratch
                card.fill(output_offset, 0xC3, rows * hidden * 4)
                card.wait()
                status = lib.exl3_expert_block_noalloc(gate, up, down, tokens,
                                                       weights.ctypes.data_as(C.POINTER(C.c_float)),
                                                       base + output_offset, rows, hidden, inner, stored, 10.0, None, 1)
                assert status == 0, status
                got = card.download(output_offset, rows * hidden * 4, np.float32)
                # the same device code, the same build flags, the same order of operations: the same bits
                assert np.array_equal(got.view(np.uint32), expected.view(np.uint32))
                assert np.abs(got - oracle_rows).max() <= 2e-2  # and the CPU oracle within the path's tolerance
            # sizes beyond the fixed scratch are refused, and nothing is written
            card.fill(output_offset, 0xC3, rows * hidden * 4)
            card.wait()
            assert lib.exl3_expert_block_noalloc(gate, up, down, tokens, None, base + output_offset, 9, hidden, inner,
                                                 stored, 10.0, None, 1) == R.STATUS_INVALID_ARGUMENT
            assert lib.exl3_expert_block_noalloc(gate, up, down, tokens, None, base + output_offset, rows, 16384,
                                                 inner, stored, 10.0, None, 1) == R.STATUS_INVALID_ARGUMENT
            assert (card.download(output_offset, rows * hidden * 4) == 0xC3).all()
        finally:
            card.close()
