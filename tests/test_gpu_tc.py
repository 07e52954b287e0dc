"""The reference's default entry points of the routed experts (exl3_tc_prepare, exl3_tcp_prepare) on a CUDA device at
the reference model's geometry (hidden 5120, six routes a row, a rank's 640 or 512 intermediate columns, a table of 384
experts), against the CPU oracle's chain on the same arena image, through the C-ABI."""
import ctypes as C

import numpy as np
import pytest

from anemone_b200 import records as R
from anemone_b200 import synthetic
from tests.exl3_cases import ChainCase
from tests.test_host_tc import bind

pytestmark = pytest.mark.gpu

HIDDEN, PICKS = 5120, 6
MAX_ABS, COSINE = 2e-2, 0.9999


@pytest.fixture(scope="module")
def api():
    from anemone_b200 import api as module
    assert module.card_count() >= 1, "no CUDA device: the CUDA path cannot run and there is no fallback"
    return module


def cosine(a, b):
    a, b = a.astype(np.float64).reshape(-1), b.astype(np.float64).reshape(-1)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-300))


def bfloat16_sum(rows, shared_bits):
    """bfloat16(FP32 row + bfloat16 shared row), one rounding (nearest even)."""
    return synthetic.to_bfloat16(rows.astype(np.float32) + synthetic.from_bfloat16(shared_bits))


@pytest.mark.parametrize("intermediate, stored, rows", [(640, 3, 8), (512, 2, 5), (640, 4, 64)])
def test_decode_entry_against_the_oracle(api, oracle, intermediate, stored, rows):
    lib = bind(api.library())
    experts = 24
    case = ChainCase(oracle, 900 + rows, hidden=HIDDEN, inner=intermediate, rows=rows, picks=PICKS,
                     expert_count=experts, widths=[stored] * experts)
    expected = case.run_oracle(False)
    want = case.view(expected, "row_output", np.float32).reshape(rows, HIDDEN)
    lib.exl3_tc_workspace_byte_count.restype = C.c_uint64
    lib.exl3_tc_workspace_byte_count.argtypes = [C.c_uint64, C.c_uint64]
    layout = api.Layout(case.arena_bytes)
    workspace_bytes = lib.exl3_tc_workspace_byte_count(rows * PICKS, intermediate)
    workspace = layout.take(workspace_bytes + 256)
    output, shared = layout.take(rows * HIDDEN * 4 + 256), layout.take(rows * HIDDEN * 2 + 256)
    arena = layout.take(0, 4096) + 4096
    record = R.Exl3Tc(case.record.jobs_offset, case.record.input_offset, workspace, output, rows, rows * PICKS,
                      intermediate, synthetic.bits_x2(stored), 10.0, 0, 0, 0, shared)
    card = api.Card(0, arena)
    try:
        card.upload(0, case.image)
        card.fill(workspace, 0xC3, workspace_bytes + 256)  # scratch starts dirty: the launches clear what they need
        card.fill(output, 0xC3, rows * HIDDEN * 4 + 256)
        launches = (R.KernelLaunch * 5)()
        for entry in (lib.exl3_tc_prepare, lib.exl3_tc_prepare_short, lib.exl3_tc_prepare_paired):
            api.check(entry(C.byref(record), arena, card.ops_pointer, card.handle, launches), "exl3_tc_prepare")
            for repeat in range(2):  # the scratch's counters are left clean for the next call
                card.run(launches)
                card.wait()
                got = card.download(output, rows * HIDDEN * 4, np.float32).reshape(rows, HIDDEN)
                assert np.isfinite(got).all()
                assert np.abs(got - want).max() <= MAX_ABS and cosine(got, want) >= COSINE
        assert (card.download(workspace + workspace_bytes, 256) == 0xC3).all()  # nothing beyond the workspace
        assert (card.download(output + rows * HIDDEN * 4, 256) == 0xC3).all()
        # shared_sum: the row sums added to the always-on expert's bfloat16 rows, one rounding, in place
        rng = np.random.default_rng(1)
        shared_rows = synthetic.to_bfloat16(rng.normal(0, 0.5, size=(rows, HIDDEN)).astype(np.float32))
        card.upload(shared, shared_rows)
        record.shared_sum = 1
        api.check(lib.exl3_tc_prepare(C.byref(record), arena, card.ops_pointer, card.handle, launches), "shared_sum")
        card.run(launches)
        card.wait()
        summed = card.download(shared, rows * HIDDEN * 2, np.uint16).reshape(rows, HIDDEN)
        assert np.array_equal(summed, bfloat16_sum(got, shared_rows))
        assert np.array_equal(card.download(output, rows * HIDDEN * 4, np.float32).reshape(rows, HIDDEN), got)
        # a job table that holds no pair: every row's sum is zero, the shared rows keep their bits
        record.shared_sum = 0
        card.fill(case.record.jobs_offset, 0, case.job_capacity * 96)
        api.check(lib.exl3_tc_prepare(C.byref(record), arena, card.ops_pointer, card.handle, launches), "empty")
        card.run(launches)
        card.wait()
        assert (card.download(output, rows * HIDDEN * 4, np.uint32) == 0).all()
    finally:
        card.close()


def prefill_world(rng, rows, intermediate, stored, experts=24):
    """An arena image for exl3_tcp_prepare: matrices of `experts` experts of a table of 384, picks [rows][6] with
    ascending distinct experts and normalised weights, tokens."""
    layout = __import__("anemone_b200.api", fromlist=["Layout"]).Layout()
    table = np.zeros((384, 3), dtype=np.uint64)
    held = np.sort(rng.choice(384, size=experts, replace=False))
    matrices = []
    for expert in held:
        for which, (inputs, outputs) in enumerate(((HIDDEN, intermediate), (HIDDEN, intermediate),
                                                   (intermediate, HIDDEN))):
            data = synthetic.exl3_matrix(rng, inputs, outputs, stored)
            table[expert, which] = layout.take(data.size, 64)
            matrices.append((int(table[expert, which]), data))
    picks = np.zeros((rows, PICKS), dtype=[("expert", np.uint32), ("weight", np.float32)])
    for row in range(rows):
        picks["expert"][row] = np.sort(rng.choice(held, size=PICKS, replace=False))
        weights = rng.uniform(0.2, 1.0, size=PICKS).astype(np.float32)
        picks["weight"][row] = weights / weights.sum() * np.float32(1.5)
    tokens = synthetic.tokens(rng, rows, HIDDEN)
    return layout, table, matrices, picks, tokens


def oracle_rows(oracle, table, matrices, picks, tokens, sample, intermediate, stored):
    """The CPU oracle's FP32 row sums of the sampled rows (a row's result depends on that row alone)."""
    from anemone_b200.api import Layout
    from oracle.binding import f32p, ptr, u32p, u64p, u8p
    rows = len(sample)
    experts = np.ascontiguousarray(picks["expert"][sample], dtype=np.uint32)
    weights = np.ascontiguousarray(picks["weight"][sample], dtype=np.float32)
    layout = Layout(max(offset + data.size for offset, data in matrices))
    capacity = rows * PICKS
    jobs = (R.ExpertJob * capacity)()
    oracle.orc_router_jobs(ptr(experts, u32p), ptr(weights, f32p), rows, PICKS, 384, 0,
                           ptr(np.ascontiguousarray(table.reshape(-1)), u64p), capacity, C.byref(jobs))
    record = R.Exl3Expert()
    record.jobs_offset = layout.take(capacity * 96)
    record.input_offset = layout.take(rows * HIDDEN * 2)
    pairs = rows * PICKS
    record.operands_offset = layout.take(pairs * HIDDEN * 4)
    record.products_offset = record.output_offset = layout.take(pairs * HIDDEN * 8)
    record.hidden_offset = layout.take(pairs * intermediate * 2)
    row_output = layout.take(rows * HIDDEN * 4)
    record.input_size, record.inner_size, record.pair_count, record.pairs_per_row = HIDDEN, intermediate, pairs, PICKS
    record.job_count, record.bits_per_weight, record.activation_limit = capacity, stored, 7.0
    image = np.zeros(layout.cursor + 64, dtype=np.uint8)
    for offset, data in matrices:
        image[offset:offset + data.size] = data
    image[record.jobs_offset:record.jobs_offset + C.sizeof(jobs)] = np.frombuffer(bytes(jobs), dtype=np.uint8)
    image[record.input_offset:record.input_offset + rows * HIDDEN * 2] = tokens[sample].reshape(-1).view(np.uint8)
    oracle.orc_exl3_experts(C.byref(record), ptr(image, u8p), None, 0)
    row_sum = R.ExpertRowSum(record.output_offset, row_output, HIDDEN, PICKS)
    oracle.orc_exl3_row_sum(C.byref(row_sum), rows, ptr(image, u8p))
    return image[row_output:row_output + rows * HIDDEN * 4].view(np.float32).reshape(rows, HIDDEN).copy()


@pytest.mark.parametrize("intermediate, stored, rows", [(512, 3, 150), (640, 2, 1100)])
def test_prefill_entry_against_the_oracle(api, oracle, intermediate, stored, rows):
    """exl3_tcp_prepare from the router's picks; 1,100 rows run as two chunks in one workspace. The oracle checks a
    sample of rows (first and last of each chunk among them); the whole call is checked against itself run as two
    calls cut at the chunk boundary, bit for bit."""
    lib = bind(api.library())
    rng = np.random.default_rng(70 + rows)
    layout, table, matrices, picks, tokens = prefill_world(rng, rows, intermediate, stored)
    lib.exl3_tcp_workspace_byte_count.restype = C.c_uint64
    lib.exl3_tcp_workspace_byte_count.argtypes = [C.c_uint64, C.c_uint64]
    picks_at, table_at = layout.take(rows * PICKS * 8), layout.take(384 * 24)
    tokens_at = layout.take(rows * HIDDEN * 2)
    workspace_bytes = lib.exl3_tcp_workspace_byte_count(rows, intermediate)
    workspace = layout.take(workspace_bytes + 256)
    output = layout.take(rows * HIDDEN * 4 + 256)
    arena = layout.take(0, 4096) + 4096
    card = api.Card(0, arena)
    try:
        for offset, data in matrices:
            card.upload(offset, data)
        card.upload(picks_at, picks.view(np.uint8).reshape(-1))
        card.upload(table_at, table)
        card.upload(tokens_at, tokens)
        card.fill(workspace, 0xC3, workspace_bytes + 256)
        card.fill(output, 0xC3, rows * HIDDEN * 4 + 256)

        def run(first, count, entry=lib.exl3_tcp_prepare):
            record = R.Exl3Tcp(picks_at + first * PICKS * 8, table_at, tokens_at + first * HIDDEN * 2, workspace,
                               output + first * HIDDEN * 4, count, intermediate, synthetic.bits_x2(stored), 0, 7.0, 0, 0,
                               0, 0, 0, 0)
            launches, launch_count = (R.KernelLaunch * 11)(), C.c_uint32()
            api.check(entry(C.byref(record), arena, card.ops_pointer, card.handle, launches, C.byref(launch_count)),
                      "exl3_tcp_prepare")
            assert launch_count.value == (10 if count > 1024 else 5)
            card.run((R.KernelLaunch * launch_count.value)(*launches[:launch_count.value]))
            card.wait()
            return card.download(output, rows * HIDDEN * 4, np.float32).reshape(rows, HIDDEN)
        got = run(0, rows)
        assert np.isfinite(got).all()
        assert (card.download(workspace + workspace_bytes, 256) == 0xC3).all()
        assert (card.download(output + rows * HIDDEN * 4, 256) == 0xC3).all()
        sample = sorted({0, 1, rows // 3, min(rows, 1024) - 1, min(rows - 1, 1024), rows - 1})
        want = oracle_rows(oracle, table, matrices, picks, tokens, sample, intermediate, stored)
        assert np.abs(got[sample] - want).max() <= MAX_ABS and cosine(got[sample], want) >= COSINE
        assert not card.waits_expired()
        if rows > 1024:  # the same rows as two calls cut where the chunks are cut: the same bits
            card.fill(output, 0, rows * HIDDEN * 4)
            run(0, 1024, lib.exl3_tcp_prepare_base)
            again = run(1024, rows - 1024, lib.exl3_tcp_prepare_hybrid)
            assert np.array_equal(again.view(np.uint32), got.view(np.uint32))
    finally:
        card.close()
