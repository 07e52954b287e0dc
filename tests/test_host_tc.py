"""The reference's default entry points of the routed experts (exl3_tc_prepare and its forms, exl3_tcp_prepare and its
forms) and the measured route table, on the host: records and workspace sizes equal to the reference's headers, and the
same verdict as the reference's own preparers (source/exl3_tc.c, source/ordered_routes_measured.c, compiled unchanged
into oracle/_ref) on a sweep of good and malformed records, with a fake backend that only hands out kernel handles."""
import ctypes as C

import numpy as np
import pytest

from anemone_b200 import api
from anemone_b200 import records as R
from tests.test_host_preparers import FakeBackend

TC_FORMS = ("exl3_tc_prepare", "exl3_tc_prepare_short", "exl3_tc_prepare_paired")
TCP_FORMS = ("exl3_tcp_prepare", "exl3_tcp_prepare_base", "exl3_tcp_prepare_hybrid")


def bind(lib):
    for name in TC_FORMS:
        getattr(lib, name).argtypes = [C.POINTER(R.Exl3Tc), C.c_uint64, C.POINTER(api.BackendOperations), C.c_void_p,
                                       C.POINTER(R.KernelLaunch)]
    for name in TCP_FORMS:
        getattr(lib, name).argtypes = [C.POINTER(R.Exl3Tcp), C.c_uint64, C.POINTER(api.BackendOperations), C.c_void_p,
                                       C.POINTER(R.KernelLaunch), C.POINTER(C.c_uint32)]
    return lib


def tc_record(lib, rows=8, intermediate=640, bits_x2=6, jobs=None, shared_sum=0):
    layout = api.Layout()
    record = R.Exl3Tc()
    record.row_count, record.intermediate, record.bits_x2 = rows, intermediate, bits_x2
    record.job_capacity = rows * 6 if jobs is None else jobs
    record.activation_limit, record.shared_sum = 10.0, shared_sum
    record.jobs_offset = layout.take(max(record.job_capacity, 1) * 96)
    record.hidden_offset = layout.take(rows * 5120 * 2)
    lib.exl3_tc_workspace_byte_count.restype = C.c_uint64
    lib.exl3_tc_workspace_byte_count.argtypes = [C.c_uint64, C.c_uint64]
    record.workspace_offset = layout.take(lib.exl3_tc_workspace_byte_count(rows * 6, intermediate))
    record.output_offset = layout.take(rows * 5120 * 4)
    record.shared_offset = layout.take(rows * 5120 * 2)
    return record, layout.take(0, 4096) + 4096


def tcp_record(lib, rows=200, intermediate=512, bits_x2=4):
    layout = api.Layout()
    record = R.Exl3Tcp()
    record.row_count, record.intermediate, record.bits_x2, record.activation_limit = rows, intermediate, bits_x2, 7.0
    record.picks_offset = layout.take(rows * 6 * 8)
    record.expert_offsets_offset = layout.take(384 * 24)
    record.hidden_offset = layout.take(rows * 5120 * 2)
    lib.exl3_tcp_workspace_byte_count.restype = C.c_uint64
    lib.exl3_tcp_workspace_byte_count.argtypes = [C.c_uint64, C.c_uint64]
    record.workspace_offset = layout.take(lib.exl3_tcp_workspace_byte_count(rows, intermediate))
    record.output_offset = layout.take(rows * 5120 * 4)
    record.step_offset = layout.take(64 + rows * 64)
    return record, layout.take(0, 4096) + 4096


def test_records_and_workspace_sizes_equal_the_reference_headers(reference):
    lib = bind(api.library())
    for name in ("ref_exl3_tc_workspace_bytes", "ref_exl3_tcp_workspace_bytes"):
        getattr(reference, name).restype = C.c_uint64
        getattr(reference, name).argtypes = [C.c_uint64, C.c_uint64]
    reference.ref_exl3_tc_record_bytes.restype = reference.ref_exl3_tcp_record_bytes.restype = C.c_uint64
    assert reference.ref_exl3_tc_record_bytes() == C.sizeof(R.Exl3Tc) == 72
    assert reference.ref_exl3_tcp_record_bytes() == C.sizeof(R.Exl3Tcp) == 88
    lib.exl3_tc_workspace_byte_count.restype = lib.exl3_tcp_workspace_byte_count.restype = C.c_uint64
    lib.exl3_tc_workspace_byte_count.argtypes = lib.exl3_tcp_workspace_byte_count.argtypes = [C.c_uint64, C.c_uint64]
    for intermediate in (512, 640):
        for pairs in (6, 48, 155, 160, 384, 2688):
            assert lib.exl3_tc_workspace_byte_count(pairs, intermediate) == \
                reference.ref_exl3_tc_workspace_bytes(pairs, intermediate)
        for rows in (1, 64, 65, 100, 1023, 1024, 1025, 2048):
            assert lib.exl3_tcp_workspace_byte_count(rows, intermediate) == \
                reference.ref_exl3_tcp_workspace_bytes(rows, intermediate)


def test_tc_launches():
    lib, fake = bind(api.library()), FakeBackend()
    record, arena = tc_record(lib)
    for name in TC_FORMS:
        launches = (R.KernelLaunch * 5)()
        assert getattr(lib, name)(C.byref(record), arena, C.byref(fake.table), fake.card, launches) == 0
        assert [key[:2] for key in fake.asked] == [("kernel_exl3_tc", kernel) for kernel in
                                                   ("exl3_tc_operands", "exl3_tc_gate_up", "exl3_tc_mark",
                                                    "exl3_tc_down", "exl3_tc_combine")]
        assert all(key[2] == 72 for key in fake.asked)
        assert [tuple(l.grid) for l in launches][0] == (10, 48, 2) and tuple(launches[4].grid) == (10, 8, 1)
        assert launches[3].grid[0] % 40 == 0 and launches[1].grid[0] % 5 == 0
        for index, launch in enumerate(launches):
            sent = R.Exl3Tc.from_buffer_copy(bytes(launch.argument[:72]))
            assert sent.pass_ == (1 if index == 3 else 0) and sent.workspace_offset == record.workspace_offset
            assert not any(launch.argument[72:])


def test_tcp_launches():
    lib, fake = bind(api.library()), FakeBackend()
    record, arena = tcp_record(lib)
    for name in TCP_FORMS:
        launches = (R.KernelLaunch * 11)()
        count = C.c_uint32(99)
        assert getattr(lib, name)(C.byref(record), arena, C.byref(fake.table), fake.card, launches, C.byref(count)) == 0
        assert count.value == 5
        assert [key[1] for key in fake.asked] == ["exl3_tcp_route", "exl3_tcp_operands", "exl3_tcp_gate_up",
                                                  "exl3_tcp_down", "exl3_tcp_combine"]
        assert tuple(launches[0].grid) == (1, 1, 1) and launches[0].block[0] == 1024
        assert not any(bytes(launches[5]))


def sweep(make, fields):
    """(description, record, arena) for a good record and one changed field at a time."""
    record, arena = make()
    yield "good", record, arena
    for field, value in fields:
        changed, arena = make()
        setattr(changed, field, value)
        yield "%s=%r" % (field, value), changed, arena


def test_tc_verdicts_equal_the_reference(reference):
    lib, fake = bind(api.library()), FakeBackend()
    bind(reference)
    fields = [("row_count", 0), ("row_count", 449), ("row_count", 448), ("intermediate", 576), ("intermediate", 0),
              ("bits_x2", 7), ("bits_x2", 0), ("bits_x2", 4), ("job_capacity", 0), ("job_capacity", 49), ("pass_", 1),
              ("activation_limit", -1.0), ("activation_limit", float("nan")), ("activation_limit", 0.0),
              ("rotation", 6), ("shared_sum", 2), ("shared_sum", 1), ("jobs_offset", 8), ("hidden_offset", 1 << 40),
              ("output_offset", 256), ("workspace_offset", 16)]
    for intermediate in (640, 512):
        for name in TC_FORMS:
            for what, record, arena in sweep(lambda: tc_record(lib, intermediate=intermediate), fields):
                ours, theirs = (R.KernelLaunch * 5)(), (R.KernelLaunch * 5)()
                got = getattr(lib, name)(C.byref(record), arena, C.byref(fake.table), fake.card, ours)
                want = getattr(reference, name)(C.byref(record), arena, C.byref(fake.table), fake.card, theirs)
                assert got == want, (name, intermediate, what, got, want)
                if got != 0:
                    assert not any(bytes(ours))  # a refusal leaves the table unchanged
    # what this library refuses and the reference takes, and the other way round: stated in the header
    record, arena = tc_record(lib)
    record.rotation = 1
    launches = (R.KernelLaunch * 5)()
    assert lib.exl3_tc_prepare(C.byref(record), arena, C.byref(fake.table), fake.card, launches) == R.STATUS_UNSUPPORTED
    record, arena = tc_record(lib, intermediate=512)
    record.rotation = 1  # mixed widths need 640 columns
    assert lib.exl3_tc_prepare(C.byref(record), arena, C.byref(fake.table), fake.card, launches) == \
        reference.exl3_tc_prepare(C.byref(record), arena, C.byref(fake.table), fake.card, launches) == 1
    record, arena = tc_record(lib, bits_x2=8)  # K4: the reference's family has no such kernels, this one has
    assert lib.exl3_tc_prepare(C.byref(record), arena, C.byref(fake.table), fake.card, launches) == 0
    assert reference.exl3_tc_prepare(C.byref(record), arena, C.byref(fake.table), fake.card, launches) == \
        R.STATUS_UNSUPPORTED


def test_tcp_verdicts_equal_the_reference(reference):
    lib, fake = bind(api.library()), FakeBackend()
    bind(reference)
    fields = [("row_count", 0), ("row_count", 2049), ("row_count", 2048), ("row_count", 1), ("intermediate", 576),
              ("bits_x2", 9), ("bits_x2", 6), ("pass_", 2), ("rotation", 6), ("activation_limit", -0.5),
              ("activation_limit", 0.0), ("half_rows", 200), ("part", 1), ("two_blocks", 2), ("two_blocks", 1),
              ("cone_layer", 1000), ("picks_offset", 4), ("output_offset", 0), ("workspace_offset", 1 << 50)]

    def make():
        return tcp_record(lib)
    for name in TCP_FORMS:
        for what, record, arena in sweep(make, fields):
            if what.startswith("row_count=20") or what == "row_count=1":  # the ranges follow the row count
                continue
            ours, theirs = (R.KernelLaunch * 11)(), (R.KernelLaunch * 11)()
            mine, other = C.c_uint32(77), C.c_uint32(77)
            got = getattr(lib, name)(C.byref(record), arena, C.byref(fake.table), fake.card, ours, C.byref(mine))
            want = getattr(reference, name)(C.byref(record), arena, C.byref(fake.table), fake.card, theirs,
                                            C.byref(other))
            assert got == want, (name, what, got, want)
            if got != 0:
                assert not any(bytes(ours)) and mine.value == 77
    for rows in (1, 2048):
        record, arena = tcp_record(lib, rows=rows, intermediate=640)
        ours, count = (R.KernelLaunch * 11)(), C.c_uint32()
        assert lib.exl3_tcp_prepare(C.byref(record), arena, C.byref(fake.table), fake.card, ours, C.byref(count)) == \
            reference.exl3_tcp_prepare(C.byref(record), arena, C.byref(fake.table), fake.card,
                                       (R.KernelLaunch * 11)(), C.byref(C.c_uint32())) == 0
    for field, value in (("rotation", 2), ("half_rows", 50), ("cone_layer", 5)):  # refused here, stated in the header
        record, arena = tcp_record(lib, intermediate=640)
        setattr(record, field, value)
        assert lib.exl3_tcp_prepare(C.byref(record), arena, C.byref(fake.table), fake.card, (R.KernelLaunch * 11)(),
                                    C.byref(C.c_uint32())) == R.STATUS_UNSUPPORTED


class RoutePolicy(C.Structure):
    _fields_ = [("rank_count", C.c_uint32), ("element_count", C.c_uint32), ("operation", C.c_int),
                ("paired_scatter_gather", C.c_bool)] + \
               [(name, C.c_uint32 * 16) for name in ("arithmetic_classes", "link_generations", "link_lane_counts",
                                                     "expected_direct_reader_masks", "host_reader_masks")]


class RouteDescription(C.Structure):
    _fields_ = [("cards", C.POINTER(R.CardDescription)), ("direct_reader_masks", C.POINTER(C.c_uint32)),
                ("rank_count", C.c_uint32), ("element_count", C.c_uint32), ("operation", C.c_int),
                ("common_numa_root", C.c_bool), ("paired_scatter_gather", C.c_bool)]


def test_measured_routes_equal_the_reference(reference):
    lib = api.library()
    rng = np.random.default_rng(9)
    ranks = 4
    cards = (R.CardDescription * ranks)()
    for card in cards:
        card.arithmetic_class, card.link_generation, card.link_lane_count = 100, 5, 18
    full = (1 << ranks) - 1

    def policy(**changes):
        row = RoutePolicy()
        row.rank_count, row.element_count, row.operation = ranks, 4096, 0
        for source in range(ranks):
            row.arithmetic_classes[source], row.link_generations[source], row.link_lane_counts[source] = 100, 5, 18
            row.expected_direct_reader_masks[source] = full & ~(1 << ((source + 1) % ranks))
            row.host_reader_masks[source] = 1 << ((source + 1) % ranks)
        for name, value in changes.items():
            if isinstance(value, tuple):
                getattr(row, name)[value[0]] = value[1]
            else:
                setattr(row, name, value)
        return row
    direct = (C.c_uint32 * ranks)(*[full & ~(1 << ((source + 1) % ranks)) for source in range(ranks)])
    cases = [[], [policy()], [policy(element_count=8192)], [policy(), policy()], [policy(rank_count=0)],
             [policy(rank_count=17)], [policy(element_count=0)], [policy(operation=4)],
             [policy(paired_scatter_gather=True)], [policy(operation=2, paired_scatter_gather=True)],
             [policy(operation=2, paired_scatter_gather=True), policy(operation=3, paired_scatter_gather=True)],
             [policy(operation=2, paired_scatter_gather=True),
              policy(operation=3, paired_scatter_gather=True, link_lane_counts=(1, 4))],
             [policy(expected_direct_reader_masks=(0, full))], [policy(host_reader_masks=(0, 1))],
             [policy(host_reader_masks=(2, 0))], [policy(expected_direct_reader_masks=(1, 0x1D))],
             [policy(arithmetic_classes=(2, 80))], [policy(link_generations=(0, 4))],
             [policy(host_reader_masks=(1, 1 << 5))]]
    for operation, paired in ((0, False), (2, True), (3, True), (1, False)):
        for index, rows in enumerate(cases):
            description = RouteDescription(cards, direct, ranks, 4096, operation, bool(rng.integers(0, 2)), paired)
            table = (RoutePolicy * max(len(rows), 1))(*rows)
            ours = (C.c_uint32 * ranks)(*[0xAAAA] * ranks)
            theirs = (C.c_uint32 * ranks)(*[0xAAAA] * ranks)
            got = lib.ordered_collective_routes_prepare_measured(C.byref(description), table, len(rows), ours)
            want = reference.ordered_collective_routes_prepare_measured(C.byref(description), table, len(rows), theirs)
            assert got == want, (operation, paired, index, got, want)
            assert list(ours) == list(theirs), (operation, paired, index)
    assert lib.ordered_collective_routes_prepare_measured(None, None, 0, None) == 1
    description = RouteDescription(cards, direct, ranks, 4096, 0, False, False)
    assert lib.ordered_collective_routes_prepare_measured(C.byref(description), None, 257, ours) == 1
