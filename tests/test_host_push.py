"""The push and exchange preparers without a GPU: the refusals of the reference's own host test
(tests/ordered_push_test.c:78-201), the launches written, and, where the reference's host code was compiled
(oracle/_ref), the same verdict as its preparers on every malformed record."""
import ctypes as C

import pytest

from anemone_b200 import api
from anemone_b200 import records as R
from tests.test_host_preparers import FakeBackend

RANKS, ELEMENTS = 5, 5120
TABLE, REGION, INPUT = 128, 512, 1280
ARRAY = ELEMENTS * 4
OUTPUT, INBOX = INPUT + ARRAY, INPUT + 2 * ARRAY
STRIDE = INBOX + RANKS * ARRAY
ARENA = REGION + 2 * STRIDE
HANDLE, NO_KERNEL = 17, 0xFFFFFFFF
OK, INVALID, UNSUPPORTED = 0, 1, 7
library = api.library


def description(**changes):
    arguments = R.OrderedPush(TABLE, REGION, INPUT, OUTPUT, INBOX, 0, STRIDE, 1_000_000, ARRAY, ELEMENTS, RANKS, 0, 0,
                              0, 0)
    value = R.OrderedPushDescription(arguments, ARENA)
    for name, change in changes.items():
        if name == "arena_byte_count":
            value.arena_byte_count = change
        else:
            setattr(value.arguments, name, change)
    return value


# the malformed records of tests/ordered_push_test.c:103-190
FAULTS = {
    "zero ranks": dict(rank_count=0),
    "excess ranks": dict(rank_count=17),
    "excess rank": dict(rank=RANKS),
    "zero elements": dict(element_count=0),
    "excess elements": dict(element_count=262144 + 1),
    "bad format": dict(payload_format=2),
    "reserved": dict(reserved_zero=1),
    "zero deadline": dict(deadline_cycles=0),
    "host self": dict(incoming_host_mask=1),
    "host excess": dict(incoming_host_mask=1 << RANKS),
    "region alignment": dict(region_offset=REGION + 1),
    "stride overflow": dict(parity_stride=2 ** 64 - 1),
    "table alignment": dict(peer_table_offset=TABLE + 1),
    "step alignment": dict(step_offset=1),
    "inbox overflow": dict(inbox_rank_stride=2 ** 64 - 1),
    "zero inbox": dict(inbox_rank_stride=0),
    "signal overlap": dict(input_offset=0),
    "array overlap": dict(output_offset=INPUT),
    "inbox range": dict(inbox_offset=2 ** 64 - 3),
    "capacity": dict(arena_byte_count=ARENA - 1),
}


def prototypes(lib):
    lib.ordered_push_prepare.argtypes = [C.POINTER(R.OrderedPushDescription), C.c_uint32, C.POINTER(R.KernelLaunch)]
    lib.tp_exchange_prepare.argtypes = [C.POINTER(R.OrderedPushDescription), C.c_uint32, C.c_uint32, C.c_uint32,
                                        C.POINTER(R.KernelLaunch)]
    lib.tp_exchange_wide_prepare.argtypes = [C.POINTER(R.OrderedPushDescription), C.c_uint32, C.c_uint32,
                                             C.POINTER(C.c_uint32), C.c_uint32, C.POINTER(R.KernelLaunch)]
    return lib


def poisoned(count=1):
    launches = (R.KernelLaunch * count)()
    C.memset(launches, 0xA5, C.sizeof(launches))
    return launches


def test_push_prepare_launch_and_refusals():
    lib = prototypes(library())
    for payload in (0, 1):
        value, launch = description(payload_format=payload), R.KernelLaunch()
        assert lib.ordered_push_prepare(C.byref(value), HANDLE, C.byref(launch)) == OK
        assert launch.kernel == HANDLE and launch.argument_byte_count == 96 and tuple(launch.block) == (256, 1, 1)
        # 5120 elements: 1281 vectors, two CTAs of up to 1024 vectors, a group each
        assert tuple(launch.grid) == (2, 1, 1)
        assert bytes(launch.argument)[:96] == bytes(value.arguments)
    big, launch = description(), R.KernelLaunch()
    big.arguments.element_count = 262144
    big.arguments.inbox_rank_stride = 4 * 262144
    big.arguments.output_offset = INPUT + 4 * 262144
    big.arguments.inbox_offset = INPUT + 8 * 262144
    big.arguments.parity_stride = INPUT + (2 + RANKS) * 4 * 262144
    big.arena_byte_count = REGION + 2 * big.arguments.parity_stride
    assert lib.ordered_push_prepare(C.byref(big), HANDLE, C.byref(launch)) == OK
    assert tuple(launch.grid) == (8, 9, 1)  # 65537 vectors: 65 CTAs asked, eight groups of nine
    launches = poisoned()
    before = bytes(launches)
    assert lib.ordered_push_prepare(C.byref(description()), NO_KERNEL, launches) == INVALID
    assert bytes(launches) == before
    for name, change in FAULTS.items():
        assert lib.ordered_push_prepare(C.byref(description(**change)), HANDLE, launches) == INVALID, name
        assert bytes(launches) == before, name
    for overlap in range(16):  # the peer table over the step block
        assert lib.ordered_push_prepare(C.byref(description(peer_table_offset=overlap)), HANDLE, launches) == INVALID
    # well formed, but a host mirror: the reference's PCIe route, not offered
    assert lib.ordered_push_prepare(C.byref(description(incoming_host_mask=2)), HANDLE, launches) == UNSUPPORTED
    assert bytes(launches) == before


def test_exchange_prepare_launches_and_refusals():
    lib = prototypes(library())
    launch = R.KernelLaunch()
    value = description()  # 5120 elements: one row of the reference's width
    assert lib.tp_exchange_prepare(C.byref(value), 3, 40, HANDLE, C.byref(launch)) == OK
    record = R.TpExchange.from_buffer_copy(bytes(launch.argument)[:112])
    assert launch.argument_byte_count == 112 and bytes(record.collective) == bytes(value.arguments)
    assert (record.layer, record.layer_count, record.row_width, record.reserved_zero) == (3, 40, 5120, 0)
    launches = poisoned(4)
    before = bytes(launches)
    for layer, layers in ((0, 0), (40, 40), (0, 1025)):
        assert lib.tp_exchange_prepare(C.byref(value), layer, layers, HANDLE, launches) == INVALID
    assert lib.tp_exchange_prepare(C.byref(description(element_count=5119)), 0, 1, HANDLE, launches) == INVALID
    for name, change in FAULTS.items():
        if name in ("zero elements", "excess elements"):
            continue  # the exchange's own row rule and limit
        assert lib.tp_exchange_prepare(C.byref(description(**change)), 0, 1, HANDLE, launches) == INVALID, name
    assert bytes(launches) == before
    kernels = (C.c_uint32 * 4)(21, 22, 23, 24)
    lib.tp_exchange_wide_rows_prepare.argtypes = [C.POINTER(R.OrderedPushDescription), C.c_uint32, C.c_uint32,
                                                  C.c_uint32, C.POINTER(C.c_uint32), C.c_uint32,
                                                  C.POINTER(R.KernelLaunch)]
    for form in (0, 1):
        four = (R.KernelLaunch * 4)()
        assert lib.tp_exchange_wide_rows_prepare(C.byref(value), 1024, 2, 8, kernels, form, four) == OK
        assert [entry.kernel for entry in four] == [21, 22, 23, 24]
        assert tuple(four[0].grid) == (2, 1, 1) and tuple(four[0].block) == (256, 1, 1)
        assert all(tuple(entry.grid) == (1, 1, 1) and tuple(entry.block) == (32, 1, 1) for entry in four[1:])
        assert R.TpExchange.from_buffer_copy(bytes(four[0].argument)[:112]).row_width == 1024
    # the owner sums: 16-byte offsets and strides, no host route
    assert lib.tp_exchange_wide_prepare(C.byref(description(input_offset=INPUT + 4, output_offset=OUTPUT + 4)), 0, 1,
                                        kernels, 1, launches) == INVALID
    assert lib.tp_exchange_wide_prepare(C.byref(description(incoming_host_mask=2)), 0, 1, kernels, 1,
                                        launches) == INVALID
    # the forms this library does not run: the ring wants four ranks and the bfloat16 wire first
    assert lib.tp_exchange_wide_prepare(C.byref(value), 0, 1, kernels, 2, launches) == INVALID
    ring = description(rank_count=4, payload_format=1)
    assert lib.tp_exchange_wide_prepare(C.byref(ring), 0, 1, kernels, 2, launches) == UNSUPPORTED
    assert lib.tp_exchange_wide_prepare(C.byref(value), 0, 1, kernels, 5, launches) == INVALID
    assert bytes(launches) == before


def test_kernel_names_asked_for():
    lib = library()
    fake = FakeBackend()
    kernel = C.c_uint32(0)
    for function, expected in ((lib.ordered_push_kernel_prepare, ("kernel_ordered_push", "ordered_push", 96)),
                               (lib.tp_exchange_kernel_prepare, ("kernel_tp_exchange", "tp_exchange", 112))):
        function.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_uint32)]
        assert function(C.byref(fake.table), fake.card, C.byref(kernel)) == OK
        assert fake.asked[-1] == expected
    lib.tp_exchange_wide_kernels_prepare.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.POINTER(C.c_uint32)]
    four = (C.c_uint32 * 4)()
    assert lib.tp_exchange_wide_kernels_prepare(C.byref(fake.table), fake.card, 1, four) == OK
    assert [name for _, name, _ in fake.asked[-2:]] == ["tp_exchange_owner", "tp_exchange_settled"]
    assert four[1] == four[2] == four[3] != four[0]  # the fake hands one handle to one name
    assert lib.tp_exchange_wide_kernels_prepare(C.byref(fake.table), fake.card, 3, four) == UNSUPPORTED
    assert lib.tp_exchange_wide_kernels_prepare(C.byref(fake.table), fake.card, 5, four) == INVALID


def test_verdicts_equal_reference(reference):
    """Every record above: accepted or refused as the reference's own preparers decide (its record bytes in the
    launch, too); the grids are this library's."""
    lib = prototypes(library())
    reference = prototypes(reference)
    cases = [dict()] + list(FAULTS.values()) + [dict(peer_table_offset=o) for o in range(16)] + \
        [dict(payload_format=1), dict(payload_format=1, inbox_rank_stride=ARRAY // 2),
         dict(payload_format=1, inbox_rank_stride=ARRAY // 2 - 4), dict(inbox_rank_stride=ARRAY + 2)]
    for change in cases:
        ours, theirs = R.KernelLaunch(), R.KernelLaunch()
        a = lib.ordered_push_prepare(C.byref(description(**change)), HANDLE, C.byref(ours))
        b = reference.ordered_push_prepare(C.byref(description(**change)), HANDLE, C.byref(theirs))
        assert a == b, change
        if a == OK:
            assert bytes(ours.argument) == bytes(theirs.argument) and ours.argument_byte_count == theirs.argument_byte_count
        for layer, layers in ((0, 1), (7, 8), (8, 8), (0, 0)):
            a = lib.tp_exchange_prepare(C.byref(description(**change)), layer, layers, HANDLE, C.byref(ours))
            b = reference.tp_exchange_prepare(C.byref(description(**change)), layer, layers, HANDLE, C.byref(theirs))
            assert a == b, (change, layer, layers)
            if a == OK:  # the reference keeps 8 reserved bytes where this library writes the row width
                assert bytes(ours.argument)[:104] == bytes(theirs.argument)[:104]
    kernels = (C.c_uint32 * 4)(21, 22, 23, 24)
    for change in cases:
        for form in (0, 1):
            ours, theirs = (R.KernelLaunch * 4)(), (R.KernelLaunch * 4)()
            a = lib.tp_exchange_wide_prepare(C.byref(description(**change)), 1, 4, kernels, form, ours)
            b = reference.tp_exchange_wide_prepare(C.byref(description(**change)), 1, 4, kernels, form, theirs)
            assert a == b, (change, form)


class RouteDescription(C.Structure):
    _fields_ = [("cards", C.c_void_p), ("direct_reader_masks", C.POINTER(C.c_uint32)), ("rank_count", C.c_uint32),
                ("element_count", C.c_uint32), ("operation", C.c_int), ("common_numa_root", C.c_bool),
                ("paired_scatter_gather", C.c_bool)]


def test_push_routes(reference):
    """tests/ordered_push_test.c:203-233: a source without write access to an owner would need the owner's host
    mirror; every qualified writer is direct. The same masks as the reference's planner."""
    cards = (R.CardDescription * RANKS)()
    everyone = (1 << RANKS) - 1
    for qualified in ([1 << rank for rank in range(RANKS)], [everyone] * RANKS, [everyone & ~2 | 1 << r for r in range(RANKS)]):
        masks = (C.c_uint32 * RANKS)(*qualified)
        value = RouteDescription(C.cast(cards, C.c_void_p), masks, RANKS, ELEMENTS, 0, False, False)
        results = []
        for lib in (api.library(), reference):
            lib.ordered_push_routes_prepare.argtypes = [C.POINTER(RouteDescription), C.POINTER(C.c_uint32)]
            host = (C.c_uint32 * RANKS)()
            assert lib.ordered_push_routes_prepare(C.byref(value), host) == OK
            results.append(list(host))
        assert results[0] == results[1] == [everyone & ~mask for mask in qualified]
    for operation, paired in ((1, False), (0, True)):  # all-reduce only
        value = RouteDescription(C.cast(cards, C.c_void_p), masks, RANKS, ELEMENTS, operation, False, paired)
        for lib in (api.library(), reference):
            assert lib.ordered_push_routes_prepare(C.byref(value), (C.c_uint32 * RANKS)()) == INVALID
