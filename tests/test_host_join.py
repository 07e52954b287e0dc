"""The local completion's preparer without a GPU: launches written, refusals, and, where the reference's host code was
compiled (oracle/_ref), the same verdict and the same record bytes as its own preparer over a sweep of descriptions;
the oracle's ring order against its definition in numpy."""
import ctypes as C
import itertools

import numpy as np

from anemone_b200 import api
from anemone_b200 import records as R
from oracle.binding import ptr

OK, INVALID = 0, 1
HANDLE = 9
ARENA = 1 << 22


def description(operation=0, width=640, rows=5, source_stride=None, output_stride=None, routed=False, slots=False,
                **changes):
    source_stride = source_stride or width
    output_stride = output_stride or width
    value = R.Tp2JoinDescription()
    value.source = R.Tp2JoinRange(4096, 1 << 20)
    value.output = R.Tp2JoinRange(4096 + (1 << 20), 1 << 20)
    if routed:
        value.routed_sums = R.Tp2JoinRange(4096 + (2 << 20), 1 << 20)
        value.routed_row_stride = width + 16
    if slots:
        value.step = R.Tp2JoinRange(0, 16)
        value.source_slot_stride, value.output_slot_stride = 1 << 19, 1 << 19
    value.width, value.row_count = width, rows
    value.source_row_stride, value.output_row_stride, value.operation = source_stride, output_stride, operation
    for name, change in changes.items():
        target, _, field = name.partition("__")
        if field:
            setattr(getattr(value, target), field, change)
        else:
            setattr(value, name, change)
    return value


def prototype(lib):
    lib.tp2_join_prepare.argtypes = [C.POINTER(R.Tp2JoinDescription), C.c_uint64, C.c_uint32, C.POINTER(R.KernelLaunch)]
    return lib


CASES = [dict(operation=op) for op in range(8)] + \
    [dict(operation=op, routed=True) for op in range(7)] + \
    [dict(operation=op, slots=True) for op in (0, 1, 3)] + \
    [dict(operation=op, source_stride=704, output_stride=768) for op in range(7)] + \
    [dict(operation=5, width=642), dict(operation=6, width=640, source_stride=704), dict(width=0), dict(rows=0),
     dict(rows=1025), dict(width=32769, rows=1), dict(width=32768, rows=1, source__byte_count=1 << 20),
     dict(source_stride=639), dict(output_stride=100), dict(reserved_zero=1), dict(source__byte_offset=4100),
     dict(output__byte_offset=4096 + 8), dict(source__byte_count=100), dict(step__byte_count=16),
     dict(slots=True, step__byte_offset=8), dict(slots=True, source_slot_stride=24), dict(slots=True, source_slot_stride=64),
     dict(routed=True, routed_row_stride=8), dict(routed_row_stride=640), dict(routed_sums__byte_offset=64),
     dict(output__byte_offset=4096), dict(slots=True, output_slot_stride=(1 << 20) - 64),
     dict(source__byte_offset=ARENA - 64)]


def test_launch_and_refusals():
    lib = prototype(api.library())
    launch = R.KernelLaunch()
    assert lib.tp2_join_prepare(C.byref(description(4, routed=True)), ARENA, HANDLE, C.byref(launch)) == OK
    record = R.Tp2Join.from_buffer_copy(bytes(launch.argument)[:80])
    assert tuple(launch.grid) == (3, 5, 1) and launch.block[0] == 256 and launch.argument_byte_count == 80
    assert (record.operation, record.has_routed_sums, record.width, record.row_count) == (4, 1, 640, 5)
    assert record.routed_row_stride == 656 and record.reserved_zero == 0
    poisoned = (R.KernelLaunch * 1)()
    C.memset(poisoned, 0xA5, C.sizeof(poisoned))
    before = bytes(poisoned)
    assert lib.tp2_join_prepare(C.byref(description()), ARENA, 0xFFFFFFFF, poisoned) == INVALID
    for case in (dict(operation=7), dict(operation=1, routed=True), dict(width=0), dict(source_stride=639),
                 dict(output__byte_offset=4096), dict(reserved_zero=1), dict(step__byte_count=16)):
        assert lib.tp2_join_prepare(C.byref(description(**case)), ARENA, HANDLE, poisoned) == INVALID, case
    assert bytes(poisoned) == before


def test_verdicts_and_records_equal_reference(reference):
    lib, theirs_lib = prototype(api.library()), prototype(reference)
    accepted = 0
    for case in CASES:
        ours, theirs = R.KernelLaunch(), R.KernelLaunch()
        a = lib.tp2_join_prepare(C.byref(description(**case)), ARENA, HANDLE, C.byref(ours))
        b = theirs_lib.tp2_join_prepare(C.byref(description(**case)), ARENA, HANDLE, C.byref(theirs))
        assert a == b, case
        if a == OK:
            accepted += 1
            assert bytes(ours) == bytes(theirs), case  # the record, and here the reference's grid too
    assert accepted >= 15


def test_oracle_ring_order_is_the_definition(oracle):
    """Owner o holds quarter o of every slab of 8 rows (the last slab what is left), slab after slab, owner after
    owner: built here with array slices, then pack and unpack by the oracle."""
    for rows, width in ((8, 16), (13, 8), (29, 12), (1, 4), (32, 640)):
        rng = np.random.default_rng(rows * 1000 + width)
        values = rng.integers(0, 0x7F00, size=(rows, width), dtype=np.uint16)
        quarters = [[] for _ in range(4)]
        for first in range(0, rows, 8):
            slab = values[first:first + 8].reshape(-1)
            for owner, part in enumerate(np.split(slab, 4)):
                quarters[owner].append(part)
        expected = np.concatenate([np.concatenate(parts) for parts in quarters])
        arena = np.zeros(1 << 18, dtype=np.uint8)
        arena[:values.nbytes] = values.reshape(-1).view(np.uint8)
        record = R.Tp2Join(0, 0, 1 << 17, 0, 0, 0, width, rows, width, 0, width, 5, 0, 0)
        oracle.orc_tp2_join(C.byref(record), arena.ctypes.data)
        packed = arena[1 << 17:(1 << 17) + values.nbytes].view(np.uint16)
        assert np.array_equal(packed, expected), (rows, width)
        back = np.zeros(1 << 18, dtype=np.uint8)
        back[:values.nbytes] = packed.view(np.uint8)
        record = R.Tp2Join(0, 0, 1 << 17, 0, 0, 0, width, rows, width, 0, width, 6, 0, 0)
        oracle.orc_tp2_join(C.byref(record), back.ctypes.data)
        assert np.array_equal(back[1 << 17:(1 << 17) + values.nbytes].view(np.uint16), values.reshape(-1))
