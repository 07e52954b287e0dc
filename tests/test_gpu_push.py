"""The one-shot push all-reduce and the exchange's owner sums on ONE CUDA device, bit for bit against the CPU oracle.

One rank is real; the others are regions of the same arena. What an absent rank would have stored into the real
rank's slot by the time it matters (its inbox, its READY and DONE lines) the host writes before the launch, so the
kernel never waits on another kernel; what the real rank stores into the others' slots is read back and checked. Runs
across real GPUs are in test_gpu_multi.py.
"""
import ctypes as C

import numpy as np
import pytest

from anemone_b200 import records as R
from oracle.binding import f32p, pointer_array, ptr, u16p

pytestmark = pytest.mark.gpu

LINE = 128
BIG = 16777216.0
POISON = 0xC3


@pytest.fixture(scope="module")
def api():
    from anemone_b200 import api as module
    assert module.card_count() >= 1, "no CUDA device: the CUDA path cannot run and there is no fallback"
    return module


def wire(values, payload):
    """What a rank's values look like in an inbox: FP32 as they are, or bfloat16 bits rounded to nearest even."""
    if payload == R.ORDERED_PUSH_FP32:
        return values.copy()
    bits = values.view(np.uint32).astype(np.uint64)
    return ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)


class Emulated:
    def __init__(self, api, ranks, real, elements, payload, skew=0, deadline=2_000_000_000):
        self.api, self.ranks, self.real, self.elements, self.payload = api, ranks, real, elements, payload
        layout = api.Layout()
        self.peer_table, self.step = layout.take(16 * 32), layout.take(16)
        self.signals = 2 * ranks * LINE
        self.inbox_stride = api.align(4 * elements, 16) + skew
        self.input = self.signals + skew  # skew 4: nothing on a 16-byte multiple, the scalar path
        self.output = self.input + api.align(4 * elements, 16)
        self.inbox = self.output + api.align(4 * elements, 16)
        self.stride = api.align(self.inbox + ranks * self.inbox_stride, LINE)
        self.regions = [layout.take(2 * self.stride, LINE) for _ in range(ranks)]
        self.arena_bytes = layout.take(4096, 4096)
        self.card = api.Card(0, self.arena_bytes)
        self.card.fill(0, 0, self.arena_bytes)
        peers = (R.OrderedPeer * ranks)()
        for rank in range(ranks):
            peers[rank].region_offset = self.regions[rank]
        self.card.upload(self.peer_table, np.frombuffer(bytes(peers), dtype=np.uint8))
        for rank in range(ranks):
            self.card.peer_connect(self.card, 0, self.peer_table + 32 * rank)
        self.deadline = deadline

    def arguments(self):
        return R.OrderedPush(self.peer_table, self.regions[self.real], self.input, self.output, self.inbox, self.step,
                             self.stride, self.deadline, self.inbox_stride, self.elements, self.ranks, self.real,
                             self.payload, 0, 0)

    def slot(self, rank, sequence):
        return self.regions[rank] + (sequence & 1) * self.stride

    def line(self, rank, sequence, phase, source):
        return self.slot(rank, sequence) + (phase * self.ranks + source) * LINE

    def write_step(self, sequence, rows):
        self.card.upload(self.step, np.frombuffer(bytes(R.StepBlock(sequence, rows, 0)), dtype=np.uint8))

    def absent_ranks_arrive(self, sequence, inputs):
        """Into the real rank's slot: every other rank's values and its READY and DONE words of all eight groups."""
        for rank in range(self.ranks):
            if rank == self.real:
                continue
            self.card.upload(self.slot(self.real, sequence) + self.inbox + rank * self.inbox_stride,
                             wire(inputs[rank], self.payload))
            for phase in range(2):
                self.card.upload(self.line(self.real, sequence, phase, rank), np.full(8, sequence, dtype=np.uint64))

    def close(self):
        self.card.close()


def fp32_inputs(rng, ranks, elements):
    inputs = [rng.normal(0, 0.05, elements).astype(np.float32) for _ in range(ranks)]
    inputs[0][:2] = [BIG, 1e-30]
    if ranks > 2:
        inputs[1][0], inputs[2][0] = 1.0, -BIG  # a changed order changes the bits
    return inputs


@pytest.mark.parametrize("payload", [0, 1])
@pytest.mark.parametrize("ranks,real,skew", [(1, 0, 0), (4, 2, 0), (8, 7, 0), (4, 0, 4)])
def test_push_bit_exact(api, oracle, payload, ranks, real, skew):
    elements = 3 * 4096 + 37
    rng = np.random.default_rng(payload * 64 + ranks * 4 + skew)
    inputs = fp32_inputs(rng, ranks, elements)
    expected = np.zeros(elements, dtype=np.float32)
    oracle.orc_ordered_push(pointer_array(inputs), ranks, elements, payload, ptr(expected, f32p))
    if payload == 0:  # the FP32 wire is the ordered sum itself
        plain = np.zeros(elements, dtype=np.float32)
        oracle.orc_ordered_sum(pointer_array(inputs), ranks, elements, ptr(plain, f32p))
        assert np.array_equal(plain.view(np.uint32), expected.view(np.uint32))
    world = Emulated(api, ranks, real, elements, payload, skew)
    try:
        card, lib = world.card, api.library()
        kernel = C.c_uint32()
        lib.ordered_push_kernel_prepare.argtypes = [C.POINTER(api.BackendOperations), C.c_void_p, C.POINTER(C.c_uint32)]
        api.check(lib.ordered_push_kernel_prepare(card.ops_pointer, card.handle, C.byref(kernel)), "kernel")
        description = R.OrderedPushDescription(world.arguments(), world.arena_bytes)
        launch = R.KernelLaunch()
        lib.ordered_push_prepare.argtypes = [C.POINTER(R.OrderedPushDescription), C.c_uint32, C.POINTER(R.KernelLaunch)]
        api.check(lib.ordered_push_prepare(C.byref(description), kernel.value, C.byref(launch)), "prepare")
        groups = launch.grid[0]
        assert 1 <= groups <= 8 and launch.grid[0] * launch.grid[1] >= 4
        sent = wire(inputs[real], payload)
        for sequence in (1, 2, 3, 7):  # both parities, a reuse, a skipped sequence
            world.write_step(sequence, 1)
            card.upload(world.slot(real, sequence) + world.input, inputs[real])
            world.absent_ranks_arrive(sequence, inputs)
            card.fill(world.slot(real, sequence) + world.output, POISON, 4 * elements)
            for rank in range(ranks):
                if rank != real:
                    card.fill(world.slot(rank, sequence) + world.inbox + real * world.inbox_stride, POISON, sent.nbytes)
            card.run([launch])
            card.wait()
            assert card.expired_bits() == 0
            got = card.download(world.slot(real, sequence) + world.output, 4 * elements, np.float32)
            assert np.array_equal(got.view(np.uint32), expected.view(np.uint32))
            for rank in range(ranks):  # what every other rank was sent, and told
                arrived = card.download(world.slot(rank, sequence) + world.inbox + real * world.inbox_stride,
                                        sent.nbytes, sent.dtype)
                assert np.array_equal(arrived.view(np.uint8), sent.view(np.uint8)), rank
                for phase in range(2):
                    words = card.download(world.line(rank, sequence, phase, real), 64, np.uint64)
                    assert (words[:groups] == sequence).all() and (rank == real or (words[groups:] == 0).all())
            counters = card.download(world.line(real, sequence, 0, real) + 64, 32, np.uint32)
            assert (counters == 0).all()  # ready for the slot's next use
    finally:
        world.close()


def exchange_launches(api, world, row_width, layer, layers, form):
    card, lib = world.card, api.library()
    kernels = (C.c_uint32 * 4)()
    lib.tp_exchange_wide_kernels_prepare.argtypes = [C.POINTER(api.BackendOperations), C.c_void_p, C.c_uint32,
                                                     C.POINTER(C.c_uint32)]
    api.check(lib.tp_exchange_wide_kernels_prepare(card.ops_pointer, card.handle, form, kernels), "kernels")
    description = R.OrderedPushDescription(world.arguments(), world.arena_bytes)
    launches = (R.KernelLaunch * 4)()
    lib.tp_exchange_wide_rows_prepare.argtypes = [C.POINTER(R.OrderedPushDescription), C.c_uint32, C.c_uint32,
                                                  C.c_uint32, C.POINTER(C.c_uint32), C.c_uint32,
                                                  C.POINTER(R.KernelLaunch)]
    api.check(lib.tp_exchange_wide_rows_prepare(C.byref(description), row_width, layer, layers, kernels, form,
                                                launches), "prepare")
    return launches


@pytest.mark.parametrize("payload", [0, 1])
@pytest.mark.parametrize("ranks,real", [(1, 0), (4, 1), (8, 5)])
def test_owner_sums_bit_exact(api, oracle, payload, ranks, real):
    """The rows a rank owns: added in rank order, rounded once to bfloat16, stored into every rank's output array; the
    rows the others own: sent to them and to nobody else. Live rows below the prepared rows, an odd row count."""
    width, capacity, layers, layer = 256, 29, 6, 4
    rng = np.random.default_rng(900 + payload * 64 + ranks)
    world = Emulated(api, ranks, real, capacity * width, payload)
    try:
        card = world.card
        launches = exchange_launches(api, world, width, layer, layers, R.TP_EXCHANGE_FORM_OWNER_SUMS)
        for step, rows in ((1, 29), (2, 13), (3, 5), (4, 0)):
            sequence = (step * layers + layer) * 2 + (step & 1)
            live = rows * width
            inputs = fp32_inputs(rng, ranks, capacity * width)
            expected = np.zeros(capacity * width, dtype=np.uint16)
            oracle.orc_owner_sums(pointer_array(inputs), ranks, live, payload, ptr(expected, u16p))
            first = [rows * shard // ranks * width for shard in range(ranks + 1)]
            world.write_step(step, rows)
            card.upload(world.slot(real, sequence) + world.input, inputs[real])
            world.absent_ranks_arrive(sequence, inputs)
            sent = wire(inputs[real], payload)
            unit = sent.itemsize
            for rank in range(ranks):
                card.fill(world.slot(rank, sequence) + world.output, POISON, 2 * capacity * width)
                if rank != real:
                    card.fill(world.slot(rank, sequence) + world.inbox + real * world.inbox_stride, POISON, sent.nbytes)
            card.run(launches)
            card.wait()
            assert card.expired_bits() == 0
            for rank in range(ranks):
                got = card.download(world.slot(rank, sequence) + world.output, 2 * capacity * width, np.uint16)
                mine = slice(first[real], first[real + 1])
                assert np.array_equal(got[mine], expected[mine]), (rows, rank)
                untouched = np.ones(capacity * width, dtype=bool)
                untouched[mine] = False
                assert (got[untouched] == POISON * 0x0101).all()  # the other owners' rows: theirs to store
                if rank != real:
                    arrived = card.download(world.slot(rank, sequence) + world.inbox + real * world.inbox_stride,
                                            sent.nbytes, np.uint8)
                    theirs = slice(first[rank] * unit, first[rank + 1] * unit)
                    assert np.array_equal(arrived[theirs], sent.view(np.uint8)[theirs]), (rows, rank)
                    other = np.ones(sent.nbytes, dtype=bool)
                    other[theirs] = False
                    assert (arrived[other] == POISON).all()
    finally:
        world.close()


def test_exchange_push_form_live_rows(api, oracle):
    """The push form of the exchange: only the step's live rows are exchanged, under the layer's own sequence."""
    width, capacity, ranks, real, layers, layer = 512, 16, 4, 3, 3, 1
    rng = np.random.default_rng(77)
    world = Emulated(api, ranks, real, capacity * width, 0)
    try:
        card = world.card
        launches = exchange_launches(api, world, width, layer, layers, R.TP_EXCHANGE_FORM_PUSH)
        for step, rows in ((1, 16), (2, 3)):
            sequence = (step * layers + layer) * 2 + (step & 1)
            inputs = fp32_inputs(rng, ranks, capacity * width)
            expected = np.zeros(rows * width, dtype=np.float32)
            oracle.orc_ordered_push(pointer_array(inputs), ranks, rows * width, 0, ptr(expected, f32p))
            world.write_step(step, rows)
            card.upload(world.slot(real, sequence) + world.input, inputs[real])
            world.absent_ranks_arrive(sequence, inputs)
            card.fill(world.slot(real, sequence) + world.output, POISON, 4 * capacity * width)
            card.run(launches)
            card.wait()
            assert card.expired_bits() == 0
            got = card.download(world.slot(real, sequence) + world.output, 4 * capacity * width, np.uint32)
            assert np.array_equal(got[:rows * width], expected.view(np.uint32))
            assert (got[rows * width:] == 0xC3C3C3C3).all()
    finally:
        world.close()


def test_failures_are_reported_without_a_fault(api):
    """A rank whose peer never arrives gives up after its deadline (here a millisecond or so), says so, and the card
    stays usable; a replayed sequence and a step of too many rows are refused on the device. Nothing traps."""
    width, capacity, ranks = 256, 8, 2
    world = Emulated(api, ranks, 0, capacity * width, 0, deadline=2_000_000)
    try:
        card = world.card
        launches = exchange_launches(api, world, width, 0, 1, R.TP_EXCHANGE_FORM_PUSH)
        values = np.ones(capacity * width, dtype=np.float32)
        world.write_step(1, capacity)
        card.upload(world.slot(0, 2 + 1) + world.input, values)
        card.fill(world.slot(0, 3) + world.output, POISON, 4 * capacity * width)
        card.run(launches)
        card.wait()
        assert card.expired_bits() == 1  # rank 1 never published READY
        got = card.download(world.slot(0, 3) + world.output, 4 * capacity * width, np.uint8)
        assert (got == POISON).all()  # nothing was added
        world.write_step(1, capacity)  # the same step again: its sequence is not above the slot's last
        card.run(launches)
        card.wait()
        assert card.expired_bits() == 1 | 2
        world.write_step(2, capacity + 1)
        card.run(launches)
        card.wait()
        assert card.expired_bits() == 1 | 2 | 4
        card.upload(world.peer_table + 512 - 8, np.arange(2, dtype=np.uint32))  # the card still answers
        assert np.array_equal(card.download(world.peer_table + 512 - 8, 8, np.uint32), np.arange(2))
    finally:
        world.close()
