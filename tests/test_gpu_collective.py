"""The fixed-order reduction kernels on a CUDA device, bit for bit against the CPU oracle and the fixtures generated
from the reference's own host code.

On one GPU the other ranks are emulated as REGIONS OF THE SAME ARENA whose payload and signal lines the host has
written before the launch: the kernel under test then reads "peer" data through the peer table exactly as it would
over NVLink, and never waits on another kernel (kernels that wait on one another must not share a GPU). Real
multi-GPU runs are in test_gpu_multi.py.
"""
import ctypes as C

import numpy as np
import pytest

from anemone_b200 import records as R
from tests import golden_util
from oracle.binding import f32p, pointer_array, ptr, u16p

pytestmark = pytest.mark.gpu

LINE = 128
SIGNALS = 3 * LINE
BIG = 16777216.0


@pytest.fixture(scope="module")
def api():
    from anemone_b200 import api as module
    assert module.card_count() >= 1, "no CUDA device: the CUDA path cannot run and there is no fallback"
    return module


class Emulated:
    """Rank 0 real, ranks 1 .. R-1 host-written regions of the same arena."""

    def __init__(self, api, ranks, elements, deadline=2_000_000_000):
        self.api, self.ranks, self.elements = api, ranks, elements
        layout = api.Layout()
        self.peer_table = layout.take(16 * 32)
        self.step = layout.take(16)
        self.status = layout.take(16)
        self.input, self.output, self.scratch = SIGNALS, SIGNALS + 4 * elements, SIGNALS + 8 * elements
        self.stride = api.align(SIGNALS + 12 * elements, LINE)
        self.regions = [layout.take(2 * self.stride, LINE) for _ in range(ranks)]
        self.result = layout.take(2 * elements)
        self.pairs = layout.take(4 * elements * 3)
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
        return R.OrderedCollective(self.peer_table, self.regions[0], self.input, self.output, self.scratch, self.step,
                                   self.stride, self.deadline, self.elements, self.ranks, 0, 0)

    def slot(self, rank, sequence):
        return self.regions[rank] + (sequence & 1) * self.stride

    def write_step(self, sequence, rows):
        self.card.upload(self.step, np.frombuffer(bytes(R.StepBlock(sequence, rows, 0)), dtype=np.uint8))

    def write_line(self, rank, sequence, phase, value):
        self.card.upload(self.slot(rank, sequence) + phase * LINE, np.array([value], dtype=np.uint64))

    def close(self):
        self.card.close()


def fp32_inputs(rng, ranks, elements):
    inputs = [rng.normal(0, 0.05, elements).astype(np.float32) for _ in range(ranks)]
    inputs[0][:2] = [BIG, 1e-30]
    if ranks > 2:
        inputs[1][0], inputs[2][0] = 1.0, -BIG  # cancellation-sensitive: a changed order changes the bits
    return inputs


@pytest.mark.parametrize("operation", [0, 1, 2, 3])
@pytest.mark.parametrize("ranks", [1, 4, 8])
def test_fp32_collectives_bit_exact(api, oracle, operation, ranks):
    elements = 4096 + 37
    rng = np.random.default_rng(operation * 16 + ranks)
    inputs = fp32_inputs(rng, ranks, elements)
    outputs = [np.zeros(elements, dtype=np.float32) for _ in range(ranks)]
    assert oracle.orc_ordered_collective(pointer_array(inputs), pointer_array(outputs), ranks, elements, operation) == 0
    reduced = np.zeros(elements, dtype=np.float32)
    oracle.orc_ordered_sum(pointer_array(inputs), ranks, elements, ptr(reduced, f32p))
    world = Emulated(api, ranks, elements)
    try:
        card, lib = world.card, api.library()
        kernels = R.OrderedCollectiveKernels()
        lib.ordered_collective_kernels_prepare.argtypes = [C.POINTER(api.BackendOperations), C.c_void_p,
                                                           C.POINTER(R.OrderedCollectiveKernels)]
        api.check(lib.ordered_collective_kernels_prepare(card.ops_pointer, card.handle, C.byref(kernels)), "kernels")
        description = R.OrderedCollectiveDescription(world.arguments(), world.arena_bytes, operation)
        launch = R.KernelLaunch()
        lib.ordered_collective_prepare.argtypes = [C.POINTER(R.OrderedCollectiveDescription),
                                                   C.POINTER(R.OrderedCollectiveKernels), C.POINTER(R.KernelLaunch)]
        api.check(lib.ordered_collective_prepare(C.byref(description), C.byref(kernels), C.byref(launch)), "prepare")
        for sequence in (1, 2, 3):  # both parities, then a reuse
            world.write_step(sequence, 1)
            for rank in range(ranks):
                card.upload(world.slot(rank, sequence) + world.input, inputs[rank])
                if rank != 0:
                    # what the emulated rank would have published by now: READY, its reduced slice, REDUCED, DONE
                    card.upload(world.slot(rank, sequence) + world.scratch, reduced)
                    for phase in range(3):
                        world.write_line(rank, sequence, phase, sequence)
            card.fill(world.slot(0, sequence) + world.output, 0xC3, 4 * elements)
            card.run([launch])
            card.wait()
            got = card.download(world.slot(0, sequence) + world.output, 4 * elements, np.float32)
            if operation == 2:  # reduce-scatter: only rank 0's slice is written
                piece = (elements + ranks - 1) // ranks
                assert np.array_equal(got[:piece].view(np.uint32), outputs[0][:piece].view(np.uint32))
                assert (got[piece:].view(np.uint32) == 0xC3C3C3C3).all()
            else:
                assert np.array_equal(got.view(np.uint32), outputs[0].view(np.uint32))
    finally:
        world.close()


def prepare_reduce(api, world, rows, width, pairs_per_row):
    lib, card = api.library(), world.card
    description = R.OrderedReduceBf16Description()
    description.reduce.collective = world.arguments()
    description.reduce.collective.output_offset = world.result
    description.reduce.collective.scratch_offset = 0
    description.reduce.status_offset, description.reduce.width = world.status, width
    description.pair_output_offset, description.arena_byte_count = world.pairs, world.arena_bytes
    description.pairs_per_row, description.row_capacity = pairs_per_row, rows
    launches = (R.KernelLaunch * 2)()
    lib.ordered_reduce_bf16_prepare.argtypes = [C.POINTER(R.OrderedReduceBf16Description),
                                                C.POINTER(api.BackendOperations), C.c_void_p, C.POINTER(R.KernelLaunch)]
    api.check(lib.ordered_reduce_bf16_prepare(C.byref(description), card.ops_pointer, card.handle, launches),
              "ordered_reduce_bf16_prepare")
    return launches


def test_reduce_bf16_matches_reference_fixtures(api, oracle):
    golden = golden_util.load("reference_vectors.json")
    for case in golden["ordered_all_reduce"]:
        ranks, rows, width = case["ranks"], case["rows"], 4096
        inputs = golden_util.golden_reduce_case(case)
        # the FP32 sums are the reference's own (checked against its fixture digest), rounded once by the oracle
        sums = np.zeros(rows * width, dtype=np.float32)
        oracle.orc_ordered_sum(pointer_array(inputs), ranks, sums.size, ptr(sums, f32p))
        assert hex(golden_util.fnv64(sums)) == case["sum_fnv64"]
        expected = np.zeros(sums.size, dtype=np.uint16)
        oracle.orc_ordered_reduce_bf16(pointer_array(inputs), ranks, sums.size, ptr(expected, u16p))
        world = Emulated(api, ranks, rows * width)
        try:
            card = world.card
            launches = prepare_reduce(api, world, rows, width, 3)
            # rank 0's partial is the sum of three pair outputs, of which two are zero
            pairs = np.zeros((rows, 3, width), dtype=np.float32)
            pairs[:, 1, :] = inputs[0].reshape(rows, width)
            card.upload(world.pairs, pairs)
            for sequence in (1, 2, 3, 4):
                world.write_step(sequence, rows)
                for rank in range(1, ranks):
                    card.upload(world.slot(rank, sequence) + world.input, inputs[rank])
                    world.write_line(rank, sequence, 0, sequence)
                    world.write_line(rank, sequence, 2, sequence)  # "has read this use": lets the slot be refilled
                card.fill(world.result, 0, 2 * rows * width)
                card.run(launches)
                card.wait()
                got = card.download(world.result, 2 * rows * width, np.uint16)
                assert np.array_equal(got, expected)
                assert (card.download(world.status, 16, np.uint32) == 0).all()
        finally:
            world.close()


def test_reduce_bf16_cancellation_and_specials(api, oracle):
    ranks, rows, width = 5, 2, 512
    order = [BIG, 1.0, -BIG, 1.0, 1.0]
    inputs = [np.full(rows * width, value, dtype=np.float32) for value in order]
    inputs[3][7], inputs[2][9], inputs[4][11] = np.float32("nan"), np.float32("inf"), np.float32(-0.0)
    expected = np.zeros(rows * width, dtype=np.uint16)
    oracle.orc_ordered_reduce_bf16(pointer_array(inputs), ranks, expected.size, ptr(expected, u16p))
    assert expected[0] == 0x4000 and expected[7] == 0x7FC0  # 2.0; the quiet not-a-number
    world = Emulated(api, ranks, rows * width)
    try:
        card = world.card
        launches = prepare_reduce(api, world, rows, width, 1)
        card.upload(world.pairs, inputs[0])
        world.write_step(1, rows)
        for rank in range(1, ranks):
            card.upload(world.slot(rank, 1) + world.input, inputs[rank])
            world.write_line(rank, 1, 0, 1)
        card.run(launches)
        card.wait()
        assert np.array_equal(card.download(world.result, 2 * rows * width, np.uint16), expected)
        # fewer live rows than the capacity: only they are reduced
        world.write_step(2, 1)
        for rank in range(1, ranks):
            card.upload(world.slot(rank, 2) + world.input, inputs[rank])
            world.write_line(rank, 2, 0, 2)
        card.fill(world.result, 0xEE, 2 * rows * width)
        card.run(launches)
        card.wait()
        got = card.download(world.result, 2 * rows * width, np.uint16)
        assert np.array_equal(got[:width], expected[:width]) and (got[width:] == 0xEEEE).all()
    finally:
        world.close()


def test_wait_runs_out_without_fault(api):
    """A peer that never publishes: the bounded wait ends, the status block says who was missing, the card lives on."""
    ranks, rows, width = 2, 1, 512
    world = Emulated(api, ranks, rows * width, deadline=2_000_000)  # about a millisecond of device clock
    try:
        card = world.card
        launches = prepare_reduce(api, world, rows, width, 1)
        card.upload(world.pairs, np.ones(rows * width, dtype=np.float32))
        world.write_step(1, rows)  # rank 1's READY line stays zero: nothing sets it
        card.run(launches)
        card.wait()
        status = card.download(world.status, 16, np.uint32)
        assert status[0] == 1 and status[1] == 0 and status[2] == 1  # timed out, READY phase, rank 1
        # the card is still usable: publish the missing line and run the next step to completion
        card.fill(world.status, 0, 16)
        world.write_step(2, rows)
        card.upload(world.slot(1, 2) + world.input, np.full(rows * width, 2.0, dtype=np.float32))
        world.write_line(1, 2, 0, 2)
        card.run(launches)
        card.wait()
        assert (card.download(world.status, 16, np.uint32) == 0).all()
        assert (card.download(world.result, 2 * rows * width, np.uint16) == 0x4040).all()  # 1 + 2 = 3.0
    finally:
        world.close()
