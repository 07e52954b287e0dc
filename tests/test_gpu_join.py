"""The local completion kernel on a CUDA device: every operation, strided rows, parity slots, bit for bit against the
CPU oracle run on a host copy of the same arena."""
import ctypes as C

import numpy as np
import pytest

from anemone_b200 import records as R

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    from anemone_b200 import api as module
    assert module.card_count() >= 1, "no CUDA device: the CUDA path cannot run and there is no fallback"
    return module


@pytest.mark.parametrize("operation", range(7))
@pytest.mark.parametrize("rows,width,gap,slots", [(5, 640, 0, False), (29, 4096, 64, True), (1, 4, 0, False),
                                                   (8, 36, 12, True)])
def test_join_bit_exact(api, oracle, operation, rows, width, gap, slots):
    rng = np.random.default_rng(operation * 100 + rows)
    ring_in, ring_out = operation == 6, operation == 5
    source_stride = width if ring_in else width + gap
    output_stride = width if ring_out else width + gap + 8
    routed = operation in (0, 4, 5)
    span = 1 << 20
    layout = api.Layout()
    step = layout.take(16)
    source, output, sums = layout.take(2 * span), layout.take(2 * span), layout.take(span)
    arena_bytes = layout.take(4096, 4096)
    description = R.Tp2JoinDescription()
    description.source, description.output = R.Tp2JoinRange(source, 2 * span), R.Tp2JoinRange(output, 2 * span)
    if routed:
        description.routed_sums, description.routed_row_stride = R.Tp2JoinRange(sums, span), width + 4
    if slots:
        description.step = R.Tp2JoinRange(step, 16)
        description.source_slot_stride = description.output_slot_stride = span
    description.width, description.row_count, description.operation = width, rows, operation
    description.source_row_stride, description.output_row_stride = source_stride, output_stride
    card = api.Card(0, arena_bytes)
    try:
        lib = api.library()
        kernel = C.c_uint32()
        lib.tp2_join_kernel_prepare.argtypes = [C.POINTER(api.BackendOperations), C.c_void_p, C.POINTER(C.c_uint32)]
        api.check(lib.tp2_join_kernel_prepare(card.ops_pointer, card.handle, C.byref(kernel)), "kernel")
        launch = R.KernelLaunch()
        lib.tp2_join_prepare.argtypes = [C.POINTER(R.Tp2JoinDescription), C.c_uint64, C.c_uint32,
                                         C.POINTER(R.KernelLaunch)]
        api.check(lib.tp2_join_prepare(C.byref(description), arena_bytes, kernel.value, C.byref(launch)), "prepare")
        record = R.Tp2Join.from_buffer_copy(bytes(launch.argument)[:80])
        for sequence in (1, 2):
            host = rng.integers(0, 256, size=arena_bytes, dtype=np.uint8)
            if operation in (0, 4, 5):  # arithmetic on bfloat16 values: finite ones (the sum of a not-a-number has
                words = host[source:source + 2 * span].view(np.uint16)  # no payload the two machines agree on)
                words[(words & 0x7F80) == 0x7F80] &= 0xBFFF
            # finite, mixed-sign FP32 routed sums and values; a few special values in front
            sums_view = host[sums:sums + span].view(np.float32)
            sums_view[:] = rng.normal(0, 1, sums_view.size).astype(np.float32)
            if operation in (1, 3):
                values = host[source:source + 2 * span].view(np.float32)
                values[:] = rng.normal(0, 1, values.size).astype(np.float32)
                for slot in range(2):
                    values[slot * span // 4:slot * span // 4 + 4] = [np.nan, -0.0, np.inf, 3.3895314e38]
            host[step:step + 16] = np.frombuffer(bytes(R.StepBlock(sequence, rows, 0)), dtype=np.uint8)
            card.upload(0, host)
            expected = host.copy()
            oracle.orc_tp2_join(C.byref(record), expected.ctypes.data)
            card.run([launch])
            card.wait()
            got = card.download(0, arena_bytes)
            assert np.array_equal(got, expected), (operation, sequence)  # the whole arena: nothing else is touched
            assert not np.array_equal(got, host)
    finally:
        card.close()
