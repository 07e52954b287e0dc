"""The load-time preparers on the host, with a fake backend whose only member is kernel_prepare (the way the
reference's own host tests drive them: tests/exl3_tp_test.c:23-48, tests/exl3_fast_prepare_test.c) and, where the
reference's host code was compiled (oracle/_ref), byte for byte against its preparers."""
import ctypes as C

import numpy as np
import pytest

from anemone_b200 import api, synthetic
from anemone_b200 import records as R

U32P = C.POINTER(C.c_uint32)


class Slice(C.Structure):
    _fields_ = [(name, C.c_uint32) for name in ("input_size", "output_size", "input_begin", "input_count",
                                                "output_begin", "output_count", "bits_per_weight", "reserved_zero")]


class SliceSizes(C.Structure):
    _fields_ = [("source_bytes", C.c_uint64), ("packed_bytes", C.c_uint64)]


class ShardPlan(C.Structure):
    _fields_ = [("gate_up", Slice), ("down", Slice), ("rank_count", C.c_uint32), ("rank", C.c_uint32),
                ("product_slices", C.c_uint32), ("order", C.c_int)]


class PassDescription(C.Structure):
    _fields_ = [("plan", C.POINTER(ShardPlan)), ("record", R.Exl3Expert), ("arena_bytes", C.c_uint64),
                ("weight_offset", C.c_uint64), ("weight_bytes", C.c_uint64), ("pass_", C.c_int),
                ("product_tiles", C.c_uint32)]


class FakeBackend:
    """kernel_prepare hands out dense handles and remembers what was asked."""

    def __init__(self):
        self.asked = []
        self.table = api.BackendOperations()
        prototype = dict(api.BackendOperations._fields_)["kernel_prepare"]

        def prepare(card, file_name, function_name, argument_bytes, kernel_out):
            key = (file_name.decode(), function_name.decode(), argument_bytes)
            if key not in self.asked:
                self.asked.append(key)
            kernel_out[0] = self.asked.index(key)
            return 0
        self.callback = prototype(prepare)
        self.table.kernel_prepare = self.callback
        self.card = C.c_void_p(0x1000)  # opaque to every preparer: never dereferenced


def chain_record(pairs=12, ppr=3, hidden=512, inner=256, jobs=7, width=3):
    layout = api.Layout()
    record = R.Exl3Expert()
    record.jobs_offset = layout.take(jobs * 96)
    record.input_offset = layout.take(pairs // ppr * hidden * 2)
    record.operands_offset = layout.take(pairs * hidden * 4)
    record.products_offset = record.output_offset = layout.take(pairs * hidden * 8)
    record.hidden_offset = layout.take(pairs * inner * 2)
    record.input_size, record.inner_size, record.pair_count, record.pairs_per_row = hidden, inner, pairs, ppr
    record.job_count, record.bits_per_weight, record.activation_limit = jobs, width, 10.0
    return record, layout.take(0, 4096) + 4096


def test_experts_prepare_launches_and_refusals():
    lib, fake = api.library(), FakeBackend()
    record, arena = chain_record()
    launches = (R.KernelLaunch * 5)()
    assert lib.exl3_experts_prepare(C.byref(record), arena, C.byref(fake.table), fake.card, 100, launches) == 0
    assert [key[1] for key in fake.asked] == ["exl3_input", "exl3_gate_up_k3", "exl3_activate", "exl3_down_k3",
                                              "exl3_finish"]
    assert all(key[0] == "kernel_exl3" and key[2] == 80 for key in fake.asked)
    grids = [tuple(l.grid) for l in launches]
    assert grids == [(1, 7, 2), (2, 7, 2), (1, 7, 1), (4, 7, 1), (1, 7, 1)]
    assert [l.block[0] for l in launches] == [128] * 5
    assert launches[1].dynamic_shared_byte_count == max(4 * 4 * 8 * 16 * 6, 16384) and launches[0].dynamic_shared_byte_count == 0
    for launch in launches:
        assert bytes(launch.argument[:80]) == bytes(record) and not any(launch.argument[80:])
    # refusals leave the whole table untouched
    untouched = bytes(launches)
    bad = []
    for field, value in (("reserved_zero", 1), ("pair_count", 0), ("pairs_per_row", 5), ("job_count", 0),
                         ("job_count", 70000), ("inner_size", 1024), ("activation_limit", 0.0),
                         ("activation_limit", float("inf")), ("bits_per_weight", 9), ("input_size", 500),
                         ("output_offset", 64), ("hidden_offset", record.products_offset + 16),
                         ("jobs_offset", 8), ("operands_offset", arena)):
        broken = R.Exl3Expert.from_buffer_copy(bytes(record))
        setattr(broken, field, value)
        bad.append(lib.exl3_experts_prepare(C.byref(broken), arena, C.byref(fake.table), fake.card, 100, launches))
    assert all(status == R.STATUS_INVALID_ARGUMENT for status in bad), bad
    assert lib.exl3_experts_prepare(C.byref(record), arena, C.byref(fake.table), fake.card, 80, launches) == \
        R.STATUS_UNSUPPORTED
    assert lib.exl3_experts_prepare(C.byref(record), arena, C.byref(fake.table), fake.card, 7, launches) == \
        R.STATUS_INVALID_ARGUMENT
    assert lib.exl3_experts_relaxed_prepare(C.byref(record), arena, C.byref(fake.table), fake.card, 100, launches) == \
        R.STATUS_UNSUPPORTED
    assert lib.exl3_experts_prepare(None, arena, C.byref(fake.table), fake.card, 100, launches) == 1
    assert bytes(launches) == untouched
    assert lib.exl3_scratch_byte_count(12, 512) == 12 * 512 * 12
    assert [lib.exl3_width_name(b) for b in (4, 5, 6, 8, 7)] == [b"k2", b"k2_5", b"k3", b"k4", None]


def test_moe_prepare():
    lib, fake = api.library(), FakeBackend()
    base, arena = chain_record()
    layout = api.Layout(arena)
    record = R.Exl3Moe()
    record.base = base
    record.base.bits_per_weight = R.EXL3_WIDTH_PER_EXPERT
    sizes = api.moe_sizes(12, 7, 512, 256)
    assert (sizes.gate_up_splits, sizes.down_splits) == (1, 1) and sizes.counter_bytes == 7 * 6 * 4
    big = api.moe_sizes(72, 65, 4096, 2048)
    assert (big.gate_up_splits, big.down_splits) == (2, 1) and big.product_bytes == 2 * 2 * 72 * 2048 * 4
    eighth = api.moe_sizes(72, 65, 4096, 256)  # a rank of eight: few outputs, so more runs of K
    assert (eighth.gate_up_splits, eighth.down_splits) == (8, 1)
    record.base.operands_offset = layout.take(sizes.operand_bytes)
    record.base.products_offset = record.base.output_offset = layout.take(max(sizes.product_bytes, 12 * 512 * 8))
    record.widths_offset, record.row_output_offset, record.expert_count = layout.take(64), layout.take(4 * 512 * 4), 9
    record.counters_offset = layout.take(sizes.counter_bytes)
    arena = layout.take(0, 4096) + 4096
    launches = (R.KernelLaunch * 4)()
    assert lib.exl3_moe_prepare(C.byref(record), arena, C.byref(fake.table), fake.card, launches) == 0
    assert [key[1] for key in fake.asked] == ["exl3_moe_input", "exl3_moe_gate_up", "exl3_moe_down", "exl3_moe_row_sum"]
    assert all(key[0] == "kernel_exl3_b200" and key[2] == 112 for key in fake.asked)
    untouched = bytes(launches)
    record.row_output_offset = record.base.products_offset  # overlaps the products
    assert lib.exl3_moe_prepare(C.byref(record), arena, C.byref(fake.table), fake.card, launches) == 1
    assert bytes(launches) == untouched


def test_slices_and_plans_against_numpy():
    lib = api.library()
    lib.bb_exl3_matrix_slice_prepare.argtypes = [C.POINTER(Slice), C.POINTER(SliceSizes)]
    lib.bb_exl3_matrix_slice_copy.argtypes = [C.POINTER(Slice), C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t]
    lib.bb_exl3_inner_shard_prepare.argtypes = [C.c_uint32] * 5 + [C.POINTER(ShardPlan)]
    rng = np.random.default_rng(4)
    for stored in (2, 40, 3, 4):
        matrix = synthetic.exl3_matrix(rng, 512, 768, stored)
        for ranks in (1, 2, 4):
            covered = 0
            for rank in range(ranks):
                plan = ShardPlan()
                assert lib.bb_exl3_inner_shard_prepare(512, 768, stored, ranks, rank, C.byref(plan)) == 0
                assert plan.gate_up.output_begin == covered and plan.down.input_begin == covered
                covered += plan.gate_up.output_count
                sizes = SliceSizes()
                assert lib.bb_exl3_matrix_slice_prepare(C.byref(plan.gate_up), C.byref(sizes)) == 0
                assert sizes.source_bytes == matrix.size
                packed = np.zeros(sizes.packed_bytes, dtype=np.uint8)
                assert lib.bb_exl3_matrix_slice_copy(C.byref(plan.gate_up), matrix.ctypes.data, matrix.size,
                                                     packed.ctypes.data, packed.size) == 0
                want = synthetic.slice_matrix(matrix, 512, 768, stored, 0, 512, plan.gate_up.output_begin,
                                              plan.gate_up.output_count)
                assert np.array_equal(packed, want)
            assert covered == 768
    plan = ShardPlan()
    assert lib.bb_exl3_inner_shard_prepare(512, 768, 3, 3, 0, C.byref(plan)) == 1  # ranks 1, 2, 4, 8 only
    assert lib.bb_exl3_inner_shard_prepare(512, 256, 3, 4, 0, C.byref(plan)) == 1  # fewer blocks than ranks


def test_slice_keeps_every_state(oracle):
    from oracle.binding import ptr, u16p, u8p
    rng = np.random.default_rng(9)
    for stored in (2, 40, 3, 4):
        matrix = synthetic.exl3_matrix(rng, 256, 256, stored)
        full = np.zeros((256, 256), dtype=np.uint16)
        oracle.orc_exl3_states(ptr(matrix, u8p), 256, 256, stored, ptr(full, u16p))
        for (ib, ic, ob, oc) in ((0, 256, 128, 128), (128, 128, 0, 256)):
            piece = synthetic.slice_matrix(matrix, 256, 256, stored, ib, ic, ob, oc)
            states = np.zeros((ic, oc), dtype=np.uint16)
            oracle.orc_exl3_states(ptr(piece, u8p), ic, oc, stored, ptr(states, u16p))
            assert np.array_equal(states, full[ib:ib + ic, ob:ob + oc])


def test_router_and_reduce_prepare():
    lib, fake = api.library(), FakeBackend()
    from anemone_b200.moe import MoeConfig, MoeLayout
    config = MoeConfig(hidden=512, inner=256, experts=32, shared=1, picks=4, row_capacity=8)
    L = MoeLayout(config, np.full(33, 3, dtype=np.uint32), 2, 1, reduce_form="pull")
    lib.router_select_b200_prepare.argtypes = [C.POINTER(R.RouterSelectB200), C.c_uint64,
                                               C.POINTER(api.BackendOperations), C.c_void_p, C.POINTER(R.KernelLaunch)]
    lib.router_b200_job_capacity.restype = C.c_uint32
    assert lib.router_b200_job_capacity(8, 4, 1) == 33 == L.job_capacity
    router = R.RouterSelectB200(L.scores, L.expert_table, L.picks, L.weights, L.jobs, L.step, 32, 1, 4, 8,
                                L.job_capacity, 0, 1.0, 0)
    launch = R.KernelLaunch()
    assert lib.router_select_b200_prepare(C.byref(router), L.arena_bytes, C.byref(fake.table), fake.card,
                                          C.byref(launch)) == 0
    assert tuple(launch.grid) == (1, 1, 1) and launch.block[0] == 1024
    untouched = bytes(launch)
    for field, value in (("picks", 0), ("picks", 17), ("expert_count", 600), ("row_capacity", 65),
                         ("job_capacity", 32), ("scoring", 2), ("route_scale", 0.0), ("jobs_offset", L.step)):
        broken = R.RouterSelectB200.from_buffer_copy(bytes(router))
        setattr(broken, field, value)
        assert lib.router_select_b200_prepare(C.byref(broken), L.arena_bytes, C.byref(fake.table), fake.card,
                                              C.byref(launch)) == 1, field
    assert bytes(launch) == untouched
    lib.ordered_reduce_bf16_prepare.argtypes = [C.POINTER(R.OrderedReduceBf16Description),
                                                C.POINTER(api.BackendOperations), C.c_void_p, C.POINTER(R.KernelLaunch)]
    description = R.OrderedReduceBf16Description()
    description.reduce.collective = R.OrderedCollective(L.peer_table, L.region, L.slot_input, L.result, 0, L.step,
                                                        L.parity_stride, 1000, 8 * 512, 2, 1, 0)
    description.reduce.status_offset, description.reduce.width = L.status, 512
    description.pair_output_offset, description.arena_byte_count = L.products, L.arena_bytes
    description.pairs_per_row, description.row_capacity = 5, 8
    launches = (R.KernelLaunch * 2)()
    assert lib.ordered_reduce_bf16_prepare(C.byref(description), C.byref(fake.table), fake.card, launches) == 0
    assert tuple(launches[0].grid) == (1, 8, 1) and tuple(launches[1].grid) == (4, 1, 1)
    untouched = bytes(launches)
    for path, value in (("rank", 2), ("rank_count", 17), ("deadline_cycles", 0), ("region_offset", L.region + 64),
                        ("input_offset", 128), ("parity_stride", L.parity_stride - 128)):
        broken = R.OrderedReduceBf16Description.from_buffer_copy(bytes(description))
        setattr(broken.reduce.collective, path, value)
        assert lib.ordered_reduce_bf16_prepare(C.byref(broken), C.byref(fake.table), fake.card, launches) == 1, path
    description.reduce.width = 510
    assert lib.ordered_reduce_bf16_prepare(C.byref(description), C.byref(fake.table), fake.card, launches) == 1
    assert bytes(launches) == untouched
    # the same reduction as one launch, by stores
    L = MoeLayout(config, np.full(33, 3, dtype=np.uint32), 2, 1, reduce_form="push")
    lib.ordered_rows_push_prepare.argtypes = [C.POINTER(R.OrderedRowsPushDescription), C.POINTER(api.BackendOperations),
                                              C.c_void_p, C.POINTER(R.KernelLaunch)]
    push = R.OrderedRowsPushDescription()
    push.arguments.push = R.OrderedPush(L.peer_table, L.region, 0, L.result, L.inbox, L.step, L.parity_stride, 1000,
                                        L.inbox_stride, 8 * 512, 2, 1, 0, 0, 0)
    push.arguments.pair_output_offset, push.arguments.width, push.arguments.pairs_per_row = L.products, 512, 5
    push.arena_byte_count = L.arena_bytes
    one = (R.KernelLaunch * 1)()
    assert lib.ordered_rows_push_prepare(C.byref(push), C.byref(fake.table), fake.card, one) == 0
    assert tuple(one[0].grid) == (2, 1, 1) and one[0].block[0] == 256 and one[0].argument_byte_count == 112
    assert fake.asked[-1] == ("kernel_ordered_b200", "ordered_rows_push", 112)
    untouched = bytes(one)
    for path, value in (("rank", 2), ("payload_format", 1), ("input_offset", 16), ("inbox_offset", 256),
                        ("inbox_rank_stride", 8 * 512 * 4 - 16), ("output_offset", L.region),
                        ("incoming_host_mask", 1), ("deadline_cycles", 0)):
        broken = R.OrderedRowsPushDescription.from_buffer_copy(bytes(push))
        setattr(broken.arguments.push, path, value)
        assert lib.ordered_rows_push_prepare(C.byref(broken), C.byref(fake.table), fake.card, one) != 0, path
    for path, value in (("width", 510), ("pairs_per_row", 0), ("pair_output_offset", L.result)):
        broken = R.OrderedRowsPushDescription.from_buffer_copy(bytes(push))
        setattr(broken.arguments, path, value)
        assert lib.ordered_rows_push_prepare(C.byref(broken), C.byref(fake.table), fake.card, one) == 1, path
    assert bytes(one) == untouched


# ---- byte for byte against the reference's own preparers (oracle/_ref) ----

def test_reconstruct_and_collective_launches_equal_reference(reference):
    lib = api.library()
    record = R.Exl3Reconstruct(0, 1 << 20, 256, 384, 3, 0)
    ours, theirs = R.KernelLaunch(), R.KernelLaunch()
    reference.exl3_reconstruct_prepare.argtypes = lib.exl3_reconstruct_prepare.argtypes
    assert lib.exl3_reconstruct_prepare(C.byref(record), 1 << 22, 5, C.byref(ours)) == 0
    assert reference.exl3_reconstruct_prepare(C.byref(record), 1 << 22, 5, C.byref(theirs)) == 0
    assert bytes(ours) == bytes(theirs)
    for field, value in (("matrix_offset", 32), ("output_offset", 1 << 22), ("bits_per_weight", 5), ("input_size", 100)):
        broken = R.Exl3Reconstruct.from_buffer_copy(bytes(record))
        setattr(broken, field, value)
        assert lib.exl3_reconstruct_prepare(C.byref(broken), 1 << 22, 5, C.byref(ours)) == \
            reference.exl3_reconstruct_prepare(C.byref(broken), 1 << 22, 5, C.byref(theirs)) != 0
    kernels = R.OrderedCollectiveKernels((C.c_uint32 * 4)(3, 4, 5, 6))
    prototype = [C.POINTER(R.OrderedCollectiveDescription), C.POINTER(R.OrderedCollectiveKernels),
                 C.POINTER(R.KernelLaunch)]
    lib.ordered_collective_prepare.argtypes = reference.ordered_collective_prepare.argtypes = prototype
    good = R.OrderedCollective(0, 4096, 384, 384 + 4096, 384 + 8192, 1024, 16384, 1000, 1000, 4, 2, 0)
    cases = [good]
    for field, value in (("rank", 4), ("element_count", 0), ("element_count", 300000), ("region_offset", 4100),
                         ("input_offset", 100), ("scratch_offset", 384 + 4096), ("deadline_cycles", 0),
                         ("step_offset", 4096), ("peer_table_offset", 4), ("parity_stride", 8192)):
        broken = R.OrderedCollective.from_buffer_copy(bytes(good))
        setattr(broken, field, value)
        cases.append(broken)
    for arguments in cases:
        for operation in range(4):
            description = R.OrderedCollectiveDescription(arguments, 1 << 20, operation)
            ours, theirs = R.KernelLaunch(), R.KernelLaunch()
            a = lib.ordered_collective_prepare(C.byref(description), C.byref(kernels), C.byref(ours))
            b = reference.ordered_collective_prepare(C.byref(description), C.byref(kernels), C.byref(theirs))
            assert a == b and bytes(ours) == bytes(theirs)


def test_output_shard_plan_and_slice_copy_equal_reference(reference):
    lib = api.library()
    prototype = [C.c_uint32] * 5 + [C.c_int, C.POINTER(ShardPlan)]
    lib.bb_exl3_output_shard_prepare.argtypes = reference.bb_exl3_output_shard_prepare.argtypes = prototype
    copy_prototype = [C.POINTER(Slice), C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t]
    lib.bb_exl3_matrix_slice_copy.argtypes = reference.bb_exl3_matrix_slice_copy.argtypes = copy_prototype
    rng = np.random.default_rng(12)
    for stored in (2, 40, 3, 4):
        for ranks in (1, 4):
            for rank in range(ranks):
                ours, theirs = ShardPlan(), ShardPlan()
                assert lib.bb_exl3_output_shard_prepare(5120, 2304, stored, ranks, rank, 0, C.byref(ours)) == 0
                assert reference.bb_exl3_output_shard_prepare(5120, 2304, stored, ranks, rank, 0, C.byref(theirs)) == 0
                assert bytes(ours) == bytes(theirs)
        matrix = synthetic.exl3_matrix(rng, 256, 384, stored)
        piece = Slice(256, 384, 128, 128, 128, 256, stored, 0)
        size = synthetic.matrix_bytes(128, 256, stored)
        a, b = np.zeros(size, dtype=np.uint8), np.ones(size, dtype=np.uint8)
        assert lib.bb_exl3_matrix_slice_copy(C.byref(piece), matrix.ctypes.data, matrix.size, a.ctypes.data, size) == 0
        assert reference.bb_exl3_matrix_slice_copy(C.byref(piece), matrix.ctypes.data, matrix.size, b.ctypes.data,
                                                   size) == 0
        assert np.array_equal(a, b)
        assert lib.bb_exl3_matrix_slice_copy(C.byref(piece), matrix.ctypes.data, matrix.size, a.ctypes.data,
                                             size - 1) == 1


def test_collective_host_equals_reference(reference):
    from oracle.binding import f32p, pointer_array
    lib = api.library()
    lib.ordered_collective_host.argtypes = [C.POINTER(f32p), C.POINTER(f32p), C.c_uint32, C.c_uint32, C.c_int]
    rng = np.random.default_rng(2)
    inputs = [rng.normal(0, 0.05, 999).astype(np.float32) for _ in range(5)]
    inputs[0][0], inputs[2][0] = 16777216.0, -16777216.0
    for operation in range(4):
        ours = [np.full(999, -99, dtype=np.float32) for _ in range(5)]
        theirs = [np.full(999, -99, dtype=np.float32) for _ in range(5)]
        assert lib.ordered_collective_host(pointer_array(inputs), pointer_array(ours), 5, 999, operation) == 0
        assert reference.ordered_collective_host(pointer_array(inputs), pointer_array(theirs), 5, 999, operation) == 0
        for a, b in zip(ours, theirs):
            assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    assert lib.ordered_collective_host(pointer_array(inputs), pointer_array(inputs), 5, 999, 0) == 1  # overlap


def layer_description(rows=8, hidden=4096, inner=2048, experts=256, picks=8, ranks=1):
    """A decode step's description laid out in an arena, for exl3_layer_prepare (fake card: nothing is read)."""
    slots, jobs = picks + 1, rows * picks + 1
    pairs = rows * slots
    sizes = api.layer_sizes(pairs, jobs, hidden, inner)
    layout = api.Layout(256)
    description = R.Exl3LayerDescription()
    route = description.route
    peer_table, status, step = layout.take(16 * 32), layout.take(16), layout.take(16)
    stride = api.align(R.EXL3_LAYER_SIGNAL_BYTES + rows * hidden * 4, 128)
    region = layout.take(2 * stride, 128)
    products = layout.take(max(sizes.product_bytes, pairs * hidden * 8))
    route.moe.base = R.Exl3Expert(layout.take(jobs * 96), layout.take(rows * hidden * 2), layout.take(sizes.operand_bytes),
                                  products, layout.take(pairs * inner * 2), products, hidden, inner, pairs, slots, jobs,
                                  R.EXL3_WIDTH_PER_EXPERT, 10.0, 0)
    route.moe.widths_offset, route.moe.row_output_offset = layout.take((experts + 1) * 4), layout.take(rows * hidden * 4)
    route.moe.counters_offset, route.moe.expert_count = layout.take(sizes.counter_bytes), experts + 1
    route.scores_offset, route.expert_table_offset = layout.take(rows * experts * 4), layout.take((experts + 1) * 24)
    route.picks_offset, route.weights_offset = layout.take(rows * picks * 4), layout.take(rows * picks * 4)
    route.step_offset, route.routed_count, route.shared_count, route.picks, route.row_capacity = step, experts, 1, picks, rows
    route.scoring, route.route_scale = 0, 1.0
    description.publish = R.Exl3LayerPublish(peer_table, region, R.EXL3_LAYER_SIGNAL_BYTES, status, step, stride,
                                             1_000_000, ranks, 0, rows, 0)
    description.result_offset = layout.take(rows * hidden * 2)
    description.arena_byte_count = layout.take(0, 4096) + 4096
    return description, sizes


def test_layer_prepare_three_launches():
    lib, fake = api.library(), FakeBackend()
    for inner, runs in ((2048, 4), (1024, 4), (512, 8), (256, 8)):  # one, two, four and eight ranks' shares
        description, sizes = layer_description(inner=inner)
        assert sizes.product_bytes == (2 * 16 * 72 * inner + 16 * 72 * 4096) * 4  # gate/up's, then down's own
        assert sizes.counter_bytes == (65 * (inner // 128 + 32) + 4 + 65) * 4
        launches = (R.KernelLaunch * R.EXL3_LAYER_LAUNCHES)()
        assert lib.exl3_layer_prepare(C.byref(description), C.byref(fake.table), fake.card, launches) == 0
        assert [key[1] for key in fake.asked[-3:]] == ["exl3_layer_route_input", "exl3_layer_products",
                                                       "ordered_publish_reduce_flags"]
        assert [key[2] for key in fake.asked[-3:]] == [184, 128, 104]
        route, products, reduce = launches
        assert tuple(route.block) == (1024, 1, 1) and route.grid[0] == 1 + 8 * 9 * 2 * 32 // 32 and route.branch == 0
        # a CTA an item: every job's gate and up items (two matrices x groups x runs), then its down items
        assert tuple(products.grid) == (65 * (2 * (inner // 128) * runs + 32), 1, 1) and products.block[0] == 128
        assert products.branch == reduce.branch == 0x100  # each is given its place while the one before it runs
        record = R.Exl3LayerProducts.from_buffer_copy(bytes(products.argument[:128]))
        assert (record.gate_up_runs, record.down_runs) == (runs, 1)
        assert record.down_products_offset == description.route.moe.base.products_offset + 2 * 16 * 72 * inner * 4
        publish = R.OrderedPublishReduce.from_buffer_copy(bytes(reduce.argument[:104]))
        assert publish.pair_output_offset == record.down_products_offset  # run 0 of down's sums: the pair outputs
    # the caller's cut; refusals leave the table untouched
    description, _ = layer_description()
    description.gate_up_runs, description.down_runs = 2, 2
    launches = (R.KernelLaunch * R.EXL3_LAYER_LAUNCHES)()
    assert lib.exl3_layer_prepare(C.byref(description), C.byref(fake.table), fake.card, launches) == 0
    assert launches[1].grid[0] == 65 * (2 * 16 * 2 + 32 * 2)
    untouched = bytes(launches)
    for change in (dict(gate_up_runs=3), dict(gate_up_runs=64), dict(down_runs=32)):
        bad, _ = layer_description()
        for name, value in change.items():
            setattr(bad, name, value)
        assert lib.exl3_layer_prepare(C.byref(bad), C.byref(fake.table), fake.card, launches) == 1
        assert bytes(launches) == untouched
    bad, _ = layer_description()
    bad.route.moe.counters_offset = bad.route.moe.base.products_offset  # overlaps the partial sums
    assert lib.exl3_layer_prepare(C.byref(bad), C.byref(fake.table), fake.card, launches) == 1
    assert bytes(launches) == untouched


def test_router_wide_prepare():
    """The job table of many rows: three launches (the prefill's picks and grouping, then router_wide_jobs)."""
    lib, fake = api.library(), FakeBackend()
    lib.router_wide_prepare.argtypes = [C.POINTER(R.RouterWide), C.c_uint64, C.POINTER(api.BackendOperations),
                                        C.c_void_p, C.POINTER(R.KernelLaunch)]
    rows, experts, picks, hidden, inner = 2048, 256, 8, 4096, 256

    def arguments(**changes):
        layout = api.Layout(256)
        routing = R.Exl3Prefill()
        routing.scores_offset, routing.expert_table_offset = layout.take(rows * experts * 4), layout.take(experts * 24)
        routing.picks_offset, routing.weights_offset = layout.take(rows * picks * 4), layout.take(rows * picks * 4)
        parts = api.prefill_parts(rows, picks, 0, experts, hidden, inner)
        routing.workspace_offset, routing.step_offset = layout.take(parts.gate_up_operands, 1024), layout.take(16)
        routing.input_size, routing.inner_size, routing.expert_count, routing.local_count = hidden, inner, experts, experts
        routing.picks, routing.row_capacity, routing.scoring, routing.route_scale = picks, rows, 0, 1.0
        value = R.RouterWide(routing, layout.take((rows * picks // 8 + experts) * 96), rows * picks // 8 + experts, 0)
        for name, change in changes.items():
            if hasattr(value, name):
                setattr(value, name, change)
            else:
                setattr(value.routing, name, change)
        return value, layout.take(0, 4096) + 4096
    value, arena = arguments()
    launches = (R.KernelLaunch * R.ROUTER_WIDE_LAUNCHES)()
    assert lib.router_wide_prepare(C.byref(value), arena, C.byref(fake.table), fake.card, launches) == 0
    assert fake.asked == [("kernel_exl3_prefill", "exl3_prefill_picks", 136), ("kernel_exl3_prefill", "exl3_prefill_group", 136),
                          ("kernel_router_b200", "router_wide_jobs", 152)]
    assert [tuple(l.grid) for l in launches] == [(rows // 32, 1, 1), (experts, 1, 1), (1, 1, 1)]
    assert [l.block[0] for l in launches] == [1024, 256, 1024]
    assert bytes(launches[2].argument[:152]) == bytes(value) and bytes(launches[0].argument[:136]) == bytes(value.routing)
    untouched = bytes(launches)
    for change in (dict(job_capacity=rows * picks // 8 + experts - 1), dict(shared_count=1), dict(local_first=1),
                   dict(local_count=experts - 1), dict(picks=17), dict(expert_count=513), dict(row_capacity=0),
                   dict(route_scale=0.0), dict(scoring=2), dict(reserved_zero=1), dict(jobs_offset=8),
                   dict(workspace_offset=256 + 512)):
        bad, size = arguments(**change)
        assert lib.router_wide_prepare(C.byref(bad), size, C.byref(fake.table), fake.card, launches) == 1, change
        assert bytes(launches) == untouched
    assert lib.router_wide_prepare(C.byref(value), arena - 8192, C.byref(fake.table), fake.card, launches) == 1


def test_routed_experts_wide_prepare():
    """The routed experts for a job table of many rows: the thin preparer's four launches with the two product
    launches given to the group kernels (slice counts and the job count in their records), and its refusals."""
    lib, fake = api.library(), FakeBackend()
    lib.linear_kernels_prepare.argtypes = [C.POINTER(api.BackendOperations), C.c_void_p, C.c_uint32,
                                           C.POINTER(R.LinearKernels)]
    kernels = R.LinearKernels()
    assert lib.linear_kernels_prepare(C.byref(fake.table), fake.card, 100, C.byref(kernels)) == 0
    thin_prepare, wide_prepare = lib.linear_routed_experts_prepare, lib.linear_routed_experts_wide_prepare
    thin_prepare.argtypes = [C.POINTER(R.LinearRoutedExpertsDescription), C.c_uint64, C.POINTER(R.LinearKernels),
                             C.POINTER(R.KernelLaunch)]
    wide_prepare.argtypes = [C.POINTER(R.LinearRoutedExpertsDescription), C.c_uint64, C.POINTER(R.LinearKernels),
                             C.POINTER(api.BackendOperations), C.c_void_p, C.POINTER(R.KernelLaunch)]

    def description(H=512, I=256, rows=64, picks=3, jobs=37, slices=(2, 4)):
        layout, pairs = api.Layout(256), rows * picks
        d = R.LinearRoutedExpertsDescription()
        sizes = dict(jobs=jobs * 96, expert_weights=max(I * H, H * I) // 2 + max(I * H, H * I) // 32,
                     codes=rows * H, exponents=rows * H // 32, operands=rows * H * 2, hidden=pairs * I * 2,
                     hidden_codes=pairs * I, hidden_exponents=pairs * I // 32, hidden_operands=pairs * I * 2,
                     pair_output=pairs * H * 2, row_output=rows * H * 4)
        for name, size in sizes.items():
            setattr(d, name, R.LinearRange(layout.take(size, 64), size))
        d.gate_up_shape, d.down_shape = R.MatrixShape(I, H, 4, 0), R.MatrixShape(H, I, 4, 0)
        d.weight_format, d.job_count, d.row_count, d.pairs_per_row = 3, jobs, rows, picks  # WEIGHT_FORMAT_E2M1_SCALED
        d.gate_up_slice_count, d.down_slice_count = slices
        d.activation_limit = 7.0
        return d, layout.take(0, 4096) + 4096
    d, arena = description()
    thin, wide = (R.KernelLaunch * 4)(), (R.KernelLaunch * 4)()
    assert thin_prepare(C.byref(d), arena, C.byref(kernels), thin) == 0
    assert wide_prepare(C.byref(d), arena, C.byref(kernels), C.byref(fake.table), fake.card, wide) == 0
    assert ("kernel_expert_linear", "expert_gate_up_many", 72) in fake.asked
    assert ("kernel_expert_linear", "expert_down_many", 64) in fake.asked
    groups = (37 + R.LINEAR_MANY_JOBS - 1) // R.LINEAR_MANY_JOBS
    assert tuple(wide[0].grid) == (256 // 64, groups, 1) and tuple(wide[2].grid) == (512 // 128, groups, 1)
    assert wide[0].block[0] == 256 and wide[2].block[0] == 256
    gate_up = R.ExpertGateUpMany.from_buffer_copy(bytes(wide[0].argument[:72]))
    down = R.ExpertDownMany.from_buffer_copy(bytes(wide[2].argument[:64]))
    assert bytes(gate_up.base) == bytes(thin[0].argument[:64]) and (gate_up.slice_count, gate_up.job_count) == (2, 37)
    assert bytes(down.base) == bytes(thin[2].argument[:56]) and (down.slice_count, down.job_count) == (4, 37)
    assert bytes(wide[1]) == bytes(thin[1]) and bytes(wide[3]) == bytes(thin[3])  # quantization and row sum as they were
    assert wide[0].kernel != thin[0].kernel and wide[2].kernel != thin[2].kernel
    untouched = bytes(wide)
    for change in (dict(I=224), dict(H=448), dict(slices=(3, 1)), dict(jobs=0)):
        bad, size = description(**change)
        assert wide_prepare(C.byref(bad), size, C.byref(kernels), C.byref(fake.table), fake.card, wide) == 1, change
        assert bytes(wide) == untouched
    assert wide_prepare(C.byref(d), arena, C.byref(kernels), None, fake.card, wide) == 1
    assert wide_prepare(C.byref(d), arena - 8192, C.byref(kernels), C.byref(fake.table), fake.card, wide) == 1


def test_router_select_quantize_prepare():
    """The router and the rows' quantizer as one launch: both records taken over as their own preparers accept them."""
    lib, fake = api.library(), FakeBackend()
    lib.linear_kernels_prepare.argtypes = [C.POINTER(api.BackendOperations), C.c_void_p, C.c_uint32,
                                           C.POINTER(R.LinearKernels)]
    kernels = R.LinearKernels()
    assert lib.linear_kernels_prepare(C.byref(fake.table), fake.card, 100, C.byref(kernels)) == 0
    lib.linear_quantize_prepare.argtypes = [C.POINTER(R.LinearQuantizeDescription), C.c_uint64,
                                            C.POINTER(R.LinearKernels), C.POINTER(R.KernelLaunch)]
    lib.router_select_quantize_prepare.argtypes = [C.POINTER(R.RouterSelectB200), C.POINTER(R.KernelLaunch), C.c_uint64,
                                                   C.POINTER(api.BackendOperations), C.c_void_p,
                                                   C.POINTER(R.KernelLaunch)]
    rows, experts, picks, H = 8, 64, 4, 1024
    layout = api.Layout(256)
    scores, table = layout.take(rows * experts * 4), layout.take(experts * 24)
    picked, weights, jobs = layout.take(rows * picks * 4), layout.take(rows * picks * 4), layout.take(rows * picks * 96)
    step, values = layout.take(16), layout.take(rows * H * 2)
    codes, exponents, operands = layout.take(rows * H), layout.take(rows * H // 32), layout.take(rows * H * 2)
    arena = layout.take(0, 4096) + 4096
    router = R.RouterSelectB200(scores, table, picked, weights, jobs, step, experts, 0, picks, rows, rows * picks, 0,
                                1.0, 0)
    quantize = R.LinearQuantizeDescription(R.LinearRange(values, rows * H * 2), R.LinearRange(codes, rows * H),
                                           R.LinearRange(exponents, rows * H // 32),
                                           R.LinearRange(operands, rows * H * 2), H, rows)
    quantize_launch, launch = R.KernelLaunch(), R.KernelLaunch()
    assert lib.linear_quantize_prepare(C.byref(quantize), arena, C.byref(kernels), C.byref(quantize_launch)) == 0
    assert lib.router_select_quantize_prepare(C.byref(router), C.byref(quantize_launch), arena, C.byref(fake.table),
                                              fake.card, C.byref(launch)) == 0
    assert ("kernel_router_b200", "router_select_quantize", 136) in fake.asked
    assert tuple(launch.grid) == (1 + (rows * H // 64 + 31) // 32, 1, 1) and launch.block[0] == 1024
    record = R.RouterSelectQuantize.from_buffer_copy(bytes(launch.argument[:136]))
    assert bytes(record.router) == bytes(router) and bytes(record.quantize) == bytes(quantize_launch.argument[:40])
    assert record.vector_count == rows and record.reserved_zero == 0
    untouched = bytes(launch)
    bad = R.RouterSelectB200.from_buffer_copy(bytes(router))
    bad.picks = 17
    assert lib.router_select_quantize_prepare(C.byref(bad), C.byref(quantize_launch), arena, C.byref(fake.table),
                                              fake.card, C.byref(launch)) == 1
    other = R.KernelLaunch.from_buffer_copy(bytes(quantize_launch))
    other.block[0] = 64
    assert lib.router_select_quantize_prepare(C.byref(router), C.byref(other), arena, C.byref(fake.table), fake.card,
                                              C.byref(launch)) == 1
    assert lib.router_select_quantize_prepare(C.byref(router), None, arena, C.byref(fake.table), fake.card,
                                              C.byref(launch)) == 1
    assert bytes(launch) == untouched


def test_publish_reduce_bf16_prepare():
    """The original-weights decode step's reduction as one launch: its record, its grid and its refusals; the step
    entries of the card interface refuse a card that is not there."""
    lib, fake = api.library(), FakeBackend()
    from anemone_b200.moe import MoeConfig
    from anemone_b200.mx import MxLayout
    config = MoeConfig(hidden=512, inner=256, experts=12, shared=1, picks=3, row_capacity=8, activation_limit=7.0)
    L = MxLayout(config, 2, 1)
    assert L.flags and L.slot_input == R.EXL3_LAYER_SIGNAL_BYTES
    prepare = lib.ordered_publish_reduce_bf16_prepare
    prepare.argtypes = [C.POINTER(R.OrderedReduceBf16Description), C.c_uint64, C.c_uint64,
                        C.POINTER(api.BackendOperations), C.c_void_p, C.POINTER(R.KernelLaunch)]
    description = R.OrderedReduceBf16Description()
    description.reduce.collective = R.OrderedCollective(L.peer_table, L.region, L.slot_input, L.result, 0, L.step,
                                                        L.parity_stride, 1000, 8 * 512, 2, 1, 0)
    description.reduce.status_offset, description.reduce.width = L.status, 512
    description.pair_output_offset, description.arena_byte_count = L.at["pair_output"], L.arena_bytes
    description.pairs_per_row, description.row_capacity = 3, 8
    launch = R.KernelLaunch()
    addend, rows_at = L.shared_at["output"], L.at["row_output"]
    assert prepare(C.byref(description), addend, rows_at, C.byref(fake.table), fake.card, C.byref(launch)) == 0
    assert fake.asked[-1] == ("kernel_ordered_b200", "ordered_publish_reduce_flags_bf16", 120)
    assert tuple(launch.grid) == (4, 1, 1) and launch.block[0] == 256 and launch.argument_byte_count == 120
    record = R.OrderedPublishReduceBf16.from_buffer_copy(bytes(launch.argument[:120]))
    assert bytes(record.base.collective) == bytes(description.reduce.collective)
    assert (record.base.status_offset, record.base.pair_output_offset, record.base.width, record.base.pairs_per_row,
            record.addend_offset, record.row_output_offset) == (L.status, L.at["pair_output"], 512, 3, addend, rows_at)
    assert prepare(C.byref(description), 0, 0, C.byref(fake.table), fake.card, C.byref(launch)) == 0  # neither
    untouched = bytes(launch)
    for path, value in (("rank", 2), ("rank_count", 17), ("deadline_cycles", 0), ("region_offset", L.region + 64),
                        ("input_offset", R.EXL3_LAYER_SIGNAL_BYTES - 128), ("parity_stride", L.parity_stride - 128),
                        ("scratch_offset", 16)):
        broken = R.OrderedReduceBf16Description.from_buffer_copy(bytes(description))
        setattr(broken.reduce.collective, path, value)
        assert prepare(C.byref(broken), addend, rows_at, C.byref(fake.table), fake.card, C.byref(launch)) == 1, path
    for change in (dict(width=510), dict(mode=R.ORDERED_REDUCE_OWNER_RUNS)):
        broken = R.OrderedReduceBf16Description.from_buffer_copy(bytes(description))
        for name, value in change.items():
            setattr(broken.reduce, name, value)
        assert prepare(C.byref(broken), addend, rows_at, C.byref(fake.table), fake.card, C.byref(launch)) == 1, change
    assert prepare(C.byref(description), addend + 8, rows_at, C.byref(fake.table), fake.card, C.byref(launch)) == 1
    assert prepare(C.byref(description), addend, L.region, C.byref(fake.table), fake.card, C.byref(launch)) == 1
    assert bytes(launch) == untouched
    graph = C.c_uint32(7)
    assert lib.backend_b200_step_capture(None, launch, 1, 0, None, 0, 0, None, 0, C.byref(graph)) == 1
    assert lib.backend_b200_graph_run_wait(None, 0) == 1 and graph.value == 7
