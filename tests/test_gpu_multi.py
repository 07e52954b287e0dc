"""Real multi-GPU runs of the reduction and of the tensor-parallel layer: one process driving R cards (the reference's
arrangement), peer loads over NVLink. Skipped on a machine with fewer than two GPUs; every rank's kernels are queued
before the host waits for any, and every device wait is bounded."""
import ctypes as C

import numpy as np
import pytest

from anemone_b200 import records as R
from anemone_b200 import synthetic
from anemone_b200.moe import MoeConfig, MoeLayer, MoeLayout, local_matrices
from oracle import moe_reference
from oracle.binding import f32p, pointer_array, ptr, u16p

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    from anemone_b200 import api as module
    if module.card_count() < 2:
        pytest.skip("needs at least two GPUs")
    return module


def world_sizes(api):
    return [size for size in (2, 4, 8) if size <= api.card_count()]


@pytest.mark.parametrize("form", ["fused", "push", "pull"])
def test_layer_tensor_parallel(api, oracle, form):
    for ranks in world_sizes(api):
        config = MoeConfig(hidden=512, inner=128 * ranks * 2, experts=24, shared=1, picks=4, row_capacity=8)
        rng = np.random.default_rng(300 + ranks)
        widths = np.concatenate([synthetic.expert_widths(rng, config.experts), [3]]).astype(np.uint32)
        matrices = [(synthetic.exl3_matrix(rng, config.hidden, config.inner, int(w)),
                     synthetic.exl3_matrix(rng, config.hidden, config.inner, int(w)),
                     synthetic.exl3_matrix(rng, config.inner, config.hidden, int(w))) for w in widths]
        cards, layers = [], []
        try:
            for rank in range(ranks):
                card = api.Card(rank, MoeLayout(config, widths, ranks, rank, reduce_form=form).arena_bytes)
                cards.append(card)
                local = [local_matrices(*matrices[e], config, int(widths[e]), ranks, rank)
                         for e in range(config.total_experts)]
                layers.append(MoeLayer(card, config, widths, local, rank=rank, rank_count=ranks, reduce_form=form))
            for layer in layers:
                layer.connect_local(layers)
            for card in cards:
                card.wait()
            for step in range(4):
                rows = [8, 3, 8, 1][step]
                tokens = synthetic.tokens(rng, rows, config.hidden)
                scores = rng.normal(0, 1, size=(rows, config.experts)).astype(np.float32)
                expected, partials, _, _ = moe_reference.layer(oracle, config, widths, matrices, tokens, scores, ranks)
                result_at = api.align(layers[0].layout.step_input_bytes, 4096)
                tickets = []
                for layer in layers:  # queue every rank before waiting for any
                    layer.sequence += 1
                    layer.stage_step(0, layer.sequence, tokens, scores)
                    tickets.append(layer.submit(0, result_at, rows))
                outputs = []
                for layer, ticket in zip(layers, tickets):
                    layer.card.transfer_wait(ticket)
                    layer.check_status()
                    nbytes = rows * config.hidden * 2
                    outputs.append(layer.card.staging_view[result_at:result_at + nbytes].view(np.uint16).copy())
                for rank in range(1, ranks):  # every rank holds the same bits
                    assert np.array_equal(outputs[rank], outputs[0])
                a = synthetic.from_bfloat16(outputs[0])
                b = synthetic.from_bfloat16(expected.reshape(-1))
                assert np.abs(a - b).max() <= 2e-2
                assert float(a.astype(np.float64) @ b.astype(np.float64)) / (np.linalg.norm(a) * np.linalg.norm(b)) >= 0.9999
                # bit-exact ordered reduction: re-reduce the FP32 rows the ranks actually published, on the CPU oracle
                published = []
                for layer in layers:
                    L = layer.layout
                    slot = L.region + (layer.sequence & 1) * L.parity_stride + L.slot_input
                    published.append(layer.card.download(slot, rows * config.hidden * 4, np.float32))
                want = np.zeros(rows * config.hidden, dtype=np.uint16)
                oracle.orc_ordered_reduce_bf16(pointer_array(published), ranks, want.size, ptr(want, u16p))
                assert np.array_equal(outputs[0], want)
        finally:
            for card in cards:
                card.close()


def test_fp32_all_reduce_across_cards(api, oracle):
    lib = api.library()
    lib.ordered_collective_kernels_prepare.argtypes = [C.POINTER(api.BackendOperations), C.c_void_p,
                                                       C.POINTER(R.OrderedCollectiveKernels)]
    lib.ordered_collective_prepare.argtypes = [C.POINTER(R.OrderedCollectiveDescription),
                                               C.POINTER(R.OrderedCollectiveKernels), C.POINTER(R.KernelLaunch)]
    for ranks in world_sizes(api):
        elements = 8 * 4096
        rng = np.random.default_rng(500 + ranks)
        inputs = [rng.normal(0, 0.05, elements).astype(np.float32) for _ in range(ranks)]
        inputs[0][0], inputs[1][0] = 16777216.0, 1.0
        layout = api.Layout()
        peer_table, step = layout.take(16 * 32), layout.take(16)
        stride = api.align(384 + 12 * elements, 128)
        region = layout.take(2 * stride, 128)
        arena_bytes = layout.take(4096, 4096)
        cards = [api.Card(rank, arena_bytes) for rank in range(ranks)]
        try:
            launches = {}
            for rank, card in enumerate(cards):
                card.fill(0, 0, arena_bytes)
                peers = (R.OrderedPeer * ranks)()
                for peer in range(ranks):
                    peers[peer].region_offset = region
                card.upload(peer_table, np.frombuffer(bytes(peers), dtype=np.uint8))
                for peer, other in enumerate(cards):
                    card.peer_connect(other, 0, peer_table + 32 * peer)
                kernels = R.OrderedCollectiveKernels()
                api.check(lib.ordered_collective_kernels_prepare(card.ops_pointer, card.handle, C.byref(kernels)), "k")
                for operation in (0, 1):
                    arguments = R.OrderedCollective(peer_table, region, 384, 384 + 4 * elements, 384 + 8 * elements,
                                                    step, stride, 2_000_000_000, elements, ranks, rank, 0)
                    description = R.OrderedCollectiveDescription(arguments, arena_bytes, operation)
                    launch = R.KernelLaunch()
                    api.check(lib.ordered_collective_prepare(C.byref(description), C.byref(kernels), C.byref(launch)),
                              "prepare")
                    launches[(rank, operation)] = launch
            expected = np.zeros(elements, dtype=np.float32)
            oracle.orc_ordered_sum(pointer_array(inputs), ranks, elements, ptr(expected, f32p))
            sequence = 0
            for operation in (0, 1, 0, 1):
                sequence += 1
                for rank, card in enumerate(cards):
                    card.upload(step, np.frombuffer(bytes(R.StepBlock(sequence, 1, 0)), dtype=np.uint8))
                    card.upload(region + (sequence & 1) * stride + 384, inputs[rank])
                for rank, card in enumerate(cards):
                    card.run([launches[(rank, operation)]])
                for rank, card in enumerate(cards):
                    card.wait()
                    got = card.download(region + (sequence & 1) * stride + 384 + 4 * elements, 4 * elements, np.float32)
                    assert np.array_equal(got.view(np.uint32), expected.view(np.uint32)), (ranks, operation, rank)
        finally:
            for card in cards:
                card.close()


@pytest.mark.parametrize("mode", [0, 1])
def test_prefill_expert_parallel(api, oracle, mode):
    """Prefill over R cards, each holding a run of the routed experts and a column slice of the always-on one; the
    ordered reduction adds the ranks' rows (mode 1: every rank its run of the result, stored into every rank)."""
    from anemone_b200.prefill import PrefillLayer, PrefillLayout, Share
    for ranks in world_sizes(api):
        config = MoeConfig(hidden=512, inner=128 * ranks, experts=8 * ranks, shared=1, picks=4, row_capacity=333)
        rng = np.random.default_rng(500 + ranks)
        widths = np.concatenate([synthetic.expert_widths(rng, config.experts), [3]]).astype(np.uint32)
        matrices = [(synthetic.exl3_matrix(rng, config.hidden, config.inner, int(w)),
                     synthetic.exl3_matrix(rng, config.hidden, config.inner, int(w)),
                     synthetic.exl3_matrix(rng, config.inner, config.hidden, int(w))) for w in widths]
        cards, layers = [], []
        try:
            for rank in range(ranks):
                share = Share.expert_parallel(config, ranks, rank)
                held = share.experts(config)
                card = api.Card(rank, PrefillLayout(config, widths[held], share).arena_bytes)
                cards.append(card)
                local = [share.matrices(config, e, int(widths[e]), *matrices[e]) for e in held]
                layers.append(PrefillLayer(card, config, widths[held], local, share, rank=rank, rank_count=ranks,
                                           reduce_mode=mode))
            for layer in layers:
                layer.connect_local(layers)
            for card in cards:
                card.wait()
            for rows in (333, 40, 333):
                tokens = synthetic.tokens(rng, rows, config.hidden)
                scores = rng.normal(0, 1, size=(rows, config.experts)).astype(np.float32)
                scores[:, :3] += 1.5  # the first rank gets more pairs than the others
                experts, weights = moe_reference.route(oracle, config, scores)
                expected = moe_reference.rank_partial(oracle, config, widths, matrices, tokens, experts, weights, 1, 0)[0]
                for layer in layers:  # queue every rank before waiting for any
                    layer.load(tokens, scores)
                for layer in layers:
                    layer.run()
                outputs = [layer.result(rows).reshape(-1) for layer in layers]
                for rank in range(1, ranks):  # every rank holds the same bits
                    assert np.array_equal(outputs[rank], outputs[0])
                a = synthetic.from_bfloat16(outputs[0]).reshape(rows, config.hidden)
                assert np.abs(a - expected).max() <= 2e-2
                assert float(a.astype(np.float64).reshape(-1) @ expected.astype(np.float64).reshape(-1)) / \
                    (np.linalg.norm(a) * np.linalg.norm(expected)) >= 0.9999
                # bit-exact ordered reduction of the FP32 rows the ranks computed
                partials = [layer.rows(rows).reshape(-1).copy() for layer in layers]
                want = np.zeros(rows * config.hidden, dtype=np.uint16)
                oracle.orc_ordered_reduce_bf16(pointer_array(partials), ranks, want.size, ptr(want, u16p))
                assert np.array_equal(outputs[0], want)
        finally:
            for card in cards:
                card.close()


@pytest.mark.parametrize("payload", [0, 1])
def test_push_and_owner_sums_across_cards(api, oracle, payload):
    """The one-shot push and the exchange's owner sums between real cards: every rank stores into every rank's inbox
    over NVLink, every wait polls local memory; FP32 sums and bfloat16 owner sums bit for bit on every rank."""
    lib = api.library()
    lib.ordered_push_kernel_prepare.argtypes = [C.POINTER(api.BackendOperations), C.c_void_p, C.POINTER(C.c_uint32)]
    lib.ordered_push_prepare.argtypes = [C.POINTER(R.OrderedPushDescription), C.c_uint32, C.POINTER(R.KernelLaunch)]
    lib.tp_exchange_wide_kernels_prepare.argtypes = [C.POINTER(api.BackendOperations), C.c_void_p, C.c_uint32,
                                                     C.POINTER(C.c_uint32)]
    lib.tp_exchange_wide_rows_prepare.argtypes = [C.POINTER(R.OrderedPushDescription), C.c_uint32, C.c_uint32,
                                                  C.c_uint32, C.POINTER(C.c_uint32), C.c_uint32,
                                                  C.POINTER(R.KernelLaunch)]
    width, capacity, layers = 4096, 64, 2
    elements = width * capacity
    for ranks in world_sizes(api):
        rng = np.random.default_rng(700 + ranks + payload)
        layout = api.Layout()
        peer_table, step = layout.take(16 * 32), layout.take(16)
        signals = 2 * ranks * 128
        input_at, output_at, inbox_at = signals, signals + 4 * elements, signals + 8 * elements
        stride = api.align(inbox_at + ranks * 4 * elements, 128)
        region = layout.take(2 * stride, 128)
        arena_bytes = layout.take(4096, 4096)
        cards = [api.Card(rank, arena_bytes) for rank in range(ranks)]
        try:
            push, owner = {}, {}
            for rank, card in enumerate(cards):
                card.fill(0, 0, arena_bytes)
                peers = (R.OrderedPeer * ranks)()
                for peer in range(ranks):
                    peers[peer].region_offset = region
                card.upload(peer_table, np.frombuffer(bytes(peers), dtype=np.uint8))
                for peer, other in enumerate(cards):
                    card.peer_connect(other, 0, peer_table + 32 * peer)
                arguments = R.OrderedPush(peer_table, region, input_at, output_at, inbox_at, step, stride,
                                          2_000_000_000, 4 * elements, elements, ranks, rank, payload, 0, 0)
                description = R.OrderedPushDescription(arguments, arena_bytes)
                kernel = C.c_uint32()
                api.check(lib.ordered_push_kernel_prepare(card.ops_pointer, card.handle, C.byref(kernel)), "kernel")
                push[rank] = R.KernelLaunch()
                api.check(lib.ordered_push_prepare(C.byref(description), kernel.value, C.byref(push[rank])), "push")
                kernels = (C.c_uint32 * 4)()
                api.check(lib.tp_exchange_wide_kernels_prepare(card.ops_pointer, card.handle, 1, kernels), "kernels")
                for layer in range(layers):
                    owner[(rank, layer)] = (R.KernelLaunch * 4)()
                    api.check(lib.tp_exchange_wide_rows_prepare(C.byref(description), width, layer, layers, kernels, 1,
                                                                owner[(rank, layer)]), "owner")
            for card in cards:
                card.wait()
            # the plain push: the step's sequence itself
            for sequence in (1, 2, 3):
                inputs = [rng.normal(0, 0.05, elements).astype(np.float32) for _ in range(ranks)]
                inputs[0][0], inputs[1][0] = 16777216.0, 1.0
                expected = np.zeros(elements, dtype=np.float32)
                oracle.orc_ordered_push(pointer_array(inputs), ranks, elements, payload, ptr(expected, f32p))
                for rank, card in enumerate(cards):
                    card.upload(step, np.frombuffer(bytes(R.StepBlock(sequence, capacity, 0)), dtype=np.uint8))
                    card.upload(region + (sequence & 1) * stride + input_at, inputs[rank])
                for rank, card in enumerate(cards):  # queue every rank before waiting for any
                    card.run([push[rank]])
                for rank, card in enumerate(cards):
                    card.wait()
                    assert card.expired_bits() == 0
                    got = card.download(region + (sequence & 1) * stride + output_at, 4 * elements, np.float32)
                    assert np.array_equal(got.view(np.uint32), expected.view(np.uint32)), (ranks, sequence, rank)
            # the owner sums, two layers a step sharing the region; the steps go on from the push's sequences
            for model_step, rows in ((40, 64), (41, 37), (42, 1)):
                for layer in range(layers):
                    sequence = (model_step * layers + layer) * 2 + (model_step & 1)
                    live = rows * width
                    inputs = [rng.normal(0, 0.05, elements).astype(np.float32) for _ in range(ranks)]
                    inputs[0][0], inputs[1][0] = 16777216.0, 1.0
                    expected = np.zeros(live, dtype=np.uint16)
                    oracle.orc_owner_sums(pointer_array(inputs), ranks, live, payload, ptr(expected, u16p))
                    for rank, card in enumerate(cards):
                        card.upload(step, np.frombuffer(bytes(R.StepBlock(model_step, rows, 0)), dtype=np.uint8))
                        card.upload(region + (sequence & 1) * stride + input_at, inputs[rank])
                    for rank, card in enumerate(cards):
                        card.run(owner[(rank, layer)])
                    for rank, card in enumerate(cards):
                        card.wait()
                        assert card.expired_bits() == 0
                        got = card.download(region + (sequence & 1) * stride + output_at, 2 * live, np.uint16)
                        assert np.array_equal(got, expected), (ranks, model_step, layer, rank)
        finally:
            for card in cards:
                card.close()


@pytest.mark.parametrize("kind,mode", [("exact", 0), ("exact", 1), ("exact", 2), ("compressed", 1), ("compressed", 2),
                                       ("round_once", 1)])
def test_output_axis_exchanges_across_cards(api, oracle, kind, mode):
    """The gather, the BF16 sum in the ring's order (plain and on the coded wire) and the round-once sum between real
    cards: every rank stores into every rank's bank over NVLink and waits on its own; bit for bit against the oracle
    on every rank, three calls in a row on the same banks."""
    from anemone_b200.ring import RingExchange
    from tests.test_gpu_ring import expected_for, values_for
    for ranks in world_sizes(api):
        packs, vectors = 32 * 24, (4 if mode != 1 else 0)
        rng = np.random.default_rng(900 + ranks + mode)
        cards, exchanges = [], []
        try:
            for rank in range(ranks):
                cards.append(api.Card(rank, 64 << 20))
                exchanges.append(RingExchange(cards[-1], kind, mode, rank, ranks, packs, vectors))
            for exchange in exchanges:
                exchange.connect_local(exchanges)
            for card in cards:
                card.wait()
            for call in range(3):
                inputs = values_for(rng, ranks, packs, "wide" if call == 1 else "near")
                expected = expected_for(oracle, kind, mode, inputs, ranks, packs, vectors)
                for exchange, values in zip(exchanges, inputs):
                    exchange.load(values)
                for exchange in exchanges:  # queue every rank before waiting for any
                    exchange.run()
                for card in cards:
                    card.wait()
                for rank, exchange in enumerate(exchanges):
                    assert np.array_equal(exchange.result(), expected[rank]), (ranks, call, rank)
        finally:
            for card in cards:
                card.close()


def test_copy_launches_to_peers_at_once(api):
    """One graph on card 0: a copy into every other card's arena, each on a side run of its own (the reference's use of
    LAUNCH_SIDE_MORE, include/anemone/backend_seam.h:183-195), and a copy behind the join."""
    for ranks in world_sizes(api):
        ranks = min(ranks, 5)  # a fork has at most four side runs
        bytes_each, arena_bytes = 1 << 20, 8 << 20
        cards = [api.Card(rank, arena_bytes) for rank in range(ranks)]
        try:
            rng = np.random.default_rng(ranks)
            payload = rng.integers(0, 256, bytes_each).astype(np.uint8)
            for card in cards:
                card.fill(0, 0, arena_bytes)
            cards[0].upload(1 << 20, payload)
            table = [R.copy_launch(1 << 20, 2 << 20, bytes_each)]
            for peer in range(1, ranks):
                cards[0].peer_connect(cards[peer], 4 << 20, 8 * peer)
                table.append(R.copy_launch(2 << 20, 0, bytes_each, R.LAUNCH_SIDE if peer == 1 else R.LAUNCH_SIDE_MORE,
                                           destination_word=8 * peer))
            table.append(R.copy_launch(2 << 20, 3 << 20, bytes_each, R.LAUNCH_JOIN))
            graph = cards[0].graph(table)
            cards[0].graph_run(graph)
            cards[0].wait()
            assert np.array_equal(cards[0].download(3 << 20, bytes_each), payload)
            for peer in range(1, ranks):
                cards[peer].wait()
                assert np.array_equal(cards[peer].download(4 << 20, bytes_each), payload)
        finally:
            for card in cards:
                card.close()


@pytest.mark.parametrize("shared", [1, 0])
def test_original_weights_layer_tensor_parallel(api, oracle, shared):
    """The original-weights decode layer on R cards (every rank its own column slice of the MXFP4 experts and of the
    always-on expert): its reduction is one launch a rank (row sums of the bfloat16 pair outputs, the always-on
    expert's rows, READY and the rank-ordered sum, flags in the reader's memory). Every rank ends with the same bits;
    they are the oracle's rank-ordered sum of the FP32 rows the ranks published; a rank's published rows are its pair
    outputs added in slot order, its always-on rows, and one addition onto +0, bit for bit."""
    from anemone_b200.mx import MxLayer, MxLayout
    from tests.test_gpu_mx import mx_matrix
    for ranks in world_sizes(api):
        config = MoeConfig(hidden=512, inner=128 * ranks, experts=12, shared=shared, picks=3, row_capacity=8,
                           activation_limit=7.0)
        rng = np.random.default_rng(700 + ranks)
        H = config.hidden
        cards, layers = [], []
        try:
            for rank in range(ranks):
                L = MxLayout(config, ranks, rank)
                assert L.flags
                I = L.inner_local
                card = api.Card(rank, L.arena_bytes)
                cards.append(card)
                matrices = [(mx_matrix(oracle, rng, I, H), mx_matrix(oracle, rng, I, H), mx_matrix(oracle, rng, H, I))
                            for _ in range(config.experts)]
                always = (synthetic.e4m3_matrix(rng, I, H), synthetic.e4m3_matrix(rng, I, H),
                          synthetic.e4m3_matrix(rng, H, I)) if shared else None
                layers.append(MxLayer(card, config, matrices, rank=rank, rank_count=ranks, slices=(2, 2),
                                      shared_matrices=always))
            for layer in layers:
                layer.connect_local(layers)
            for card in cards:
                card.wait()
            for step in range(4):
                rows = [8, 3, 8, 1][step]
                tokens = synthetic.tokens(rng, rows, H)
                scores = rng.normal(0, 1, size=(rows, config.experts)).astype(np.float32)
                result_at = api.align(layers[0].layout.step_input_bytes, 4096)
                tickets = []
                for layer in layers:  # queue every rank before waiting for any
                    layer.sequence += 1
                    layer.stage_step(0, layer.sequence, tokens, scores)
                    tickets.append(layer.submit(0, result_at, rows))
                outputs, published = [], []
                for layer, ticket in zip(layers, tickets):
                    layer.card.transfer_wait(ticket)
                    layer.check_status()
                    outputs.append(layer.card.staging_view[result_at:result_at + rows * H * 2].view(np.uint16).copy())
                for rank in range(1, ranks):
                    assert np.array_equal(outputs[rank], outputs[0])
                for layer in layers:
                    L = layer.layout
                    slot = L.region + (layer.sequence & 1) * L.parity_stride + L.slot_input
                    mine = layer.card.download(slot, rows * H * 4, np.float32)
                    published.append(mine)
                    pairs = synthetic.from_bfloat16(layer.card.download(L.at["pair_output"], rows * config.picks * H * 2,
                                                                       np.uint16)).reshape(rows, config.picks, H)
                    resummed = np.zeros((rows, H), dtype=np.float32)
                    for slot_index in range(config.picks):
                        resummed = (resummed + pairs[:, slot_index, :]).astype(np.float32)
                    if shared:
                        resummed = (resummed + synthetic.from_bfloat16(layer.card.download(
                            L.shared_at["output"], rows * H * 2, np.uint16)).reshape(rows, H)).astype(np.float32)
                    row_output = layer.card.download(L.at["row_output"], rows * H * 4, np.float32).reshape(rows, H)
                    assert np.array_equal(resummed.view(np.uint32), row_output.view(np.uint32))
                    assert np.array_equal((np.float32(0.0) + resummed).view(np.uint32).reshape(-1), mine.view(np.uint32))
                    assert np.any(mine != 0)
                want = np.zeros(rows * H, dtype=np.uint16)
                oracle.orc_ordered_reduce_bf16(pointer_array(published), ranks, want.size, ptr(want, u16p))
                assert np.array_equal(outputs[0], want)
        finally:
            for card in cards:
                card.close()
