"""The N > 1 host logic with two CPU ranks over gloo: every rank slices its own shard with the library's plan, computes
its partial rows (CPU oracle standing in for the card), the partials meet through the process group, and the
rank-ordered reduction equals the single-process result bit for bit. Also the plumbing bench.py uses for the
inter-process arena handles (all_gather_object) and that the arena layout is the same on every rank."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def worker(rank, world, port, queue):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from anemone_b200 import synthetic
    from anemone_b200.moe import MoeConfig, MoeLayout, rank_columns
    from oracle import binding, moe_reference
    from oracle.binding import pointer_array, ptr, u16p
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        oracle = binding.load_oracle()
        config = MoeConfig(hidden=256, inner=256, experts=12, shared=1, picks=3, row_capacity=4)
        rng = np.random.default_rng(77)  # the same stream on every rank: the same weights and inputs
        widths = np.concatenate([synthetic.expert_widths(rng, config.experts), [3]]).astype(np.uint32)
        matrices = [(synthetic.exl3_matrix(rng, 256, 256, int(w)), synthetic.exl3_matrix(rng, 256, 256, int(w)),
                     synthetic.exl3_matrix(rng, 256, 256, int(w))) for w in widths]
        tokens = synthetic.tokens(rng, 4, 256)
        scores = rng.normal(0, 1, size=(4, config.experts)).astype(np.float32)
        experts, weights = moe_reference.route(oracle, config, scores)
        mine, _, _ = moe_reference.rank_partial(oracle, config, widths, matrices, tokens, experts, weights, world, rank, 1)
        gathered = [torch.zeros(mine.shape, dtype=torch.float32) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(mine))
        partials = [np.ascontiguousarray(t.numpy().reshape(-1)) for t in gathered]
        out = np.zeros(mine.size, dtype=np.uint16)
        oracle.orc_ordered_reduce_bf16(pointer_array(partials), world, out.size, ptr(out, u16p))
        handles = [None] * world
        dist.all_gather_object(handles, bytes([rank]) * 64)  # what bench.py does with the arena handles
        layouts = [None] * world
        layout = MoeLayout(config, widths, world, rank)
        dist.all_gather_object(layouts, (layout.region, layout.parity_stride, layout.peer_table, layout.step,
                                         layout.result, rank_columns(config.inner, world, rank)))
        if rank == 0:
            expected = moe_reference.layer(oracle, config, widths, matrices, tokens, scores, world, threads=1)[0]
            queue.put({"equal": bool(np.array_equal(out.reshape(expected.shape), expected)),
                       "handles": [h[0] for h in handles], "layouts": layouts})
    finally:
        dist.destroy_process_group()


def test_two_ranks_over_gloo():
    import torch.multiprocessing as mp
    context = mp.get_context("spawn")
    queue = context.Queue()
    port = 29400 + os.getpid() % 500
    processes = [context.Process(target=worker, args=(rank, 2, port, queue)) for rank in range(2)]
    for process in processes:
        process.start()
    try:
        result = queue.get(timeout=180)
    finally:
        for process in processes:
            process.join(timeout=60)
            if process.is_alive():
                process.kill()
    assert all(process.exitcode == 0 for process in processes)
    assert result["equal"]
    assert result["handles"] == [0, 1]
    first, second = result["layouts"]
    assert first[:5] == second[:5]  # every shared offset is the same on both ranks
    assert first[5] == (0, 128) and second[5] == (128, 128)  # the ranks' column blocks tile the intermediate width


def exchange_worker(rank, world, port, queue):
    """Each rank prepares its own exchange and one-launch reduction (a fake backend hands out handles); the owner
    shards a rank would send and add are taken with the record's own rule and must tile the step's rows; the owner sums
    of the shards, gathered, equal the ordered reduction of the whole step bit for bit."""
    sys.path.insert(0, ROOT)
    import ctypes as C
    import torch
    import torch.distributed as dist
    from anemone_b200 import api
    from anemone_b200 import records as R
    from anemone_b200.moe import MoeConfig, MoeLayout
    from oracle import binding
    from oracle.binding import pointer_array, ptr, u16p
    from tests.test_host_preparers import FakeBackend
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        oracle, lib, fake = binding.load_oracle(), api.library(), FakeBackend()
        config = MoeConfig(hidden=256, inner=256, experts=12, shared=1, picks=3, row_capacity=7)
        L = MoeLayout(config, [3] * 13, world, rank, reduce_form="push")
        rows_push = R.OrderedRowsPushDescription()
        rows_push.arguments.push = R.OrderedPush(L.peer_table, L.region, 0, L.result, L.inbox, L.step, L.parity_stride,
                                                 1_000_000, L.inbox_stride, 7 * 256, world, rank, 0, 0, 0)
        rows_push.arguments.pair_output_offset, rows_push.arguments.width = L.products, 256
        rows_push.arguments.pairs_per_row, rows_push.arena_byte_count = config.pairs_per_row, L.arena_bytes
        lib.ordered_rows_push_prepare.argtypes = [C.POINTER(R.OrderedRowsPushDescription), C.c_void_p, C.c_void_p,
                                                  C.POINTER(R.KernelLaunch)]
        one = (R.KernelLaunch * 1)()
        assert lib.ordered_rows_push_prepare(C.byref(rows_push), C.byref(fake.table), fake.card, one) == 0
        record = R.OrderedRowsPush.from_buffer_copy(bytes(one[0].argument)[:112])
        # the step's values of this rank, and the exchange's owner rule: rank d owns rows [R d / ranks, R (d + 1) / ranks)
        rows, width = 7, 256
        mine = np.random.default_rng(900 + rank).normal(0, 0.05, rows * width).astype(np.float32)
        gathered = [torch.zeros(rows * width, dtype=torch.float32) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(mine))
        partials = [np.ascontiguousarray(t.numpy()) for t in gathered]
        first, last = rows * rank // world * width, rows * (rank + 1) // world * width
        shard = np.zeros(last - first, dtype=np.uint16)
        pieces = [p[first:last].copy() for p in partials]  # kept alive over the call
        oracle.orc_owner_sums(pointer_array(pieces), world, last - first, 0, ptr(shard, u16p))
        shards = [None] * world
        dist.all_gather_object(shards, (first, last, shard.tobytes()))
        records = [None] * world
        dist.all_gather_object(records, (bytes(record), tuple(one[0].grid), one[0].kernel))
        if rank == 0:
            whole = np.zeros(rows * width, dtype=np.uint16)
            oracle.orc_ordered_reduce_bf16(pointer_array(partials), world, whole.size, ptr(whole, u16p))
            joined = np.concatenate([np.frombuffer(data, dtype=np.uint16) for _, _, data in shards])
            tiled = [shards[0][0] == 0, shards[-1][1] == rows * width] + \
                [shards[r][1] == shards[r + 1][0] for r in range(world - 1)]
            queue.put({"tiled": all(tiled), "equal": bool(np.array_equal(joined, whole)), "records": records})
    finally:
        dist.destroy_process_group()


def test_exchange_shards_over_gloo():
    import torch.multiprocessing as mp
    from anemone_b200 import records as R
    context = mp.get_context("spawn")
    queue = context.Queue()
    port = 29400 + (os.getpid() + 250) % 500
    processes = [context.Process(target=exchange_worker, args=(rank, 2, port, queue)) for rank in range(2)]
    for process in processes:
        process.start()
    try:
        result = queue.get(timeout=180)
    finally:
        for process in processes:
            process.join(timeout=60)
            if process.is_alive():
                process.kill()
    assert all(process.exitcode == 0 for process in processes)
    assert result["tiled"] and result["equal"]
    (first, first_grid, first_kernel), (second, second_grid, second_kernel) = result["records"]
    a, b = R.OrderedRowsPush.from_buffer_copy(first), R.OrderedRowsPush.from_buffer_copy(second)
    assert (a.push.rank, b.push.rank) == (0, 1) and first_grid == second_grid and first_kernel == second_kernel
    b.push.rank = 0
    assert bytes(a) == bytes(b)  # identical launches on every rank but for the rank itself
