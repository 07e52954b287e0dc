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
