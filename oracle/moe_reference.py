"""The whole MoE layer on the CPU oracle: router, per-rank expert chains on local slices, rank-ordered reduction.
Test infrastructure (uses oracle/): the checker of the CUDA layer, never a product path."""
import ctypes as C

import numpy as np

from anemone_b200 import records as R
from anemone_b200.api import Layout
from anemone_b200.moe import local_matrices, rank_columns
from oracle.binding import f32p, pointer_array, ptr, u16p, u32p, u64p, u8p


def route(oracle, config, scores):
    rows = scores.shape[0]
    experts = np.zeros((rows, config.picks), dtype=np.uint32)
    weights = np.zeros((rows, config.picks), dtype=np.float32)
    for row in range(rows):
        line = np.ascontiguousarray(scores[row], dtype=np.float32)
        oracle.orc_router_row(ptr(line, f32p), config.experts, config.picks, config.scoring, config.route_scale,
                              ptr(experts[row], u32p), ptr(weights[row], f32p))
    return experts, weights


def rank_partial(oracle, config, widths, matrices, tokens, experts, weights, rank_count, rank, threads=0,
                 job_limit=None):
    """FP32 [rows][hidden] row sums of one rank. matrices: per expert the FULL (gate, up, down) stored bytes, as a
    sequence or as a function of the expert index (called only for experts that stand in a job); sliced here.
    job_limit: keep only the first so many jobs (a bounded sample for timing). Returns (rows, jobs, job count)."""
    rows = tokens.shape[0]
    H = config.hidden
    I = rank_columns(config.inner, rank_count, rank)[1]
    ppr, pairs = config.pairs_per_row, rows * config.pairs_per_row
    job_capacity = rows * config.picks + config.shared * ((rows + 7) // 8)
    # a first pass with a dummy table finds the experts in use; only their matrices are placed
    jobs = (R.ExpertJob * job_capacity)()
    table = np.zeros((config.total_experts, 3), dtype=np.uint64)
    experts = np.ascontiguousarray(experts, dtype=np.uint32)
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    count = oracle.orc_router_jobs(ptr(experts, u32p), ptr(weights, f32p), rows, config.picks, config.experts,
                                   config.shared, ptr(table, u64p), job_capacity, C.byref(jobs))
    assert count != 0xFFFFFFFF
    kept = count if job_limit is None else min(count, job_limit)
    active = sorted(set(jobs[index].expert for index in range(kept)))
    layout = Layout()
    placed = []
    for expert in active:
        gate, up, down = matrices(expert) if callable(matrices) else matrices[expert]
        for which, data in enumerate(local_matrices(gate, up, down, config, int(widths[expert]), rank_count, rank)):
            offset = layout.take(data.size, 64)
            table[expert, which] = offset
            placed.append((offset, data))
    record = R.Exl3Expert()
    record.jobs_offset = layout.take(job_capacity * 96)
    record.input_offset = layout.take(rows * H * 2)
    record.operands_offset = layout.take(pairs * max(H, I) * 4)
    record.products_offset = record.output_offset = layout.take(pairs * max(H, I) * 8)
    record.hidden_offset = layout.take(pairs * I * 2)
    row_output = layout.take(rows * H * 4)
    record.input_size, record.inner_size, record.pair_count, record.pairs_per_row = H, I, pairs, ppr
    record.job_count, record.bits_per_weight, record.activation_limit = kept, 3, config.activation_limit
    image = np.zeros(layout.cursor + 64, dtype=np.uint8)
    for offset, data in placed:
        image[offset:offset + data.size] = data
    count = oracle.orc_router_jobs(ptr(experts, u32p), ptr(weights, f32p), rows, config.picks, config.experts,
                                   config.shared, ptr(table, u64p), job_capacity, C.byref(jobs))
    image[record.jobs_offset:record.jobs_offset + C.sizeof(jobs)] = np.frombuffer(bytes(jobs), dtype=np.uint8)
    image[record.input_offset:record.input_offset + tokens.nbytes] = tokens.reshape(-1).view(np.uint8)
    widths32 = np.ascontiguousarray(widths, dtype=np.uint32)
    oracle.orc_exl3_experts(C.byref(record), ptr(image, u8p), ptr(widths32, u32p), threads)
    row_sum = R.ExpertRowSum(record.output_offset, row_output, H, ppr)
    oracle.orc_exl3_row_sum(C.byref(row_sum), rows, ptr(image, u8p))
    return image[row_output:row_output + rows * H * 4].view(np.float32).reshape(rows, H).copy(), jobs, kept


def layer(oracle, config, widths, matrices, tokens, scores, rank_count, threads=0):
    """bfloat16 bits [rows][hidden] of the whole layer on rank_count ranks, and the ranks' FP32 partials."""
    experts, weights = route(oracle, config, scores)
    partials = [rank_partial(oracle, config, widths, matrices, tokens, experts, weights, rank_count, rank, threads)[0]
                for rank in range(rank_count)]
    out = np.zeros(tokens.shape[0] * config.hidden, dtype=np.uint16)
    flat = [np.ascontiguousarray(p.reshape(-1)) for p in partials]
    oracle.orc_ordered_reduce_bf16(pointer_array(flat), rank_count, out.size, ptr(out, u16p))
    return out.reshape(tokens.shape[0], config.hidden), partials, experts, weights
