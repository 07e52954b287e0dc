"""Builds one arena image of a routed-expert chain (matrices, job table, tokens, scratch) that both the CPU oracle and
the CUDA launches run on, in the manner of the reference's card-test fixture (tests/linear_card_fixture.h:7-69):
a host image uploaded verbatim, a received mirror downloaded after the launches, guard bytes behind every work range."""
import ctypes as C

import numpy as np

from anemone_b200 import records as R
from anemone_b200 import synthetic
from anemone_b200.api import Layout
from oracle.binding import f32p, ptr, u32p, u64p, u8p

GUARD = 64
GUARD_BYTE = 0xC3


class ChainCase:
    def __init__(self, oracle, seed, hidden, inner, rows, picks, expert_count, widths, limit=10.0, shared=0):
        rng = np.random.default_rng(seed)
        self.oracle = oracle
        self.H, self.I, self.rows, self.picks = hidden, inner, rows, picks
        self.ppr = picks + shared
        self.pairs = rows * self.ppr
        self.widths = np.asarray(widths, dtype=np.uint32)
        total = expert_count + shared
        assert self.widths.size == total
        layout = Layout()
        self.ranges = {}

        def take(name, size, alignment=256, guarded=True):
            offset = layout.take(size + (GUARD if guarded else 0), alignment)
            self.ranges[name] = (offset, size)
            return offset

        matrices = []
        table = np.zeros((total, 3), dtype=np.uint64)
        for expert in range(total):
            width = int(self.widths[expert])
            for which, (inputs, outputs) in enumerate(((hidden, inner), (hidden, inner), (inner, hidden))):
                data = synthetic.exl3_matrix(rng, inputs, outputs, width)
                offset = take("matrix_%d_%d" % (expert, which), data.size, 64, guarded=False)
                table[expert, which] = offset
                matrices.append((offset, data))
        # routing: `picks` distinct experts a row, slots ascending, weights normalised
        experts = np.stack([np.sort(rng.choice(expert_count, size=picks, replace=False)) for _ in range(rows)])
        weights = rng.uniform(0.2, 1.0, size=(rows, picks)).astype(np.float32)
        weights /= weights.sum(axis=1, keepdims=True)
        self.job_capacity = rows * picks + shared * ((rows + 7) // 8) + 2  # with empty jobs at the end
        jobs = (R.ExpertJob * self.job_capacity)()
        experts32 = experts.astype(np.uint32)
        self.job_count = oracle.orc_router_jobs(ptr(experts32, u32p), ptr(weights, f32p), rows, picks, expert_count,
                                                shared, ptr(table, u64p), self.job_capacity, C.byref(jobs))
        self.jobs = jobs
        record = R.Exl3Expert()
        record.jobs_offset = take("jobs", C.sizeof(jobs))
        record.input_offset = take("input", rows * hidden * 2)
        from anemone_b200 import api
        sizes = api.moe_sizes(self.pairs, self.job_capacity, hidden, inner)
        record.operands_offset = take("operands", sizes.operand_bytes)
        record.products_offset = take("products", max(sizes.product_bytes, self.pairs * hidden * 8))
        self.counters_offset = take("counters", sizes.counter_bytes)
        record.output_offset = record.products_offset
        record.hidden_offset = take("hidden", self.pairs * inner * 2)
        self.row_output_offset = take("row_output", rows * hidden * 4)
        self.widths_offset = take("widths", total * 4)
        record.input_size, record.inner_size = hidden, inner
        record.pair_count, record.pairs_per_row = self.pairs, self.ppr
        record.job_count = self.job_capacity
        record.bits_per_weight = int(self.widths[0])
        record.activation_limit = limit
        self.record = record
        self.arena_bytes = layout.take(0, 4096) + 4096
        image = np.full(self.arena_bytes, GUARD_BYTE, dtype=np.uint8)
        for offset, data in matrices:
            image[offset:offset + data.size] = data
        image[record.jobs_offset:record.jobs_offset + C.sizeof(jobs)] = np.frombuffer(bytes(jobs), dtype=np.uint8)
        tokens = synthetic.tokens(rng, rows, hidden)
        image[record.input_offset:record.input_offset + tokens.nbytes] = tokens.view(np.uint8).reshape(-1)
        image[self.widths_offset:self.widths_offset + total * 4] = self.widths.view(np.uint8)
        image[self.counters_offset:self.counters_offset + sizes.counter_bytes] = 0
        self.image = image
        self.expected = None

    def view(self, image, name, dtype):
        offset, size = self.ranges[name]
        return image[offset:offset + size].view(dtype)

    def guards_intact(self, image):
        for name, (offset, size) in self.ranges.items():
            if name.startswith("matrix_"):
                continue
            if not (image[offset + size:offset + size + GUARD] == GUARD_BYTE).all():
                return name
        return None

    def run_oracle(self, per_expert_widths):
        """The five passes and the row sum on a copy of the image; returns that copy."""
        expected = self.image.copy()
        widths = ptr(self.widths, u32p) if per_expert_widths else None
        self.oracle.orc_exl3_experts(C.byref(self.record), ptr(expected, u8p), widths, 0)
        row_sum = R.ExpertRowSum(self.record.output_offset, self.row_output_offset, self.H, self.ppr)
        self.oracle.orc_exl3_row_sum(C.byref(row_sum), self.rows, ptr(expected, u8p))
        return expected

    def live_pairs(self):
        pairs = []
        for job in self.jobs[:self.job_count]:
            pairs.extend(job.pair_index[c] for c in range(job.row_count))
        return sorted(pairs)
