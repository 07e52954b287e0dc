"""One rank's routed-expert layer for many rows (prefill), prepared once and run through the C-ABI library.

Launches of one call, all from libanemone_b200.so (kernel file kernel_exl3_prefill):
    exl3_prefill_picks -> exl3_prefill_group -> exl3_prefill_tiles -> exl3_prefill_operands
    -> exl3_prefill_gate_up -> exl3_prefill_down -> exl3_prefill_row_sum
Rows are grouped per expert into tiles of 128; each (row tile, 128 outputs) is a tensor-core contraction with the
expert's trellis tiles decoded on the way. The result is this rank's FP32 [rows][hidden] row sums (a rank of a
tensor-parallel group holds a slice of the intermediate columns; the ranks' rows are then reduced in rank order as in
the decode layer). Nothing here computes on the host.
"""
import ctypes as C

import numpy as np

from . import api
from . import records as R
from . import synthetic
from .moe import rank_columns


class PrefillLayout:
    """Byte offsets of everything the prefill launches use in the arena."""

    def __init__(self, config, widths, rank_count=1, rank=0):
        self.config = config
        self.inner_local = rank_columns(config.inner, rank_count, rank)[1]
        c, H, I = config, config.hidden, self.inner_local
        rows = c.row_capacity
        layout = api.Layout()
        self.step = layout.take(256)
        self.tokens = layout.take(rows * H * 2)
        self.scores = layout.take(rows * c.experts * 4)
        self.picks = layout.take(rows * c.picks * 4)
        self.weights = layout.take(rows * c.picks * 4)
        self.expert_table = layout.take(c.total_experts * 24)
        self.widths = layout.take(c.total_experts * 4)
        self.parts = api.prefill_parts(rows, c.picks, c.shared, c.experts, H, I)
        self.workspace = layout.take(self.parts.total, 1024)
        self.pair_outputs = layout.take(rows * c.pairs_per_row * H * 4)
        self.row_output = layout.take(rows * H * 4)
        self.matrices = []
        for expert in range(c.total_experts):
            width = int(widths[expert])
            sizes = (synthetic.matrix_bytes(H, I, width), synthetic.matrix_bytes(H, I, width),
                     synthetic.matrix_bytes(I, H, width))
            self.matrices.append(tuple(layout.take(size, 64) for size in sizes))
        self.arena_bytes = api.align(layout.cursor, 4096) + 4096


class PrefillLayer:
    def __init__(self, card, config, widths, matrices, rank=0, rank_count=1):
        """matrices: iterable over experts (routed, then shared) of this rank's (gate, up, down) stored bytes."""
        self.card, self.config = card, config
        self.widths = np.asarray(widths, dtype=np.uint32)
        self.layout = L = PrefillLayout(config, self.widths, rank_count, rank)
        assert card.arena_bytes >= L.arena_bytes
        self.weight_bytes = 0
        table = np.zeros((config.total_experts, 3), dtype=np.uint64)
        for expert, triple in enumerate(matrices):
            for which, data in enumerate(triple):
                offset = L.matrices[expert][which]
                card.upload(offset, data)
                table[expert, which] = offset
                self.weight_bytes += data.size
        card.upload(L.expert_table, table)
        card.upload(L.widths, self.widths)
        card.fill(L.step, 0, 256)
        c = config
        self.record = R.Exl3Prefill(L.scores, L.tokens, L.expert_table, L.widths, L.picks, L.weights, L.workspace,
                                    L.pair_outputs, L.row_output, L.step, c.hidden, L.inner_local, c.experts, c.shared,
                                    c.picks, c.row_capacity, c.scoring, c.route_scale, c.activation_limit, 0)
        self.launches = (R.KernelLaunch * 7)()
        api.check(api.library().exl3_prefill_prepare(C.byref(self.record), card.arena_bytes, card.ops_pointer,
                                                     card.handle, self.launches), "exl3_prefill_prepare")
        self.graph = card.graph(self.launches)
        self.sequence = 0

    def load(self, tokens, scores):
        """Place one call's inputs on the card: tokens bfloat16 bits [rows][hidden], scores FP32 [rows][experts]."""
        L, card = self.layout, self.card
        self.sequence += 1
        block = R.StepBlock(self.sequence, tokens.shape[0], 0)
        card.upload(L.step, np.frombuffer(bytes(block), dtype=np.uint8))
        card.upload(L.tokens, tokens)
        card.upload(L.scores, np.ascontiguousarray(scores, dtype=np.float32))

    def run(self):
        self.card.graph_run(self.graph)

    def rows(self, count):
        """FP32 [count][hidden] row sums of the last run. Raises if a CTA gave up a bounded wait."""
        if self.card.waits_expired():
            raise RuntimeError("a prefill CTA gave up a bounded wait: the result is incomplete")
        H = self.config.hidden
        return self.card.download(self.layout.row_output, count * H * 4, np.float32).reshape(count, H)

    def step(self, tokens, scores):
        self.load(tokens, scores)
        self.run()
        return self.rows(tokens.shape[0])
