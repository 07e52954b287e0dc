"""One rank's routed-expert layer for many rows (prefill), prepared once and run through the C-ABI library.

Launches of one call, all from libanemone_b200.so (kernel file kernel_exl3_prefill):
    exl3_prefill_picks -> exl3_prefill_group -> exl3_prefill_tiles -> exl3_prefill_operands
    -> exl3_prefill_gate_up -> exl3_prefill_down -> exl3_prefill_row_sum
    -> ordered_row_sum_publish -> ordered_reduce_bf16 (owner runs)
Rows are grouped per expert into tiles of 128; each (row tile, 128 outputs) is a tensor-core contraction with the
expert's trellis tiles decoded on the way. The result is this rank's FP32 [rows][hidden] row sums over the pairs whose
experts it holds. A rank holds a run of the routed experts with their full intermediate width (expert parallelism) or
all of them with a slice of the intermediate columns (tensor parallelism), and a column slice of the always-on experts;
the ranks' rows are then summed in rank order by the ordered reduction (each rank adds its run of the result and stores
it into every rank's memory) and rounded once to bfloat16. Nothing here computes on the host.
"""
import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import api
from . import records as R
from . import synthetic
from .moe import LINE, SIGNAL_BYTES, rank_columns


@dataclass
class Share:
    """What one rank holds of the layer's experts."""
    local_first: int
    local_count: int
    inner: int  # intermediate width of the routed experts' matrices held here (0 if local_count is 0)
    inner_begin: int  # first intermediate column of those matrices (tensor parallelism), else 0
    shared_inner: int  # the same for the always-on experts
    shared_begin: int

    @staticmethod
    def whole(config):
        return Share(0, config.experts, config.inner, 0, config.inner if config.shared else 0, 0)

    @staticmethod
    def tensor_parallel(config, rank_count, rank):
        begin, count = rank_columns(config.inner, rank_count, rank)
        return Share(0, config.experts, count, begin, count if config.shared else 0, begin)

    @staticmethod
    def expert_parallel(config, rank_count, rank):
        first = config.experts * rank // rank_count
        begin, count = rank_columns(config.inner, rank_count, rank)
        return Share(first, config.experts * (rank + 1) // rank_count - first, config.inner, 0,
                     count if config.shared else 0, begin)

    def shared_count(self, config):
        return config.shared if self.shared_inner else 0

    def experts(self, config):
        """Global numbers of the experts held, in local order: routed run, then the always-on ones."""
        return list(range(self.local_first, self.local_first + self.local_count)) + \
            [config.experts + s for s in range(self.shared_count(config))]

    def matrices(self, config, expert, width, gate, up, down):
        """This rank's part of one expert's three FULL stored matrices."""
        H, I = config.hidden, config.inner
        begin, count = (self.inner_begin, self.inner) if expert < config.experts else \
            (self.shared_begin, self.shared_inner)
        if count == I:
            return gate, up, down
        return (synthetic.slice_matrix(gate, H, I, width, 0, H, begin, count),
                synthetic.slice_matrix(up, H, I, width, 0, H, begin, count),
                synthetic.slice_matrix(down, I, H, width, begin, count, 0, H))


class PrefillLayout:
    """Byte offsets of everything the prefill launches use in the arena. widths: by local expert."""

    def __init__(self, config, widths, share=None):
        self.config = config
        self.share = share = share or Share.whole(config)
        c, H = config, config.hidden
        rows = c.row_capacity
        self.shared_count = share.shared_count(c)
        self.local_experts = share.local_count + self.shared_count
        self.pairs_per_row = c.picks + self.shared_count
        assert len(widths) == self.local_experts
        layout = api.Layout()
        self.peer_table = layout.take(16 * 32)
        # one call's inputs, contiguous so that one copy brings them: step block, tokens, scores
        self.step = layout.take(256)
        self.tokens = layout.take(rows * H * 2)
        self.scores = layout.take(rows * c.experts * 4)
        self.input_bytes = layout.cursor - self.step
        assert self.tokens == self.step + 256 and self.scores == self.tokens + rows * H * 2
        self.picks = layout.take(rows * c.picks * 4)
        self.weights = layout.take(rows * c.picks * 4)
        self.expert_table = layout.take(self.local_experts * 24)
        self.widths = layout.take(self.local_experts * 4)
        self.parts = api.prefill_parts(rows, c.picks, self.shared_count, share.local_count, H,
                                       max(share.inner, share.shared_inner))
        self.workspace = layout.take(self.parts.total, 1024)
        self.pair_outputs = layout.take(rows * self.pairs_per_row * H * 4)
        self.row_output = layout.take(rows * H * 4)
        # the reduction's region (two parity slots of signal lines and this rank's FP32 rows) and its result
        self.slot_input = SIGNAL_BYTES
        self.parity_stride = api.align(SIGNAL_BYTES + rows * H * 4, LINE)
        self.region = layout.take(2 * self.parity_stride, LINE)
        # the status block stands directly in front of the result: one copy brings both back
        self.status = layout.take(16 + rows * H * 2)
        self.result = self.status + 16
        self.matrices = []
        for local in range(self.local_experts):
            width = int(widths[local])
            I = share.inner if local < share.local_count else share.shared_inner
            sizes = (synthetic.matrix_bytes(H, I, width), synthetic.matrix_bytes(H, I, width),
                     synthetic.matrix_bytes(I, H, width))
            self.matrices.append(tuple(layout.take(size, 64) for size in sizes))
        self.arena_bytes = api.align(layout.cursor, 4096) + 4096


class PrefillLayer:
    def __init__(self, card, config, widths, matrices, share=None, rank=0, rank_count=1,
                 reduce_mode=R.ORDERED_REDUCE_OWNER_RUNS):
        """widths, matrices: by LOCAL expert (the rank's routed run, then its always-on experts): stored widths and
        this rank's (gate, up, down) stored bytes."""
        self.card, self.config = card, config
        self.widths = np.asarray(widths, dtype=np.uint32)
        self.layout = L = PrefillLayout(config, self.widths, share)
        share = L.share
        assert card.arena_bytes >= L.arena_bytes
        self.rank, self.rank_count = rank, rank_count
        self.weight_bytes = 0
        table = np.zeros((L.local_experts, 3), dtype=np.uint64)
        for local, triple in enumerate(matrices):
            for which, data in enumerate(triple):
                offset = L.matrices[local][which]
                card.upload(offset, data)
                table[local, which] = offset
                self.weight_bytes += data.size
        card.upload(L.expert_table, table)
        card.upload(L.widths, self.widths)
        card.fill(L.step, 0, 256)
        card.fill(L.peer_table, 0, 16 * 32)
        card.fill(L.status, 0, 16)
        card.fill(L.region, 0, 2 * L.parity_stride)
        peers = (R.OrderedPeer * rank_count)()
        for peer in range(rank_count):
            peers[peer].region_offset = L.region
        card.upload(L.peer_table, np.frombuffer(bytes(peers), dtype=np.uint8))
        c = config
        self.record = R.Exl3Prefill(L.scores, L.tokens, L.expert_table, L.widths, L.picks, L.weights, L.workspace,
                                    L.pair_outputs, L.row_output, L.step, c.hidden, share.inner, share.shared_inner,
                                    c.experts, share.local_first, share.local_count, L.shared_count, c.picks,
                                    c.row_capacity, c.scoring, c.route_scale, c.activation_limit)
        self.launches = (R.KernelLaunch * 7)()
        api.check(api.library().exl3_prefill_prepare(C.byref(self.record), card.arena_bytes, card.ops_pointer,
                                                     card.handle, self.launches), "exl3_prefill_prepare")
        lib = api.library()
        reduce = R.OrderedReduceBf16Description()
        reduce.reduce.collective = R.OrderedCollective(L.peer_table, L.region, L.slot_input, L.result, 0, L.step,
                                                       L.parity_stride, c.deadline_cycles, c.row_capacity * c.hidden,
                                                       rank_count, rank, 0)
        reduce.reduce.status_offset, reduce.reduce.width, reduce.reduce.mode = L.status, c.hidden, reduce_mode
        # the rows are already summed over the pairs: one "pair" a row
        reduce.pair_output_offset, reduce.arena_byte_count = L.row_output, card.arena_bytes
        reduce.pairs_per_row, reduce.row_capacity = 1, c.row_capacity
        lib.ordered_reduce_bf16_prepare.argtypes = [C.POINTER(R.OrderedReduceBf16Description),
                                                    C.POINTER(api.BackendOperations), C.c_void_p,
                                                    C.POINTER(R.KernelLaunch)]
        self.reduce_launches = (R.KernelLaunch * 2)()
        api.check(lib.ordered_reduce_bf16_prepare(C.byref(reduce), card.ops_pointer, card.handle,
                                                  self.reduce_launches), "ordered_reduce_bf16_prepare")
        self.graph = card.graph(list(self.launches) + list(self.reduce_launches))
        self.sequence = 0

    def connect_local(self, layers):
        """All ranks in this process: peer_connect every card to every card."""
        for peer, other in enumerate(layers):
            self.card.peer_connect(other.card, 0, self.layout.peer_table + 32 * peer)

    def connect_handles(self, handles):
        """One process per GPU: handles[r] is rank r's exported arena handle (all-gathered by the caller)."""
        for peer, handle in enumerate(handles):
            if peer == self.rank:
                self.card.peer_connect(self.card, 0, self.layout.peer_table + 32 * peer)
            else:
                self.card.ipc_connect(handle, 0, self.layout.peer_table + 32 * peer)

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

    def stage(self, staging_offset, tokens, scores):
        """Write one call's inputs into the card's page-locked staging block, in the layout of the input area (a caller
        that produces its tokens and scores in page-locked memory does this once, in place). The rows must fill the
        capacity, so that tokens and scores are one contiguous range."""
        L, view = self.layout, self.card.staging_view
        assert tokens.shape[0] == self.config.row_capacity
        at = staging_offset + 256
        view[at:at + tokens.nbytes] = tokens.reshape(-1).view(np.uint8)
        at += tokens.nbytes
        scores = np.ascontiguousarray(scores, dtype=np.float32)
        view[at:at + scores.nbytes] = scores.reshape(-1).view(np.uint8)

    def call(self, staging_offset, result_staging_offset):
        """One whole call on staged inputs in ONE library call: inputs in, the graph, status block and bfloat16 result
        out, wait. Returns the result as a view of the staging block (bfloat16 bits [rows][hidden])."""
        L, card, rows = self.layout, self.card, self.config.row_capacity
        self.sequence += 1
        block = R.StepBlock(self.sequence, rows, 0)
        card.staging_view[staging_offset:staging_offset + 16] = np.frombuffer(bytes(block), dtype=np.uint8)
        nbytes = rows * self.config.hidden * 2
        card.step_run(self.graph, L.step, staging_offset, L.input_bytes, L.status, result_staging_offset, 16 + nbytes)
        status = card.staging_view[result_staging_offset:result_staging_offset + 16].view(np.uint32)
        if status[0] != 0:
            raise RuntimeError("ordered reduction failed: code %d (1 timed out, 2 bad sequence), phase %d, rank %d"
                               % (status[0], status[1], status[2]))
        return card.staging_view[result_staging_offset + 16:result_staging_offset + 16 + nbytes].view(
            np.uint16).reshape(rows, self.config.hidden)

    def rows(self, count):
        """FP32 [count][hidden] row sums of the last run. Raises if a CTA gave up a bounded wait."""
        if self.card.waits_expired():
            raise RuntimeError("a prefill CTA gave up a bounded wait: the result is incomplete")
        H = self.config.hidden
        return self.card.download(self.layout.row_output, count * H * 4, np.float32).reshape(count, H)

    def result(self, count):
        """bfloat16 bits [count][hidden]: the ranks' rows added in rank order, of the last run."""
        if self.card.waits_expired():
            raise RuntimeError("a prefill CTA gave up a bounded wait: the result is incomplete")
        status = self.card.download(self.layout.status, 16, np.uint32)
        if status[0] != 0:
            raise RuntimeError("ordered reduction failed: code %d (1 timed out, 2 bad sequence), phase %d, rank %d"
                               % (status[0], status[1], status[2]))
        H = self.config.hidden
        return self.card.download(self.layout.result, count * H * 2, np.uint16).reshape(count, H)

    def step(self, tokens, scores):
        self.load(tokens, scores)
        self.run()
        return self.rows(tokens.shape[0])
