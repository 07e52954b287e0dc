"""One rank's quantized MoE expert layer, prepared once and run per step through the C-ABI library.

Host-side mirror of how the reference's model program uses the path (source/model_v41_program.c:4227-4531, 2618-2770):
at load, matrices are placed in the arena, every launch is prepared by the library's preparers and captured into one
graph; per step the caller writes the step block, the tokens and the router scores, runs the graph and reads the
bfloat16 result. Launches of one step, all from libanemone_b200.so, in the default form ("fused", exl3_layer_prepare):
    exl3_layer_route_input -> exl3_layer_gate_up -> exl3_layer_down_publish -> ordered_reduce_flags
and in the forms kept for callers of the separate preparers ("pull": six launches, "push": five):
    router_select_b200 -> exl3_moe_input -> exl3_moe_gate_up -> exl3_moe_down -> ordered_row_sum_publish
    -> ordered_reduce_bf16
Tensor parallelism is by intermediate columns: this rank holds columns [begin, begin + inner_local) of every expert's
gate and up and the matching input rows of down; the ranks' FP32 partial rows are summed in rank order by peer loads
and rounded once to bfloat16. Nothing here computes on the host.
"""
import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import api
from . import records as R
from . import synthetic

LINE = 128
SIGNAL_BYTES = 3 * LINE


@dataclass
class MoeConfig:
    hidden: int = 4096
    inner: int = 2048  # full intermediate width of an expert
    experts: int = 256  # routed
    shared: int = 1  # always-on experts, weight 1
    picks: int = 8
    row_capacity: int = 8
    activation_limit: float = 10.0
    scoring: int = 0  # ROUTER_SCORING_SIGMOID
    route_scale: float = 1.0
    deadline_cycles: int = 2_000_000_000  # about a second of device clock
    bias: bool = False  # a per-expert selection bias (FP32 [experts]) is added to the affinities for the choice

    @property
    def pairs_per_row(self):
        return self.picks + self.shared

    @property
    def total_experts(self):
        return self.experts + self.shared


def rank_columns(inner, rank_count, rank):
    """The 128-column blocks of a rank: [blocks r / R, blocks (r + 1) / R), as bb_exl3_inner_shard_prepare cuts them."""
    blocks = inner // 128
    begin = blocks * rank // rank_count * 128
    return begin, blocks * (rank + 1) // rank_count * 128 - begin


def local_matrices(gate, up, down, config, width, rank_count, rank):
    """This rank's slices of one expert's three stored matrices."""
    begin, count = rank_columns(config.inner, rank_count, rank)
    if rank_count == 1:
        return gate, up, down
    H, I = config.hidden, config.inner
    return (synthetic.slice_matrix(gate, H, I, width, 0, H, begin, count),
            synthetic.slice_matrix(up, H, I, width, 0, H, begin, count),
            synthetic.slice_matrix(down, I, H, width, begin, count, 0, H))


class MoeLayout:
    """Byte offsets of everything one rank keeps in its arena. Identical on every rank of a group."""

    def __init__(self, config, widths, rank_count, rank, pool_entries=0, reduce_form="fused"):
        self.config, self.rank_count, self.rank = config, rank_count, rank
        self.pool_entries = pool_entries
        self.reduce_form = reduce_form
        self.inner_local = rank_columns(config.inner, rank_count, rank)[1]
        c, H, I = config, config.hidden, self.inner_local
        rows, pairs = c.row_capacity, c.row_capacity * c.pairs_per_row
        self.pairs = pairs
        self.job_capacity = rows * c.picks + c.shared * ((rows + 7) // 8)
        layout = api.Layout()
        self.peer_table = layout.take(16 * 32)
        # per-step inputs, contiguous so that one copy brings a whole step: step block, tokens, scores
        self.step = layout.take(256)
        self.tokens = layout.take(rows * H * 2)
        self.scores = layout.take(rows * c.experts * 4)
        self.step_input_bytes = layout.cursor - self.step
        # the status block stands directly in front of the result: one copy brings both back
        self.status = layout.take(16 + rows * H * 2)
        self.result = self.status + 16
        # optional: a pool of prepared step inputs resident on the card (step_input_select walks it)
        self.pool_stride = api.align(self.step_input_bytes, 256)
        self.cursor = layout.take(16)
        self.pool = layout.take(self.pool_stride * pool_entries) if pool_entries else 0
        # the reduction's region: two parity slots of signal lines and this rank's FP32 partial rows
        if reduce_form == "fused":  # exl3_layer_prepare: READY and DONE words arrive in the reader's own memory
            self.slot_input = R.EXL3_LAYER_SIGNAL_BYTES
            self.parity_stride = api.align(self.slot_input + rows * H * 4, LINE)
        elif reduce_form == "pull":  # ordered_row_sum_publish + ordered_reduce_bf16: peers read this rank's rows
            self.slot_input = SIGNAL_BYTES
            self.parity_stride = api.align(SIGNAL_BYTES + rows * H * 4, LINE)
        else:  # ordered_rows_push: one launch; every rank stores its rows into an inbox of every rank's slot
            assert reduce_form == "push"
            self.inbox = 2 * rank_count * LINE
            self.inbox_stride = rows * H * 4
            self.slot_input = self.inbox + rank * self.inbox_stride  # where this rank's own rows end up
            self.parity_stride = api.align(self.inbox + rank_count * self.inbox_stride, LINE)
        self.region = layout.take(2 * self.parity_stride, LINE)
        self.picks = layout.take(rows * c.picks * 4)
        self.weights = layout.take(rows * c.picks * 4)
        self.jobs = layout.take(self.job_capacity * 96)
        self.expert_table = layout.take(c.total_experts * 24)
        self.widths = layout.take(c.total_experts * 4)
        self.bias = layout.take(c.experts * 4) if c.bias else 0
        sizes = (api.layer_sizes if reduce_form == "fused" else api.moe_sizes)(pairs, self.job_capacity, H, I)
        self.operands = layout.take(sizes.operand_bytes)
        self.products = layout.take(max(sizes.product_bytes, pairs * H * 8))
        self.counters = layout.take(sizes.counter_bytes)
        self.counter_bytes = sizes.counter_bytes
        self.hidden = layout.take(pairs * I * 2)
        self.row_output = layout.take(rows * H * 4)
        self.matrices = []
        for expert in range(c.total_experts):
            width = int(widths[expert])
            sizes = (synthetic.matrix_bytes(H, I, width), synthetic.matrix_bytes(H, I, width),
                     synthetic.matrix_bytes(I, H, width))
            self.matrices.append(tuple(layout.take(size, 64) for size in sizes))
        self.arena_bytes = api.align(layout.cursor, 4096) + 4096


class MoeLayer:
    def __init__(self, card, config, widths, matrices, rank=0, rank_count=1, pool_entries=0, reduce_form="fused",
                 bias=None, cut=(0, 0)):
        """matrices: iterable over experts (routed, then shared) of this rank's (gate, up, down) stored bytes.
        reduce_form: "fused" (the step in three launches: the router with the input transform; the products as one
        resident grid that walks the step's items; row sums, READY and the reduction, with flags that arrive in the
        reader's memory),
        "pull" (router, four expert launches, two reduction launches: the ranks read each other's rows) or "push"
        (one reduction launch: the ranks store their rows into each other's inboxes); the same sums of the ranks'
        rows and the same bits given those rows. bias: FP32 [experts] for a config with bias=True. cut: (gate/up
        runs of K, down runs of K) of the fused form, 0 for the library's choice."""
        self.card, self.config = card, config
        self.widths = np.asarray(widths, dtype=np.uint32)
        self.layout = L = MoeLayout(config, self.widths, rank_count, rank, pool_entries, reduce_form)
        assert card.arena_bytes >= L.arena_bytes
        self.rank, self.rank_count = rank, rank_count
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
        card.fill(L.peer_table, 0, 16 * 32)
        card.fill(L.status, 0, 16)
        card.fill(L.step, 0, 256)
        card.fill(L.region, 0, 2 * L.parity_stride)
        card.fill(L.counters, 0, L.counter_bytes)
        if config.bias:
            card.upload(L.bias, np.ascontiguousarray(bias, dtype=np.float32))
        self.cut = cut
        peers = (R.OrderedPeer * rank_count)()
        for peer in range(rank_count):
            peers[peer].region_offset = L.region
        card.upload(L.peer_table, np.frombuffer(bytes(peers), dtype=np.uint8))
        self._prepare()
        self.sequence = 0

    # ---- load time ----
    def connect_local(self, layers):
        """All ranks in this process (the reference's arrangement): peer_connect every card to every card."""
        for peer, other in enumerate(layers):
            self.card.peer_connect(other.card, 0, self.layout.peer_table + 32 * peer)

    def connect_handles(self, handles):
        """One process per GPU: handles[r] is rank r's exported arena handle (all-gathered by the caller)."""
        for peer, handle in enumerate(handles):
            if peer == self.rank:
                self.card.peer_connect(self.card, 0, self.layout.peer_table + 32 * peer)
            else:
                self.card.ipc_connect(handle, 0, self.layout.peer_table + 32 * peer)

    def _prepare_fused(self):
        c, L, card, lib = self.config, self.layout, self.card, api.library()
        description = R.Exl3LayerDescription()
        route = description.route
        route.moe.base = R.Exl3Expert(L.jobs, L.tokens, L.operands, L.products, L.hidden, L.products, c.hidden,
                                      L.inner_local, L.pairs, c.pairs_per_row, L.job_capacity,
                                      R.EXL3_WIDTH_PER_EXPERT, c.activation_limit, 0)
        route.moe.widths_offset, route.moe.row_output_offset = L.widths, L.row_output
        route.moe.counters_offset, route.moe.expert_count = L.counters, c.total_experts
        route.scores_offset, route.expert_table_offset, route.picks_offset = L.scores, L.expert_table, L.picks
        route.weights_offset, route.bias_offset, route.step_offset = L.weights, L.bias, L.step
        route.routed_count, route.shared_count, route.picks, route.row_capacity = (c.experts, c.shared, c.picks,
                                                                                     c.row_capacity)
        route.scoring, route.route_scale = c.scoring, c.route_scale
        description.publish = R.Exl3LayerPublish(L.peer_table, L.region, L.slot_input, L.status, L.step,
                                                 L.parity_stride, c.deadline_cycles, self.rank_count, self.rank,
                                                 c.row_capacity, 0)
        description.result_offset, description.arena_byte_count = L.result, card.arena_bytes
        description.gate_up_runs, description.down_runs = self.cut
        launches = (R.KernelLaunch * R.EXL3_LAYER_LAUNCHES)()
        api.check(lib.exl3_layer_prepare(C.byref(description), card.ops_pointer, card.handle, launches),
                  "exl3_layer_prepare")
        return list(launches)

    def _prepare(self):
        c, L, card, lib = self.config, self.layout, self.card, api.library()
        # which launches stand before the gate/up products, and which launch they are (for callers that time them)
        self.step_graph = None  # step(): the copies and the launches as one graph, captured at its first call
        self.gate_up_index = 1 if L.reduce_form == "fused" else 2
        self.gate_up_kernel = "exl3_layer_products" if L.reduce_form == "fused" else "exl3_moe_gate_up"
        # the launch at gate_up_index holds the down products too (callers that count a launch's bytes ask)
        self.products_in_one_launch = L.reduce_form == "fused"
        if L.reduce_form == "fused":
            self.launches = self._prepare_fused()
            self._capture()
            return
        router = R.RouterSelectB200(L.scores, L.expert_table, L.picks, L.weights, L.jobs, L.step, c.experts, c.shared,
                                    c.picks, c.row_capacity, L.job_capacity, c.scoring, c.route_scale, 0, L.bias)
        lib.router_select_b200_prepare.argtypes = [C.POINTER(R.RouterSelectB200), C.c_uint64,
                                                   C.POINTER(api.BackendOperations), C.c_void_p,
                                                   C.POINTER(R.KernelLaunch)]
        router_launch = R.KernelLaunch()
        api.check(lib.router_select_b200_prepare(C.byref(router), card.arena_bytes, card.ops_pointer, card.handle,
                                                 C.byref(router_launch)), "router_select_b200_prepare")
        moe = R.Exl3Moe()
        moe.base = R.Exl3Expert(L.jobs, L.tokens, L.operands, L.products, L.hidden, L.products, c.hidden,
                                L.inner_local, L.pairs, c.pairs_per_row, L.job_capacity, R.EXL3_WIDTH_PER_EXPERT,
                                c.activation_limit, 0)
        moe.widths_offset, moe.row_output_offset, moe.expert_count = L.widths, L.row_output, c.total_experts
        moe.counters_offset = L.counters
        moe_launches = (R.KernelLaunch * 4)()
        api.check(lib.exl3_moe_prepare(C.byref(moe), card.arena_bytes, card.ops_pointer, card.handle, moe_launches),
                  "exl3_moe_prepare")
        if L.reduce_form == "pull":
            reduce = R.OrderedReduceBf16Description()
            reduce.reduce.collective = R.OrderedCollective(L.peer_table, L.region, L.slot_input, L.result, 0, L.step,
                                                           L.parity_stride, c.deadline_cycles,
                                                           c.row_capacity * c.hidden, self.rank_count, self.rank, 0)
            reduce.reduce.status_offset, reduce.reduce.width = L.status, c.hidden
            reduce.pair_output_offset, reduce.arena_byte_count = L.products, card.arena_bytes
            reduce.pairs_per_row, reduce.row_capacity = c.pairs_per_row, c.row_capacity
            lib.ordered_reduce_bf16_prepare.argtypes = [C.POINTER(R.OrderedReduceBf16Description),
                                                        C.POINTER(api.BackendOperations), C.c_void_p,
                                                        C.POINTER(R.KernelLaunch)]
            reduce_launches = (R.KernelLaunch * 2)()
            api.check(lib.ordered_reduce_bf16_prepare(C.byref(reduce), card.ops_pointer, card.handle, reduce_launches),
                      "ordered_reduce_bf16_prepare")
        else:
            push = R.OrderedRowsPushDescription()
            push.arguments.push = R.OrderedPush(L.peer_table, L.region, 0, L.result, L.inbox, L.step, L.parity_stride,
                                                c.deadline_cycles, L.inbox_stride, c.row_capacity * c.hidden,
                                                self.rank_count, self.rank, R.ORDERED_PUSH_FP32, 0, 0)
            push.arguments.pair_output_offset, push.arguments.width = L.products, c.hidden
            push.arguments.pairs_per_row, push.arena_byte_count = c.pairs_per_row, card.arena_bytes
            lib.ordered_rows_push_prepare.argtypes = [C.POINTER(R.OrderedRowsPushDescription),
                                                      C.POINTER(api.BackendOperations), C.c_void_p,
                                                      C.POINTER(R.KernelLaunch)]
            reduce_launches = (R.KernelLaunch * 1)()
            api.check(lib.ordered_rows_push_prepare(C.byref(push), card.ops_pointer, card.handle, reduce_launches),
                      "ordered_rows_push_prepare")
        # the fused chain's own row sum is replaced by the reduction's, which sums straight into the exchange slot
        self.launches = [router_launch, moe_launches[0], moe_launches[1], moe_launches[2]] + list(reduce_launches)
        self._capture()

    def _capture(self):
        c, L, card, lib = self.config, self.layout, self.card, api.library()
        self.graph = card.graph(self.launches)
        self.resident_graph = None
        if L.pool_entries:
            select = R.StepInputSelect(L.pool, L.pool_stride, L.step, L.cursor, L.pool_entries, L.step_input_bytes)
            lib.step_input_select_prepare.argtypes = [C.POINTER(R.StepInputSelect), C.c_uint64,
                                                      C.POINTER(api.BackendOperations), C.c_void_p,
                                                      C.POINTER(R.KernelLaunch)]
            select_launch = R.KernelLaunch()
            api.check(lib.step_input_select_prepare(C.byref(select), card.arena_bytes, card.ops_pointer, card.handle,
                                                    C.byref(select_launch)), "step_input_select_prepare")
            self.resident_graph = card.graph([select_launch] + self.launches)

    def load_pool(self, steps):
        """steps: pool_entries tuples (sequence, tokens, scores), sequences strictly increasing. Their input areas go
        to the card's pool; run_resident() then takes them one after the other without touching the host."""
        L, card = self.layout, self.card
        assert len(steps) == L.pool_entries
        for index, (sequence, tokens, scores) in enumerate(steps):
            self.stage_step(0, sequence, tokens, scores)
            card.transfer_wait(card.upload_async(L.pool + index * L.pool_stride, 0, L.step_input_bytes))
        card.fill(L.cursor, 0, 16)
        card.wait()

    def run_resident(self):
        self.card.graph_run(self.resident_graph)

    # ---- per step ----
    def stage_step(self, staging_offset, sequence, tokens, scores):
        """Write one step's inputs into the card's staging block at staging_offset (layout of the step input area)."""
        L, view = self.layout, self.card.staging_view
        rows = tokens.shape[0]
        block = R.StepBlock(sequence, rows, 0)
        base = staging_offset
        view[base:base + 16] = np.frombuffer(bytes(block), dtype=np.uint8)
        at = base + (L.tokens - L.step)
        view[at:at + tokens.nbytes] = tokens.reshape(-1).view(np.uint8)
        at = base + (L.scores - L.step)
        view[at:at + scores.nbytes] = np.ascontiguousarray(scores, dtype=np.float32).reshape(-1).view(np.uint8)

    def submit(self, staging_offset, result_staging_offset, rows):
        """Queue: copy the staged step in, run the layer's graph, copy the bfloat16 result out. Returns the ticket of
        the result copy; nothing waits."""
        L, card = self.layout, self.card
        card.upload_async(L.step, staging_offset, L.step_input_bytes)
        card.graph_run(self.graph)
        return card.download_async(L.result, result_staging_offset, rows * self.config.hidden * 2)

    def step(self, tokens, scores):
        """One layer call on host arrays: tokens bfloat16 bits [rows][hidden], scores FP32 [rows][experts].
        Returns bfloat16 bits [rows][hidden]. Raises if the reduction reported a failed wait."""
        L, card = self.layout, self.card
        rows = tokens.shape[0]
        self.sequence += 1
        result_at = api.align(L.step_input_bytes, 4096)
        nbytes = rows * self.config.hidden * 2
        self.stage_step(0, self.sequence, tokens, scores)
        # one library call: inputs in, the graph, status block and result out, wait. The copies are nodes of the
        # step's own graph where its table is a plain chain (one graph launch a step)
        if self.step_graph is None:
            captured = card.step_capture(self.launches, L.step, 0, L.step_input_bytes, L.status, result_at,
                                         16 + self.config.row_capacity * self.config.hidden * 2)
            self.step_graph = -1 if captured is None else captured
        if self.step_graph >= 0:
            card.graph_run_wait(self.step_graph)
        else:
            card.step_run(self.graph, L.step, 0, L.step_input_bytes, L.status, result_at, 16 + nbytes)
        if L.reduce_form == "push":
            self.check_status()
        else:
            self._raise_on(card.staging_view[result_at:result_at + 16].view(np.uint32))
        return card.staging_view[result_at + 16:result_at + 16 + nbytes].view(np.uint16).reshape(
            rows, self.config.hidden).copy()

    def check_status(self):
        if self.layout.reduce_form == "push":
            bits = self.card.expired_bits()
            if bits != 0:
                raise RuntimeError("ordered reduction failed: bits %d (1 a wait ran out, 2 bad sequence, 4 too many "
                                   "rows)" % bits)
            return
        self._raise_on(self.card.download(self.layout.status, 16, np.uint32))

    @staticmethod
    def _raise_on(status):
        if status[0] != 0:
            raise RuntimeError("ordered reduction failed: code %d (1 timed out, 2 bad sequence), phase %d, rank %d"
                               % (status[0], status[1], status[2]))
