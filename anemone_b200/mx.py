"""One rank's original-weights routed-expert layer (MXFP4 weights by E4M3 block-quantized activations), prepared once
and run per step through the C-ABI library. Launches of one step, all from libanemone_b200.so:
    router_select_b200 -> activation_quantize_entry -> expert_gate_up_<S> -> activation_quantize_entry (hidden)
    -> expert_down_<S> -> expert_row_sum_entry
    [-> trunk_linear_quantized_<S> (gate, up) -> trunk_hidden_entry -> activation_quantize_entry
     -> trunk_linear_quantized_<S> (down) -> trunk_rows_add_entry]          the always-on expert, E4M3 matrices
    -> ordered_row_sum_publish -> ordered_reduce_bf16
(linear_routed_experts_prepare's four, linear_shared_expert_prepare's four). Tensor parallelism is by intermediate columns, as in the
EXL3 decode layer; the ranks' FP32 rows are added in rank order and rounded once. Nothing here computes on the host.

wide=True is the same layer for MANY rows (the profile's prefill): the router's launch gives way to the three of
router_wide_prepare (the prefill's picks and grouping, then a job table of eight rows a job), the always-on expert to
linear_shared_expert_wide_prepare (a block column per eight rows), and the reduction adds by owner runs. The routed
experts' products are linear_routed_experts_wide_prepare's (a group of jobs and several tiles a block, the thin
instances' arithmetic; many=False keeps the thin instances, where every job streams its expert's matrices again).
"""
import ctypes as C

import numpy as np

from . import api
from . import records as R
from .moe import LINE, SIGNAL_BYTES, rank_columns

WEIGHT_FORMAT_E2M1_SCALED = 3
WEIGHT_FORMAT_E4M3_SCALED = 5
WEIGHT_FORMAT_E4M3_BLOCK128 = 6


def matrix_bytes(outputs, inputs):
    return outputs * inputs // 2 + outputs * inputs // 32


def shared_matrix_bytes(outputs, inputs, block128=False):
    """Stored bytes of an E4M3 matrix: one E8M0 code per 32 by 32 weights (the reference's format), or one FP32 scale
    per 128 by 128 (the original-weights checkpoints' block-scaled FP8)."""
    if block128:
        return outputs * inputs + (outputs + 127) // 128 * (inputs // 128) * 4
    return outputs * inputs + (outputs + 31) // 32 * (inputs // 32)


class MxLayout:
    def __init__(self, config, rank_count, rank, pool_entries=0, block128=False, wide=False):
        assert config.shared in (0, 1)
        self.block128, self.wide = block128, wide
        self.pool_entries = pool_entries
        self.config = c = config
        self.inner_local = I = rank_columns(c.inner, rank_count, rank)[1]
        H, rows = c.hidden, c.row_capacity
        self.pairs = pairs = rows * c.picks
        self.job_capacity = rows * c.picks // 8 + c.experts if wide else rows * c.picks
        layout = api.Layout()
        self.peer_table = layout.take(16 * 32)
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
        # a decode step's reduction is one launch whose flags arrive in the reader's own memory (the slot layout of the
        # EXL3 layer's step); many rows (owner runs) and steps beyond that launch's size keep the two-launch form
        self.flags = not wide and rows * H <= R.ORDERED_COLLECTIVE_MAXIMUM_ELEMENTS
        self.slot_input = R.EXL3_LAYER_SIGNAL_BYTES if self.flags else SIGNAL_BYTES
        self.parity_stride = api.align(self.slot_input + rows * H * 4, LINE)
        self.region = layout.take(2 * self.parity_stride, LINE)
        self.picks = layout.take(rows * c.picks * 4)
        self.weights = layout.take(rows * c.picks * 4)
        self.jobs = layout.take(self.job_capacity * 96)
        self.expert_table = layout.take(c.experts * 24)
        # many rows: counts and entries of the grouping launch (the head of the prefill's workspace)
        self.workspace_bytes = api.prefill_parts(rows, c.picks, 0, c.experts, H, I).gate_up_operands if wide else 0
        self.workspace = layout.take(self.workspace_bytes, 1024) if wide else 0
        self.sizes = {"codes": rows * H, "exponents": rows * H // 32, "operands": rows * H * 2,
                      "hidden": pairs * I * 2, "hidden_codes": pairs * I, "hidden_exponents": pairs * I // 32,
                      "hidden_operands": pairs * I * 2, "pair_output": pairs * H * 2, "row_output": rows * H * 4}
        self.at = {name: layout.take(size) for name, size in self.sizes.items()}
        self.shared_sizes = {"gate_output": rows * I * 2, "up_output": rows * I * 2, "hidden": rows * I * 2,
                             "hidden_codes": rows * I, "hidden_exponents": rows * I // 32,
                             "hidden_operands": rows * I * 2, "output": rows * H * 2} if c.shared else {}
        self.shared_at = {name: layout.take(size) for name, size in self.shared_sizes.items()}
        self.weights_begin = api.align(layout.cursor, 64)
        self.matrices = []
        for _ in range(c.experts):
            self.matrices.append((layout.take(matrix_bytes(I, H), 64), layout.take(matrix_bytes(I, H), 64),
                                  layout.take(matrix_bytes(H, I), 64)))
        self.weights_end = layout.cursor
        self.shared_matrices = (layout.take(shared_matrix_bytes(I, H, block128), 64),
                                layout.take(shared_matrix_bytes(I, H, block128), 64),
                                layout.take(shared_matrix_bytes(H, I, block128), 64)) if c.shared else ()
        self.arena_bytes = api.align(layout.cursor, 4096) + 4096


class MxLayer:
    def __init__(self, card, config, matrices, rank=0, rank_count=1, slices=(4, 4), shared_matrices=None,
                 shared_slices=(2, 2), pool_entries=0, block128=False, wide=False, many=True, side_run=True):
        """matrices: iterable over the routed experts of this rank's (gate, up, down) stored MXFP4 bytes;
        shared_matrices: the always-on expert's (gate, up, down) stored E4M3 bytes, where the configuration has one:
        WEIGHT_FORMAT_E4M3_SCALED, or with block128 WEIGHT_FORMAT_E4M3_BLOCK128 (one FP32 scale per 128 by 128).
        side_run: the always-on expert's launches as a side run of the step's graph, beside the routed experts' (the
        same values either way: the two touch disjoint ranges until the launch that joins them)."""
        self.card, self.config = card, config
        self.layout = L = MxLayout(config, rank_count, rank, pool_entries, block128, wide)
        assert card.arena_bytes >= L.arena_bytes
        self.rank, self.rank_count = rank, rank_count
        self.weight_bytes = 0
        table = np.zeros((config.experts, 3), dtype=np.uint64)
        for expert, triple in enumerate(matrices):
            for which, data in enumerate(triple):
                card.upload(L.matrices[expert][which], data)
                table[expert, which] = L.matrices[expert][which]
                self.weight_bytes += data.size
        card.upload(L.expert_table, table)
        if config.shared:
            for which, data in enumerate(shared_matrices):
                assert data.size == shared_matrix_bytes(*((L.inner_local, config.hidden) if which < 2 else
                                                          (config.hidden, L.inner_local)), block128)
                card.upload(L.shared_matrices[which], data)
                self.weight_bytes += data.size
        for offset, size in ((L.peer_table, 16 * 32), (L.status, 16), (L.step, 256), (L.region, 2 * L.parity_stride)):
            card.fill(offset, 0, size)
        peers = (R.OrderedPeer * rank_count)()
        for peer in range(rank_count):
            peers[peer].region_offset = L.region
        card.upload(L.peer_table, np.frombuffer(bytes(peers), dtype=np.uint8))
        c, lib, H, I = config, api.library(), config.hidden, L.inner_local
        router = R.RouterSelectB200(L.scores, L.expert_table, L.picks, L.weights, L.jobs, L.step, c.experts, 0,
                                    c.picks, c.row_capacity, L.job_capacity, c.scoring, c.route_scale, 0)
        lib.router_select_b200_prepare.argtypes = [C.POINTER(R.RouterSelectB200), C.c_uint64,
                                                   C.POINTER(api.BackendOperations), C.c_void_p,
                                                   C.POINTER(R.KernelLaunch)]
        router_launch = R.KernelLaunch()
        if wide:
            routing = R.Exl3Prefill()
            routing.scores_offset, routing.expert_table_offset = L.scores, L.expert_table
            routing.picks_offset, routing.weights_offset, routing.workspace_offset = L.picks, L.weights, L.workspace
            routing.step_offset, routing.input_size, routing.inner_size = L.step, H, I
            routing.expert_count, routing.local_count, routing.picks = c.experts, c.experts, c.picks
            routing.row_capacity, routing.scoring, routing.route_scale = c.row_capacity, c.scoring, c.route_scale
            lib.router_wide_prepare.argtypes = [C.POINTER(R.RouterWide), C.c_uint64, C.POINTER(api.BackendOperations),
                                                C.c_void_p, C.POINTER(R.KernelLaunch)]
            router_launches = (R.KernelLaunch * R.ROUTER_WIDE_LAUNCHES)()
            api.check(lib.router_wide_prepare(C.byref(R.RouterWide(routing, L.jobs, L.job_capacity, 0)),
                                              card.arena_bytes, card.ops_pointer, card.handle, router_launches),
                      "router_wide_prepare")
            router_launches = list(router_launches)
        else:
            api.check(lib.router_select_b200_prepare(C.byref(router), card.arena_bytes, card.ops_pointer, card.handle,
                                                     C.byref(router_launch)), "router_select_b200_prepare")
            router_launches = [router_launch]
        kernels = R.LinearKernels()
        lib.linear_kernels_prepare.argtypes = [C.POINTER(api.BackendOperations), C.c_void_p, C.c_uint32,
                                               C.POINTER(R.LinearKernels)]
        api.check(lib.linear_kernels_prepare(card.ops_pointer, card.handle, 100, C.byref(kernels)),
                  "linear_kernels_prepare")

        def span(name):
            return R.LinearRange(L.at[name], L.sizes[name])
        quantize = R.LinearQuantizeDescription(R.LinearRange(L.tokens, c.row_capacity * H * 2), span("codes"),
                                               span("exponents"), span("operands"), H, c.row_capacity)
        lib.linear_quantize_prepare.argtypes = [C.POINTER(R.LinearQuantizeDescription), C.c_uint64,
                                                C.POINTER(R.LinearKernels), C.POINTER(R.KernelLaunch)]
        quantize_launch = R.KernelLaunch()
        api.check(lib.linear_quantize_prepare(C.byref(quantize), card.arena_bytes, C.byref(kernels),
                                              C.byref(quantize_launch)), "linear_quantize_prepare")
        head = router_launches + [quantize_launch]
        if not wide:
            # a decode step begins with the router and the rows' quantization, neither of which reads the other's
            # output: one launch (block 0 routes, the others quantize)
            lib.router_select_quantize_prepare.argtypes = [C.POINTER(R.RouterSelectB200), C.POINTER(R.KernelLaunch),
                                                           C.c_uint64, C.POINTER(api.BackendOperations), C.c_void_p,
                                                           C.POINTER(R.KernelLaunch)]
            first = R.KernelLaunch()
            api.check(lib.router_select_quantize_prepare(C.byref(router), C.byref(quantize_launch), card.arena_bytes,
                                                         card.ops_pointer, card.handle, C.byref(first)),
                      "router_select_quantize_prepare")
            head = [first]
        description = R.LinearRoutedExpertsDescription()
        description.jobs = R.LinearRange(L.jobs, L.job_capacity * 96)
        description.expert_weights = R.LinearRange(L.weights_begin, L.weights_end - L.weights_begin)
        for name in L.sizes:
            setattr(description, name, span(name))
        description.gate_up_shape, description.down_shape = R.MatrixShape(I, H, 4, 0), R.MatrixShape(H, I, 4, 0)
        description.weight_format, description.job_count = WEIGHT_FORMAT_E2M1_SCALED, L.job_capacity
        description.row_count, description.pairs_per_row = c.row_capacity, c.picks
        description.activation_limit = c.activation_limit
        description.gate_up_slice_count, description.down_slice_count = slices
        lib.linear_routed_experts_prepare.argtypes = [C.POINTER(R.LinearRoutedExpertsDescription), C.c_uint64,
                                                      C.POINTER(R.LinearKernels), C.POINTER(R.KernelLaunch)]
        lib.linear_routed_experts_wide_prepare.argtypes = [C.POINTER(R.LinearRoutedExpertsDescription), C.c_uint64,
                                                           C.POINTER(R.LinearKernels),
                                                           C.POINTER(api.BackendOperations), C.c_void_p,
                                                           C.POINTER(R.KernelLaunch)]
        self.expert_launches = (R.KernelLaunch * 4)()
        if wide and many:
            api.check(lib.linear_routed_experts_wide_prepare(C.byref(description), card.arena_bytes, C.byref(kernels),
                                                             card.ops_pointer, card.handle, self.expert_launches),
                      "linear_routed_experts_wide_prepare")
        else:
            api.check(lib.linear_routed_experts_prepare(C.byref(description), card.arena_bytes, C.byref(kernels),
                                                        self.expert_launches), "linear_routed_experts_prepare")
        shared_launches = []
        if c.shared:
            shared = R.LinearSharedExpertDescription()
            for which, (name, (o, i)) in enumerate((("gate", (I, H)), ("up", (I, H)), ("down", (H, I)))):
                setattr(shared, name, R.LinearMatrix(R.LinearRange(L.shared_matrices[which],
                                                                   shared_matrix_bytes(o, i, L.block128)),
                                                     R.MatrixShape(o, i, 8, 0),
                                                     WEIGHT_FORMAT_E4M3_BLOCK128 if L.block128 else
                                                     WEIGHT_FORMAT_E4M3_SCALED,
                                                     shared_slices[0 if which < 2 else 1], 0, 0))
            shared.codes, shared.exponents, shared.operands = span("codes"), span("exponents"), span("operands")
            for name in L.shared_sizes:
                setattr(shared, name, R.LinearRange(L.shared_at[name], L.shared_sizes[name]))
            shared.row_count, shared.activation_limit = c.row_capacity, c.activation_limit
            lib.linear_shared_expert_prepare.argtypes = [C.POINTER(R.LinearSharedExpertDescription), C.c_uint64,
                                                         C.POINTER(R.LinearKernels), C.POINTER(R.KernelLaunch)]
            lib.linear_shared_expert_block128_prepare.argtypes = [C.POINTER(R.LinearSharedExpertDescription), C.c_uint64,
                                                                  C.POINTER(R.LinearKernels),
                                                                  C.POINTER(api.BackendOperations), C.c_void_p,
                                                                  C.POINTER(R.KernelLaunch)]
            lib.linear_shared_expert_wide_prepare.argtypes = lib.linear_shared_expert_block128_prepare.argtypes
            four = (R.KernelLaunch * 4)()
            if wide:
                api.check(lib.linear_shared_expert_wide_prepare(C.byref(shared), card.arena_bytes, C.byref(kernels),
                                                                card.ops_pointer, card.handle, four),
                          "linear_shared_expert_wide_prepare")
            elif L.block128:
                api.check(lib.linear_shared_expert_block128_prepare(C.byref(shared), card.arena_bytes, C.byref(kernels),
                                                                    card.ops_pointer, card.handle, four),
                          "linear_shared_expert_block128_prepare")
            else:
                api.check(lib.linear_shared_expert_prepare(C.byref(shared), card.arena_bytes, C.byref(kernels), four),
                          "linear_shared_expert_prepare")
            lib.linear_rows_add_prepare.argtypes = [C.POINTER(R.LinearRange), C.POINTER(R.LinearRange), C.c_uint32,
                                                    C.c_uint32, C.c_uint64, C.POINTER(api.BackendOperations),
                                                    C.c_void_p, C.POINTER(R.KernelLaunch)]
            add = R.KernelLaunch()
            sums, values = span("row_output"), R.LinearRange(L.shared_at["output"], L.shared_sizes["output"])
            api.check(lib.linear_rows_add_prepare(C.byref(sums), C.byref(values), H, c.row_capacity, card.arena_bytes,
                                                  card.ops_pointer, card.handle, C.byref(add)), "linear_rows_add_prepare")
            shared_launches = list(four) + [add]
        reduce = R.OrderedReduceBf16Description()
        reduce.reduce.collective = R.OrderedCollective(L.peer_table, L.region, L.slot_input, L.result, 0, L.step,
                                                       L.parity_stride, c.deadline_cycles, c.row_capacity * H,
                                                       rank_count, rank, 0)
        reduce.reduce.status_offset, reduce.reduce.width = L.status, H
        reduce.reduce.mode = R.ORDERED_REDUCE_OWNER_RUNS if wide else R.ORDERED_REDUCE_EVERY_RANK
        reduce.pair_output_offset, reduce.arena_byte_count = L.at["row_output"], card.arena_bytes
        reduce.pairs_per_row, reduce.row_capacity = 1, c.row_capacity
        lib.ordered_reduce_bf16_prepare.argtypes = [C.POINTER(R.OrderedReduceBf16Description),
                                                    C.POINTER(api.BackendOperations), C.c_void_p,
                                                    C.POINTER(R.KernelLaunch)]
        lib.ordered_publish_reduce_bf16_prepare.argtypes = [C.POINTER(R.OrderedReduceBf16Description), C.c_uint64,
                                                            C.c_uint64, C.POINTER(api.BackendOperations), C.c_void_p,
                                                            C.POINTER(R.KernelLaunch)]
        if L.flags:
            # row sums of the pair outputs, the always-on expert's rows, READY and the ranks' sum in one launch: it
            # stands for expert_row_sum_entry, trunk_rows_add_entry and the reduction's two
            reduce.pair_output_offset, reduce.pairs_per_row = L.at["pair_output"], c.picks
            reduce_launches = (R.KernelLaunch * 1)()
            api.check(lib.ordered_publish_reduce_bf16_prepare(
                C.byref(reduce), L.shared_at["output"] if c.shared else 0, L.at["row_output"], card.ops_pointer,
                card.handle, reduce_launches), "ordered_publish_reduce_bf16_prepare")
            self.step_launches = list(self.expert_launches)[:3]
            shared_launches = shared_launches[:4]
        else:
            reduce_launches = (R.KernelLaunch * 2)()
            api.check(lib.ordered_reduce_bf16_prepare(C.byref(reduce), card.ops_pointer, card.handle, reduce_launches),
                      "ordered_reduce_bf16_prepare")
            self.step_launches = list(self.expert_launches)
        # the always-on expert reads the quantized rows alone: its four launches are a side run of the graph beside the
        # routed experts' launches (a decode step's trunk launches are too small to fill the card by themselves);
        # the join is the launch that adds its rows to the routed experts' sums
        behind = shared_launches[4:] + list(reduce_launches)  # the launch that joins the two runs first
        if shared_launches and side_run:
            for launch in shared_launches[:4]:
                launch.branch = R.LAUNCH_SIDE
            self.expert_launches[0].branch = R.LAUNCH_RESUME
            behind[0].branch = R.LAUNCH_JOIN
            self.launches = head + shared_launches[:4] + self.step_launches + behind
        else:
            self.launches = head + self.step_launches + shared_launches[:4] + behind
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
        self.sequence = 0

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

    def connect_local(self, layers):
        for peer, other in enumerate(layers):
            self.card.peer_connect(other.card, 0, self.layout.peer_table + 32 * peer)

    def connect_handles(self, handles):
        for peer, handle in enumerate(handles):
            if peer == self.rank:
                self.card.peer_connect(self.card, 0, self.layout.peer_table + 32 * peer)
            else:
                self.card.ipc_connect(handle, 0, self.layout.peer_table + 32 * peer)

    def stage_step(self, staging_offset, sequence, tokens, scores):
        L, view = self.layout, self.card.staging_view
        block = R.StepBlock(sequence, tokens.shape[0], 0)
        view[staging_offset:staging_offset + 16] = np.frombuffer(bytes(block), dtype=np.uint8)
        at = staging_offset + (L.tokens - L.step)
        view[at:at + tokens.nbytes] = tokens.reshape(-1).view(np.uint8)
        at = staging_offset + (L.scores - L.step)
        view[at:at + scores.nbytes] = np.ascontiguousarray(scores, dtype=np.float32).reshape(-1).view(np.uint8)

    def submit(self, staging_offset, result_staging_offset, rows):
        L, card = self.layout, self.card
        card.upload_async(L.step, staging_offset, L.step_input_bytes)
        card.graph_run(self.graph)
        return card.download_async(L.result, result_staging_offset, rows * self.config.hidden * 2)

    def step(self, tokens, scores):
        """One layer call on host arrays; returns bfloat16 bits [rows][hidden]."""
        L, card = self.layout, self.card
        rows = tokens.shape[0]
        self.sequence += 1
        result_at = api.align(L.step_input_bytes, 4096)
        self.stage_step(0, self.sequence, tokens, scores)
        nbytes = rows * self.config.hidden * 2
        # one library call: inputs in, the graph, status block and result out, wait
        card.step_run(self.graph, L.step, 0, L.step_input_bytes, L.status, result_at, 16 + nbytes)
        status = card.staging_view[result_at:result_at + 16].view(np.uint32)
        if status[0] != 0:
            raise RuntimeError("ordered reduction failed: code %d (1 timed out, 2 bad sequence), phase %d, rank %d"
                               % (status[0], status[1], status[2]))
        return card.staging_view[result_at + 16:result_at + 16 + nbytes].view(np.uint16).reshape(
            rows, self.config.hidden).copy()

    def check_status(self):
        status = self.card.download(self.layout.status, 16, np.uint32)
        if status[0] != 0:
            raise RuntimeError("ordered reduction failed: code %d (1 timed out, 2 bad sequence), phase %d, rank %d"
                               % (status[0], status[1], status[2]))
