"""Benchmark of the quantized MoE expert-layer hot path: one step = one layer call over one batch of M tokens.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--rows M] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Workload (synthetic, seeded; no checkpoint is available offline): the EXL3 MoE layer of the headline metric, 256 routed
+ 1 shared experts, top-8 sigmoid routing, hidden 4096, intermediate 2048, a stored width per expert drawn from
{2, 3, 4} bits with probabilities {0.2, 0.5, 0.3}, M = 8 decode tokens, sharded over N GPUs by intermediate columns
with the fixed-order FP32 -> bfloat16 reduction at the end. Every step draws its own tokens and router scores, so each
step streams a different set of about 58 experts (about 0.55 GB at N = 1, more than the 126 MB L2).

One JSON line on rank 0:
  value     tokens/s with every step's inputs already resident in HBM (a device-side step_input_select hands them over),
            timed with CUDA events on the card's stream, max over ranks; behind the barrier one untimed step lets
            the ranks meet on the device, so that the events hold the K steps and no rank's wait for a late one;
  e2e       the same through the public call with host buffers: per step the host -> device copy of the step's inputs
            from pinned memory, the layer's graph, the device -> host copy of the bfloat16 result, and the wait for it;
  roofline  the dominant kernel (exl3_layer_products: every product of the step) timed alone, launch by launch, with
            CUDA events, against the
            measured HBM copy bandwidth of MEASURED_PEAKS.json;
  cpu_baseline  the CPU oracle (OpenMP, all host cores) on a bounded sample of the same step, scaled to the step.
Further objects of the same line, each with its own value, e2e and roofline where they apply:
  prefill            cfg4: the same layer for M = 4096 rows, Zipf(1.1) routing, experts sharded over the ranks,
                     tensor-core (tcgen05) grouped products, ordered reduction with owner runs;
  original_weights   cfg5 decode: MXFP4 routed experts and the E4M3 always-on expert, E4M3 block-quantized activations;
  original_weights_prefill  cfg5 prefill: the same layer for M = 2048 rows (group products: two jobs of eight rows a block);
  reduction          (N > 1) cfg2: the fixed-order reduction alone, FP32 [M][4096] a rank, M in {1, 8, 64}, in this
                     library's four forms, microseconds a call and NVLink bytes a second;
  reference_kernels  (N = 1) the reference's own EXL3 kernels, recompiled for sm_100a from its sources into oracle/_ref,
                     timed on this card beside this library's expert launches on the same inputs (every expert K3).
--impl reference times that CPU restatement of the reference's arithmetic alone (the reference has no engine CPU path
for this layer), on the same metric and config.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "MoE expert-layer tok/s (decode M=8, prefill M=4096) at 1/2/4/8 B200"
SEED = 20261125
# dram bytes moved per algorithmic byte by the gate/up product kernel: dram__bytes_read.sum + dram__bytes_write.sum of
# one ncu capture of a 64-expert, 8-row launch over that launch's algorithmic bytes (the capture is too large for the
# full workload; traffic grows in proportion to the experts streamed)
GATE_UP_TRAFFIC_RATIO = 1.03
# the same for the prefill's gate/up products (one capture at 32 experts and 1024 rows: 401.3 MB read and 45.0 MB
# written against 444 MB of codes, scales, operand blocks read and down operand blocks written) and for the
# original-weights gate/up products (one capture at 64 experts: 360.1 MB against 356.8 MB)
PREFILL_TRAFFIC_RATIO = 1.00
MX_GATE_UP_TRAFFIC_RATIO = 1.01


def parse():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--rows", type=int, default=8)
    parser.add_argument("--impl", default="ours")
    parser.add_argument("--experts", type=int, default=256)
    parser.add_argument("--hidden", type=int, default=4096)
    parser.add_argument("--inner", type=int, default=2048)
    parser.add_argument("--prefill-rows", type=int, default=4096, help="0 skips the prefill part")
    parser.add_argument("--prefill-steps", type=int, default=5)
    parser.add_argument("--cut", default="0,0",
                        help="runs of K of the decode products (gate/up,down); 0: the library's measured default")
    parser.add_argument("--no-original-weights", action="store_true", help="skip the MXFP4 part")
    parser.add_argument("--original-prefill-rows", type=int, default=2048,
                        help="rows of the original-weights prefill (cfg5); 0 skips it")
    parser.add_argument("--no-reduction", action="store_true",
                        help="skip the reduction-alone measurement of runs on two or more GPUs")
    parser.add_argument("--no-reference-kernels", action="store_true",
                        help="skip the reference's own kernels on this card (N = 1 only)")
    return parser.parse_args()


def expert_matrices(config, widths):
    """expert -> its three FULL stored matrices, drawn from a stream of its own so that every rank draws the same."""
    from anemone_b200 import synthetic

    def draw(expert):
        rng = np.random.default_rng([SEED, 1000 + expert])
        width = int(widths[expert])
        return (synthetic.exl3_matrix(rng, config.hidden, config.inner, width),
                synthetic.exl3_matrix(rng, config.hidden, config.inner, width),
                synthetic.exl3_matrix(rng, config.inner, config.hidden, width))
    return draw


def step_inputs(config, rows, count):
    from anemone_b200 import synthetic
    steps = []
    for index in range(count):
        rng = np.random.default_rng([SEED, 7, index])
        steps.append((synthetic.tokens(rng, rows, config.hidden),
                      rng.normal(0.0, 1.0, size=(rows, config.experts)).astype(np.float32)))
    return steps


def layer_widths(config):
    from anemone_b200 import synthetic
    rng = np.random.default_rng([SEED, 3])
    return np.concatenate([synthetic.expert_widths(rng, config.experts), [3] * config.shared]).astype(np.uint32)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons every 200 ms while a timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.samples, self.process = [], None
        try:
            self.process = subprocess.Popen(["nvidia-smi", "-i", str(device), "--query-gpu=" + self.QUERY,
                                             "--format=csv,noheader,nounits", "-lms", "200"],
                                            stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.process = None

    def _read(self):
        for line in self.process.stdout:
            self.samples.append([field.strip() for field in line.split(",")])

    def stop(self):
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.process.terminate()
        self.thread.join(timeout=2)
        clocks = [float(s[0]) for s in self.samples if s and s[0].replace(".", "").isdigit()]
        maxima = [float(s[1]) for s in self.samples if len(s) > 1 and s[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for s in self.samples if len(s) >= 8 for i in range(4) if s[4 + i] == "Active"})
        return {"sm_mhz": float(np.median(clocks)) if clocks else None,
                "sm_max_mhz": max(maxima) if maxima else None, "reasons": reasons, "samples": len(clocks)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            return float(json.load(handle)["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    return 6650.0, "fallback (6.65 TB/s, an earlier measurement on this pool)"


def measured_tensor_peak():
    """Dense bf16 TFLOP/s of a kernel timed alone (the burst figure)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            return float(json.load(handle)["bf16_tflops"]), "measured burst (MEASURED_PEAKS.json)"
    return 1590.0, "fallback (1.59 PFLOP/s, an earlier measurement on this pool)"


def prefill_inputs(config, rows, index):
    """Tokens and router scores of one prefill call: expert popularity Zipf(1.1) over a seeded order of the experts."""
    from anemone_b200 import synthetic
    rng = np.random.default_rng([SEED, 11, index])
    order = np.random.default_rng([SEED, 12]).permutation(config.experts)
    popularity = 1.0 / np.arange(1, config.experts + 1, dtype=np.float64) ** 1.1
    bias = np.log(popularity / popularity.mean())[order]
    scores = (rng.normal(0.0, 1.0, size=(rows, config.experts)) + bias).astype(np.float32)
    return synthetic.tokens(rng, rows, config.hidden), scores


def run_prefill(args, api, base, widths, draw, rank, world, local_rank, dist, barrier, maximum):
    """cfg4: the same layer for M = 4096 rows, experts sharded over the ranks (a run of routed experts each, the
    always-on expert by columns), Zipf(1.1) routing, tensor-core products, ordered reduction to bfloat16."""
    from anemone_b200 import records as R
    from anemone_b200 import synthetic
    from anemone_b200.moe import MoeConfig
    from anemone_b200.prefill import PrefillLayer, PrefillLayout, Share
    rows, steps, warmup = args.prefill_rows, args.prefill_steps, 3
    config = MoeConfig(hidden=base.hidden, inner=base.inner, experts=base.experts, shared=base.shared,
                       picks=base.picks, row_capacity=rows)
    share = Share.expert_parallel(config, world, rank)
    held = share.experts(config)
    local_widths = widths[held]
    layout = PrefillLayout(config, local_widths, share)
    card = api.Card(local_rank, layout.arena_bytes, staging_bytes=128 << 20)
    matrices = (share.matrices(config, e, int(widths[e]), *draw(e)) for e in held)
    layer = PrefillLayer(card, config, local_widths, matrices, share, rank=rank, rank_count=world)
    if dist is None:
        layer.connect_local([layer])
    else:
        handles = [None] * world
        dist.all_gather_object(handles, card.ipc_export())
        layer.connect_handles(handles)
    card.wait()
    barrier()
    inputs = [prefill_inputs(config, rows, index) for index in range(2)]

    # ---- value: tokens and scores resident; only the 16-byte step block (the reduction's sequence) goes in ----
    layer.load(*inputs[0])
    first = layer.sequence
    for index in range(warmup + steps + 1):  # one more: the untimed call behind the barrier that aligns the ranks
        block = R.StepBlock(first + 1 + index, rows, 0)
        card.staging_view[64 * index:64 * index + 16] = np.frombuffer(bytes(block), dtype=np.uint8)

    tickets = []

    def resident(index):
        if len(tickets) >= 4:  # the card takes a bounded number of copies in flight
            card.transfer_wait(tickets[-4])
        tickets.append(card.upload_async(layout.step, 64 * index, 16))
        layer.run()
    for index in range(warmup):
        resident(index)
    card.wait()
    barrier()
    resident(warmup)  # untimed: the ranks meet in its reduction, so the timed region begins together on every card
    launches_before = card.launch_count()
    card.measure_begin()
    for index in range(warmup + 1, warmup + 1 + steps):
        resident(index)
    card.measure_end()
    device_ms = maximum(card.measure_elapsed_us() / 1000.0) / steps
    card.wait()
    launches = (card.launch_count() - launches_before) // steps
    layer.sequence = first + warmup + steps + 1
    layer.result(1)  # raises if a wait expired or the reduction failed
    barrier()

    # ---- e2e: a call's inputs in page-locked host memory, its result back in page-locked host memory, every call ----
    # (two input sets staged once, as a caller that produces its tokens and scores in page-locked buffers has them;
    # every call copies its 37.7 MB in, runs, copies status and result out and waits, in one library call)
    stride = api.align(layout.input_bytes, 4096)
    result_at = 2 * stride
    for index in range(2):
        layer.stage(index * stride, *inputs[index])
    for index in range(2):
        layer.call((index % 2) * stride, result_at)
    if card.waits_expired():
        raise RuntimeError("a prefill CTA gave up a bounded wait")
    barrier()
    wall_begin = time.perf_counter()
    for index in range(steps):
        layer.call((index % 2) * stride, result_at)
    e2e_ms = maximum(1000.0 * (time.perf_counter() - wall_begin)) / steps
    if card.waits_expired():
        raise RuntimeError("a prefill CTA gave up a bounded wait")
    barrier()

    # ---- roofline: the dominant kernel alone ----
    roofline = None
    counts = card.download(layout.workspace + layout.parts.counts, (len(held) + 1) * 4, np.uint32)
    if rank == 0:
        gate_up = (R.KernelLaunch * 1)(layer.launches[4])
        card.run(gate_up)
        card.wait()
        card.measure_begin()
        for _ in range(3):
            card.run(gate_up)
        card.measure_end()
        us = card.measure_elapsed_us() / 3
        flops = sum(int(counts[local]) * 2 * 2 * config.hidden *
                    (share.inner if expert < config.experts else share.shared_inner)
                    for local, expert in enumerate(held))
        peak, source = measured_tensor_peak()
        achieved = flops / us / 1e6  # TFLOP/s
        # bytes of the launch: gate and up of every expert that has a row; a row tile's operand blocks of both in, its
        # down operand blocks out (whole tiles of 128 rows move, filled or not)
        tiles_of = [(int(counts[local]) + 127) // 128 for local in range(len(held))]
        byte_total = sum((2 * synthetic.matrix_bytes(config.hidden, share.inner if expert < config.experts else
                                                     share.shared_inner, int(widths[expert])) if tiles else 0) +
                         tiles * 128 * (2 * config.hidden * 2 +
                                        (share.inner if expert < config.experts else share.shared_inner) * 2)
                         for (local, expert), tiles in zip(enumerate(held), tiles_of))
        roofline = {"kernel": "exl3_prefill_gate_up", "bound": "tensor", "achieved": achieved, "peak": peak,
                    "unit": "TFLOP/s", "frac": achieved / peak, "peak_source": source,
                    "traffic": PREFILL_TRAFFIC_RATIO * byte_total, "algorithmic_bytes_per_launch": byte_total,
                    "algorithmic_flops_per_launch": flops, "us_per_launch": us,
                    "row_tiles": int(counts[len(held)]), "pairs": int(counts[:len(held)].sum())}
    card.wait()
    barrier()
    card.close()
    return {"value": rows * 1000.0 / device_ms, "unit": "tok/s", "ms_per_step": device_ms, "rows": rows,
            "steps": steps, "warmup": warmup, "gpu_launches_per_step": int(launches),
            "e2e": {"value": rows * 1000.0 / e2e_ms, "unit": "tok/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": layout.input_bytes,
                    "d2h_bytes_per_step": rows * config.hidden * 2 + 16},
            "roofline": roofline,
            "config": {"workload": "cfg4 EXL3 MoE layer prefill: M=%d, Zipf(1.1) expert popularity, %d of %d routed "
                                   "experts a GPU and 1/%d of the shared expert's columns" %
                                   (rows, share.local_count, config.experts, world),
                       "parallelism": "ep%d, ordered FP32->bf16 reduce (owner runs)" % world,
                       "l2": "inputs larger than L2: a call streams its operand blocks (1 GB at N=1) and every "
                             "local expert's matrices"}}


def host_threads():
    """The threads the CPU legs use: every core this process may run on (a launcher's OMP_NUM_THREADS is not obeyed:
    the thread count is handed to the oracle explicitly)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_step(config, widths, cached, tokens, scores, threads):
    """Seconds of ONE whole layer call on the CPU oracle (every expert job of the step, all columns: the CPU has no
    ranks), matrices drawn before the clock starts."""
    from oracle import binding, moe_reference
    oracle = binding.load_oracle()
    experts, weights = moe_reference.route(oracle, config, scores)
    for expert in sorted(set(experts.reshape(-1).tolist())) + list(range(config.experts, config.total_experts)):
        cached(expert)
    begin = time.perf_counter()
    experts, weights = moe_reference.route(oracle, config, scores)
    _, _, kept = moe_reference.rank_partial(oracle, config, widths, cached, tokens, experts, weights, 1, 0, threads)
    return time.perf_counter() - begin, kept


def matrix_cache(draw):
    cache = {}

    def cached(expert):
        if expert not in cache:
            cache[expert] = draw(expert)
        return cache[expert]
    return cached


def cpu_baseline(config, widths, draw, steps, rows):
    """The CPU oracle beside the GPU number: whole steps of the same workload on every host thread."""
    threads = host_threads()
    cached = matrix_cache(draw)
    seconds, jobs = [], 0
    for index, (tokens, scores) in enumerate(steps):
        elapsed, jobs = cpu_step(config, widths, cached, tokens, scores, threads)
        if index > 0 or len(steps) == 1:
            seconds.append(elapsed)
    mean = float(np.mean(seconds))
    return {"value": rows / mean, "unit": "tok/s", "cores": threads, "kind": "port", "extrapolated": False,
            "sample": "%d whole steps (the last of %d expert jobs) of the same workload on the OpenMP CPU oracle, "
                      "%d threads, %.2f s a step; one more step first as warm-up" % (len(seconds), jobs, threads, mean)}


def run_reference(args, config, widths, draw, rank, world):
    """--impl reference: the CPU restatement of the reference's arithmetic, every host thread, WHOLE steps of the
    whole layer (a CPU has no ranks: the value does not depend on the GPU count the arm is launched for)."""
    if rank != 0:
        return
    threads = host_threads()
    steps = step_inputs(config, args.rows, args.warmup + args.steps)
    cached = matrix_cache(draw)
    times, jobs = [], 0
    wall_begin = time.perf_counter()
    for index, (tokens, scores) in enumerate(steps):
        seconds, jobs = cpu_step(config, widths, cached, tokens, scores, threads)
        if index >= args.warmup:
            times.append(seconds)
    ms = 1000.0 * float(np.mean(times))
    value = args.rows * 1000.0 / ms
    info = {"value": value, "unit": "tok/s", "cores": threads, "kind": "port", "extrapolated": False,
            "sample": "%d whole steps of the whole layer (about %d expert jobs a step), %d threads; drawing a step's "
                      "matrices is outside its timed region (%.0f s of wall clock in all)" %
                      (len(times), jobs, threads, time.perf_counter() - wall_begin)}
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16xf16->f32", "data": "synthetic",
        "config": workload_config(args, config, world), "cpu_baseline": info,
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference has no engine CPU path for this layer and no sm_100 kernel build; this arm times the "
                "CPU restatement of its arithmetic (oracle/, pinned to its known-answer vectors and to its own host "
                "code compiled from its sources) on the host cores"}))


def checked_step(config, widths, draw, layer, step, rank, world, dist):
    """One more step whose result is CHECKED: every rank's bfloat16 result against the rank-ordered FP32 sum of the rows
    the ranks really published, rounded once, bit for bit (the CPU oracle's ordered reduction), and against the CPU
    oracle's whole layer within the path's tolerance (max-abs 2e-2, cosine 0.9999). Rank 0 gathers and checks."""
    from anemone_b200 import synthetic
    tokens, scores = step
    rows = tokens.shape[0]
    got = layer.step(tokens, scores).reshape(-1)
    L = layer.layout
    slot = L.region + (layer.sequence & 1) * L.parity_stride + L.slot_input
    published = layer.card.download(slot, rows * config.hidden * 4, np.float32)
    picks = layer.card.download(L.picks, rows * config.picks * 4, np.uint32).reshape(rows, config.picks)
    if dist is None:
        everyone = [(published, got, picks)]
    else:
        everyone = [None] * world if rank == 0 else None
        dist.gather_object((published, got, picks), everyone, dst=0)
    if rank != 0:
        return None
    from oracle import binding, moe_reference
    from oracle.binding import pointer_array, ptr, u16p
    oracle = binding.load_oracle()
    want = np.zeros(rows * config.hidden, dtype=np.uint16)
    inputs = [np.ascontiguousarray(entry[0]) for entry in everyone]
    oracle.orc_ordered_reduce_bf16(pointer_array(inputs), world, want.size, ptr(want, u16p))
    bit_exact = all(np.array_equal(entry[1], want) for entry in everyone)
    expected, partials, experts, _ = moe_reference.layer(oracle, config, widths, matrix_cache(draw), tokens, scores,
                                                         world, host_threads())
    a = synthetic.from_bfloat16(got).astype(np.float64)
    b = synthetic.from_bfloat16(expected.reshape(-1)).astype(np.float64)
    worst = float(np.abs(a - b).max())
    cosine = float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-300))
    # before the one rounding: the rank-ordered FP32 sums of the published rows against the oracle's
    total, wanted = np.zeros(rows * config.hidden, dtype=np.float32), np.zeros(rows * config.hidden, dtype=np.float32)
    for entry, partial in zip(everyone, partials):
        total = total + entry[0]
        wanted = wanted + partial.reshape(-1)
    worst_fp32 = float(np.abs(total.astype(np.float64) - wanted.astype(np.float64)).max())
    # a bfloat16 value of magnitude 4 or more has steps of 2^-5 and more: where the FP32 sums straddle a rounding
    # boundary the results differ by one such step, which the 2e-2 bound on the sums does not forbid
    step = float(2.0 ** (np.floor(np.log2(max(np.abs(b).max(), 1e-30))) - 7))
    picks_exact = all(np.array_equal(entry[2], experts) for entry in everyone)
    ok = bit_exact and picks_exact and cosine >= 0.9999 and worst_fp32 <= 2e-2 and worst <= max(2e-2, step)
    return {"ok": bool(ok), "ordered_reduction_bit_exact_on_every_rank": bool(bit_exact),
            "router_picks_bit_exact": bool(picks_exact), "layer_max_abs_vs_cpu_oracle": worst,
            "layer_cosine_vs_cpu_oracle": cosine, "fp32_sums_max_abs_vs_cpu_oracle": worst_fp32,
            "bfloat16_step_at_largest_output": step, "ranks": world,
            "what": "one more step after the timed regions: every rank's result against the oracle's rank-ordered "
                    "sum of the FP32 rows the ranks published over NVLink (bit for bit), the ranks' FP32 sums before "
                    "the one rounding and the bfloat16 layer output against the oracle's whole layer (max-abs 2e-2, "
                    "or one bfloat16 step where outputs reach magnitude 4; cosine 0.9999)"}


def workload_config(args, config, world):
    return {"workload": "cfg3 EXL3 MoE layer decode: %d routed + %d shared experts, top-%d, hidden %d, intermediate %d, "
                        "per-expert widths {2,3,4} p={0.2,0.5,0.3}, M=%d" % (config.experts, config.shared,
                                                                                 config.picks, config.hidden,
                                                                                 config.inner, args.rows),
            "rows": args.rows, "parallelism": "tp%d by intermediate columns, ordered FP32->bf16 reduce" % world,
            "l2": "inputs larger than L2: every step routes to a different expert set (~58 experts of 257)",
            "timing": "W warm-up steps, barrier and synchronize, one more untimed step in which the ranks meet on the "
                      "device, then K steps between two CUDA events on the launching stream, max over ranks"}


def run_reference_kernels(args, api, base, draw_k3, local_rank):
    """The reference's own EXL3 kernels on this card, beside this library's, on the same inputs: its retained chain
    and its fast form (source/kernel_exl3.cu, source/kernel_exl3_wide.cu), recompiled for sm_100a from its sources into
    oracle/_ref and launched through its own preparer. Its chain takes ONE stored width a record, so every expert is
    K3 here (3 bits a weight; the headline workload's mix averages 3.1). Two comparisons, each the mean of three
    passes over the steps with the spread between the passes:
      expert launches alone (input transform, products, activation, output transform, row sum; the job table written
      before the clock starts): the reference's two chains and this library's launches of the separate preparers;
      the step WITH its router: the reference's fast chain behind a router launch (up to its FP32 row sums), against
      this library's four launches of the whole decode step (router and input transform; gate/up; down, row sums,
      READY; the one-rank reduction to bfloat16, which the reference's side of this comparison does not have)."""
    from oracle import binding, reference_kernels
    if not reference_kernels.available():
        return {"unavailable": "oracle/_ref holds no reference kernel images (built where the reference tree is present)"}
    import ctypes as C
    from anemone_b200 import records as R
    from anemone_b200.moe import MoeLayer, MoeLayout
    reference = binding.load_reference()
    widths = np.full(base.total_experts, 3, dtype=np.uint32)
    layout = MoeLayout(base, widths, 1, 0, reduce_form="pull")
    fused_layout = MoeLayout(base, widths, 1, 0, reduce_form="fused")
    passes = 3
    steps = step_inputs(base, args.rows, 3 + args.steps)
    names = ("retained", "fast", "ours", "fast_with_router", "ours_step_with_router")
    elapsed = {name: [0.0] * passes for name in names}
    rows_of = {}

    def timed(where, chains, before, each, rows_at):
        """Every chain on every step, `passes` times over; before(): what runs untimed in front of a step's chains."""
        for repeat in range(passes):
            for index, (tokens, scores) in enumerate(steps):
                each.sequence += 1
                each.stage_step(0, each.sequence, tokens, scores)
                where.transfer_wait(where.upload_async(each.layout.step, 0, each.layout.step_input_bytes))
                before()
                for name, launches in chains.items():
                    where.measure_begin()
                    where.run(launches)
                    where.measure_end()
                    us = where.measure_elapsed_us()
                    if index >= 3:
                        elapsed[name][repeat] += us
                    if repeat == 0:
                        rows_of[name] = where.download(rows_at(), args.rows * base.hidden * 4, np.float32)

    # one card of a device at a time: the reference's chains and this library's separate launches first
    card = api.Card(local_rank, layout.arena_bytes)
    try:
        layer = MoeLayer(card, base, widths, (draw_k3(expert) for expert in range(base.total_experts)),
                         reduce_form="pull")
        layer.connect_local([layer])
        record = R.Exl3Expert(layout.jobs, layout.tokens, layout.operands, layout.products, layout.hidden,
                              layout.products, base.hidden, layout.inner_local, layout.pairs, base.pairs_per_row,
                              layout.job_capacity, 3, base.activation_limit, 0)
        backend = reference_kernels.RenamingBackend()
        chains = {"retained": list(reference_kernels.chain_launches(reference, backend, card, record,
                                                                    card.arena_bytes, False)),
                  "fast": list(reference_kernels.chain_launches(reference, backend, card, record, card.arena_bytes,
                                                                True)),
                  "ours": list(layer.launches[1:4])}
        row_sum = R.ExpertRowSum(layout.products, layout.row_output, base.hidden, base.pairs_per_row)
        sum_launch = R.KernelLaunch()
        api.check(api.library().bb_exl3_row_sum_prepare(C.byref(row_sum), base.row_capacity, card.arena_bytes,
                                                        card.ops_pointer, card.handle, C.byref(sum_launch)),
                  "bb_exl3_row_sum_prepare")
        for name in chains:
            chains[name].append(sum_launch)
        chains["fast_with_router"] = list(layer.launches[0:1]) + chains["fast"]

        def route():  # the router: the job table every chain reads
            card.run(layer.launches[0:1])
            card.wait()
        timed(card, chains, route, layer, lambda: layout.row_output)
    finally:
        card.close()
    # then the decode step's four launches on a card of their own
    card = api.Card(local_rank, fused_layout.arena_bytes)
    try:
        fused = MoeLayer(card, base, widths, (draw_k3(expert) for expert in range(base.total_experts)),
                         reduce_form="fused")
        fused.connect_local([fused])
        timed(card, {"ours_step_with_router": list(fused.launches)}, lambda: None, fused,
              lambda: fused_layout.region + (fused.sequence & 1) * fused_layout.parity_stride + fused_layout.slot_input)
        fused.check_status()
    finally:
        card.close()
    worst = float(max(np.abs(rows_of["ours"] - rows_of[name]).max() for name in ("retained", "fast")))
    worst_fused = float(np.abs(rows_of["ours_step_with_router"] - rows_of["fast"]).max())
    out = {}
    for name, totals in elapsed.items():
        per_step = [total / args.steps for total in totals]
        out[name + "_us_per_step"] = float(np.mean(per_step))
        out[name + "_spread"] = float((max(per_step) - min(per_step)) / np.mean(per_step))
    out.update({"unit": "us of one decode step's launches, CUDA events; mean of %d passes over %d steps, spread = "
                        "(max - min) / mean of the passes" % (passes, args.steps), "rows": args.rows, "stored_width": 3,
                "speedup_over_fast": out["fast_us_per_step"] / out["ours_us_per_step"],
                "speedup_over_retained": out["retained_us_per_step"] / out["ours_us_per_step"],
                "step_speedup_over_fast_with_router": out["fast_with_router_us_per_step"] /
                                                      out["ours_step_with_router_us_per_step"],
                "max_abs_difference_of_row_sums": worst,
                "max_abs_difference_of_row_sums_step": worst_fused,
                "kernels": "the reference's source/kernel_exl3.cu (retained) and source/kernel_exl3_wide.cu (fast), "
                           "recompiled for sm_100a, through its own exl3_experts_prepare / exl3_experts_fast_prepare"})
    return out


def run_original_weights(args, api, base, rank, world, local_rank, dist, barrier, maximum):
    """cfg5: routed experts MXFP4 (E8M0 scales 2^-8 .. 2^-4), the always-on expert E4M3 with one FP32 scale per 128 by 128
    weights drawn U(0.5, 2) / 448 (the configuration's block-scaled FP8; the reference's own E4M3 format, one E8M0 code
    per 32 by 32 weights, is the library's other option), E4M3 block-quantized activations, decode M = 8, tensor
    parallel by intermediate columns."""
    from anemone_b200 import records as R
    from anemone_b200 import synthetic
    from anemone_b200.moe import MoeConfig
    from anemone_b200.mx import MxLayer, MxLayout, matrix_bytes
    rows, steps, warmup = args.rows, args.steps, args.warmup
    config = MoeConfig(hidden=base.hidden, inner=base.inner, experts=base.experts, shared=1, picks=base.picks,
                       row_capacity=rows, activation_limit=7.0)
    pool_entries = warmup + steps + 1  # the last: the untimed step behind the barrier
    layout = MxLayout(config, world, rank, pool_entries, block128=True)
    H, I = config.hidden, layout.inner_local
    card = api.Card(local_rank, layout.arena_bytes)

    def draw(expert):
        rng = np.random.default_rng([SEED, 2000 + expert, rank])
        return (synthetic.mx_matrix(rng, I, H), synthetic.mx_matrix(rng, I, H), synthetic.mx_matrix(rng, H, I))
    always_rng = np.random.default_rng([SEED, 2999, rank])
    always = (synthetic.e4m3_block128_matrix(always_rng, I, H), synthetic.e4m3_block128_matrix(always_rng, I, H),
              synthetic.e4m3_block128_matrix(always_rng, H, I))
    layer = MxLayer(card, config, (draw(expert) for expert in range(config.experts)), rank=rank, rank_count=world,
                    slices=(2, 2), shared_matrices=always, pool_entries=pool_entries, block128=True)
    if dist is None:
        layer.connect_local([layer])
    else:
        handles = [None] * world
        dist.all_gather_object(handles, card.ipc_export())
        layer.connect_handles(handles)
    card.wait()
    barrier()
    inputs = step_inputs(config, rows, pool_entries)
    # ---- value: every step's inputs wait in a pool on the card; a select launch in front of each step takes the next
    layer.load_pool([(index + 1, tokens, scores) for index, (tokens, scores) in enumerate(inputs)])
    barrier()
    for _ in range(warmup):
        layer.run_resident()
    card.wait()
    barrier()
    layer.run_resident()  # untimed: the ranks meet in its reduction, so the timed region begins together on every card
    launches_before = card.launch_count()
    card.measure_begin()
    for _ in range(steps):
        layer.run_resident()
    card.measure_end()
    device_ms = maximum(card.measure_elapsed_us() / 1000.0) / steps
    card.wait()
    launches = (card.launch_count() - launches_before) // steps
    layer.sequence = warmup + steps + 1
    layer.check_status()
    barrier()
    # ---- e2e ----
    for tokens, scores in inputs[:warmup]:
        layer.step(tokens, scores)
    barrier()
    wall_begin = time.perf_counter()
    for tokens, scores in inputs[warmup:warmup + steps]:
        layer.step(tokens, scores)
    e2e_ms = maximum(1000.0 * (time.perf_counter() - wall_begin)) / steps
    barrier()
    # ---- roofline: expert_gate_up alone ----
    roofline = None
    if rank == 0:
        peak, source = measured_peaks()
        gate_up = (R.KernelLaunch * 1)(R.KernelLaunch.from_buffer_copy(bytes(layer.expert_launches[0])))
        gate_up[0].branch = 0  # alone: in the step's graph it resumes the main run beside the always-on expert's
        card.run(gate_up)
        card.wait()
        card.measure_begin()
        for _ in range(5):
            card.run(gate_up)
        card.measure_end()
        us = card.measure_elapsed_us() / 5
        picks = card.download(layout.picks, rows * config.picks * 4, np.uint32)
        active = len(set(picks.tolist()))
        pairs = rows * config.picks
        byte_total = active * 2 * matrix_bytes(I, H) + rows * H * 2 + rows * H // 32 + pairs * I * 2
        achieved = byte_total / us / 1000.0
        roofline = {"kernel": "expert_gate_up_2", "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                    "frac": achieved / peak, "peak_source": source, "traffic": MX_GATE_UP_TRAFFIC_RATIO * byte_total,
                    "algorithmic_bytes_per_launch": byte_total, "us_per_launch": us, "active_experts": active}
    card.wait()
    barrier()
    card.close()
    return {"value": rows * 1000.0 / device_ms, "unit": "tok/s", "ms_per_step": device_ms, "rows": rows,
            "steps": steps, "warmup": warmup, "gpu_launches_per_step": int(launches),
            "e2e": {"value": rows * 1000.0 / e2e_ms, "unit": "tok/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": layout.step_input_bytes, "d2h_bytes_per_step": rows * H * 2},
            "roofline": roofline, "dtype": "e2m1 x e4m3 -> f32",
            "config": {"workload": "cfg5 original-weights MoE layer decode: %d routed MXFP4 experts (E2M1, one E8M0 "
                                   "scale per 32 inputs, exponents -8..-4), top-%d, 1 always-on expert E4M3 with one "
                                   "FP32 scale per 128x128 weights U(0.5,2)/448, hidden %d, intermediate %d, M=%d" %
                                   (config.experts, config.picks, H, config.inner, rows),
                       "parallelism": "tp%d by intermediate columns, ordered FP32->bf16 reduce" % world,
                       "l2": "inputs larger than L2: every step routes to a different expert set; a step's inputs are taken "
                             "from a pool on the card by a select launch"}}


def run_original_weights_prefill(args, api, base, rank, world, local_rank, dist, barrier, maximum):
    """cfg5 prefill: the same original-weights layer for M = 2048 rows, tensor parallel by intermediate columns. The
    products are linear_routed_experts_wide_prepare's (a group of two jobs of eight rows and several tiles a block, the
    thin instances' arithmetic bit for bit), not yet a tcgen05 grouped GEMM: the number says where that stands."""
    from anemone_b200 import synthetic
    from anemone_b200.moe import MoeConfig
    from anemone_b200.mx import MxLayer, MxLayout
    rows, steps, warmup = args.original_prefill_rows, 3, 2
    config = MoeConfig(hidden=base.hidden, inner=base.inner, experts=base.experts, shared=1, picks=base.picks,
                       row_capacity=rows, activation_limit=7.0)
    layout = MxLayout(config, world, rank, block128=True, wide=True)
    H, I = config.hidden, layout.inner_local
    card = api.Card(local_rank, layout.arena_bytes)

    def draw(expert):
        rng = np.random.default_rng([SEED, 2000 + expert, rank])
        return (synthetic.mx_matrix(rng, I, H), synthetic.mx_matrix(rng, I, H), synthetic.mx_matrix(rng, H, I))
    always_rng = np.random.default_rng([SEED, 2999, rank])
    always = (synthetic.e4m3_block128_matrix(always_rng, I, H), synthetic.e4m3_block128_matrix(always_rng, I, H),
              synthetic.e4m3_block128_matrix(always_rng, H, I))
    layer = MxLayer(card, config, (draw(expert) for expert in range(config.experts)), rank=rank, rank_count=world,
                    slices=(2, 2), shared_matrices=always, block128=True, wide=True)
    if dist is None:
        layer.connect_local([layer])
    else:
        handles = [None] * world
        dist.all_gather_object(handles, card.ipc_export())
        layer.connect_handles(handles)
    card.wait()
    barrier()
    inputs = [prefill_inputs(config, rows, 50 + index) for index in range(2)]
    # ---- e2e: the public call on host arrays (inputs up, graph, result down, wait) ----
    for index in range(warmup):
        layer.step(*inputs[index % 2])
    barrier()
    wall_begin = time.perf_counter()
    for index in range(steps):
        layer.step(*inputs[index % 2])
    e2e_ms = maximum(1000.0 * (time.perf_counter() - wall_begin)) / steps
    barrier()
    # ---- value: the inputs of the last call wait in the arena; a step's 16-byte block goes up, then the graph is timed
    device_us = 0.0
    launches_before = card.launch_count()
    for _ in range(steps):
        layer.sequence += 1
        card.upload(layout.step, np.frombuffer(bytes(R_step(layer.sequence, rows)), dtype=np.uint8))
        barrier()
        card.measure_begin()
        card.graph_run(layer.graph)
        card.measure_end()
        device_us += maximum(card.measure_elapsed_us())
        card.wait()
    launches = (card.launch_count() - launches_before) // steps
    layer.check_status()
    expired = card.expired_bits()
    barrier()
    card.close()
    if expired:
        raise RuntimeError("a kernel of the original-weights prefill gave up a bounded wait (bits %d)" % expired)
    device_ms = device_us / 1000.0 / steps
    return {"value": rows * 1000.0 / device_ms, "unit": "tok/s", "ms_per_step": device_ms, "rows": rows,
            "steps": steps, "warmup": warmup, "gpu_launches_per_step": int(launches),
            "e2e": {"value": rows * 1000.0 / e2e_ms, "unit": "tok/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": layout.step_input_bytes, "d2h_bytes_per_step": rows * H * 2},
            "dtype": "e2m1 x e4m3 -> f32", "jobs": layout.job_capacity,
            "config": {"workload": "cfg5 original-weights MoE layer prefill: M=%d, %d routed MXFP4 experts, top-%d, 1 "
                                   "always-on expert E4M3 with one FP32 scale per 128x128 weights, hidden %d, "
                                   "intermediate %d; group products (two jobs of eight rows a block, mma.sync, the thin instances' bits)" %
                                   (rows, config.experts, config.picks, H, config.inner),
                       "parallelism": "tp%d by intermediate columns, ordered FP32->bf16 reduce (owner runs)" % world}}


def R_step(sequence, rows):
    from anemone_b200 import records as R
    return R.StepBlock(sequence, rows, 0)


def run_reduction(args, api, hidden, rank, world, local_rank, dist, barrier, maximum):
    """cfg2: the fixed-order reduction ALONE between the ranks: FP32 [M][hidden] a rank, added in rank order, rounded
    once to bfloat16, M in {1, 8, 64}. Four forms of this library: every rank stores its rows into every rank's inbox and adds
    its inboxes (one launch: what a decode step uses), every rank pulls every rank's rows, owner runs (every rank adds its run and stores it into every rank), and the exchange's owner sums
    (every rank stores each owner's rows into the owner's inbox: the reference's tp_exchange entry points). Times are
    device times of a captured graph a call, the 16-byte step block copied in before each, max over ranks."""
    import ctypes as C
    from anemone_b200 import records as R
    lib = api.library()
    most = 64
    elements = most * hidden
    layout = api.Layout()
    peer_table, step, status = layout.take(16 * 32), layout.take(16), layout.take(16)
    pull_stride = api.align(384 + 4 * elements, 128)
    pull_region = layout.take(2 * pull_stride, 128)
    result, rows_at = layout.take(2 * elements), layout.take(4 * elements)
    signals = 2 * world * 128
    push_input, push_output, push_inbox = signals, signals + 4 * elements, signals + 8 * elements
    push_stride = api.align(push_inbox + world * 4 * elements, 128)
    push_region = layout.take(2 * push_stride, 128)
    # every call's step block waits in a pool on the card; a select launch in front of each call takes the next
    # the order the timings run in; the exchange last: its sequences (twice a step's and more) leave no room above
    forms = ("pull_every_rank", "pull_owner_runs", "push_every_rank", "exchange_owner_sums")
    row_counts, repeats, warm_graphs, timed_graphs = (1, 8, 64), 10, 1, 4
    pool_entries = len(forms) * len(row_counts) * repeats * (warm_graphs + 1 + timed_graphs)
    pool, cursor = layout.take(64 * pool_entries, 64), layout.take(16)
    copy_bytes = 64 << 20  # a peer copy's rate, measured here: what the calls' NVLink bytes a second are set against
    copy_from, copy_to = layout.take(copy_bytes, 4096), layout.take(copy_bytes, 4096)
    arena_bytes = layout.take(4096, 4096)
    card = api.Card(local_rank, arena_bytes)
    card.fill(0, 0, arena_bytes)
    card.fill(copy_from, rank + 1, copy_bytes)
    blocks = np.zeros(64 * pool_entries, dtype=np.uint8)
    entry = 0
    for form in forms:  # the order the timings below run in; sequences strictly increasing
        for rows in row_counts:
            for _ in range(repeats * (warm_graphs + 1 + timed_graphs)):
                blocks[64 * entry:64 * entry + 16] = np.frombuffer(bytes(R.StepBlock(entry + 1, rows, 0)), dtype=np.uint8)
                entry += 1
    card.upload(pool, blocks)
    select = R.StepInputSelect(pool, 64, step, cursor, pool_entries, 16)
    lib.step_input_select_prepare.argtypes = [C.POINTER(R.StepInputSelect), C.c_uint64,
                                              C.POINTER(api.BackendOperations), C.c_void_p, C.POINTER(R.KernelLaunch)]
    select_launch = R.KernelLaunch()
    api.check(lib.step_input_select_prepare(C.byref(select), arena_bytes, card.ops_pointer, card.handle,
                                            C.byref(select_launch)), "step_input_select_prepare")
    rng = np.random.default_rng([SEED, 4000, rank])
    values = rng.normal(0, 0.05, elements).astype(np.float32)
    card.upload(rows_at, values)
    for parity in range(2):
        card.upload(push_region + parity * push_stride + push_input, values)
    lib.ordered_reduce_bf16_prepare.argtypes = [C.POINTER(R.OrderedReduceBf16Description),
                                                C.POINTER(api.BackendOperations), C.c_void_p,
                                                C.POINTER(R.KernelLaunch)]
    lib.tp_exchange_wide_kernels_prepare.argtypes = [C.POINTER(api.BackendOperations), C.c_void_p, C.c_uint32,
                                                     C.POINTER(C.c_uint32)]
    lib.tp_exchange_wide_rows_prepare.argtypes = [C.POINTER(R.OrderedPushDescription), C.c_uint32, C.c_uint32,
                                                  C.c_uint32, C.POINTER(C.c_uint32), C.c_uint32,
                                                  C.POINTER(R.KernelLaunch)]
    graphs = {}

    def connect(region_of):
        peers = (R.OrderedPeer * world)()
        for peer in range(world):
            peers[peer].region_offset = region_of
        card.upload(peer_table, np.frombuffer(bytes(peers), dtype=np.uint8))
        if dist is None:
            card.peer_connect(card, 0, peer_table)
        else:
            handles = [None] * world
            dist.all_gather_object(handles, card.ipc_export())
            for peer, handle in enumerate(handles):
                if peer == rank:
                    card.peer_connect(card, 0, peer_table + 32 * peer)
                else:
                    card.ipc_connect(handle, 0, peer_table + 32 * peer)
    # the peer table names a rank's region: written for the pull forms first, rewritten for the exchange below
    connect(pull_region)
    # every rank copies 64 MB into its right neighbour's arena at once (a copy launch: the card's copy engine), eight
    # times between two events; the rate is the slowest rank's
    neighbour = (rank + 1) % world
    copies = [R.copy_launch(copy_from, copy_to, copy_bytes, destination_word=peer_table + 32 * neighbour)] * 8
    card.run(copies[:1])
    card.wait()
    barrier()
    card.measure_begin()
    card.run(copies)
    card.measure_end()
    peer_copy_gbs = len(copies) * copy_bytes / maximum(card.measure_elapsed_us()) / 1000.0
    received = card.download(copy_to, 64, np.uint8)  # the left neighbour's bytes have arrived (its rank in every byte)
    barrier()
    if not (received == (rank - 1) % world + 1).all():
        raise RuntimeError("the peer copy did not arrive")
    for mode, name in ((R.ORDERED_REDUCE_EVERY_RANK, "pull_every_rank"), (R.ORDERED_REDUCE_OWNER_RUNS, "pull_owner_runs")):
        for rows in (1, 8, 64):
            reduce = R.OrderedReduceBf16Description()
            reduce.reduce.collective = R.OrderedCollective(peer_table, pull_region, 384, result, 0, step, pull_stride,
                                                           2_000_000_000, rows * hidden, world, rank, 0)
            reduce.reduce.status_offset, reduce.reduce.width, reduce.reduce.mode = status, hidden, mode
            reduce.pair_output_offset, reduce.arena_byte_count = rows_at, arena_bytes
            reduce.pairs_per_row, reduce.row_capacity = 1, rows
            launches = (R.KernelLaunch * 2)()
            api.check(lib.ordered_reduce_bf16_prepare(C.byref(reduce), card.ops_pointer, card.handle, launches),
                      "ordered_reduce_bf16_prepare")
            graphs[(name, rows)] = (card.graph(([select_launch] + list(launches)) * repeats), 2)
    results = {}

    def timed(name, rows):
        graph, launches = graphs[(name, rows)]
        barrier()
        for _ in range(warm_graphs):
            card.graph_run(graph)
        card.wait()
        barrier()
        card.graph_run(graph)  # untimed: the ranks meet on the device before the timed graphs begin
        card.measure_begin()
        for _ in range(timed_graphs):
            card.graph_run(graph)
        card.measure_end()
        card.wait()
        return maximum(card.measure_elapsed_us() / (timed_graphs * repeats)), launches
    for name in ("pull_every_rank", "pull_owner_runs"):
        for rows in (1, 8, 64):
            results[(name, rows)] = timed(name, rows)
    if card.download(status, 16, np.uint32)[0] != 0:
        raise RuntimeError("ordered reduction failed in the reduction bench")
    barrier()
    connect(push_region)
    lib.ordered_rows_push_prepare.argtypes = [C.POINTER(R.OrderedRowsPushDescription), C.POINTER(api.BackendOperations),
                                              C.c_void_p, C.POINTER(R.KernelLaunch)]
    for rows in (1, 8, 64):
        push = R.OrderedRowsPushDescription()
        push.arguments.push = R.OrderedPush(peer_table, push_region, 0, result, push_inbox, step, push_stride,
                                            2_000_000_000, 4 * elements, rows * hidden, world, rank,
                                            R.ORDERED_PUSH_FP32, 0, 0)
        push.arguments.pair_output_offset, push.arguments.width, push.arguments.pairs_per_row = rows_at, hidden, 1
        push.arena_byte_count = arena_bytes
        one = (R.KernelLaunch * 1)()
        api.check(lib.ordered_rows_push_prepare(C.byref(push), card.ops_pointer, card.handle, one),
                  "ordered_rows_push_prepare")
        graphs[("push_every_rank", rows)] = (card.graph(([select_launch] + list(one)) * repeats), 1)
    for rows in (1, 8, 64):
        results[("push_every_rank", rows)] = timed("push_every_rank", rows)
    kernels = (C.c_uint32 * 4)()
    api.check(lib.tp_exchange_wide_kernels_prepare(card.ops_pointer, card.handle, R.TP_EXCHANGE_FORM_OWNER_SUMS, kernels),
              "tp_exchange_wide_kernels_prepare")
    for rows in (1, 8, 64):
        arguments = R.OrderedPush(peer_table, push_region, push_input, push_output, push_inbox, step, push_stride,
                                  2_000_000_000, 4 * elements, rows * hidden, world, rank, R.ORDERED_PUSH_FP32, 0, 0)
        description = R.OrderedPushDescription(arguments, arena_bytes)
        launches = (R.KernelLaunch * 4)()
        api.check(lib.tp_exchange_wide_rows_prepare(C.byref(description), hidden, 0, 1, kernels,
                                                    R.TP_EXCHANGE_FORM_OWNER_SUMS, launches),
                  "tp_exchange_wide_rows_prepare")
        graphs[("exchange_owner_sums", rows)] = (card.graph(([select_launch] + list(launches)) * repeats), 4)
    for rows in (1, 8, 64):
        results[("exchange_owner_sums", rows)] = timed("exchange_owner_sums", rows)
    expired = card.expired_bits()
    barrier()
    card.close()
    if expired:
        raise RuntimeError("an exchange kernel gave up (bits %d) in the reduction bench" % expired)
    share = (world - 1) / world
    remote = {"pull_every_rank": lambda rows: (world - 1) * rows * hidden * 4,
              "pull_owner_runs": lambda rows: share * rows * hidden * (4 + 2),
              "exchange_owner_sums": lambda rows: share * rows * hidden * (4 + 2),
              "push_every_rank": lambda rows: (world - 1) * rows * hidden * 4}
    out = []
    for (name, rows), (us, launches) in sorted(results.items()):
        moved = remote[name](rows)
        out.append({"form": name, "rows": rows, "us_per_call": us, "launches_per_call": launches,
                    "remote_bytes_per_rank": int(moved), "nvlink_gbs": moved / us / 1000.0,
                    "frac_of_peer_copy_measured": moved / us / 1000.0 / peer_copy_gbs,
                    "frac_of_900_nominal": moved / us / 1000.0 / 900.0})
    return {"config": {"workload": "cfg2 ordered reduction alone: FP32 [M][%d] a rank, N(0, 0.05^2), rank order, one "
                                   "rounding to bfloat16, M in {1, 8, 64}, %d ranks" % (hidden, world)},
            "note": "a call is a select launch (the next step block from a pool on the card) and the form's "
                    "launches; ten calls a captured graph, four graphs timed back to back; the exchange's rows "
                    "wait in its slot, the pull forms first add one 'pair' a row into theirs (their publish launch)",
            "peer_copy_gbs": peer_copy_gbs,
            "peer_copy": "every rank copies 64 MB into its right neighbour's arena at once, eight copies between two "
                         "CUDA events, the slowest rank's rate: GB/s a direction a GPU, measured in this run",
            "calls": out}


def main():
    args = parse()
    from anemone_b200.moe import MoeConfig
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    config = MoeConfig(hidden=args.hidden, inner=args.inner, experts=args.experts, shared=1, picks=8,
                       row_capacity=args.rows)
    widths = layer_widths(config)
    draw = expert_matrices(config, widths)
    if args.impl == "reference":
        run_reference(args, config, widths, draw, rank, world)
        return

    from anemone_b200 import api, synthetic
    from anemone_b200 import records as R
    from anemone_b200.moe import MoeLayer, MoeLayout, local_matrices
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if dist is not None:
            dist.barrier()

    def maximum(value):
        if dist is None:
            return value
        import torch
        tensor = torch.tensor([value], dtype=torch.float64, device="cuda")
        dist.all_reduce(tensor, op=dist.ReduceOp.MAX)
        return float(tensor.item())

    if api.card_count() <= local_rank:
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    # one step more than the warm-up and the timed ones: it runs untimed behind the barrier (see below)
    total_steps = args.warmup + args.steps + 1
    layout = MoeLayout(config, widths, world, rank, pool_entries=total_steps)
    card = api.Card(local_rank, layout.arena_bytes)
    matrices = (local_matrices(*draw(expert), config, int(widths[expert]), world, rank)
                for expert in range(config.total_experts))
    layer = MoeLayer(card, config, widths, matrices, rank=rank, rank_count=world, pool_entries=total_steps,
                     cut=tuple(int(part) for part in args.cut.split(",")))
    if dist is None:
        layer.connect_local([layer])
    else:
        handles = [None] * world
        dist.all_gather_object(handles, card.ipc_export())
        layer.connect_handles(handles)
    card.wait()
    barrier()
    steps = step_inputs(config, args.rows, total_steps)
    aligning, steps = steps[-1], steps[:-1]

    # ---- value: inputs resident on the card ----
    order = steps[:args.warmup] + [aligning] + steps[args.warmup:]
    layer.load_pool([(index + 1, tokens, scores) for index, (tokens, scores) in enumerate(order)])
    barrier()
    for _ in range(args.warmup):
        layer.run_resident()
    card.wait()
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    # The ranks leave the barrier microseconds to milliseconds apart on the host. One untimed step queued first makes
    # them meet on the device (its reduction waits for every rank), so the timed region begins at the same moment on
    # every card and holds exactly the timed steps, not a rank's wait for a late one.
    layer.run_resident()
    launches_before = card.launch_count()
    card.measure_begin()
    for _ in range(args.steps):
        layer.run_resident()
    card.measure_end()
    device_ms = maximum(card.measure_elapsed_us() / 1000.0)
    card.wait()
    launches = card.launch_count() - launches_before
    barrier()
    layer.check_status()
    ms_per_step = device_ms / args.steps

    # ---- e2e: host buffers in, host buffer out, every step ----
    layer.sequence = total_steps
    result_at = api.align(layout.step_input_bytes, 4096)
    for tokens, scores in steps[:args.warmup]:
        layer.step(tokens, scores)
    barrier()
    card.measure_begin()
    wall_begin = time.perf_counter()
    for tokens, scores in steps[args.warmup:]:
        layer.step(tokens, scores)  # host arrays in, host array out: one library call a step
    wall_ms = 1000.0 * (time.perf_counter() - wall_begin)
    card.measure_end()
    e2e_ms = maximum(max(card.measure_elapsed_us() / 1000.0, wall_ms)) / args.steps
    clocks = sampler.stop() if sampler is not None else None
    layer.check_status()
    barrier()

    # ---- parity of this very build on these very cards: one checked step at every N ----
    parity = checked_step(config, widths, draw, layer, steps[args.warmup], rank, world, dist)
    barrier()

    # ---- roofline: the dominant kernel alone, launch by launch ----
    roofline = None
    if rank == 0:
        peak, peak_source = measured_peaks()
        gate_up = layer.launches[layer.gate_up_index:layer.gate_up_index + 1]
        prologue = layer.launches[0:layer.gate_up_index]
        elapsed_us, byte_total = 0.0, 0
        inner_local = layout.inner_local
        for index, (tokens, scores) in enumerate(steps[args.warmup:]):
            layer.sequence += 1
            layer.stage_step(0, layer.sequence, tokens, scores)
            card.transfer_wait(card.upload_async(layout.step, 0, layout.step_input_bytes))
            card.run(prologue)
            card.wait()
            card.measure_begin()
            card.run(gate_up)
            card.measure_end()
            elapsed_us += card.measure_elapsed_us()
            picks = card.download(layout.picks, args.rows * config.picks * 4, np.uint32)
            active = sorted(set(picks.tolist())) + list(range(config.experts, config.total_experts))
            pairs = args.rows * config.pairs_per_row
            matrices = 3 if getattr(layer, "products_in_one_launch", False) else 2  # gate, up (and down) in the launch
            byte_total += sum(matrices * synthetic.matrix_bytes(config.hidden, inner_local, int(widths[e]))
                              for e in active)
            byte_total += 2 * pairs * config.hidden * 2 + pairs * inner_local * 4  # operands in, hidden + operands out
            if matrices == 3:
                byte_total += pairs * inner_local * 2 + pairs * config.hidden * 4  # down operands in, pair outputs out
        achieved = byte_total / elapsed_us / 1000.0  # GB/s
        roofline = {"kernel": layer.gate_up_kernel, "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                    "frac": achieved / peak, "peak_source": peak_source,
                    "traffic": GATE_UP_TRAFFIC_RATIO * byte_total / args.steps,
                    "algorithmic_bytes_per_launch": byte_total / args.steps,
                    "us_per_launch": elapsed_us / args.steps}
    card.wait()
    barrier()

    # ---- the CPU oracle beside it (rank 0 at N = 1 only) ----
    cpu = None
    if rank == 0 and world == 1:
        cpu = cpu_baseline(config, widths, draw, steps[args.warmup:args.warmup + 4], args.rows)
    if rank == 0:
        line = {
            "metric": METRIC, "value": args.rows * 1000.0 / ms_per_step, "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16xf16->f32", "data": "synthetic",
            "config": workload_config(args, config, world),
            "e2e": {"value": args.rows * 1000.0 / e2e_ms, "unit": "tok/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": layout.step_input_bytes, "d2h_bytes_per_step": args.rows * config.hidden * 2},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline,
            "parity_checked": parity["ok"], "parity": parity,
        }
        line = dict(line)
        if cpu is not None:
            line["cpu_baseline"] = cpu
    card.close()
    prefill = None
    if args.prefill_rows > 0:
        prefill = run_prefill(args, api, config, widths, draw, rank, world, local_rank, dist, barrier, maximum)
    reference_kernels = None
    if rank == 0 and world == 1 and not args.no_reference_kernels:
        def draw_k3(expert):
            rng = np.random.default_rng([SEED, 3000 + expert])
            return (synthetic.exl3_matrix(rng, config.hidden, config.inner, 3),
                    synthetic.exl3_matrix(rng, config.hidden, config.inner, 3),
                    synthetic.exl3_matrix(rng, config.inner, config.hidden, 3))
        try:
            reference_kernels = run_reference_kernels(args, api, config, draw_k3, local_rank)
        except Exception as error:  # this leg is a comparison beside the numbers: it must not take the line with it
            reference_kernels = {"error": "%s: %s" % (type(error).__name__, error)}
    original = None
    if not args.no_original_weights:
        original = run_original_weights(args, api, config, rank, world, local_rank, dist, barrier, maximum)
    original_prefill = None
    if not args.no_original_weights and args.original_prefill_rows:
        try:
            original_prefill = run_original_weights_prefill(args, api, config, rank, world, local_rank, dist, barrier,
                                                            maximum)
        except Exception as error:  # a secondary object of the line: it must not take the line with it
            original_prefill = {"error": "%s: %s" % (type(error).__name__, error)}
    reduction = None
    if world > 1 and not args.no_reduction:
        reduction = run_reduction(args, api, config.hidden, rank, world, local_rank, dist, barrier, maximum)
    if rank == 0:
        if reduction is not None:
            line["reduction"] = reduction
        if prefill is not None:
            line["prefill"] = prefill
        if original is not None:
            line["original_weights"] = original
        if original_prefill is not None:
            line["original_weights_prefill"] = original_prefill
        if reference_kernels is not None:
            line["reference_kernels"] = reference_kernels
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()
    if rank == 0 and not line["parity_checked"]:
        raise SystemExit("bench.py: the checked step differs from the CPU oracle: " + json.dumps(line["parity"]))


if __name__ == "__main__":
    main()
