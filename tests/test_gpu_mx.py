"""The original-weights routed experts (MXFP4 weights by E4M3 block-quantized activations) on a CUDA device through the
C-ABI library, against the CPU oracle (itself pinned to the reference's test references). Mirrors the reference's
expert card tests (tests/linear_expert_card_test.c): quantization bit for bit, products within the tolerance of a
bfloat16 result, row sums bit for bit given the pair outputs."""
import ctypes as C

import numpy as np
import pytest

from anemone_b200 import records as R
from anemone_b200 import synthetic
from oracle.binding import f32p, ptr, u16p, u32p, u64p, u8p

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    from anemone_b200 import api as module
    assert module.card_count() >= 1, "no CUDA device: the CUDA path cannot run and there is no fallback"
    return module


def mx_matrix(oracle, rng, outputs, inputs, scale_codes=(119, 124)):
    """Stored MXFP4 matrix of the original-weights profile: uniform E2M1 nibbles, E8M0 codes 127 + e, e in [-8, -4]
    (or from the given half-open range)."""
    codes = rng.integers(0, 16, size=outputs * inputs, dtype=np.uint8)
    scales = rng.integers(scale_codes[0], scale_codes[1], size=outputs * inputs // 32).astype(np.uint8)
    stored = np.zeros(outputs * inputs // 2 + outputs * inputs // 32, dtype=np.uint8)
    oracle.orc_mx_weights_lay_out(ptr(codes, u8p), ptr(scales, u8p), outputs, inputs, ptr(stored, u8p))
    return stored


def prepare_kernels(api, card):
    lib = api.library()
    kernels = R.LinearKernels()
    lib.linear_kernels_prepare.argtypes = [C.POINTER(api.BackendOperations), C.c_void_p, C.c_uint32,
                                           C.POINTER(R.LinearKernels)]
    api.check(lib.linear_kernels_prepare(card.ops_pointer, card.handle, 100, C.byref(kernels)), "linear_kernels_prepare")
    return kernels


def test_activation_quantize_is_bit_exact(api, oracle):
    rng = np.random.default_rng(31)
    width, rows = 512, 6
    values = synthetic.to_bfloat16((rng.normal(0, 1, (rows, width)) * np.array([1, 1e-3, 300, 1e-6, 1, 30])[:, None])
                                   .astype(np.float32))
    values[4, :40] = 0
    values[4, 5] = 0x8000
    values[4, 64:96] = synthetic.to_bfloat16(np.full(32, 0.4375, dtype=np.float32))
    layout = api.Layout()
    at = {name: layout.take(size) for name, size in (("values", rows * width * 2), ("codes", rows * width),
                                                     ("exponents", rows * width // 32), ("operands", rows * width * 2))}
    card = api.Card(0, layout.take(4096, 4096))
    try:
        kernels = prepare_kernels(api, card)
        card.upload(at["values"], values)
        description = R.LinearQuantizeDescription(
            R.LinearRange(at["values"], rows * width * 2), R.LinearRange(at["codes"], rows * width),
            R.LinearRange(at["exponents"], rows * width // 32), R.LinearRange(at["operands"], rows * width * 2), width, rows)
        launch = R.KernelLaunch()
        lib = api.library()
        lib.linear_quantize_prepare.argtypes = [C.POINTER(R.LinearQuantizeDescription), C.c_uint64,
                                                C.POINTER(R.LinearKernels), C.POINTER(R.KernelLaunch)]
        api.check(lib.linear_quantize_prepare(C.byref(description), card.arena_bytes, C.byref(kernels), C.byref(launch)),
                  "linear_quantize_prepare")
        card.run([launch])
        card.wait()
        codes = card.download(at["codes"], rows * width).reshape(rows, width)
        exponents = card.download(at["exponents"], rows * width // 32).reshape(rows, width // 32)
        operands = card.download(at["operands"], rows * width * 2, np.uint16).reshape(rows, width)
    finally:
        card.close()
    for row in range(rows):
        natural, want_exponents = np.zeros(width, np.uint8), np.zeros(width // 32, np.uint8)
        line = np.ascontiguousarray(values[row])
        oracle.orc_mx_quantize(ptr(line, u16p), width, ptr(natural, u8p), ptr(want_exponents, u8p))
        want_codes, want_operands = np.zeros(width, np.uint8), np.zeros(width, np.uint16)
        oracle.orc_mx_codes_lay_out(ptr(natural, u8p), width, ptr(want_codes, u8p))
        oracle.orc_mx_operands_lay_out(ptr(natural, u8p), width, ptr(want_operands, u16p))
        assert np.array_equal(exponents[row], want_exponents), row
        assert np.array_equal(codes[row], want_codes), row
        assert np.array_equal(operands[row], want_operands), row


@pytest.mark.parametrize("slices,edge", [((1, 1), False), ((4, 4), False), ((8, 2), False), ((16, 8), False),
                                         ((2, 2), True)])
def test_routed_experts_match_oracle(api, oracle, slices, edge):
    """edge: the block scales' codes straddle the window inside which the kernels form a scale as a product of two
    powers of two (53 .. 179) and outside which they clamp the sum: weights' codes 50 .. 56, the rows' blocks scaled so
    that their codes are about 176 .. 182, so that lanes of one warp go both ways and the scales stay near one."""
    rng = np.random.default_rng(32 + slices[0])
    H, I, experts, rows, picks = 1024, 512, 6, 11, 2
    pairs = rows * picks
    layout = api.Layout()
    table = np.zeros((experts, 3), dtype=np.uint64)
    matrices = []
    for expert in range(experts):
        for which, (outputs, inputs) in enumerate(((I, H), (I, H), (H, I))):
            data = mx_matrix(oracle, rng, outputs, inputs, (50, 57) if edge and which < 2 else (119, 124))
            table[expert, which] = layout.take(data.size, 64)
            matrices.append((int(table[expert, which]), data))
    weights_end = layout.cursor
    chosen = np.stack([np.sort(rng.choice(experts, size=picks, replace=False)) for _ in range(rows)]).astype(np.uint32)
    route = rng.uniform(0.3, 1.0, size=(rows, picks)).astype(np.float32)
    job_capacity = rows * picks + 1
    jobs = (R.ExpertJob * job_capacity)()
    oracle.orc_router_jobs(ptr(chosen, u32p), ptr(route, f32p), rows, picks, experts, 0, ptr(table, u64p),
                           job_capacity, C.byref(jobs))
    sizes = {"jobs": job_capacity * 96, "values": rows * H * 2, "codes": rows * H, "exponents": rows * H // 32,
             "operands": rows * H * 2, "hidden": pairs * I * 2, "hidden_codes": pairs * I,
             "hidden_exponents": pairs * I // 32, "hidden_operands": pairs * I * 2, "pair_output": pairs * H * 2,
             "row_output": rows * H * 4}
    at = {name: layout.take(size) for name, size in sizes.items()}
    arena_bytes = layout.take(4096, 4096)
    image = np.zeros(arena_bytes, dtype=np.uint8)
    for offset, data in matrices:
        image[offset:offset + data.size] = data
    image[at["jobs"]:at["jobs"] + sizes["jobs"]] = np.frombuffer(bytes(jobs), dtype=np.uint8)
    tokens = synthetic.tokens(rng, rows, H)
    if edge:
        blocks = synthetic.from_bfloat16(tokens).reshape(rows, H // 32, 32)
        blocks = blocks * np.exp2(rng.integers(56, 63, size=(rows, H // 32, 1))).astype(np.float32)
        tokens = synthetic.to_bfloat16(blocks.reshape(rows, H).astype(np.float32))
    image[at["values"]:at["values"] + sizes["values"]] = tokens.view(np.uint8).reshape(-1)
    description = R.LinearRoutedExpertsDescription()
    description.jobs = R.LinearRange(at["jobs"], sizes["jobs"])
    description.expert_weights = R.LinearRange(0, weights_end)
    for name in ("codes", "exponents", "operands", "hidden", "hidden_codes", "hidden_exponents", "hidden_operands",
                 "pair_output", "row_output"):
        setattr(description, name, R.LinearRange(at[name], sizes[name]))
    description.gate_up_shape, description.down_shape = R.MatrixShape(I, H, 4, 0), R.MatrixShape(H, I, 4, 0)
    description.weight_format, description.job_count, description.row_count = 3, job_capacity, rows
    description.pairs_per_row, description.activation_limit = picks, 7.0
    description.gate_up_slice_count, description.down_slice_count = slices
    lib = api.library()
    lib.linear_quantize_prepare.argtypes = [C.POINTER(R.LinearQuantizeDescription), C.c_uint64,
                                            C.POINTER(R.LinearKernels), C.POINTER(R.KernelLaunch)]
    lib.linear_routed_experts_prepare.argtypes = [C.POINTER(R.LinearRoutedExpertsDescription), C.c_uint64,
                                                  C.POINTER(R.LinearKernels), C.POINTER(R.KernelLaunch)]
    card = api.Card(0, arena_bytes)
    try:
        kernels = prepare_kernels(api, card)
        card.upload(0, image)
        quantize = R.LinearQuantizeDescription(R.LinearRange(at["values"], sizes["values"]), description.codes,
                                               description.exponents, description.operands, H, rows)
        first = R.KernelLaunch()
        api.check(lib.linear_quantize_prepare(C.byref(quantize), arena_bytes, C.byref(kernels), C.byref(first)), "quantize")
        launches = (R.KernelLaunch * 4)()
        api.check(lib.linear_routed_experts_prepare(C.byref(description), arena_bytes, C.byref(kernels), launches),
                  "linear_routed_experts_prepare")
        card.run([first] + list(launches))
        card.wait()
        received = card.download(0, arena_bytes)
    finally:
        card.close()
    if edge:
        seen = received[at["exponents"]:at["exponents"] + sizes["exponents"]]
        assert (seen > 179).any() and (seen <= 179).any() and seen.min() >= 170
    # the oracle on the same image, from the card's own (bit-exact, checked above) quantized rows
    expected = image.copy()
    for name in ("codes", "exponents", "operands"):
        expected[at[name]:at[name] + sizes[name]] = received[at[name]:at[name] + sizes[name]]
    gate_up = R.ExpertGateUp(at["jobs"], at["codes"], at["exponents"], at["operands"], at["hidden"], I, H, pairs, picks,
                             7.0, 0)
    down = R.ExpertDown(at["jobs"], at["hidden_codes"], at["hidden_exponents"], at["hidden_operands"], at["pair_output"],
                        H, I, pairs, 0)
    oracle.orc_mx_experts(C.byref(gate_up), C.byref(down), job_capacity, slices[0], slices[1], at["hidden_codes"],
                          at["hidden_exponents"], at["hidden_operands"], ptr(expected, u8p))
    row_sum = R.ExpertRowSum(at["pair_output"], at["row_output"], H, picks)
    oracle.orc_mx_row_sum(C.byref(row_sum), rows, ptr(expected, u8p))

    def ordinals(bits):
        bits = bits.astype(np.int32)
        return np.where(bits & 0x8000, -(bits & 0x7FFF), bits & 0x7FFF)

    def region(data, name, dtype):
        return data[at[name]:at[name] + sizes[name]].view(dtype)
    hidden_got, hidden_want = region(received, "hidden", np.uint16), region(expected, "hidden", np.uint16)
    distance = np.abs(ordinals(hidden_got) - ordinals(hidden_want))
    assert distance.max() <= 2 and (distance == 0).mean() > 0.98  # the tensor cores' sum of a block may round otherwise
    out_got = synthetic.from_bfloat16(region(received, "pair_output", np.uint16))
    out_want = synthetic.from_bfloat16(region(expected, "pair_output", np.uint16))
    assert np.isfinite(out_got).all() and np.abs(out_want).max() > 0
    assert np.abs(out_got - out_want).max() <= max(2e-2, 2.0 ** -6 * np.abs(out_want).max())
    cosine = float(out_got.astype(np.float64) @ out_want.astype(np.float64) /
                   (np.linalg.norm(out_got) * np.linalg.norm(out_want)))
    assert cosine >= 0.9999
    # the row sum is bit-exact given the pair outputs the card wrote
    pair_values = out_got.reshape(rows, picks, H)
    resummed = np.zeros((rows, H), dtype=np.float32)
    for slot in range(picks):
        resummed = (resummed + pair_values[:, slot, :]).astype(np.float32)
    assert np.array_equal(resummed.view(np.uint32), region(received, "row_output", np.uint32).reshape(rows, H))
    # weights and inputs untouched
    assert np.array_equal(received[:weights_end], image[:weights_end])


@pytest.mark.parametrize("shared", [0, 1])
def test_layer_matches_oracle(api, oracle, shared):
    """The whole original-weights layer (router -> quantize -> experts -> row sum -> ordered reduction) through
    anemone_b200.mx.MxLayer: the card's own job table and quantized rows, then the oracle's experts on the same image."""
    from anemone_b200.moe import MoeConfig
    from anemone_b200.mx import MxLayer, MxLayout
    from oracle import moe_reference
    config = MoeConfig(hidden=512, inner=256, experts=12, shared=shared, picks=3, row_capacity=8, activation_limit=7.0)
    rng = np.random.default_rng(91)
    H, I, rows = config.hidden, config.inner, 7
    matrices = [(mx_matrix(oracle, rng, I, H), mx_matrix(oracle, rng, I, H), mx_matrix(oracle, rng, H, I))
                for _ in range(config.experts)]
    tokens = synthetic.tokens(rng, rows, H)
    scores = rng.normal(0, 1, size=(rows, config.experts)).astype(np.float32)
    L = MxLayout(config, 1, 0)
    card = api.Card(0, L.arena_bytes)
    try:
        always = (synthetic.e4m3_matrix(rng, I, H), synthetic.e4m3_matrix(rng, I, H),
                  synthetic.e4m3_matrix(rng, H, I)) if shared else None
        layer = MxLayer(card, config, matrices, slices=(2, 2), shared_matrices=always)
        layer.connect_local([layer])
        result = layer.step(tokens, scores)
        received = card.download(0, L.arena_bytes)
    finally:
        card.close()
    experts, weights = moe_reference.route(oracle, config, scores)
    picks = received[L.picks:L.picks + rows * config.picks * 4].view(np.uint32).reshape(rows, config.picks)
    assert np.array_equal(picks, experts)
    expected = received.copy()
    at, pairs = L.at, L.pairs
    gate_up = R.ExpertGateUp(L.jobs, at["codes"], at["exponents"], at["operands"], at["hidden"], I, H, pairs,
                             config.picks, 7.0, 0)
    down = R.ExpertDown(L.jobs, at["hidden_codes"], at["hidden_exponents"], at["hidden_operands"], at["pair_output"],
                        H, I, pairs, 0)
    oracle.orc_mx_experts(C.byref(gate_up), C.byref(down), L.job_capacity, 2, 2, at["hidden_codes"],
                          at["hidden_exponents"], at["hidden_operands"], ptr(expected, u8p))
    live = rows * config.picks
    out_got = synthetic.from_bfloat16(received[at["pair_output"]:at["pair_output"] + live * H * 2].view(np.uint16))
    out_want = synthetic.from_bfloat16(expected[at["pair_output"]:at["pair_output"] + live * H * 2].view(np.uint16))
    assert np.isfinite(out_got).all() and np.abs(out_want).max() > 0
    assert np.abs(out_got - out_want).max() <= max(2e-2, 2.0 ** -6 * np.abs(out_want).max())
    # row sums and the reduction are bit-exact given the pair outputs the card wrote
    resummed = np.zeros((rows, H), dtype=np.float32)
    for slot in range(config.picks):
        resummed = (resummed + out_got.reshape(rows, config.picks, H)[:, slot, :]).astype(np.float32)
    row_output = received[at["row_output"]:at["row_output"] + rows * H * 4].view(np.float32).reshape(rows, H)
    if shared:
        # the always-on expert's rows (checked against the oracle in test_shared_expert_matches_oracle) joined by one
        # FP32 addition each
        where = L.shared_at["output"]
        joined = synthetic.from_bfloat16(received[where:where + rows * H * 2].view(np.uint16)).reshape(rows, H)
        assert np.abs(joined).max() > 0
        resummed = (resummed + joined).astype(np.float32)
    assert np.array_equal(resummed.view(np.uint32), row_output.view(np.uint32))
    assert np.array_equal(result, synthetic.to_bfloat16(np.float32(0.0) + row_output))


@pytest.mark.parametrize("block128", [False, True])
@pytest.mark.parametrize("rows,slices", [(1, (1, 1)), (5, (2, 4)), (8, (8, 2))])
def test_shared_expert_matches_oracle(api, oracle, rows, slices, block128):
    """linear_shared_expert_prepare's four launches (E4M3 matrices, one scale per 32 by 32 weights) and
    linear_shared_expert_block128_prepare's (one FP32 scale per 128 by 128 weights) against the oracle on the same
    image, from the card's own quantized rows: gate, up and down within the tolerance of a bfloat16 result, the
    hidden rows' quantization bit for bit given the hidden rows."""
    rng = np.random.default_rng(60 + rows)
    # 320 = 10 blocks of 32, 5 loads of 64, a last scale block of 16 outputs; the FP32-scaled format wants whole
    # blocks of 128 inputs: 384 outputs = three blocks, 512 = four
    H, I = (512, 384) if block128 else (512, 320)
    layout = api.Layout()
    draw = synthetic.e4m3_block128_matrix if block128 else synthetic.e4m3_matrix
    stored = {name: draw(rng, o, i) for name, (o, i) in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I)))}
    where = {name: layout.take(data.size, 64) for name, data in stored.items()}
    sizes = {"values": rows * H * 2, "codes": rows * H, "exponents": rows * H // 32, "operands": rows * H * 2,
             "gate_output": rows * I * 2, "up_output": rows * I * 2, "hidden": rows * I * 2, "hidden_codes": rows * I,
             "hidden_exponents": rows * I // 32, "hidden_operands": rows * I * 2, "output": rows * H * 2}
    at = {name: layout.take(size + 64) for name, size in sizes.items()}
    arena_bytes = layout.take(4096, 4096)
    image = np.full(arena_bytes, 0xC3, dtype=np.uint8)
    for name, data in stored.items():
        image[where[name]:where[name] + data.size] = data
    tokens = synthetic.tokens(rng, rows, H)
    image[at["values"]:at["values"] + sizes["values"]] = tokens.view(np.uint8).reshape(-1)
    lib = api.library()
    description = R.LinearSharedExpertDescription()
    for name, (o, i), count in (("gate", (I, H), slices[0]), ("up", (I, H), slices[0]), ("down", (H, I), slices[1])):
        setattr(description, name, R.LinearMatrix(R.LinearRange(where[name], stored[name].size), R.MatrixShape(o, i, 8, 0),
                                                  6 if block128 else 5, count, 0, 0))
    for name in ("codes", "exponents", "operands", "gate_output", "up_output", "hidden", "hidden_codes",
                 "hidden_exponents", "hidden_operands", "output"):
        setattr(description, name, R.LinearRange(at[name], sizes[name]))
    description.row_count, description.activation_limit = rows, 7.0
    lib.linear_quantize_prepare.argtypes = [C.POINTER(R.LinearQuantizeDescription), C.c_uint64,
                                            C.POINTER(R.LinearKernels), C.POINTER(R.KernelLaunch)]
    lib.linear_shared_expert_prepare.argtypes = [C.POINTER(R.LinearSharedExpertDescription), C.c_uint64,
                                                 C.POINTER(R.LinearKernels), C.POINTER(R.KernelLaunch)]
    lib.linear_shared_expert_block128_prepare.argtypes = [C.POINTER(R.LinearSharedExpertDescription), C.c_uint64,
                                                          C.POINTER(R.LinearKernels),
                                                          C.POINTER(api.BackendOperations), C.c_void_p,
                                                          C.POINTER(R.KernelLaunch)]
    card = api.Card(0, arena_bytes)

    def prepare(description, launches):
        if block128:
            return lib.linear_shared_expert_block128_prepare(C.byref(description), arena_bytes, C.byref(kernels),
                                                             card.ops_pointer, card.handle, launches)
        return lib.linear_shared_expert_prepare(C.byref(description), arena_bytes, C.byref(kernels), launches)
    try:
        kernels = prepare_kernels(api, card)
        card.upload(0, image)
        quantize = R.LinearQuantizeDescription(R.LinearRange(at["values"], sizes["values"]), description.codes,
                                               description.exponents, description.operands, H, rows)
        first = R.KernelLaunch()
        api.check(lib.linear_quantize_prepare(C.byref(quantize), arena_bytes, C.byref(kernels), C.byref(first)), "quantize")
        launches = (R.KernelLaunch * 4)()
        api.check(prepare(description, launches), "linear_shared_expert_prepare")
        if block128:  # a matrix of the other format is refused by either preparer
            assert lib.linear_shared_expert_prepare(C.byref(description), arena_bytes, C.byref(kernels),
                                                    (R.KernelLaunch * 4)()) == 1
        assert launches[0].grid[0] == 2 * I // 16 and launches[0].block[0] == 32 * slices[0]
        assert launches[3].grid[0] == H // 16 and launches[3].block[0] == 32 * slices[1]
        before = bytes(launches)
        description.row_count = 9  # more rows than a thin launch takes
        assert prepare(description, launches) == 1
        assert bytes(launches) == before
        card.run([first] + list(launches))
        card.wait()
        received = card.download(0, arena_bytes)
    finally:
        card.close()
    expected = image.copy()
    for name in ("codes", "exponents", "operands"):
        expected[at[name]:at[name] + sizes[name]] = received[at[name]:at[name] + sizes[name]]
    gate_up = R.TrunkLinearQuantized((C.c_uint64 * 2)(where["gate"], where["up"]),
                                     (C.c_uint64 * 2)(at["gate_output"], at["up_output"]), at["codes"],
                                     at["exponents"], at["operands"], (C.c_uint32 * 2)(I, I), H, rows)
    hidden = R.TrunkHidden(at["gate_output"], at["up_output"], at["hidden"], I, 7.0)
    requantize = R.ActivationQuantize(at["hidden"], at["hidden_codes"], at["hidden_exponents"], at["hidden_operands"], I, 0)
    down = R.TrunkLinearQuantized((C.c_uint64 * 2)(where["down"], 0), (C.c_uint64 * 2)(at["output"], 0),
                                  at["hidden_codes"], at["hidden_exponents"], at["hidden_operands"],
                                  (C.c_uint32 * 2)(H, 0), I, rows)
    (oracle.orc_shared_expert_block128 if block128 else oracle.orc_shared_expert)(
        C.byref(gate_up), C.byref(hidden), C.byref(requantize), C.byref(down), slices[0], slices[1], ptr(expected, u8p))

    def ordinals(bits):
        bits = bits.astype(np.int32)
        return np.where(bits & 0x8000, -(bits & 0x7FFF), bits & 0x7FFF)

    def region(data, name):
        return data[at[name]:at[name] + sizes[name]].view(np.uint16)
    for name in ("gate_output", "up_output"):
        distance = np.abs(ordinals(region(received, name)) - ordinals(region(expected, name)))
        assert distance.max() <= 2 and (distance == 0).mean() > 0.98, name
    out_got = synthetic.from_bfloat16(region(received, "output"))
    out_want = synthetic.from_bfloat16(region(expected, "output"))
    assert np.isfinite(out_got).all() and np.abs(out_want).max() > 0
    assert np.abs(out_got - out_want).max() <= max(2e-2, 2.0 ** -6 * np.abs(out_want).max())
    cosine = float(out_got.astype(np.float64) @ out_want.astype(np.float64) /
                   (np.linalg.norm(out_got) * np.linalg.norm(out_want)))
    assert cosine >= 0.9999
    # the hidden rows' quantization: the card's own kernel on the card's own hidden rows, against the oracle's quantizer
    hidden_rows = region(received, "hidden").reshape(rows, I)
    for row in range(rows):
        natural, exponents = np.zeros(I, np.uint8), np.zeros(I // 32, np.uint8)
        line = np.ascontiguousarray(hidden_rows[row])
        oracle.orc_mx_quantize(ptr(line, u16p), I, ptr(natural, u8p), ptr(exponents, u8p))
        lane_order = np.zeros(I, np.uint8)
        oracle.orc_mx_codes_lay_out(ptr(natural, u8p), I, ptr(lane_order, u8p))
        got = received[at["hidden_codes"] + row * I:at["hidden_codes"] + (row + 1) * I]
        assert np.array_equal(got, lane_order), row
    for name, size in sizes.items():  # nothing written behind a range, weights untouched
        assert (received[at[name] + size:at[name] + size + 64] == 0xC3).all(), name
    for name, data in stored.items():
        assert np.array_equal(received[where[name]:where[name] + data.size], data)


@pytest.mark.parametrize("block128", [False, True])
def test_wide_layer_matches_oracle(api, oracle, block128):
    """The original-weights layer for MANY rows (MxLayer(wide=True): the prefill's picks and grouping, a job table of
    eight rows a job, the thin expert launches, the always-on expert a block column per eight rows, owner-run
    reduction): the job table against the oracle's picks grouped by the same rule, bit for bit; then the oracle's
    experts and always-on expert on the card's own quantized rows."""
    from anemone_b200.moe import MoeConfig
    from anemone_b200.mx import MxLayer, MxLayout
    from oracle import moe_reference
    rows = 203
    config = MoeConfig(hidden=512, inner=384 if block128 else 256, experts=12, shared=1, picks=3, row_capacity=256,
                       activation_limit=7.0)
    rng = np.random.default_rng(123)
    H, I = config.hidden, config.inner
    matrices = [(mx_matrix(oracle, rng, I, H), mx_matrix(oracle, rng, I, H), mx_matrix(oracle, rng, H, I))
                for _ in range(config.experts)]
    draw = synthetic.e4m3_block128_matrix if block128 else synthetic.e4m3_matrix
    always = (draw(rng, I, H), draw(rng, I, H), draw(rng, H, I))
    tokens = synthetic.tokens(rng, rows, H)
    scores = rng.normal(0, 1, size=(rows, config.experts)).astype(np.float32)
    scores[:, 1] += 1.0  # one expert with many jobs
    L = MxLayout(config, 1, 0, block128=block128, wide=True)
    card = api.Card(0, L.arena_bytes)
    try:
        layer = MxLayer(card, config, matrices, slices=(2, 2), shared_matrices=always, block128=block128, wide=True)
        layer.connect_local([layer])
        for _ in range(2):  # both parity slots
            result = layer.step(tokens, scores)
        received = card.download(0, L.arena_bytes)
    finally:
        card.close()
    experts, weights = moe_reference.route(oracle, config, scores)
    picks = received[L.picks:L.picks + rows * config.picks * 4].view(np.uint32).reshape(rows, config.picks)
    assert np.array_equal(picks, experts)
    # the job table: expert e's rows ascending, eight to a job, experts ascending; everything else zero
    table = np.frombuffer(received[L.expert_table:L.expert_table + config.experts * 24].tobytes(), dtype=np.uint64)
    want = (R.ExpertJob * L.job_capacity)()
    job = 0
    for expert in range(config.experts):
        held = [(row, slot) for row in range(rows) for slot in range(config.picks) if experts[row, slot] == expert]
        for first in range(0, len(held), 8):
            record = want[job]
            record.gate_offset, record.up_offset, record.down_offset = (int(x) for x in table[3 * expert:3 * expert + 3])
            record.expert, record.row_count = expert, min(8, len(held) - first)
            for column, (row, slot) in enumerate(held[first:first + 8]):
                record.pair_index[column] = row * config.picks + slot
                record.route_weight[column] = float(weights[row, slot])
            job += 1
    assert job > config.experts and bytes(received[L.jobs:L.jobs + L.job_capacity * 96]) == bytes(want)
    # the routed experts: the oracle on the card's own job table and quantized rows
    expected = received.copy()
    at, pairs = L.at, L.pairs
    gate_up = R.ExpertGateUp(L.jobs, at["codes"], at["exponents"], at["operands"], at["hidden"], I, H, pairs,
                             config.picks, 7.0, 0)
    down = R.ExpertDown(L.jobs, at["hidden_codes"], at["hidden_exponents"], at["hidden_operands"], at["pair_output"],
                        H, I, pairs, 0)
    oracle.orc_mx_experts(C.byref(gate_up), C.byref(down), L.job_capacity, 2, 2, at["hidden_codes"],
                          at["hidden_exponents"], at["hidden_operands"], ptr(expected, u8p))
    live = rows * config.picks
    out_got = synthetic.from_bfloat16(received[at["pair_output"]:at["pair_output"] + live * H * 2].view(np.uint16))
    out_want = synthetic.from_bfloat16(expected[at["pair_output"]:at["pair_output"] + live * H * 2].view(np.uint16))
    assert np.isfinite(out_got).all() and np.abs(out_want).max() > 0
    assert np.abs(out_got - out_want).max() <= max(2e-2, 2.0 ** -6 * np.abs(out_want).max())
    # the always-on expert on all rows: the oracle on the same quantized rows
    S = L.shared_at
    trunk_gate_up = R.TrunkLinearQuantized((C.c_uint64 * 2)(L.shared_matrices[0], L.shared_matrices[1]),
                                           (C.c_uint64 * 2)(S["gate_output"], S["up_output"]), at["codes"],
                                           at["exponents"], at["operands"], (C.c_uint32 * 2)(I, I), H, rows)
    hidden = R.TrunkHidden(S["gate_output"], S["up_output"], S["hidden"], I, 7.0)
    requantize = R.ActivationQuantize(S["hidden"], S["hidden_codes"], S["hidden_exponents"], S["hidden_operands"], I, 0)
    trunk_down = R.TrunkLinearQuantized((C.c_uint64 * 2)(L.shared_matrices[2], 0), (C.c_uint64 * 2)(S["output"], 0),
                                        S["hidden_codes"], S["hidden_exponents"], S["hidden_operands"],
                                        (C.c_uint32 * 2)(H, 0), I, rows)
    (oracle.orc_shared_expert_block128 if block128 else oracle.orc_shared_expert)(
        C.byref(trunk_gate_up), C.byref(hidden), C.byref(requantize), C.byref(trunk_down), 2, 2, ptr(expected, u8p))
    joined = synthetic.from_bfloat16(received[S["output"]:S["output"] + rows * H * 2].view(np.uint16)).reshape(rows, H)
    joined_want = synthetic.from_bfloat16(expected[S["output"]:S["output"] + rows * H * 2].view(np.uint16)).reshape(rows, H)
    assert np.abs(joined_want).max() > 0
    assert np.abs(joined - joined_want).max() <= max(2e-2, 2.0 ** -6 * np.abs(joined_want).max())
    # row sums, the join and the reduction are bit-exact given what the card wrote
    resummed = np.zeros((rows, H), dtype=np.float32)
    for slot in range(config.picks):
        resummed = (resummed + out_got.reshape(rows, config.picks, H)[:, slot, :]).astype(np.float32)
    resummed = (resummed + joined).astype(np.float32)
    row_output = received[at["row_output"]:at["row_output"] + rows * H * 4].view(np.float32).reshape(rows, H)
    assert np.array_equal(resummed.view(np.uint32), row_output.view(np.uint32))
    assert np.array_equal(result, synthetic.to_bfloat16(np.float32(0.0) + row_output))


def test_layer_at_the_configured_shapes(api, oracle):
    """The original-weights layer at the configured shapes (256 MXFP4 routed experts, top-8, hidden 4096, intermediate
    2048, the always-on expert E4M3 with 128 x 128 FP32 scales, 8 rows) against the oracle: the card's own picks, job
    table and quantized rows, then the oracle's experts on an image that holds the matrices of the experts a job
    names (the others are never read)."""
    from anemone_b200.moe import MoeConfig
    from anemone_b200.mx import MxLayer, MxLayout
    from oracle import moe_reference
    config = MoeConfig(hidden=4096, inner=2048, experts=256, shared=1, picks=8, row_capacity=8, activation_limit=7.0)
    rng = np.random.default_rng(555)
    H, I, rows = config.hidden, config.inner, 8
    tokens = synthetic.tokens(rng, rows, H)
    scores = rng.normal(0, 1, size=(rows, config.experts)).astype(np.float32)
    experts, weights = moe_reference.route(oracle, config, scores)
    active = set(experts.reshape(-1).tolist())
    filler = (synthetic.mx_matrix(rng, I, H), synthetic.mx_matrix(rng, I, H), synthetic.mx_matrix(rng, H, I))
    matrices = [(synthetic.mx_matrix(rng, I, H), synthetic.mx_matrix(rng, I, H), synthetic.mx_matrix(rng, H, I))
                if expert in active else filler for expert in range(config.experts)]
    always = (synthetic.e4m3_block128_matrix(rng, I, H), synthetic.e4m3_block128_matrix(rng, I, H),
              synthetic.e4m3_block128_matrix(rng, H, I))
    L = MxLayout(config, 1, 0, block128=True)
    card = api.Card(0, L.arena_bytes)
    at, S = L.at, L.shared_at
    try:
        layer = MxLayer(card, config, matrices, slices=(4, 4), shared_matrices=always, block128=True)
        layer.connect_local([layer])
        result = layer.step(tokens, scores)
        expected = np.zeros(L.arena_bytes, dtype=np.uint8)  # pages are taken as they are written
        for offset, size in [(L.picks, rows * config.picks * 4), (L.jobs, L.job_capacity * 96)] + \
                [(at[name], L.sizes[name]) for name in L.sizes] + [(S[name], L.shared_sizes[name]) for name in S]:
            expected[offset:offset + size] = card.download(offset, size)
        received = {name: expected[at[name]:at[name] + L.sizes[name]].copy() for name in ("pair_output", "row_output")}
        joined_bits = expected[S["output"]:S["output"] + rows * H * 2].copy()
    finally:
        card.close()
    picks = expected[L.picks:L.picks + rows * config.picks * 4].view(np.uint32).reshape(rows, config.picks)
    assert np.array_equal(picks, experts)
    for expert in active:
        for which in range(3):
            data = matrices[expert][which]
            expected[L.matrices[expert][which]:L.matrices[expert][which] + data.size] = data
    for which in range(3):
        expected[L.shared_matrices[which]:L.shared_matrices[which] + always[which].size] = always[which]
    pairs = L.pairs
    gate_up = R.ExpertGateUp(L.jobs, at["codes"], at["exponents"], at["operands"], at["hidden"], I, H, pairs,
                             config.picks, 7.0, 0)
    down = R.ExpertDown(L.jobs, at["hidden_codes"], at["hidden_exponents"], at["hidden_operands"], at["pair_output"],
                        H, I, pairs, 0)
    oracle.orc_mx_experts(C.byref(gate_up), C.byref(down), L.job_capacity, 4, 4, at["hidden_codes"],
                          at["hidden_exponents"], at["hidden_operands"], ptr(expected, u8p))
    out_got = synthetic.from_bfloat16(received["pair_output"].view(np.uint16))
    out_want = synthetic.from_bfloat16(expected[at["pair_output"]:at["pair_output"] + pairs * H * 2].view(np.uint16))
    assert np.isfinite(out_got).all() and np.abs(out_want).max() > 0
    assert np.abs(out_got - out_want).max() <= max(2e-2, 2.0 ** -6 * np.abs(out_want).max())
    cosine = float(out_got.astype(np.float64) @ out_want.astype(np.float64) /
                   (np.linalg.norm(out_got) * np.linalg.norm(out_want)))
    assert cosine >= 0.9999
    # the always-on expert
    trunk_gate_up = R.TrunkLinearQuantized((C.c_uint64 * 2)(L.shared_matrices[0], L.shared_matrices[1]),
                                           (C.c_uint64 * 2)(S["gate_output"], S["up_output"]), at["codes"],
                                           at["exponents"], at["operands"], (C.c_uint32 * 2)(I, I), H, rows)
    hidden = R.TrunkHidden(S["gate_output"], S["up_output"], S["hidden"], I, 7.0)
    requantize = R.ActivationQuantize(S["hidden"], S["hidden_codes"], S["hidden_exponents"], S["hidden_operands"], I, 0)
    trunk_down = R.TrunkLinearQuantized((C.c_uint64 * 2)(L.shared_matrices[2], 0), (C.c_uint64 * 2)(S["output"], 0),
                                        S["hidden_codes"], S["hidden_exponents"], S["hidden_operands"],
                                        (C.c_uint32 * 2)(H, 0), I, rows)
    oracle.orc_shared_expert_block128(C.byref(trunk_gate_up), C.byref(hidden), C.byref(requantize),
                                      C.byref(trunk_down), 2, 2, ptr(expected, u8p))
    joined = synthetic.from_bfloat16(joined_bits.view(np.uint16)).reshape(rows, H)
    joined_want = synthetic.from_bfloat16(expected[S["output"]:S["output"] + rows * H * 2].view(np.uint16)).reshape(rows, H)
    assert np.abs(joined - joined_want).max() <= max(2e-2, 2.0 ** -6 * np.abs(joined_want).max())
    # row sums, the join and the reduction: bit for bit given what the card wrote
    resummed = np.zeros((rows, H), dtype=np.float32)
    for slot in range(config.picks):
        resummed = (resummed + out_got.reshape(rows, config.picks, H)[:, slot, :]).astype(np.float32)
    resummed = (resummed + joined).astype(np.float32)
    row_output = received["row_output"].view(np.float32).reshape(rows, H)
    assert np.array_equal(resummed.view(np.uint32), row_output.view(np.uint32))
    assert np.array_equal(result, synthetic.to_bfloat16(np.float32(0.0) + row_output))


@pytest.mark.parametrize("slices", [(1, 1), (2, 2), (4, 4)])
def test_many_row_products_equal_the_thin_instances(api, oracle, slices):
    """linear_routed_experts_wide_prepare (a group of jobs and several tiles a block) against the thin instances on the
    same layer, rows and routing: hidden values and pair outputs bit for bit, for runs of one expert that fill a group,
    runs that end inside one, and experts with a single job or none."""
    from anemone_b200.moe import MoeConfig
    from anemone_b200.mx import MxLayer, MxLayout
    rows = 171
    config = MoeConfig(hidden=512, inner=256, experts=12, shared=1, picks=3, row_capacity=256, activation_limit=7.0)
    rng = np.random.default_rng(321)
    H, I = config.hidden, config.inner
    matrices = [(mx_matrix(oracle, rng, I, H), mx_matrix(oracle, rng, I, H), mx_matrix(oracle, rng, H, I))
                for _ in range(config.experts)]
    always = (synthetic.e4m3_matrix(rng, I, H), synthetic.e4m3_matrix(rng, I, H), synthetic.e4m3_matrix(rng, H, I))
    tokens = synthetic.tokens(rng, rows, H)
    scores = rng.normal(0, 1, size=(rows, config.experts)).astype(np.float32)
    scores[:, 1] += 1.5  # one expert with many jobs
    scores[:, 7] -= 30.0  # one with none
    L = MxLayout(config, 1, 0, wide=True)
    got = {}
    for many in (False, True):
        card = api.Card(0, L.arena_bytes)
        try:
            layer = MxLayer(card, config, matrices, slices=slices, shared_matrices=always, wide=True, many=many)
            layer.connect_local([layer])
            result = layer.step(tokens, scores)
            received = card.download(0, L.arena_bytes)
        finally:
            card.close()
        live = rows * config.picks
        got[many] = (received[L.at["hidden"]:L.at["hidden"] + live * I * 2].copy(),
                     received[L.at["pair_output"]:L.at["pair_output"] + live * H * 2].copy(), result.copy(),
                     tuple(tuple(launch.grid) for launch in layer.expert_launches))
    assert got[True][3] != got[False][3]  # other launches
    assert got[True][3][0] == (I // 64, (L.job_capacity + R.LINEAR_MANY_JOBS - 1) // R.LINEAR_MANY_JOBS, 1)
    assert got[True][3][2] == (H // 128, (L.job_capacity + R.LINEAR_MANY_JOBS - 1) // R.LINEAR_MANY_JOBS, 1)
    assert np.any(got[False][1] != 0)
    assert np.array_equal(got[True][0], got[False][0])
    assert np.array_equal(got[True][1], got[False][1])
    assert np.array_equal(got[True][2], got[False][2])
