"""Generates tests/golden/reference_vectors.json by running the REFERENCE's own host code (oracle/_ref, compiled from
the reference sources by `make -C oracle ref`) on seeded inputs. Run where the reference tree is present:

    make -C oracle ref && python tests/golden/make_golden.py

The fixtures travel with the repository, so the oracle and the CUDA path are checked against the reference's outputs
on machines that do not have the reference tree.
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle.binding import f32p, load_oracle, load_reference, pointer_array, ptr, u32p, u64p, u8p  # noqa: E402
from tests.golden_util import router_case_inputs  # noqa: E402


def fnv64(values):
    digest = 0xCBF29CE484222325
    for byte in np.ascontiguousarray(values).reshape(-1).view(np.uint8).tolist():
        digest = ((digest ^ byte) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return digest


def bits_x2(stored):
    return 2 * stored if stored <= 8 else stored // 8


def main():
    reference = load_reference()
    if reference is None:
        raise SystemExit("oracle/_ref/libanemone_ref.so missing: run `make -C oracle ref` first")
    out = {"_generator": "tests/golden/make_golden.py over oracle/_ref (the reference's tests/exl3_reference.c and "
                         "source/ordered_collective.c compiled unchanged)"}
    decode = []
    for stored in (2, 40, 3, 4):
        rng = np.random.default_rng(0xE3100 + stored)
        inputs, outputs = 64, 48
        codes = rng.integers(0, 256, size=inputs * outputs // 16 * bits_x2(stored), dtype=np.uint8)
        weights = np.array([[reference.test_exl3_reconstruct(ptr(codes, u8p), inputs, outputs, stored, i, o)
                             for o in range(outputs)] for i in range(inputs)], dtype=np.uint16)
        decode.append({"stored": stored, "seed": 0xE3100 + stored, "inputs": inputs, "outputs": outputs,
                       "weights_fnv64": hex(fnv64(weights)), "first_row": [hex(v) for v in weights[0, :8].tolist()]})
    out["decode"] = decode
    out["codebook_fnv64"] = hex(fnv64(np.array([reference.test_exl3_codebook(s) for s in range(65536)],
                                               dtype=np.uint16)))
    reduce = []
    for ranks in (2, 4, 8):
        for rows in (1, 8):
            rng = np.random.default_rng(0x0C011 + 16 * ranks + rows)
            count = rows * 4096
            inputs = [rng.normal(0.0, 0.05, count).astype(np.float32) for _ in range(ranks)]
            outputs = [np.zeros(count, dtype=np.float32) for _ in range(ranks)]
            status = reference.ordered_collective_host(pointer_array(inputs), pointer_array(outputs), ranks, count, 0)
            assert status == 0
            reduce.append({"ranks": ranks, "rows": rows, "seed": 0x0C011 + 16 * ranks + rows,
                           "sum_fnv64": hex(fnv64(outputs[0])),
                           "first": [hex(v) for v in outputs[0][:8].view(np.uint32).tolist()]})
    out["ordered_all_reduce"] = reduce
    # the router at the reference's geometry (384 experts, 6 picks, scale 1.5, sqrt(softplus) affinities): its own
    # test_router_select / test_router_jobs on the affinities of seeded scores. The affinities are this library's
    # fixed FP32 sequence (the reference takes a card's affinities as given and bounds them by
    # test_router_affinity_holds, which make_golden asserts for every one of them).
    import ctypes as C
    oracle = load_oracle()
    reference.test_router_affinity_holds.restype = C.c_bool
    reference.test_router_affinity_holds.argtypes = [C.c_float, C.c_float]
    reference.test_router_select.argtypes = [f32p, f32p, C.c_bool, u32p, f32p]
    router = []
    for seed in (0x707E0, 0x707E1, 0x707E2, 0x707E7):
        scores, bias, table = router_case_inputs(seed)
        rows = scores.shape[0]
        affinities = np.array([[oracle.orc_router_affinity(float(s), 1) for s in row] for row in scores],
                              dtype=np.float32)
        for row in range(rows):
            for expert in range(384):
                assert reference.test_router_affinity_holds(float(scores[row, expert]), float(affinities[row, expert]))
        experts = np.zeros((rows, 6), dtype=np.uint32)
        weights = np.zeros((rows, 6), dtype=np.float32)
        for row in range(rows):
            reference.test_router_select(ptr(affinities[row], f32p), ptr(bias, f32p), False, ptr(experts[row], u32p),
                                         ptr(weights[row], f32p))
        jobs = np.zeros(rows * 6 * 96, dtype=np.uint8)
        reference.test_router_jobs(ptr(experts, u32p), ptr(weights, f32p), rows, rows, ptr(table, u64p),
                                   jobs.ctypes.data_as(C.c_void_p))
        router.append({"seed": seed, "rows": rows, "experts": experts.tolist(),
                       "weights": [[hex(v) for v in row] for row in weights.view(np.uint32).tolist()],
                       "jobs_fnv64": hex(fnv64(jobs))})
    out["router_select"] = router
    with open(os.path.join(ROOT, "tests", "golden", "reference_vectors.json"), "w") as handle:
        json.dump(out, handle, indent=1)
    print("wrote tests/golden/reference_vectors.json")


if __name__ == "__main__":
    main()
