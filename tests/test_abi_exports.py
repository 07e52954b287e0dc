"""The C-ABI library loads on a machine without a GPU and exports every symbol the public headers declare."""
import ctypes as C
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for path in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = re.sub(r"/\*.*?\*/", "", open(path).read(), flags=re.S)
        text = re.sub(r"AB_INLINE[^{;]*\{", "{", text)  # inline helpers are not exports
        for match in re.finditer(r"(?:result_status|const char \*|uint64_t|uint32_t|void|const struct backend_operations \*)\s*"
                                 r"([a-z_0-9]+)\s*\(", text):
            names.add(match.group(1))
        for match in re.finditer(r"extern const struct [a-z_]+ ([a-z_0-9]+);", text):
            names.add(match.group(1))
    inline = {"exl3_bits_x2", "exl3_window_end", "exl3_code_bytes", "exl3_matrix_bytes", "exl3_tile_position",
              "bf16_wire_byte", "bf16_wire_half", "bf16_wire_high_exponent", "bf16_wire_low_exponent",
              "bf16_wire_pair_pack", "bf16_wire_pair_unpack"}
    return sorted(names - inline)


def test_library_loads_and_exports_every_declared_symbol():
    from anemone_b200 import api
    lib = api.library()
    names = declared_symbols()
    assert len(names) >= 30 and "exl3_experts_prepare" in names and "backend_cuda_value" in names
    missing = [name for name in names if not hasattr(lib, name)]
    assert not missing, missing


def test_no_card_without_a_driver_is_not_an_error():
    from anemone_b200 import api
    assert api.card_count() >= 0  # 0 here; the table answers, nothing computes
    operations = api.operations().contents
    assert operations.name == b"cuda-sm_100a"
    for absent in ("digest", "exchange_allocate", "peer_attach", "staging_retire"):
        assert not getattr(operations, absent)
    assert api.library().status_text(6) == b"timed out" and api.library().status_text(99) == b"unknown status"


def test_record_sizes_match_the_headers():
    from anemone_b200 import records as R
    header = open(os.path.join(ROOT, "include", "anemone_b200_records.h")).read()
    declared = dict(re.findall(r"AB_RECORD_HAS\(([a-z_0-9]+), (\d+)\);", header))
    mirror = {"exl3_reconstruct_record": R.Exl3Reconstruct, "exl3_expert_record": R.Exl3Expert,
              "expert_job_record": R.ExpertJob, "expert_row_sum_arguments": R.ExpertRowSum,
              "bb_exl3_shard_activation_record": R.Exl3ShardActivation, "exl3_moe_record": R.Exl3Moe,
              "exl3_prefill_record": R.Exl3Prefill, "exl3_prefill_tile": R.Exl3PrefillTile,
              "exl3_prefill_entry": R.Exl3PrefillEntry,
              "step_block": R.StepBlock, "ordered_collective_peer": R.OrderedPeer,
              "ordered_collective_arguments": R.OrderedCollective, "ordered_reduce_bf16_arguments": R.OrderedReduceBf16,
              "ordered_row_sum_publish_arguments": R.OrderedRowSumPublish,
              "ordered_push_arguments": R.OrderedPush, "tp_exchange_arguments": R.TpExchange,
              "ordered_rows_push_arguments": R.OrderedRowsPush, "tp2_join_arguments": R.Tp2Join,
              "router_select_b200_arguments": R.RouterSelectB200, "step_input_select_arguments": R.StepInputSelect,
              "activation_quantize_arguments": R.ActivationQuantize, "expert_gate_up_arguments": R.ExpertGateUp,
              "expert_down_arguments": R.ExpertDown, "trunk_linear_quantized_arguments": R.TrunkLinearQuantized,
              "trunk_hidden_arguments": R.TrunkHidden, "trunk_rows_add_arguments": R.TrunkRowsAdd,
              "exl3_layer_route_record": R.Exl3LayerRoute, "exl3_layer_publish_arguments": R.Exl3LayerPublish,
              "ordered_publish_reduce_arguments": R.OrderedPublishReduce,
              "exact_ring_arguments": R.ExactRing, "exl3_layer_products_record": R.Exl3LayerProducts,
              "router_wide_arguments": R.RouterWide, "expert_gate_up_many_arguments": R.ExpertGateUpMany,
              "expert_down_many_arguments": R.ExpertDownMany,
              "ordered_publish_reduce_bf16_arguments": R.OrderedPublishReduceBf16,
              "router_select_quantize_arguments": R.RouterSelectQuantize}
    assert set(declared) == set(mirror)
    for name, record in mirror.items():
        assert C.sizeof(record) == int(declared[name]), name


REFERENCE = os.environ.get("ANEMONE_REFERENCE", "/root/reference")

# every function the reference's boundary for this path names (its own headers declare them), and its card table
BOUNDARY = {
    "anemone/exl3.h": ["exl3_width_name", "exl3_reconstruct_prepare", "exl3_scratch_byte_count", "exl3_experts_prepare",
                       "exl3_experts_fast_prepare", "exl3_experts_relaxed_prepare"],
    "anemone/exl3_layout.h": ["bb_exl3_matrix_slice_prepare", "bb_exl3_matrix_slice_copy",
                              "bb_exl3_output_shard_prepare"],
    "anemone/exl3_tp.h": ["bb_exl3_pass_prepare", "bb_exl3_row_sum_prepare"],
    "anemone/exl3_tc.h": ["exl3_tc_prepare", "exl3_tc_prepare_short", "exl3_tc_prepare_paired", "exl3_tcp_prepare",
                          "exl3_tcp_prepare_base", "exl3_tcp_prepare_hybrid"],
    "anemone/ordered_collective.h": ["ordered_collective_routes_prepare", "ordered_collective_routes_prepare_measured",
                                     "ordered_collective_kernels_prepare", "ordered_collective_prepare",
                                     "ordered_collective_host"],
    "anemone/ordered_push.h": ["ordered_push_kernel_prepare", "ordered_push_prepare", "ordered_push_routes_prepare"],
    "anemone/tp_exchange.h": ["tp_exchange_kernel_prepare", "tp_exchange_prepare", "tp_exchange_wide_kernels_prepare",
                              "tp_exchange_wide_prepare"],
}


def test_a_caller_built_on_the_reference_headers_links_against_the_library(tmp_path):
    """A C file that includes the REFERENCE's own headers and takes the address of every function of its boundary for
    this path (and of its card table) compiles against those headers and links against libanemone_b200.so alone: the
    reference's callers find every symbol they bind. Runs where the reference tree is present."""
    import shutil
    import subprocess
    import pytest
    if not os.path.isdir(os.path.join(REFERENCE, "include", "anemone")):
        pytest.skip("the reference tree is not on this machine")
    from anemone_b200 import api
    api.library()
    lines = ['#include "%s"' % header for header in BOUNDARY] + ['#include "anemone/backend_seam.h"', "#include <stdio.h>",
                                                                  "int main(void)", "{",
                                                                  "\tconst void *const bound[] = {"]
    lines += ["\t\t(const void *)%s," % name for names in BOUNDARY.values() for name in names]
    lines += ["\t\t(const void *)&backend_cuda_value, (const void *)&exl3_weight_operations,", "\t};",
              "\tunsigned found = 0;", "\tfor (unsigned i = 0; i < sizeof(bound) / sizeof(bound[0]); i++)",
              "\t\tfound += bound[i] != NULL;", '\tprintf("%u\\n", found);',
              "\treturn backend_cuda_value.card_count == NULL;", "}"]
    source = tmp_path / "caller.c"
    source.write_text("\n".join(lines) + "\n")
    binary = tmp_path / "caller"
    library_dir = os.path.dirname(api.LIBRARY)
    compiler = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else shutil.which("gcc")
    build = subprocess.run([compiler, "-std=c11", "-D_GNU_SOURCE", "-DCHECKING_HOOKS_ENABLED=0",
                            "-DTIMING_HOOKS_ENABLED=0", "-I" + os.path.join(REFERENCE, "include"), "-o", str(binary),
                            str(source), "-L" + library_dir, "-lanemone_b200", "-Wl,-rpath," + library_dir],
                           capture_output=True, text=True)
    assert build.returncode == 0, build.stderr
    ran = subprocess.run([str(binary)], capture_output=True, text=True)
    assert ran.returncode == 0 and int(ran.stdout) == sum(len(names) for names in BOUNDARY.values()) + 2
