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
    inline = {"exl3_bits_x2", "exl3_window_end", "exl3_code_bytes", "exl3_matrix_bytes", "exl3_tile_position"}
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
              "exl3_layer_down_record": R.Exl3LayerDown}
    assert set(declared) == set(mirror)
    for name, record in mirror.items():
        assert C.sizeof(record) == int(declared[name]), name
