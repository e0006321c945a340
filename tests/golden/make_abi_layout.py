"""Generates tests/golden/abi_layout.json from the REFERENCE's own headers: sizeof and the
offset of every field of the structures that cross the drop-in boundary, as the reference's
compiler lays them out. The headers are compiled where they lie (YVEX_REFERENCE_TREE, or a
checkout named `reference` beside this repository):

    python tests/golden/make_abi_layout.py

tests/test_abi_cpu.py compiles the same probe against include/yvex_b200/*.h and compares.
"""
import json
import os
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
HERE = os.path.dirname(os.path.abspath(__file__))

STRUCTS = {
    "yvex_error": ["code", "where", "message"],
    "yvex_device_tensor": ["owner", "owner_id", "name", "dtype", "rank", "dims", "bytes", "data", "host_data",
                           "backend_allocation", "resident_bytes", "virtual_reserved", "is_written",
                           "host_accessible", "borrowed_host"],
    "yvex_backend_operation_facts": ["h2d_bytes", "d2h_bytes", "d2d_bytes", "kernel_launches", "upload_count",
                                     "download_count", "queue_synchronizations", "device_synchronizations",
                                     "active_weight_bytes", "state_bytes", "activation_bytes", "temporary_bytes",
                                     "accelerated_matrix_launches", "compulsory_memory_facts_available"],
    "yvex_transformer_attention_requirement": ["query_tokens", "key_value_tokens", "query_start", "query_heads",
                                               "key_value_heads", "head_dimension", "query_token_stride",
                                               "key_token_stride", "value_token_stride", "query_dtype", "key_dtype",
                                               "value_dtype", "output_dtype", "layout", "mask", "numeric_contract",
                                               "deterministic"],
    "yvex_transformer_attention_request": ["requirement", "query", "key", "value", "output"],
    "yvex_backend_attention_weight": ["encoded", "encoded_bytes", "row_bytes", "row_width", "row_count", "qtype",
                                      "present"],
    "yvex_backend_attention_position": ["theta", "scaling_factor", "original_context", "beta_fast", "beta_slow",
                                        "rope_dimensions"],
    "yvex_backend_attention_activation": ["required", "block_width", "quantization", "hadamard"],
    "yvex_backend_attention_rolling": ["present", "overlap", "next_token_position", "ratio", "head_dimension",
                                       "state_width", "state_slots", "cursor", "previous_fill", "current_fill",
                                       "kv_state", "score_state", "kv_state_capacity", "score_state_capacity"],
    "yvex_backend_attention_job": [
        "schema", "phase", "attention_class", "compute_contract", "operation_scope", "token_position", "token_count",
        "input_stride", "hidden_width", "q_rank", "query_heads", "head_dimension", "kv_width", "sliding_window",
        "compression_ratio", "output_groups", "output_group_input_width", "output_rank", "indexer_heads",
        "indexer_head_dimension", "indexer_topk", "residual_stream_count", "residual_stream_width",
        "residual_expanded_width", "mhc_mixing_rows", "mhc_sinkhorn_iterations", "rms_epsilon", "mhc_epsilon",
        "mhc_residual_post_multiplier", "position", "attention_kv_activation", "compressor_activation",
        "compressor_rotated_activation", "indexer_query_activation", "weights", "input", "local_kv", "compressed_kv",
        "indexer_kv", "device_input", "device_output", "local_positions", "compressed_positions",
        "indexer_positions", "local_count", "local_stride", "compressed_count", "compressed_stride", "indexer_count",
        "indexer_stride", "main_rolling", "indexer_rolling", "cancellation", "device_completion", "evidence_level",
        "measure_device_time", "candidate_block_visible", "retain_prefix_checkpoints", "native_execution",
        "max_host_bytes", "max_device_bytes"],
    "yvex_backend_attention_output": [
        "core_input", "q_low", "query", "raw_kv", "compressed_kv", "indexer_kv", "index_query", "index_weights",
        "attention_values", "output", "envelope_output", "compressed_positions", "indexer_positions",
        "topk_positions", "topk_counts", "valid_candidate_counts", "main_kv_state", "main_score_state",
        "indexer_kv_state", "indexer_score_state", "tokens_executed", "compressed_count", "indexer_count",
        "topk_count", "valid_candidate_count", "host_bytes", "peak_host_bytes", "device_bytes", "peak_device_bytes",
        "kernel_launches", "accelerated_matrix_launches", "h2d_bytes", "d2h_bytes", "d2d_bytes",
        "device_state_staged_bytes", "queue_synchronizations", "device_synchronizations",
        "device_execution_elapsed_ns", "host_workspace_capacity", "host_workspace_used", "host_workspace_peak",
        "host_workspace_allocation_count", "host_workspace_reused", "device_state_staged"],
    "yvex_backend_attention_failure": ["code", "stage", "expected", "actual"],
    "yvex_backend_attention_completion_transfer": ["output", "staged", "capacity", "output_capacity", "used",
                                                   "width", "stage"],
    "struct yvex_backend_attention_completion": [
        "defer", "stack_start", "pending", "barrier_observed", "output", "failure", "host_status",
        "host_selected_counts", "host_candidate_counts", "attention_class", "token_count", "indexer_topk",
        "candidate_capacity", "transfer_count", "transfers"],
    "yvex_backend_capability_result": ["backend_kind", "variant", "state", "reason", "input_dtype", "weight_dtype",
                                       "output_dtype", "context_available", "kernel_bundle_available",
                                       "function_available"],
}
ENUMS = ["YVEX_BACKEND_ATTENTION_JOB_SCHEMA", "YVEX_BACKEND_ATTENTION_WEIGHT_COUNT",
         "YVEX_BACKEND_ATTENTION_WEIGHT_INPUT_NORM", "YVEX_BACKEND_ATTENTION_HCA",
         "YVEX_BACKEND_ATTENTION_COMPUTE_BF16_F32_RNE_V1", "YVEX_BACKEND_ATTENTION_SCOPE_ENVELOPE",
         "YVEX_BACKEND_ATTENTION_PHASE_MIXED", "YVEX_BACKEND_ATTENTION_PHASE_COUNT",
         "YVEX_BACKEND_ATTENTION_FAILURE_CANCELLED", "YVEX_BACKEND_ATTENTION_FAILURE_CLEANUP",
         "YVEX_BACKEND_VARIANT_QTYPE_ROW_DOT", "YVEX_BACKEND_VARIANT_ATTENTION_ENCODED", "YVEX_BACKEND_VARIANT_COUNT",
         "YVEX_BACKEND_CAPABILITY_FAILED", "YVEX_BACKEND_CAPABILITY_REASON_CLEANUP_FAILED", "YVEX_ERR_TIMEOUT",
         "YVEX_ERR_CANCELLED", "YVEX_DTYPE_BF16", "YVEX_DTYPE_I64", "YVEX_TENSOR_MAX_DIMS",
         "YVEX_TRANSFORMER_ATTENTION_MASK_CAUSAL", "YVEX_TRANSFORMER_ATTENTION_NUMERIC_EXACT_F32"]


def probe_source(includes):
    lines = ["#include <stddef.h>", "#include <stdio.h>"] + [f"#include <{h}>" for h in includes]
    lines.append("int main(void) {")
    for name, fields in STRUCTS.items():
        lines.append(f'  printf("%s %zu\\n", "{name}", sizeof({name}));')
        for field in fields:
            lines.append(f'  printf("%s.%s %zu\\n", "{name}", "{field}", offsetof({name}, {field}));')
    for name in ENUMS:
        lines.append(f'  printf("%s %lld\\n", "{name}", (long long){name});')
    lines += ["  return 0;", "}"]
    return "\n".join(lines)


def layout(include_dirs, includes):
    """Compiles and runs the probe; returns {name: number}."""
    with tempfile.TemporaryDirectory() as tmp:
        src, exe = os.path.join(tmp, "probe.c"), os.path.join(tmp, "probe")
        with open(src, "w") as f:
            f.write(probe_source(includes))
        cmd = ["gcc", "-std=c11", "-D_GNU_SOURCE"] + [f"-I{d}" for d in include_dirs] + [src, "-o", exe]
        subprocess.run(cmd, check=True)
        out = subprocess.run([exe], check=True, capture_output=True, text=True).stdout
    return {line.rsplit(" ", 1)[0]: int(line.rsplit(" ", 1)[1]) for line in out.splitlines()}


REFERENCE_HEADERS = ["yvex/core.h", "yvex/backend.h", "yvex/internal/backend.h", "yvex/internal/transformer.h"]
LIBRARY_HEADERS = ["yvex_b200/abi.h", "yvex_b200/attention.h", "yvex_b200/attention_job.h"]


def main():
    from oracle.binding import reference_tree
    tree = reference_tree()
    assert tree, "the reference tree is required"
    result = layout([os.path.join(tree, "include"), tree], REFERENCE_HEADERS)
    with open(os.path.join(HERE, "abi_layout.json"), "w") as f:
        json.dump(result, f, indent=0, sort_keys=True)
    print("written", len(result), "entries")


if __name__ == "__main__":
    main()
