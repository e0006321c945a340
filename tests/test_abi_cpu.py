"""The C-ABI library loads without a GPU and exports every declared symbol;
host-side logic that needs no device (page and block indexing, admission
errors raised before any device call) behaves as the reference's."""
import ctypes as C
import os
import re

import numpy as np

import clori_b200
from clori_b200 import abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    names = set()
    pattern = re.compile(r"^\s*(?:const\s+)?[A-Za-z_][\w\s\*]*?\b(yv(?:ex|x)_\w+)\s*\(", re.M)
    for header in ("attention.h", "cuda_shim.h"):
        text = open(os.path.join(ROOT, "include", "yvex_b200", header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        for m in pattern.finditer(text):
            names.add(m.group(1))
    return names


def test_library_exports_every_declared_symbol(library):
    declared = _declared_functions()
    assert len(declared) >= 45
    missing = [n for n in sorted(declared) if not hasattr(library, n)]
    assert not missing, missing
    assert set(abi.EXPORTED_SYMBOLS) >= declared


def test_struct_sizes_match_the_reference_abi():
    # include/yvex/core.h: code + 96 + 256; include/yvex/internal/backend.h:215-228
    assert C.sizeof(abi.Error) == 356
    assert C.sizeof(abi.DeviceTensor) == 120          # four dims: include/yvex/model.h:85
    assert C.sizeof(abi.OperationFacts) == 13 * 8 + 8
    assert C.sizeof(abi.AttentionRequirement) == 9 * 8 + 8 * 4
    assert C.sizeof(abi.AttentionRequest) == C.sizeof(abi.AttentionRequirement) + 4 * 8


def test_open_refuses_without_a_fallback(library):
    err = abi.Error()
    handle = C.c_void_p()
    options = abi.BackendOptions(abi.BACKEND_KIND_CPU, None, 0)
    rc = library.yvex_backend_open(C.byref(handle), C.byref(options), C.byref(err))
    assert rc == abi.YVEX_ERR_UNSUPPORTED and not handle.value
    assert b"no CPU fallback" in err.message


def test_workspace_admission_codes(library):
    # src/backend/cuda/exact_attention.c:8-53 refusal order.
    def ask(**changes):
        r = clori_b200.attention_requirement(2, 4, 2, 8, 2, 128)
        for k, v in changes.items():
            setattr(r, k, v)
        nbytes = abi.u64(123)
        err = abi.Error()
        rc = library.yvex_b200_transformer_attention_workspace_required(
            C.byref(r), C.byref(nbytes), C.byref(err))
        return rc, nbytes.value
    assert ask() == (abi.YVEX_OK, 0)
    assert ask(query_start=3)[0] == abi.YVEX_ERR_INVALID_ARG      # query range beyond KV
    assert ask(query_heads=7)[0] == abi.YVEX_ERR_INVALID_ARG      # not a multiple of KV heads
    assert ask(value_token_stride=255)[0] == abi.YVEX_ERR_INVALID_ARG
    assert ask(head_dimension=257)[0] == abi.YVEX_ERR_UNSUPPORTED
    assert ask(output_dtype=abi.DTYPE_BF16)[0] == abi.YVEX_ERR_UNSUPPORTED
    assert ask(deterministic=0)[0] == abi.YVEX_ERR_UNSUPPORTED
    assert ask(numeric_contract=abi.NUMERIC_BF16_F32_ACCUMULATE)[0] == abi.YVEX_ERR_UNSUPPORTED
    assert ask(mask=0)[0] == abi.YVEX_ERR_UNSUPPORTED


def test_page_geometry_matches_reference_fixtures(library):
    # tests/unit/runtime_execution.c:203-279 expectations of the capacity plan.
    def page(**kw):
        r = abi.PageRequest()
        base = dict(logical_block_tokens=1, kernel_tile_tokens=1, promotion_granularity_tokens=1,
                    alignment_bytes=256, bytes_per_block=256, page_table_entry_bytes=16,
                    device_page_bytes=65536, logical_tokens=131072)
        base.update(kw)
        for k, v in base.items():
            setattr(r, k, v)
        tokens, nbytes = abi.u64(), abi.u64()
        assert library.yvex_b200_kv_page_tokens(C.byref(r), C.byref(tokens), C.byref(nbytes))
        return tokens.value, nbytes.value
    assert page(bytes_per_block=4096, logical_tokens=128) == (16, 65536)
    assert page(logical_block_tokens=8, kernel_tile_tokens=8, bytes_per_block=4096)[0] == 128
    assert page(bytes_per_block=32768, promotion_granularity_tokens=6, logical_tokens=5,
                candidate_extent=1)[0] == 6
    assert page(bytes_per_block=4104, logical_tokens=128, device_page_bytes=4096) == (32, 131328)
    # tests/unit/runtime_state.c:2069-2105: page_bytes = page_tokens / block * bytes_per_block
    for block, tokens in ((1, 16), (128, 128), (128, 256)):
        assert tokens // block * 4096 == {16: 65536, 128: 4096, 256: 8192}[tokens]


def test_page_and_block_indexing_equal_the_oracle(library, oracle):
    rng = np.random.default_rng(3)
    for _ in range(200):
        start, count, page = int(rng.integers(0, 10**6)), int(rng.integers(1, 10**4)), int(rng.integers(1, 5000))
        first, last = abi.u64(), abi.u64()
        assert library.yvex_b200_kv_page_touch(start, count, page, C.byref(first), C.byref(last))
        assert (first.value, last.value) == oracle.page_touch(start, count, page)
    assert not library.yvex_b200_kv_page_touch(1, 0, 4, C.byref(first), C.byref(last))
    table = rng.permutation(500).astype(np.int32)
    ptr = table.ctypes.data_as(C.POINTER(C.c_int))
    for row in rng.integers(0, 500 * 64, 300):
        assert library.yvex_b200_kv_block_row(ptr, 64, int(row)) == oracle.block_row(table, 64, int(row))


def test_split_plan_is_deterministic_and_bounded(library):
    p = abi.GqaProblem()
    p.sessions, p.kv_heads, p.kv_tokens_max, p.query_rows, p.query_heads, p.head_dim = 1, 8, 4096, 1, 32, 128
    library.yvx_cuda_gqa_plan_splits(C.byref(p), 148)
    assert (p.chunk_tokens, p.max_splits) == (64, 64)
    p.sessions, p.kv_tokens_max = 64, 32768
    library.yvx_cuda_gqa_plan_splits(C.byref(p), 148)
    assert p.chunk_tokens == 4096 and p.max_splits == 8
    assert library.yvx_cuda_gqa_partials_bytes(C.byref(p)) == 64 * 32 * 8 * 130 * 4
    p.sessions, p.kv_tokens_max, p.query_rows = 1, 131072, 4   # one long session: exactly one wave
    library.yvx_cuda_gqa_plan_splits(C.byref(p), 148)
    assert p.chunk_tokens == 3584 and p.max_splits == 37
    p.sessions, p.kv_tokens_max = 1, 3
    library.yvx_cuda_gqa_plan_splits(C.byref(p), 148)
    assert p.max_splits == 1 and library.yvx_cuda_gqa_partials_bytes(C.byref(p)) == 0


def test_bf16_helpers_equal_the_oracle(oracle):
    rng = np.random.default_rng(9)
    x = rng.standard_normal(5000).astype(np.float32) * np.float32(10.0) ** rng.integers(-20, 20, 5000).astype(np.float32)
    x[:4] = [np.nan, np.inf, -np.inf, -0.0]
    bits, widened = oracle.bf16_round(x)
    assert np.array_equal(clori_b200.f32_to_bf16_bits(x), bits)
    assert np.array_equal(clori_b200.bf16_bits_to_f32(bits).view(np.uint32), widened.view(np.uint32))


def test_struct_layouts_equal_the_reference_headers():
    """sizeof and every field offset of the structures that cross the boundary, and the enum
    values the caller passes, against tests/golden/abi_layout.json (written from the
    reference's own headers by tests/golden/make_abi_layout.py): once for the C headers of
    this library, once for the ctypes mirrors the Python tests use."""
    import json
    import sys
    golden = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    sys.path.insert(0, golden)
    import make_abi_layout as probe
    with open(os.path.join(golden, "abi_layout.json")) as f:
        reference = json.load(f)
    ours = probe.layout([os.path.join(os.path.dirname(golden), "..", "include")], probe.LIBRARY_HEADERS)
    assert ours == reference
    mirrors = {"yvex_error": abi.Error, "yvex_device_tensor": abi.DeviceTensor,
               "yvex_backend_operation_facts": abi.OperationFacts,
               "yvex_transformer_attention_requirement": abi.AttentionRequirement,
               "yvex_transformer_attention_request": abi.AttentionRequest,
               "yvex_backend_attention_weight": abi.JobWeight, "yvex_backend_attention_position": abi.JobPosition,
               "yvex_backend_attention_activation": abi.JobActivation,
               "yvex_backend_attention_rolling": abi.JobRolling, "yvex_backend_attention_job": abi.AttentionJob,
               "yvex_backend_attention_output": abi.AttentionJobOutput,
               "yvex_backend_attention_failure": abi.AttentionJobFailure,
               "yvex_backend_attention_completion_transfer": abi.CompletionTransfer,
               "struct yvex_backend_attention_completion": abi.AttentionCompletion,
               "yvex_backend_capability_result": abi.CapabilityResult}
    for name, mirror in mirrors.items():
        assert C.sizeof(mirror) == reference[name], name
        for field, _ in mirror._fields_[:]:
            assert getattr(mirror, field).offset == reference[f"{name}.{field}"], (name, field)
        assert len(mirror._fields_) == len(probe.STRUCTS[name]), name


def test_latent_decode_plans(library, monkeypatch):
    """The latent decode planner needs no device: a grid of sessions x splits, or (uniform lengths only, and only
    where it saves an eighth of the estimated cost) equal runs of the sessions' tiles, one per pair of SMs."""
    monkeypatch.delenv("YVEX_B200_MLA_PLAN", raising=False)
    monkeypatch.delenv("YVEX_B200_MLA_INDEPENDENT", raising=False)

    def plan(sessions, tokens, uniform=True, sms=148):
        p = abi.MlaProblem()
        p.sessions, p.heads, p.nope_dim, p.latent_dim, p.rope_dim = sessions, 128, 128, 512, 64
        p.kv_tokens_max = tokens
        if uniform:
            p.kv_tokens, p.kv_tokens_uniform = None, tokens
        else:
            p.kv_tokens = 0x1000     # a device address as far as the planner is concerned: lengths it cannot read
        library.yvx_cuda_mla_plan(C.byref(p), sms)
        return p.chunk_tokens, p.max_splits, p.balanced_pairs

    assert plan(32, 16384) == (8192, 2, 0)                 # 128 work items in one wave: nothing to gain
    assert plan(32, 16384, uniform=False) == (8192, 2, 0)
    chunk, pieces, pairs = plan(20, 16384)                 # 40 x 7 splits would be two waves
    assert pairs == 74 and pieces == 5 and chunk == 16384
    assert plan(20, 16384, uniform=False)[2] == 0          # lengths on the device: the grid
    monkeypatch.setenv("YVEX_B200_MLA_PLAN", "balanced")
    assert plan(32, 16384) == (16384, 4, 74)
    assert plan(3, 700, sms=10) == (704, 2, 5)
    assert plan(1, 100)[2] == 0                            # fewer cost units than pairs: some runs would be empty
    monkeypatch.setenv("YVEX_B200_MLA_PLAN", "grid")
    assert plan(20, 16384)[2] == 0
    # the scratch grows with the partial slots
    p = abi.MlaProblem()
    p.sessions, p.heads, p.latent_dim, p.max_splits = 2, 128, 512, 3
    assert library.yvx_cuda_mla_partials_bytes(C.byref(p)) == 2 * 128 * 2 * 3 * 258 * 4
