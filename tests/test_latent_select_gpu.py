"""Sparse index selection and the fused output rotation of the shared-latent stage
on a B200. Scores and selected rows are integer / bit-exact work: the float score of
every candidate and the ranked row lists must equal the CPU checker's (which the CPU
suite pins to the reference's compiled code). The rotation epilogue is exact given
the published values it starts from; the whole stage (select -> reduce -> rotate)
is compared with the reference-made golden fixtures within the reduce stage's
tolerance (5e-4 absolute and relative plus bf16 ulps of the rotated pair)."""
import ctypes as C
import os

import numpy as np
import pytest

import clori_b200
from clori_b200 import abi
from latent_cases import bf16_valued, build, host_args
from oracle.binding import PositionPolicy, indexer_struct
from test_latent_reduce_gpu import run_gpu

pytestmark = pytest.mark.gpu
u64 = np.uint64
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "latent_attention.npz")


def run_select(backend, keys, positions, query, weights, heads, hd, topk, ratio, start, expect_rc=0):
    lib, s = backend.lib, backend.stream
    tokens, rows = query.shape[0], keys.shape[0]
    t = dict(keys=backend.tensor("keys", keys), query=backend.tensor("iq", query), weights=backend.tensor("iw", weights),
             positions=backend.tensor("pos", positions.view(np.int64), dtype=abi.DTYPE_I64),
             scores=backend.alloc("scores", abi.DTYPE_F32, (tokens, rows)),
             selected=backend.alloc("sel", abi.DTYPE_I64, (tokens, topk)),
             count=backend.alloc("cnt", abi.DTYPE_I64, (tokens,)),
             status=backend.tensor("status", np.zeros(1, np.int32)))
    nbytes = lib.yvx_cuda_csa_select_workspace_bytes(rows, tokens, topk)
    work = backend.alloc("work", abi.DTYPE_I8, (int(nbytes),))
    a = abi.CsaSelectArgs()
    a.keys, a.positions, a.rows, a.key_stride = t["keys"].data_ptr, t["positions"].data_ptr, rows, keys.shape[1]
    a.query, a.weights, a.heads, a.head_dim, a.topk = t["query"].data_ptr, t["weights"].data_ptr, heads, hd, topk
    a.ratio, a.phase_start_position, a.token_count = ratio, start, tokens
    a.scores, a.selected, a.selected_count = t["scores"].data_ptr, t["selected"].data_ptr, t["count"].data_ptr
    a.topk_capacity, a.workspace, a.status = topk, work.data_ptr, t["status"].data_ptr
    launches = C.c_uint()
    rc = lib.yvx_cuda_csa_select(C.byref(a), s, C.byref(launches))
    assert rc == expect_rc, lib.yvx_cuda_last_error_text()
    if rc:
        return None
    assert lib.yvx_cuda_stream_synchronize(s) == 0, lib.yvx_cuda_last_error_text()
    for name in ("scores", "selected", "count"):
        t[name].struct.is_written = 1
    return (t["scores"].read(), t["selected"].read().view(u64), t["count"].read().view(u64),
            int(t["status"].read()[0]), launches.value)


def check_against_oracle(oracle, got, keys, positions, query, weights, heads, hd, topk, ratio, start):
    scores, selected, counts, status, _ = got
    assert status == 0
    ix = indexer_struct(keys, positions, query, weights, heads, hd, topk, ratio)
    for t in range(query.shape[0]):
        picked, valid, ref_scores = oracle.csa_select(ix, t, start + t)
        candidates = ~np.isnan(ref_scores)
        assert candidates.sum() == valid
        assert np.array_equal(scores[t][candidates].view(np.uint32), ref_scores[candidates].view(np.uint32))
        assert int(counts[t]) == len(picked)
        assert np.array_equal(selected[t, :len(picked)], picked)


@pytest.mark.parametrize("heads,hd,rows,topk,tokens,start_offset", [
    (4, 32, 75, 8, 3, 0),            # a few rows
    (64, 128, 575, 512, 2, 0),       # the reference configuration's widths: 575 candidates for 512
    (8, 64, 9000, 512, 3, 0),        # three chunks of rows -> one merge level
    (4, 32, 40000, 1024, 1, 0),      # ten chunks, fan-in 4 -> three merge levels
    (48, 96, 300, 64, 2, -700),      # heads that do not divide the block; only part of the rows visible
    (64, 128, 100, 512, 4, 0),       # fewer candidates than k
])
def test_scores_and_selection_equal_the_checker(backend, oracle, heads, hd, rows, topk, tokens, start_offset):
    rng = np.random.default_rng(rows + heads)
    ratio = 4
    keys = bf16_valued(rng, (rows, hd + 8))[:, :hd + 8]
    positions = np.arange(rows, dtype=u64) * u64(ratio)
    query = bf16_valued(rng, (tokens, heads * hd))
    weights = bf16_valued(rng, (tokens, heads), 0.5)
    start = rows * ratio + start_offset
    got = run_select(backend, keys, positions, query, weights, heads, hd, topk, ratio, start)
    check_against_oracle(oracle, got, keys, positions, query, weights, heads, hd, topk, ratio, start)
    lists, expected_launches = -(-rows // 4096), 2
    while lists > 1:
        lists, expected_launches = -(-lists // (4096 // topk)), expected_launches + 1
    assert got[4] == expected_launches


def test_ties_zeros_and_signed_zero(backend, oracle):
    # small integers: many exactly equal scores; zero weights: scores of +0 and -0 that must tie
    rng = np.random.default_rng(8)
    heads, hd, rows, topk, ratio = 4, 32, 6000, 512, 4
    keys = rng.integers(-1, 2, (rows, hd)).astype(np.float32)
    positions = np.arange(rows, dtype=u64) * u64(ratio) + u64(3)
    query = rng.integers(-1, 2, (2, heads * hd)).astype(np.float32)
    weights = rng.integers(-1, 2, (2, heads)).astype(np.float32)
    weights[1] = [0.0, -0.0, 0.0, -0.0]
    start = rows * ratio + 10
    got = run_select(backend, keys, positions, query, weights, heads, hd, topk, ratio, start)
    check_against_oracle(oracle, got, keys, positions, query, weights, heads, hd, topk, ratio, start)
    # all scores of token 1 are zero: the first k rows in position order
    assert np.array_equal(got[1][1, :topk], np.arange(topk, dtype=u64))


def test_refusals(backend):
    rng = np.random.default_rng(9)
    heads, hd, rows, topk, ratio = 4, 32, 50, 8, 4
    keys = bf16_valued(rng, (rows, hd))
    positions = np.arange(rows, dtype=u64) * u64(ratio)
    query, weights = bf16_valued(rng, (1, heads * hd)), bf16_valued(rng, (1, heads))
    start = rows * ratio
    bad = positions.copy()
    bad[20] = bad[19]                                   # duplicate position
    assert run_select(backend, keys, bad, query, weights, heads, hd, topk, ratio, start)[3] == 2
    nan_keys = keys.copy()
    nan_keys[7, 3] = np.nan
    assert run_select(backend, nan_keys, positions, query, weights, heads, hd, topk, ratio, start)[3] == 1
    # a non-finite key in a row that is not yet visible is not inspected
    assert run_select(backend, nan_keys, positions, query, weights, heads, hd, topk, ratio, 20)[3] == 0
    run_select(backend, keys, positions, query, weights, 65, hd, topk, ratio, start, expect_rc=abi.YVEX_ERR_UNSUPPORTED)
    run_select(backend, keys, positions, query, weights, heads, hd, 2048, ratio, start, expect_rc=abi.YVEX_ERR_UNSUPPORTED)


def run_reduce_rotated(backend, case, frequency):
    """The reduce launch with the rotation epilogue; returns (out, status)."""
    freq = backend.tensor("freq", frequency)
    t = {}
    for name in ("query", "local", "compressed", "sinks"):
        t[name] = backend.tensor(name, case[name])
    for name in ("local_positions", "compressed_positions", "selected", "selected_count"):
        t[name] = backend.tensor(name, case[name].view(np.int64), dtype=abi.DTYPE_I64)
    out = backend.alloc("out", abi.DTYPE_F32, (case["tokens"], case["heads"] * case["hd"]))
    status = backend.tensor("status", np.zeros(1, np.int32))
    a = host_args(case)
    for name in t:
        setattr(a, name, t[name].data_ptr)
    a.out, a.status = out.data_ptr, status.data_ptr
    a.rope_dims, a.rope_frequency = 2 * len(frequency), freq.data_ptr
    nbytes = int(backend.lib.yvx_cuda_latent_reduce_workspace_bytes(C.byref(a)))
    if nbytes:
        a.workspace = backend.alloc("work", abi.DTYPE_I8, (nbytes,)).data_ptr
    assert backend.lib.yvx_cuda_latent_reduce(C.byref(a), backend.stream) == 0, backend.lib.yvx_cuda_last_error_text()
    assert backend.lib.yvx_cuda_stream_synchronize(backend.stream) == 0
    out.struct.is_written = 1
    return out.read(), int(status.read()[0])


@pytest.mark.parametrize("policy", [(10000, 0, 0, 0, 0), (10000, 16, 65536, 32, 1)])
@pytest.mark.parametrize("heads,hd,rope,start", [(16, 512, 64, 70000), (10, 64, 16, 40), (8, 128, 128, 999983)])
def test_rotation_epilogue_is_exact(backend, oracle, policy, heads, hd, rope, start):
    rng = np.random.default_rng(start)
    tokens = 3
    case = build(rng, heads, hd, 128, 0, tokens, start)
    frequency = oracle.rope_frequencies(PositionPolicy(*policy), rope)
    device_frequency = np.zeros(rope // 2, np.float64)
    assert backend.lib.yvex_b200_rope_frequencies(C.byref(abi.PositionPolicy(*policy)), rope,
                                                  device_frequency.ctypes.data) == 0
    assert np.array_equal(device_frequency, frequency)
    plain, status = run_gpu(backend, case)
    rotated, status2 = run_reduce_rotated(backend, case, frequency)
    assert status == 0 and status2 == 0
    for t in range(tokens):
        for h in range(heads):
            row = plain[t, h * hd:(h + 1) * hd]
            expect = oracle.rope_apply(row, rope, start + t, frequency, True)
            expect = clori_b200.bf16_bits_to_f32(clori_b200.f32_to_bf16_bits(expect))
            assert np.array_equal(rotated[t, h * hd:(h + 1) * hd].view(np.uint32), expect.view(np.uint32))


def test_rotation_refusals(backend):
    rng = np.random.default_rng(1)
    case = build(rng, 8, 128, 128, 0, 1, 10)
    a = host_args(case)
    a.out = a.status = a.rope_frequency = 1
    for bad in (0, 3, 130):
        a.rope_dims = bad
        assert backend.lib.yvx_cuda_latent_reduce(C.byref(a), backend.stream) == abi.YVEX_ERR_INVALID_ARG


def ptr(tensor):
    return C.cast(tensor.ptr, C.c_void_p) if tensor is not None else None


def test_select_then_reduce_operators_against_the_reference_fixtures(backend):
    g = np.load(GOLDEN)
    checked = 0
    for i in range(int(g["count"])):
        heads, hd, cls, tokens, start, topk, ih, idim, rope = (int(x) for x in g[f"meta{i}"])
        f32 = lambda name: clori_b200.bf16_bits_to_f32(g[f"{name}_{i}"])
        rows = int(g[f"rows{i}"])
        ratio = {0: 0, 1: 4, 2: 128}[cls]
        t = dict(query=backend.tensor("q", f32("query")), local=backend.tensor("l", f32("local")),
                 compressed=backend.tensor("c", f32("compressed")), sinks=backend.tensor("s", g[f"sinks_{i}"]),
                 local_positions=backend.tensor("lp", g[f"local_positions_{i}"].view(np.int64), dtype=abi.DTYPE_I64),
                 compressed_positions=backend.tensor("cp", g[f"compressed_positions_{i}"].view(np.int64), dtype=abi.DTYPE_I64),
                 frequency=backend.tensor("f", g[f"frequency{i}"]),
                 selected=backend.alloc("sel", abi.DTYPE_I64, (tokens, topk)),
                 selected_count=backend.alloc("cnt", abi.DTYPE_I64, (tokens,)),
                 out=backend.alloc("out", abi.DTYPE_F32, (tokens, heads * hd)))
        failure, facts, err = abi.AttentionFailure(), abi.OperationFacts(), abi.Error()
        if cls == 1:
            t.update(keys=backend.tensor("ik", f32("index_keys")), iq=backend.tensor("iq", f32("index_query")),
                     iw=backend.tensor("iw", f32("index_weights")),
                     scores=backend.alloc("sc", abi.DTYPE_F32, (tokens, rows)))
            s = abi.AttentionSelectRequest()
            s.token_position, s.token_count = start, tokens
            s.indexer_heads, s.indexer_head_dimension, s.indexer_topk, s.compression_ratio = ih, idim, topk, ratio
            s.index_keys, s.positions, s.count, s.key_stride = ptr(t["keys"]), ptr(t["compressed_positions"]), rows, idim
            s.index_query, s.index_weights = ptr(t["iq"]), ptr(t["iw"])
            s.scores, s.selected, s.selected_count = ptr(t["scores"]), ptr(t["selected"]), ptr(t["selected_count"])
            rc = backend.lib.yvex_b200_attention_select_execute(backend.handle, C.byref(s), C.byref(failure),
                                                                C.byref(facts), C.byref(err))
            assert rc == 0, err.message
            assert facts.kernel_launches == 2 and failure.code == 0
            counts = t["selected_count"].read().view(u64)
            assert np.array_equal(counts, g[f"counts{i}"])
            selected = t["selected"].read().view(u64)
            for tok in range(tokens):
                n = int(counts[tok])
                assert np.array_equal(g[f"compressed_positions_{i}"][selected[tok, :n]], g[f"positions{i}"][tok, :n])
        r = abi.AttentionReduceRequest()
        r.attention_class, r.token_position, r.token_count = cls, start, tokens
        r.query_heads, r.head_dimension = heads, hd
        r.sliding_window, r.compression_ratio, r.indexer_topk = 128, ratio, topk
        r.query, r.local, r.local_positions = ptr(t["query"]), ptr(t["local"]), ptr(t["local_positions"])
        r.local_count, r.local_stride = min(start, 127), hd + 16
        r.compressed, r.compressed_positions = ptr(t["compressed"]), ptr(t["compressed_positions"])
        r.compressed_count, r.compressed_stride = max(rows, 1), hd
        r.selected, r.selected_count = ptr(t["selected"]), ptr(t["selected_count"])
        r.sinks, r.output = ptr(t["sinks"]), ptr(t["out"])
        r.rope_dimension, r.rope_frequency = rope, ptr(t["frequency"])
        rc = backend.lib.yvex_b200_attention_reduce_execute(backend.handle, C.byref(r), C.byref(failure),
                                                            C.byref(facts), C.byref(err))
        assert rc == 0, err.message
        got, ref = t["out"].read(), g[f"out{i}"]
        # rotated lanes mix two published values: twice the publication tolerance there
        bound = 1e-3 + (5e-4 + 2.0 ** -6) * np.maximum(np.abs(got), np.abs(ref))
        assert np.all(np.abs(got - ref) <= bound)
        a, c = got.astype(np.float64).ravel(), ref.astype(np.float64).ravel()
        assert a @ c / np.sqrt((a @ a) * (c @ c)) >= 0.9999
        checked += 1
    assert checked == 5
