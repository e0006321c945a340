"""Publication chain of projected rows on a B200 against the CPU checker (pinned to the
reference's compiled code by the CPU suite) and the reference-made fixtures.

Without a norm the chain is rotation -> bf16 -> activation: exact given its inputs, so rows must
be bit-equal. With a norm the sum of squares is reduced in a tree instead of serially and the
device square root / sine / cosine may differ from libm in the last place, so a published bf16
lane may land on the other side of a rounding tie: at most 1 lane in 200, by one bf16 ulp
(relative 2^-7). The activation is exact given the published row, so it is checked bit for bit
against the checker's activation of the device's own published rows."""
import ctypes as C
import os

import numpy as np
import pytest

from clori_b200 import abi
from oracle.binding import PositionPolicy
from publish_cases import CASES, POLICY, build

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "rows_publish.npz")


def same_bits(a, b):
    return a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))


def run_gpu(backend, x, rpt, start, norm_mode=0, norm_weights=None, epsilon=1e-6, rope_dims=0, rope_frequency=None,
            quantization=0, activation_count=0, block_width=0, hadamard=0, expect_rc=0):
    lib, s = backend.lib, backend.stream
    t = backend.tensor("x", x)
    status = backend.tensor("status", np.zeros(1, np.int32))
    a = abi.RowsPublishArgs()
    a.values, a.rows, a.rows_per_token, a.row_stride, a.width = t.data_ptr, x.shape[0], rpt, x.shape[1], x.shape[1]
    a.norm_mode, a.epsilon = norm_mode, epsilon
    keep = []
    if norm_mode == 2:
        keep.append(backend.tensor("w", norm_weights))
        a.norm_weights = keep[-1].data_ptr
    if rope_dims:
        keep.append(backend.tensor("f", np.ascontiguousarray(rope_frequency, np.float64), dtype=abi.DTYPE_F64))
        a.rope_dims, a.rope_frequency = rope_dims, keep[-1].data_ptr
    a.start_position = start
    a.quantization, a.activation_count, a.block_width, a.hadamard = quantization, activation_count, block_width, hadamard
    a.status = status.data_ptr
    rc = lib.yvx_cuda_rows_publish(C.byref(a), s)
    assert rc == expect_rc, lib.yvx_cuda_last_error_text()
    if rc:
        return None
    assert lib.yvx_cuda_stream_synchronize(s) == 0, lib.yvx_cuda_last_error_text()
    return t.read(), int(status.read()[0])


def check(backend, oracle, x, w, rpt, start, chain, freq, reference_rows=None):
    plain = {k: v for k, v in chain.items() if k not in ("quantization", "activation_count", "block_width", "hadamard")}
    expected = oracle.rows_publish(x, rpt, start, norm_weights=w, rope_frequency=freq, **plain)
    got, status = run_gpu(backend, x, rpt, start, norm_weights=w, rope_frequency=freq, **plain)
    assert status == 0
    if chain.get("norm_mode"):
        differ = got != expected
        assert differ.sum() <= max(1, got.size // 200)
        assert np.all(np.abs(got - expected)[differ] <= 2.0 ** -7 * np.abs(expected)[differ])
    else:
        assert same_bits(got, expected)
    if chain.get("quantization"):
        full, status = run_gpu(backend, x, rpt, start, norm_weights=w, rope_frequency=freq, **chain)
        assert status == 0
        count = chain["activation_count"]
        device_expected = got.copy()
        device_expected[:, :count] = oracle.activation_quant(np.ascontiguousarray(got[:, :count]), chain["quantization"],
                                                             chain["block_width"], chain.get("hadamard", 0))
        assert same_bits(full, device_expected)
        if reference_rows is not None and same_bits(got, expected):
            assert same_bits(full, reference_rows)
    elif reference_rows is not None and same_bits(got, expected):
        assert same_bits(got, reference_rows)


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_rows_against_the_checker(backend, oracle, case):
    name, width, rpt, tokens, start, chain = case
    x, w = build(400 + width, width, rpt * tokens)
    freq = oracle.rope_frequencies(PositionPolicy(*POLICY), chain["rope_dims"]) if chain.get("rope_dims") else None
    check(backend, oracle, x, w, rpt, start, chain, freq)


def test_reference_fixtures(backend, oracle):
    g = np.load(GOLDEN)
    for i, (name, width, rpt, tokens, start, chain) in enumerate(CASES):
        freq = g[f"frequency{i}"] if chain.get("rope_dims") else None
        check(backend, oracle, g[f"in{i}"], g[f"weights{i}"], rpt, start, chain, freq, reference_rows=g[f"out{i}"])


def test_prefill_sized_batch(backend, oracle):
    # 4096 tokens x 64 query heads of 512 lanes (537 MB): a sample of rows against the checker
    name, width, rpt, tokens, start, chain = CASES[0]
    x, w = build(77, width, rpt * 4096)
    freq = oracle.rope_frequencies(PositionPolicy(*POLICY), 64)
    got, status = run_gpu(backend, x, rpt, start, rope_frequency=freq, **chain)
    assert status == 0
    for token in (0, 1777, 4095):
        rows = slice(token * rpt, token * rpt + rpt)
        expected = oracle.rows_publish(x[rows], rpt, start + token, rope_frequency=freq, **chain)
        differ = got[rows] != expected
        assert differ.sum() <= max(1, expected.size // 200)
        assert np.all(np.abs(got[rows] - expected)[differ] <= 2.0 ** -7 * np.abs(expected)[differ])
    # publishing a published, unit-norm row again moves nothing but rounding ties: idempotent norm, new rotation
    again, _ = run_gpu(backend, got, rpt, start, norm_mode=1)
    assert np.abs(again - got).max() <= 2.0 ** -6 * np.abs(got).max()


def test_refusals_and_status(backend):
    x = np.ones((4, 128), np.float32)
    f = np.ones(32, np.float64)
    assert run_gpu(backend, x[:, :126].copy(), 1, 0, norm_mode=1, expect_rc=abi.YVEX_ERR_UNSUPPORTED) is None
    assert run_gpu(backend, x, 1, 0, norm_mode=1, epsilon=0.0, expect_rc=abi.YVEX_ERR_INVALID_ARG) is None
    assert run_gpu(backend, x, 1, 0, rope_dims=63, rope_frequency=f, expect_rc=abi.YVEX_ERR_INVALID_ARG) is None
    assert run_gpu(backend, x, 1, 0, quantization=8, activation_count=96, block_width=64,
                   expect_rc=abi.YVEX_ERR_BOUNDS) is None
    assert run_gpu(backend, x, 1, 0, quantization=3, activation_count=64, block_width=64,
                   expect_rc=abi.YVEX_ERR_FORMAT) is None
    x[2, 9] = np.inf
    assert run_gpu(backend, x, 1, 0, norm_mode=1)[1] == 1


def test_batched_launch_equals_separate_launches(backend, oracle):
    """The three row sets of a decode step in one launch: bit-equal to one launch per set."""
    lib, s = backend.lib, backend.stream
    freq = backend.tensor("f", oracle.rope_frequencies(PositionPolicy(*POLICY), 64), dtype=abi.DTYPE_F64)
    status = backend.tensor("status", np.zeros(1, np.int32))
    inputs, tensors, descriptors = [], [], (abi.RowsPublishArgs * 3)()
    for i, (name, width, rpt, tokens, start, chain) in enumerate(CASES[:3]):
        x, w = build(700 + i, width, rpt * 2)
        weights = backend.tensor("w", w)
        inputs.append(x)
        tensors.append((backend.tensor("x", x), weights))
        a = descriptors[i]
        a.values, a.rows, a.rows_per_token, a.row_stride, a.width = tensors[i][0].data_ptr, x.shape[0], rpt, width, width
        a.norm_mode, a.norm_weights, a.epsilon = chain.get("norm_mode", 0), weights.data_ptr, 1e-6
        a.rope_dims, a.rope_frequency, a.start_position = 64, freq.data_ptr, start
        a.quantization, a.activation_count = chain.get("quantization", 0), chain.get("activation_count", 0)
        a.block_width, a.hadamard, a.status = chain.get("block_width", 0), chain.get("hadamard", 0), status.data_ptr
    for i in range(3):
        assert lib.yvx_cuda_rows_publish(C.byref(descriptors[i]), s) == 0, lib.yvx_cuda_last_error_text()
    assert lib.yvx_cuda_stream_synchronize(s) == 0
    separate = [t.read() for t, _ in tensors]
    for (t, _), x in zip(tensors, inputs):
        t.write(x)
    assert lib.yvx_cuda_rows_publish_batch(descriptors, 3, s) == 0, lib.yvx_cuda_last_error_text()
    assert lib.yvx_cuda_stream_synchronize(s) == 0, lib.yvx_cuda_last_error_text()
    for (t, _), expected in zip(tensors, separate):
        assert same_bits(t.read(), expected)
    assert int(status.read()[0]) == 0
    assert lib.yvx_cuda_rows_publish_batch(descriptors, 5, s) == abi.YVEX_ERR_INVALID_ARG
    descriptors[1].width = 510
    assert lib.yvx_cuda_rows_publish_batch(descriptors, 3, s) == abi.YVEX_ERR_UNSUPPORTED


def ptr(tensor):
    return C.cast(tensor.ptr, C.c_void_p) if tensor is not None else None


def test_operator_entry(backend, oracle):
    name, width, rpt, tokens, start, chain = CASES[2]          # index queries: exact chain
    x, w = build(5, width, rpt * tokens)
    freq = oracle.rope_frequencies(PositionPolicy(*POLICY), chain["rope_dims"])
    t, f = backend.tensor("x", x), backend.tensor("f", freq, dtype=abi.DTYPE_F64)
    r = abi.AttentionPublishRequest()
    r.values, r.rows, r.rows_per_token, r.row_stride, r.width = ptr(t), x.shape[0], rpt, width, width
    r.token_position, r.norm_mode, r.rope_dimension, r.rope_frequency = start, 0, chain["rope_dims"], ptr(f)
    r.activation_quantization, r.activation_count, r.activation_block_width, r.activation_hadamard = 4, 128, 32, 1
    failure, facts, err = abi.AttentionFailure(), abi.OperationFacts(), abi.Error()
    call = lambda: backend.lib.yvex_b200_attention_publish_execute(backend.handle, C.byref(r), C.byref(failure),
                                                                   C.byref(facts), C.byref(err))
    assert call() == 0, err.message
    assert facts.kernel_launches == 1
    assert same_bits(t.read(), oracle.rows_publish(x, rpt, start, rope_frequency=freq, **chain))
    r.activation_block_width = 48
    assert call() == abi.YVEX_ERR_BOUNDS and failure.stage == b"publish"
    r.activation_block_width, r.rows = 32, x.shape[0] + 1
    assert call() == abi.YVEX_ERR_FORMAT


def test_chain_compressor_and_activation_inside_a_stream_capture(backend, oracle):
    """The three stage entries enqueue work only (no allocation, no synchronisation), so a decode
    step's calls can be captured once and replayed: the replayed graph leaves the same bits as the
    direct calls."""
    from compressor_cases import build as build_compressor
    from oracle.binding import compressor_initial_state
    lib, s = backend.lib, backend.stream
    name, width, rpt, tokens, start, chain = CASES[0]
    x, w = build(31, width, rpt)
    freq = oracle.rope_frequencies(PositionPolicy(*POLICY), 64)
    ratio, hd = 4, 128
    case = build_compressor(32, ratio, hd, 1, (ratio,))
    kv0, score0 = compressor_initial_state(ratio, hd, 1)
    t = dict(x=backend.tensor("x", x), f=backend.tensor("f", freq, dtype=abi.DTYPE_F64),
             kv=backend.tensor("kv", case["token_kv"]), sc=backend.tensor("sc", case["token_score"]),
             ape=backend.tensor("ape", case["ape"]), skv=backend.tensor("skv", kv0), ssc=backend.tensor("ssc", score0),
             akv=backend.alloc("akv", abi.DTYPE_F32, kv0.shape), asc=backend.alloc("asc", abi.DTYPE_F32, kv0.shape),
             norm=backend.tensor("norm", case["norm"]), rows=backend.alloc("rows", abi.DTYPE_F32, (1, hd)),
             status=backend.tensor("status", np.zeros(1, np.int32)))
    p = abi.RowsPublishArgs()
    p.values, p.rows, p.rows_per_token, p.row_stride, p.width = t["x"].data_ptr, rpt, rpt, width, width
    p.norm_mode, p.epsilon, p.rope_dims, p.rope_frequency, p.start_position = 1, 1e-6, 64, t["f"].data_ptr, start
    p.status = t["status"].data_ptr
    c = abi.CompressorArgs()
    c.ratio, c.head_dim, c.overlap, c.start_position, c.token_count = ratio, hd, 1, 0, ratio
    c.token_kv, c.token_score, c.token_stride, c.ape = t["kv"].data_ptr, t["sc"].data_ptr, 2 * hd, t["ape"].data_ptr
    c.state_kv, c.state_score, c.after_kv, c.after_score = (t[k].data_ptr for k in ("skv", "ssc", "akv", "asc"))
    c.compressed, c.compressed_stride = t["rows"].data_ptr, hd
    c.norm_weights, c.epsilon, c.rope_dims, c.rope_frequency = t["norm"].data_ptr, 1e-6, 64, t["f"].data_ptr
    c.status = t["status"].data_ptr
    q = abi.ActivationArgs()
    q.values, q.rows, q.row_stride, q.count = t["rows"].data_ptr, 1, hd, hd
    q.quantization, q.block_width, q.hadamard = 4, 32, 1
    q.hadamard_scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))
    q.status = t["status"].data_ptr
    emitted = C.c_ulonglong()

    def step():
        assert lib.yvx_cuda_rows_publish(C.byref(p), s) == 0
        assert lib.yvx_cuda_compressor_chunk(C.byref(c), s, C.byref(emitted)) == 0
        assert lib.yvx_cuda_activation_quant(C.byref(q), s) == 0

    step()
    assert lib.yvx_cuda_stream_synchronize(s) == 0, lib.yvx_cuda_last_error_text()
    for k in ("rows", "akv", "asc"):
        t[k].struct.is_written = 1
    direct = [t[k].read() for k in ("x", "rows", "akv", "asc")]
    assert emitted.value == 1 and int(t["status"].read()[0]) == 0
    t["x"].write(x)                      # the publication is in place: start again from the projected rows
    assert lib.yvx_cuda_graph_capture_begin(s) == 0, lib.yvx_cuda_last_error_text()
    step()
    graph = C.c_void_p()
    assert lib.yvx_cuda_graph_capture_end(s, C.byref(graph)) == 0, lib.yvx_cuda_last_error_text()
    assert lib.yvx_cuda_graph_launch(graph, s) == 0
    assert lib.yvx_cuda_stream_synchronize(s) == 0, lib.yvx_cuda_last_error_text()
    replayed = [t[k].read() for k in ("x", "rows", "akv", "asc")]
    for a, b in zip(direct, replayed):
        assert same_bits(a, b)
    assert lib.yvx_cuda_graph_destroy(graph) == 0


def test_python_stage_wrappers(backend, oracle):
    """Backend.attention_publish / _activation / _compress: the operator entries behind keyword calls."""
    from compressor_cases import build as build_compressor
    from oracle.binding import compressor_initial_state
    name, width, rpt, tokens, start, chain = CASES[2]
    x, _ = build(15, width, rpt * tokens)
    freq = oracle.rope_frequencies(PositionPolicy(*POLICY), 64)
    t, f = backend.tensor("x", x), backend.tensor("f", freq, dtype=abi.DTYPE_F64)
    rc, facts, failure = backend.attention_publish(
        t, rows_per_token=rpt, token_position=start, rope_dimension=64, rope_frequency=f,
        activation_quantization=4, activation_count=width, activation_block_width=32, activation_hadamard=1)
    assert rc == 0 and facts.kernel_launches == 1
    assert same_bits(t.read(), oracle.rows_publish(x, rpt, start, rope_frequency=freq, **chain))
    y = backend.tensor("y", x)
    rc, facts, failure = backend.attention_activation(y, quantization=8, block_width=64)
    assert rc == 0 and same_bits(y.read(), oracle.activation_quant(x, 8, 64, 0))
    rc, _, failure = backend.attention_activation(y, quantization=8, block_width=48, check=False)
    assert rc == abi.YVEX_ERR_BOUNDS and failure.stage == b"activation"
    ratio, hd = 4, 128
    case = build_compressor(16, ratio, hd, 1, (9,))
    kv0, score0 = compressor_initial_state(ratio, hd, 1)
    ref = oracle.compressor_chunk(ratio, hd, 1, 0, case["token_kv"], case["token_score"], case["ape"], kv0, score0)
    rows = backend.alloc("rows", abi.DTYPE_F32, (2, hd))
    akv, asc = backend.alloc("akv", abi.DTYPE_F32, kv0.shape), backend.alloc("asc", abi.DTYPE_F32, kv0.shape)
    rc, facts, failure, emitted = backend.attention_compress(
        kind=2, attention_class=1, token_position=0, token_count=9, compression_ratio=ratio, head_dimension=hd,
        token_kv=backend.tensor("kv", case["token_kv"]), token_score=backend.tensor("sc", case["token_score"]),
        token_stride=2 * hd, position_rows=backend.tensor("ape", case["ape"]), state_kv=backend.tensor("skv", kv0),
        state_score=backend.tensor("ssc", score0), next_state_kv=akv, next_state_score=asc, compressed=rows)
    assert rc == 0 and emitted == 2
    assert np.all(np.abs(rows.read() - ref[0]) <= 5e-7 * np.abs(ref[0]) + 1e-30)
    assert same_bits(akv.read(), ref[2]) and same_bits(asc.read(), ref[3])
