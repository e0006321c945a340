"""Rolling compressor on a B200 against the CPU checker (which the CPU suite pins to the
reference's compiled code) and against the reference-made fixtures.

The state after a chunk and the emitted positions are copies and integer work: bit-exact.
An unpublished emission is a double-precision softmax per lane narrowed to float; the
device exponential may differ from libm's in the last place, so rows agree to 4 float ulps
(relative 5e-7). Published rows are bf16 values: equal except where that last-place
difference straddles a rounding tie, so at most 1 lane in 200 may differ, by one bf16 ulp
(relative 2^-7). Splitting a chunk changes nothing, bit for bit."""
import ctypes as C
import os

import numpy as np
import pytest

import clori_b200
from clori_b200 import abi
from compressor_cases import CASES, build
from oracle.binding import PositionPolicy, compressor_initial_state

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "compressor.npz")


def run_gpu(backend, ratio, hd, overlap, start, token_kv, token_score, ape, state_kv, state_score,
            norm=None, epsilon=1e-6, rope=0, frequency=None, expect_rc=0, alias=False):
    lib, s = backend.lib, backend.stream
    tokens = token_kv.shape[0]
    capacity = max(1, tokens // ratio + 1)
    t = dict(kv=backend.tensor("kv", token_kv if tokens else np.zeros((1, 1), np.float32)),
             score=backend.tensor("score", token_score if tokens else np.zeros((1, 1), np.float32)),
             ape=backend.tensor("ape", ape), skv=backend.tensor("skv", state_kv), ssc=backend.tensor("ssc", state_score),
             akv=backend.alloc("akv", abi.DTYPE_F32, state_kv.shape), asc=backend.alloc("asc", abi.DTYPE_F32, state_kv.shape),
             rows=backend.alloc("rows", abi.DTYPE_F32, (capacity, hd)),
             positions=backend.alloc("pos", abi.DTYPE_I64, (capacity,)),
             status=backend.tensor("status", np.zeros(1, np.int32)))
    a = abi.CompressorArgs()
    a.ratio, a.head_dim, a.overlap, a.start_position, a.token_count = ratio, hd, int(overlap), start, tokens
    a.token_kv, a.token_score, a.token_stride = t["kv"].data_ptr, t["score"].data_ptr, token_kv.shape[1]
    a.ape, a.state_kv, a.state_score = t["ape"].data_ptr, t["skv"].data_ptr, t["ssc"].data_ptr
    a.after_kv, a.after_score = (t["skv"] if alias else t["akv"]).data_ptr, t["asc"].data_ptr
    a.compressed, a.compressed_stride, a.positions = t["rows"].data_ptr, hd, t["positions"].data_ptr
    if norm is not None:
        t["norm"] = backend.tensor("norm", norm)
        a.norm_weights, a.epsilon, a.rope_dims = t["norm"].data_ptr, epsilon, rope
        if rope:
            t["freq"] = backend.tensor("freq", np.ascontiguousarray(frequency, np.float64), dtype=abi.DTYPE_F64)
            a.rope_frequency = t["freq"].data_ptr
    a.status = t["status"].data_ptr
    emitted = C.c_ulonglong()
    rc = lib.yvx_cuda_compressor_chunk(C.byref(a), s, C.byref(emitted))
    assert rc == expect_rc, lib.yvx_cuda_last_error_text()
    if rc:
        return None
    assert lib.yvx_cuda_stream_synchronize(s) == 0, lib.yvx_cuda_last_error_text()
    for name in ("akv", "asc", "rows", "positions"):
        t[name].struct.is_written = 1
    n = emitted.value
    return (t["rows"].read()[:n], t["positions"].read().view(np.uint64)[:n], t["akv"].read(), t["asc"].read(),
            int(t["status"].read()[0]))


def same_bits(a, b):
    return a.shape == b.shape and np.array_equal(np.ascontiguousarray(a).view(np.uint8), np.ascontiguousarray(b).view(np.uint8))


def check_rows(got, ref, published):
    assert got.shape == ref.shape
    if not published:
        assert np.all(np.abs(got - ref) <= 5e-7 * np.abs(ref) + 1e-30)
        return
    differ = got != ref
    assert differ.sum() <= max(1, got.size // 200)
    assert np.all(np.abs(got - ref)[differ] <= 2.0 ** -7 * np.abs(ref)[differ])


@pytest.mark.parametrize("case_index", range(len(CASES)))
@pytest.mark.parametrize("published", [False, True])
def test_chunks_against_the_checker(backend, oracle, case_index, published):
    kind, ratio, hd, overlap, rope, policy, chunks = CASES[case_index]
    case = build(300 + case_index, ratio, hd, overlap, chunks)
    freq = oracle.rope_frequencies(PositionPolicy(*policy), rope)
    norm = case["norm"] if published else None
    kv, score = case["state"]
    start = 0
    for n in chunks:
        tk, ts = case["token_kv"][start:start + n], case["token_score"][start:start + n]
        ref = oracle.compressor_chunk(ratio, hd, overlap, start, tk, ts, case["ape"], kv, score, norm, 1e-6, rope, freq)
        got = run_gpu(backend, ratio, hd, overlap, start, tk, ts, case["ape"], kv, score, norm, 1e-6, rope, freq)
        assert got[4] == 0
        check_rows(got[0], ref[0], published)
        assert np.array_equal(got[1], ref[1])
        assert same_bits(got[2], ref[2]) and same_bits(got[3], ref[3])
        kv, score, start = ref[2], ref[3], start + n


def test_reference_fixtures(backend):
    g = np.load(GOLDEN)
    for i in range(int(g["count"])):
        kind, ratio, hd, overlap, rope = (int(x) for x in g[f"meta{i}"])
        f32 = lambda name: clori_b200.bf16_bits_to_f32(g[f"{name}_{i}"])
        kv, score = compressor_initial_state(ratio, hd, overlap)
        got = run_gpu(backend, ratio, hd, overlap, 0, f32("token_kv"), f32("token_score"), f32("ape"), kv, score,
                      f32("norm"), float(g["epsilon"]), rope, g[f"frequency{i}"])
        assert got[4] == 0
        check_rows(got[0], clori_b200.bf16_bits_to_f32(g[f"rows{i}"]), True)
        assert np.array_equal(got[1], g[f"positions{i}"])
        assert same_bits(got[2], g[f"state_kv{i}"]) and same_bits(got[3], g[f"state_score{i}"])


@pytest.mark.parametrize("ratio,hd,overlap,tokens", [(4, 512, 1, 8192), (128, 512, 0, 8192), (4, 128, 1, 4099)])
def test_prefill_sized_chunk_does_not_depend_on_the_split(backend, oracle, ratio, hd, overlap, tokens):
    case = build(500 + ratio, ratio, hd, overlap, (tokens,))
    freq = oracle.rope_frequencies(PositionPolicy(10000, 16, 65536, 32, 1), 64)
    kv, score = case["state"]
    whole = run_gpu(backend, ratio, hd, overlap, 0, case["token_kv"], case["token_score"], case["ape"], kv, score,
                    case["norm"], 1e-6, 64, freq)
    assert whole[4] == 0 and len(whole[1]) == tokens // ratio
    rows, positions, start = [], [], 0
    for n in (1, ratio - 1, 1000, 3, tokens - 1000 - ratio - 3):
        part = run_gpu(backend, ratio, hd, overlap, start, case["token_kv"][start:start + n],
                       case["token_score"][start:start + n], case["ape"], kv, score, case["norm"], 1e-6, 64, freq)
        rows.append(part[0]), positions.append(part[1])
        kv, score, start = part[2], part[3], start + n
    assert same_bits(np.concatenate(rows), whole[0]) and np.array_equal(np.concatenate(positions), whole[1])
    assert same_bits(kv, whole[2]) and same_bits(score, whole[3])
    # a sample of rows against the checker: the last 3 groups, from a state the checker rolls up itself
    tail = 3 * ratio
    head = oracle.compressor_chunk(ratio, hd, overlap, 0, case["token_kv"][:tokens - tokens % ratio - tail],
                                   case["token_score"][:tokens - tokens % ratio - tail], case["ape"], *case["state"])
    begin = tokens - tokens % ratio - tail
    ref = oracle.compressor_chunk(ratio, hd, overlap, begin, case["token_kv"][begin:], case["token_score"][begin:],
                                  case["ape"], head[2], head[3], case["norm"], 1e-6, 64, freq)
    check_rows(whole[0][-3:], ref[0], True)
    assert same_bits(whole[2], ref[2]) and same_bits(whole[3], ref[3])


@pytest.mark.parametrize("ratio,hd,overlap,pad", [
    (4, 6, 1, 0),        # lanes that are no multiple of four: the one-lane-per-thread kernel
    (3, 34, 0, 0),       # odd ratio
    (4, 64, 1, 3),       # token rows whose stride breaks the 16-byte alignment
    (2, 1024, 1, 0),     # the widest head: 2048-lane rows
    (2, 1022, 0, 0),     # the widest head of the one-lane-per-thread kernel
])
def test_geometries_off_the_fast_path_and_at_the_limits(backend, oracle, ratio, hd, overlap, pad):
    rope = 2 if hd < 8 else 16
    case = build(600 + hd, ratio, hd, overlap, (3 * ratio + 1,))
    freq = oracle.rope_frequencies(PositionPolicy(10000, 0, 0, 0, 0), rope)
    kv, score = case["state"]
    width = case["token_kv"].shape[1]
    tk = np.zeros((case["token_kv"].shape[0], width + pad), np.float32)
    ts = np.zeros_like(tk)
    tk[:, :width], ts[:, :width] = case["token_kv"], case["token_score"]
    ref = oracle.compressor_chunk(ratio, hd, overlap, 0, case["token_kv"], case["token_score"], case["ape"], kv, score,
                                  case["norm"], 1e-6, rope, freq)
    got = run_gpu(backend, ratio, hd, overlap, 0, tk, ts, case["ape"], kv, score, case["norm"], 1e-6, rope, freq)
    assert got[4] == 0 and np.array_equal(got[1], ref[1])
    check_rows(got[0], ref[0], True)
    assert same_bits(got[2], ref[2]) and same_bits(got[3], ref[3])
    raw = run_gpu(backend, ratio, hd, overlap, 0, tk, ts, case["ape"], kv, score)
    check_rows(raw[0], oracle.compressor_chunk(ratio, hd, overlap, 0, case["token_kv"], case["token_score"],
                                               case["ape"], kv, score)[0], False)


def test_random_geometries_positions_and_chunk_lengths(backend, oracle):
    """The next-state arithmetic (which row the serial process wrote to a slot last) and the row
    sources of an emission (chunk, or the state the chunk started from) over random ratios, widths,
    start positions and chunk lengths, empty chunks and chunks shorter than a group included."""
    rng = np.random.default_rng(2026)
    for trial in range(40):
        ratio = int(rng.choice([2, 3, 4, 5, 8, 16, 128]))
        hd = int(rng.choice([4, 6, 8, 32, 64, 100, 128]))
        overlap = int(rng.integers(0, 2))
        start = int(rng.integers(0, 3 * ratio + 1))
        length = int(rng.choice([0, 1, ratio - 1, ratio, ratio + 1, 2 * ratio, int(rng.integers(0, 4 * ratio + 2))]))
        case = build(3000 + trial, ratio, hd, overlap, (start + length,))
        kv, score = case["state"]
        head = oracle.compressor_chunk(ratio, hd, overlap, 0, case["token_kv"][:start], case["token_score"][:start],
                                       case["ape"], kv, score)
        tk, ts = case["token_kv"][start:], case["token_score"][start:]
        ref = oracle.compressor_chunk(ratio, hd, overlap, start, tk, ts, case["ape"], head[2], head[3])
        if length == 0:
            tk = ts = np.zeros((0, case["token_kv"].shape[1]), np.float32)
        got = run_gpu(backend, ratio, hd, overlap, start, tk, ts, case["ape"], head[2], head[3])
        label = (trial, ratio, hd, overlap, start, length)
        assert got[4] == 0, label
        assert np.array_equal(got[1], ref[1]), label
        assert same_bits(got[2], ref[2]) and same_bits(got[3], ref[3]), label
        check_rows(got[0], ref[0], False)


def test_refusals_and_status(backend):
    ratio, hd = 4, 64
    kv, score = compressor_initial_state(ratio, hd, 0)
    tk = np.ones((ratio, hd), np.float32)
    ape = np.zeros((ratio, hd), np.float32)
    assert run_gpu(backend, ratio, hd, 0, 0, tk, tk, ape, kv, score, expect_rc=abi.YVEX_ERR_INVALID_ARG, alias=True) is None
    assert run_gpu(backend, ratio, 63, 0, 0, tk, tk, ape, kv, score, expect_rc=abi.YVEX_ERR_UNSUPPORTED) is None
    assert run_gpu(backend, ratio, hd, 1, 0, tk, tk, ape, kv, score, expect_rc=abi.YVEX_ERR_FORMAT) is None  # rows too narrow
    bad = tk.copy()
    bad[2, 5] = np.inf
    assert run_gpu(backend, ratio, hd, 0, 0, bad, tk, ape, kv, score)[4] == 1
    assert run_gpu(backend, ratio, hd, 0, 0, tk, bad, ape, kv, score)[4] == 1
    assert run_gpu(backend, ratio, hd, 0, 0, tk[:2], bad[:2] * 0 + np.nan, ape, kv, score)[4] == 1  # caught by the state copy
    none = run_gpu(backend, ratio, hd, 0, 0, tk[:0], tk[:0], ape, kv, score)
    assert none[4] == 0 and len(none[1]) == 0 and same_bits(none[2], kv)


def ptr(tensor):
    return C.cast(tensor.ptr, C.c_void_p) if tensor is not None else None


def test_operator_entry(backend, oracle):
    kind, ratio, hd, overlap, rope, policy, chunks = CASES[1]
    case = build(901, ratio, hd, overlap, (11,))
    freq = oracle.rope_frequencies(PositionPolicy(*policy), rope)
    kv, score = case["state"]
    ref = oracle.compressor_chunk(ratio, hd, overlap, 0, case["token_kv"], case["token_score"], case["ape"], kv, score,
                                  case["norm"], 1e-6, rope, freq)
    t = dict(kv=backend.tensor("kv", case["token_kv"]), score=backend.tensor("sc", case["token_score"]),
             ape=backend.tensor("ape", case["ape"]), skv=backend.tensor("skv", kv), ssc=backend.tensor("ssc", score),
             akv=backend.alloc("akv", abi.DTYPE_F32, kv.shape), asc=backend.alloc("asc", abi.DTYPE_F32, kv.shape),
             norm=backend.tensor("norm", case["norm"]), freq=backend.tensor("freq", freq, dtype=abi.DTYPE_F64),
             rows=backend.alloc("rows", abi.DTYPE_F32, (2, hd)), positions=backend.alloc("pos", abi.DTYPE_I64, (2,)))
    r = abi.AttentionCompressRequest()
    r.kind, r.attention_class, r.token_position, r.token_count = 2, 1, 0, 11
    r.compression_ratio, r.head_dimension = ratio, hd
    r.token_kv, r.token_score, r.token_stride = ptr(t["kv"]), ptr(t["score"]), 2 * hd
    r.position_rows, r.state_kv, r.state_score = ptr(t["ape"]), ptr(t["skv"]), ptr(t["ssc"])
    r.next_state_kv, r.next_state_score = ptr(t["akv"]), ptr(t["asc"])
    r.norm_weights, r.rms_norm_epsilon, r.rope_dimension, r.rope_frequency = ptr(t["norm"]), 1e-6, rope, ptr(t["freq"])
    r.compressed, r.compressed_positions = ptr(t["rows"]), ptr(t["positions"])
    failure, facts, err = abi.AttentionFailure(), abi.OperationFacts(), abi.Error()
    call = lambda: backend.lib.yvex_b200_attention_compress_execute(backend.handle, C.byref(r), C.byref(failure),
                                                                    C.byref(facts), C.byref(err))
    assert call() == 0, err.message
    assert r.emitted == 2 and facts.kernel_launches == 1 and failure.code == 0
    check_rows(t["rows"].read(), ref[0], True)
    assert np.array_equal(t["positions"].read().view(np.uint64), ref[1])
    assert same_bits(t["akv"].read(), ref[2]) and same_bits(t["asc"].read(), ref[3])
    # index rows exist for the sparse class only; the dense compressed class has one half
    r.attention_class = 2
    assert call() == abi.YVEX_ERR_UNSUPPORTED and failure.stage == b"compress"
    r.attention_class, r.token_stride = 1, hd
    assert call() == abi.YVEX_ERR_INVALID_ARG
    r.token_stride, r.next_state_kv = 2 * hd, ptr(t["skv"])
    assert call() == abi.YVEX_ERR_INVALID_ARG
