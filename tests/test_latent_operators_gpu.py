"""The operator-level entry points for the latent reduce stage, the KV append and
the split-rope latent decode: borrowed device tensors, the reference's refusal
codes and typed failure record, facts, and results that are bit-equal to the
plain-pointer entries they wrap (whose parity the other test files establish)."""
import ctypes as C

import numpy as np
import pytest

import clori_b200
from clori_b200 import abi, workloads
from test_latent_reduce_gpu import build, host_args, run_gpu
from test_mla_gpu import run_mla

pytestmark = pytest.mark.gpu
u64 = np.uint64


def ptr(tensor):
    return C.cast(tensor.ptr, C.c_void_p) if tensor is not None else None


def reduce_request(backend, case, block_visible=0):
    t = {name: backend.tensor(name, case[name]) for name in ("query", "local", "compressed", "sinks")}
    for name in ("local_positions", "compressed_positions", "selected", "selected_count"):
        t[name] = backend.tensor(name, case[name].view(np.int64), dtype=abi.DTYPE_I64)
    t["out"] = backend.alloc("out", abi.DTYPE_F32, (case["tokens"], case["heads"] * case["hd"]))
    r = abi.AttentionReduceRequest()
    r.attention_class, r.token_position, r.token_count = case["cls"], case["start"], case["tokens"]
    r.query_heads, r.head_dimension = case["heads"], case["hd"]
    r.sliding_window, r.compression_ratio, r.indexer_topk = case["window"], case["ratio"], case["topk"]
    r.candidate_block_visible = block_visible
    r.query, r.local, r.local_positions = ptr(t["query"]), ptr(t["local"]), ptr(t["local_positions"])
    r.local_count, r.local_stride = case["initial"], case["local"].shape[1]
    r.compressed, r.compressed_positions = ptr(t["compressed"]), ptr(t["compressed_positions"])
    r.compressed_count, r.compressed_stride = case["compressed"].shape[0], case["hd"]
    r.selected, r.selected_count = ptr(t["selected"]), ptr(t["selected_count"])
    r.sinks, r.output = ptr(t["sinks"]), ptr(t["out"])
    return r, t


@pytest.mark.parametrize("cls", [0, 1, 2])
def test_reduce_operator_equals_the_plain_entry(backend, cls):
    rng = np.random.default_rng(40 + cls)
    case = build(rng, heads=16, hd=512, window=128, attention_class=cls, tokens=3, start=700)
    expect, status = run_gpu(backend, case)
    assert status == 0
    r, t = reduce_request(backend, case)
    failure, facts, err = abi.AttentionFailure(), abi.OperationFacts(), abi.Error()
    rc = backend.lib.yvex_b200_attention_reduce_execute(backend.handle, C.byref(r), C.byref(failure),
                                                        C.byref(facts), C.byref(err))
    assert rc == 0, err.message
    assert failure.code == 0 and facts.kernel_launches == 2 and t["out"].struct.is_written == 1
    assert np.array_equal(t["out"].read(), expect)


def test_reduce_operator_refusals(backend):
    rng = np.random.default_rng(44)
    case = build(rng, heads=4, hd=64, window=128, attention_class=1, tokens=2, start=300)
    lib = backend.lib
    failure, facts, err = abi.AttentionFailure(), abi.OperationFacts(), abi.Error()

    def call(r):
        return lib.yvex_b200_attention_reduce_execute(backend.handle, C.byref(r), C.byref(failure),
                                                      C.byref(facts), C.byref(err))
    r, t = reduce_request(backend, case)
    r.sinks = None
    assert call(r) == abi.YVEX_ERR_INVALID_ARG and failure.code == 1 and failure.stage == b"reduce"
    r, t = reduce_request(backend, case)
    r.head_dimension = 1024
    r.local_stride = 1024
    assert call(r) == abi.YVEX_ERR_UNSUPPORTED and failure.code == 2
    r, t = reduce_request(backend, case)
    r.token_count = 50                      # views too small for 50 tokens
    assert call(r) == abi.YVEX_ERR_FORMAT and failure.code == 1
    r, t = reduce_request(backend, case)
    r.selected = None                       # sparse attention without its lists
    assert call(r) == abi.YVEX_ERR_INVALID_ARG
    # a non-finite sink is a numeric failure reported after the launch
    bad = dict(case)
    bad["sinks"] = np.array([np.nan, 0, 0, 0], np.float32)
    r, t = reduce_request(backend, bad)
    assert call(r) == abi.YVEX_ERR_FORMAT and failure.code == 8 and failure.stage == b"reduce"


def append_request(backend, sessions, tokens, hq, hkv, hd, rotary, lengths, capacity, block=64, query=True):
    rng = np.random.default_rng(sessions + tokens)
    host = dict(q=rng.standard_normal((sessions, tokens, hq * hd)).astype(np.float32),
                k=rng.standard_normal((sessions, tokens, hkv * hd)).astype(np.float32),
                v=rng.standard_normal((sessions, tokens, hkv * hd)).astype(np.float32),
                cos=rng.uniform(-1, 1, (sessions, tokens, rotary)).astype(np.float32),
                sin=rng.uniform(-1, 1, (sessions, tokens, rotary)).astype(np.float32),
                state=np.zeros((sessions, capacity, 2 * hkv * hd), np.float32),
                pos=np.zeros((sessions, capacity), np.int64))
    blocks_per = (capacity + block - 1) // block
    host["table"] = rng.permutation(sessions * blocks_per).reshape(sessions, blocks_per).astype(np.int32)
    host["kp"] = np.zeros((sessions * blocks_per, block, hkv * hd), np.uint16)
    host["vp"] = np.zeros_like(host["kp"])
    host["len"] = np.asarray(lengths, np.int32)
    t = {name: backend.tensor(name, a) for name, a in host.items() if name not in ("pos",)}
    t["pos"] = backend.tensor("pos", host["pos"], dtype=abi.DTYPE_I64)
    r = abi.KvAppendRequest()
    r.session_count, r.token_count = sessions, tokens
    r.query_heads, r.key_value_heads, r.head_dimension, r.rotary_dimension = hq, hkv, hd, rotary
    r.bf16_staged_products = 1
    r.query = ptr(t["q"]) if query else None
    r.key, r.value, r.cosines, r.sines = ptr(t["k"]), ptr(t["v"]), ptr(t["cos"]), ptr(t["sin"])
    r.kv_tokens, r.max_kv_tokens = ptr(t["len"]), int(max(lengths))
    r.state_values, r.state_positions = ptr(t["state"]), ptr(t["pos"])
    r.state_capacity, r.state_row_stride = capacity, 2 * hkv * hd
    r.key_pool, r.value_pool, r.block_table = ptr(t["kp"]), ptr(t["vp"]), ptr(t["table"])
    r.block_tokens, r.max_blocks_per_session, r.pool_blocks = block, blocks_per, sessions * blocks_per
    return r, t, host


def test_append_operator_matches_the_restatement(backend, oracle):
    sessions, tokens, hq, hkv, hd, rotary = 2, 3, 8, 2, 128, 128
    lengths = [5, 70]
    r, t, host = append_request(backend, sessions, tokens, hq, hkv, hd, rotary, lengths, capacity=128)
    facts, err = abi.OperationFacts(), abi.Error()
    rc = backend.lib.yvex_b200_kv_append_rotary_execute(backend.handle, C.byref(r), C.byref(facts), C.byref(err))
    assert rc == 0, err.message
    assert facts.kernel_launches == 1 and facts.d2d_bytes == sessions * tokens * 2 * hkv * hd * (4 + 2)
    state, pos = t["state"].read(), t["pos"].read()
    kp = t["kp"].read()
    for b in range(sessions):
        q_ref = oracle.rotary_half(host["q"][b], host["cos"][b], host["sin"][b], hq, hd, rotary, True)
        k_ref = oracle.rotary_half(host["k"][b], host["cos"][b], host["sin"][b], hkv, hd, rotary, True)
        assert np.array_equal(t["q"].read()[b], q_ref)
        for i in range(tokens):
            row = lengths[b] + i
            assert np.array_equal(state[b, row, :hkv * hd], k_ref[i])
            assert np.array_equal(state[b, row, hkv * hd:], host["v"][b, i])
            assert pos[b, row] == row
            assert np.array_equal(kp[host["table"][b, row // 64], row % 64], clori_b200.f32_to_bf16_bits(k_ref[i]))


def test_append_operator_refusals(backend):
    lib = backend.lib
    facts, err = abi.OperationFacts(), abi.Error()

    def call(r):
        return lib.yvex_b200_kv_append_rotary_execute(backend.handle, C.byref(r), C.byref(facts), C.byref(err))
    r, t, _ = append_request(backend, 1, 2, 4, 2, 128, 128, [126], capacity=128)
    assert call(r) == 0
    r, t, _ = append_request(backend, 1, 3, 4, 2, 128, 128, [126], capacity=128)
    assert call(r) == abi.YVEX_ERR_BOUNDS                      # 126 + 3 rows > 128
    r, t, _ = append_request(backend, 1, 2, 4, 2, 128, 127, [0], capacity=128)
    assert call(r) == abi.YVEX_ERR_INVALID_ARG                 # odd rotary width
    r, t, _ = append_request(backend, 1, 2, 4, 2, 128, 128, [0], capacity=128)
    r.token_count = 9                                          # views hold two rows per session
    assert call(r) == abi.YVEX_ERR_FORMAT
    r, t, _ = append_request(backend, 1, 2, 4, 2, 128, 128, [0], capacity=128)
    r.state_values, r.key_pool = None, None
    assert call(r) == abi.YVEX_ERR_INVALID_ARG


def test_mla_operator_equals_the_plain_entry(backend):
    sessions, context = 2, 300
    qn, qr, w, lat, rk = workloads.mla_decode_bf16(seed=9, batch=sessions, context=context)
    lengths = [context, context - 41]
    scale = 1.0 / np.sqrt(192.0)
    expect, _, status, _, _ = run_mla(backend, qn, qr, w, lat, rk, lengths, scale)
    assert status == 0
    t = {n: backend.tensor(n, a) for n, a in (("qn", qn), ("qr", qr), ("w", w), ("lat", lat), ("rk", rk))}
    t["len"] = backend.tensor("len", np.asarray(lengths, np.int32))
    t["out"] = backend.alloc("out", abi.DTYPE_F32, (sessions, 128, 512))
    r = abi.MlaDecodeRequest()
    r.session_count, r.heads, r.nope_dimension, r.latent_dimension, r.rope_dimension = sessions, 128, 128, 512, 64
    r.context_capacity, r.max_kv_tokens, r.scale = context, context, scale
    r.q_nope, r.q_rope, r.w_uk = ptr(t["qn"]), ptr(t["qr"]), ptr(t["w"])
    r.latent, r.rope_key, r.kv_tokens, r.output = ptr(t["lat"]), ptr(t["rk"]), ptr(t["len"]), ptr(t["out"])
    facts, err = abi.OperationFacts(), abi.Error()
    rc = backend.lib.yvex_b200_mla_decode_execute(backend.handle, C.byref(r), C.byref(facts), C.byref(err))
    assert rc == 0, err.message
    assert facts.kernel_launches == 3 and facts.temporary_bytes > 0
    assert np.array_equal(t["out"].read(), expect)
    r.heads = 64
    assert backend.lib.yvex_b200_mla_decode_execute(backend.handle, C.byref(r), C.byref(facts),
                                                    C.byref(err)) == abi.YVEX_ERR_UNSUPPORTED
    r.heads, r.scale = 128, 0.0
    assert backend.lib.yvex_b200_mla_decode_execute(backend.handle, C.byref(r), C.byref(facts),
                                                    C.byref(err)) == abi.YVEX_ERR_INVALID_ARG
