"""KV append with rotary embedding on a B200 against the CPU restatement of the
reference's rotate-half kernels and state append: bit-exact in both arithmetic
variants, both destinations (F32 state rows and bf16 pools behind a block
table), positions exact, plus the reference's two known-answer vectors
(tests/unit/cuda/quant_qtype.c:1989-2062 and :3057-3104), checked
over both destinations."""
import ctypes as C

import numpy as np
import pytest

import clori_b200
from clori_b200 import abi

pytestmark = pytest.mark.gpu


def append(backend, q, k, v, cos, sin, heads, kv_heads, hd, rotary, staged, kv_tokens=None, uniform=0,
           state=None, positions=None, token_position=None, pools=None, row_capacity=0):
    """q/k/v [sessions, tokens, heads*hd] float32. Returns dict of device results."""
    sessions, tokens = k.shape[0], k.shape[1]
    t = dict(k=backend.tensor("k", k), v=backend.tensor("v", v), cos=backend.tensor("cos", cos),
             sin=backend.tensor("sin", sin), status=backend.tensor("status", np.zeros(1, np.int32)))
    a = abi.KvAppendArgs()
    a.sessions, a.tokens, a.query_heads, a.kv_heads, a.head_dim, a.rotary_dim = sessions, tokens, heads, kv_heads, hd, rotary
    a.staged_bf16 = int(staged)
    if q is not None:
        t["q"] = backend.tensor("q", q)
        a.query = t["q"].data_ptr
    a.key, a.value, a.cosines, a.sines = t["k"].data_ptr, t["v"].data_ptr, t["cos"].data_ptr, t["sin"].data_ptr
    if kv_tokens is not None:
        t["len"] = backend.tensor("len", kv_tokens.astype(np.int32))
        a.kv_tokens = t["len"].data_ptr
    a.kv_tokens_uniform = uniform
    if state is not None:
        t["state"] = backend.tensor("state", state)
        a.state_values = t["state"].data_ptr
        a.state_session_stride, a.state_row_stride = state.shape[1] * state.shape[2], state.shape[2]
    if positions is not None:
        t["pos"] = backend.tensor("pos", positions.view(np.int64), dtype=abi.DTYPE_I64)
        a.state_positions, a.state_position_stride = t["pos"].data_ptr, positions.shape[1]
    if token_position is not None:
        t["tp"] = backend.tensor("tp", token_position.view(np.int64), dtype=abi.DTYPE_I64)
        a.token_position = t["tp"].data_ptr
    if pools is not None:
        kp, vp, table, block_tokens = pools
        t["kp"] = backend.tensor("kp", kp, dtype=abi.DTYPE_BF16)
        t["vp"] = backend.tensor("vp", vp, dtype=abi.DTYPE_BF16)
        t["table"] = backend.tensor("table", table.astype(np.int32))
        a.key_pool, a.value_pool, a.block_table = t["kp"].data_ptr, t["vp"].data_ptr, t["table"].data_ptr
        a.block_tokens, a.block_table_stride, a.pool_blocks = block_tokens, table.shape[1], kp.shape[0]
        a.pool_token_stride, a.pool_head_stride, a.pool_block_stride = kv_heads * hd, hd, block_tokens * kv_heads * hd
    a.status = t["status"].data_ptr
    a.row_capacity = row_capacity
    rc = backend.lib.yvx_cuda_kv_append_rotary(C.byref(a), backend.stream)
    assert rc == 0, backend.lib.yvx_cuda_last_error_text()
    assert backend.lib.yvx_cuda_stream_synchronize(backend.stream) == 0
    out = {"status": int(t["status"].read()[0])}
    for name, key in (("q", "q"), ("state", "state")):
        if key in t:
            t[key].struct.is_written = 1
            out[name] = t[key].read()
    if "pos" in t:
        out["positions"] = t["pos"].read(np.int64).view(np.uint64)
    if "kp" in t:
        out["key_pool"], out["value_pool"] = t["kp"].read(np.uint16), t["vp"].read(np.uint16)
    return out


def test_reference_known_answers(backend):
    # bf16-staged variant: tokens 1, heads 1, head_dim 4, rotary 2
    k = np.array([[[-1.34375, -2.0625, 3.0, 4.0]]], np.float32)
    cos = np.full((1, 1, 2), 0.63671875, np.float32)
    sin = np.full((1, 1, 2), 0.546875, np.float32)
    state = np.zeros((1, 2, 8), np.float32)
    got = append(backend, k.copy(), k, k, cos, sin, 1, 1, 4, 2, True, uniform=1, state=state)
    rb = lambda x: np.float32(clori_b200.bf16_bits_to_f32(clori_b200.f32_to_bf16_bits(np.array([x], np.float32)))[0])
    first = rb(rb(np.float32(-1.34375) * np.float32(0.63671875)) - rb(np.float32(-2.0625) * np.float32(0.546875)))
    second = rb(rb(np.float32(-2.0625) * np.float32(0.63671875)) + rb(np.float32(-1.34375) * np.float32(0.546875)))
    expect = np.array([first, second, 3.0, 4.0], np.float32)
    assert got["status"] == 0
    assert np.array_equal(got["q"].reshape(-1), expect)
    assert np.array_equal(got["state"][0, 1, :4], expect) and np.array_equal(got["state"][0, 1, 4:], k.reshape(-1))
    assert not got["state"][0, 0].any()
    # plain variant: tokens 1, heads 2, head_dim 2, rotary 2
    q = np.array([[[1.0, 2.0, 7.0, 8.0]]], np.float32)
    cos = np.full((1, 1, 2), 0.75, np.float32)
    sin = np.full((1, 1, 2), 0.5, np.float32)
    got = append(backend, q, q.copy(), q.copy(), cos, sin, 2, 2, 2, 2, False, uniform=0,
                 state=np.zeros((1, 1, 8), np.float32))
    assert np.array_equal(got["q"].reshape(-1), np.array([-0.25, 2.0, 1.25, 9.5], np.float32))
    assert np.array_equal(got["state"][0, 0, :4], np.array([-0.25, 2.0, 1.25, 9.5], np.float32))


@pytest.mark.parametrize("staged", [True, False])
@pytest.mark.parametrize("tokens,rotary", [(1, 128), (5, 64), (130, 128)])
def test_append_is_bit_exact_in_both_destinations(backend, oracle, staged, tokens, rotary):
    rng = np.random.default_rng(tokens * 7 + rotary + int(staged))
    sessions, hq, hkv, hd, block = 3, 8, 2, 128, 64
    lengths = np.array([0, 77, 191], np.int64)
    capacity = int(lengths.max()) + tokens
    q = rng.standard_normal((sessions, tokens, hq * hd)).astype(np.float32)
    k = rng.standard_normal((sessions, tokens, hkv * hd)).astype(np.float32)
    v = rng.standard_normal((sessions, tokens, hkv * hd)).astype(np.float32)
    cos = np.empty((sessions, tokens, rotary), np.float32)
    sin = np.empty_like(cos)
    for b in range(sessions):
        cos[b], sin[b] = oracle.rope_tables(int(lengths[b]), tokens, rotary, 1.0e6)
    state = rng.standard_normal((sessions, capacity, 2 * hkv * hd)).astype(np.float32)
    positions = np.full((sessions, capacity), 2 ** 63, np.uint64)
    start = np.array([1000, 2000, 3000], np.uint64)
    blocks_per = (capacity + block - 1) // block
    table = rng.permutation(sessions * blocks_per).reshape(sessions, blocks_per)
    kp = rng.integers(0, 2 ** 16, (sessions * blocks_per, block, hkv * hd)).astype(np.uint16)
    vp = rng.integers(0, 2 ** 16, (sessions * blocks_per, block, hkv * hd)).astype(np.uint16)
    got = append(backend, q, k, v, cos, sin, hq, hkv, hd, rotary, staged, kv_tokens=lengths, state=state,
                 positions=positions, token_position=start, pools=(kp, vp, table, block))
    assert got["status"] == 0
    want_state, want_pos, want_kp, want_vp = state.copy(), positions.copy(), kp.copy(), vp.copy()
    for b in range(sessions):
        q_ref = oracle.rotary_half(q[b], cos[b], sin[b], hq, hd, rotary, staged)
        k_ref = oracle.rotary_half(k[b], cos[b], sin[b], hkv, hd, rotary, staged)
        assert np.array_equal(got["q"][b], q_ref)
        for t in range(tokens):
            row = int(lengths[b]) + t
            want_state[b, row, :hkv * hd], want_state[b, row, hkv * hd:] = k_ref[t], v[b, t]
            want_pos[b, row] = start[b] + np.uint64(t)
            pool_block, slot = table[b, row // block], row % block
            want_kp[pool_block, slot] = clori_b200.f32_to_bf16_bits(k_ref[t])
            want_vp[pool_block, slot] = clori_b200.f32_to_bf16_bits(v[b, t])
    assert np.array_equal(got["state"], want_state)
    assert np.array_equal(got["positions"], want_pos)
    assert np.array_equal(got["key_pool"].reshape(kp.shape), want_kp)
    assert np.array_equal(got["value_pool"].reshape(vp.shape), want_vp)


def test_bad_block_table_entry_is_reported_not_followed(backend):
    k = np.ones((1, 1, 128), np.float32)
    cos, sin = np.ones((1, 1, 128), np.float32), np.zeros((1, 1, 128), np.float32)
    kp = np.zeros((2, 64, 128), np.uint16)
    got = append(backend, None, k, k, cos, sin, 0, 1, 128, 128, True, uniform=3,
                 pools=(kp, kp.copy(), np.array([[7]]), 64))
    assert got["status"] == 2 and not got["key_pool"].any()


def test_refusals(backend):
    a = abi.KvAppendArgs()
    assert backend.lib.yvx_cuda_kv_append_rotary(C.byref(a), backend.stream) == abi.YVEX_ERR_INVALID_ARG
    assert backend.lib.yvx_cuda_kv_append_rotary(None, backend.stream) == abi.YVEX_ERR_INVALID_ARG
