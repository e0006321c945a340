"""Parity of batched decode / speculative verify over session KV caches
(block-tabled and contiguous, BF16 and F32) on a B200 against the CPU oracle.
Tolerance for bf16 operands: max-abs <= 2e-3 and cosine >= 0.9999."""
import numpy as np
import pytest

import clori_b200
from clori_b200 import abi, workloads

pytestmark = pytest.mark.gpu


def cosine(a, b):
    a, b = a.astype(np.float64).ravel(), b.astype(np.float64).ravel()
    return float(a @ b / np.sqrt((a @ a) * (b @ b)))


def oracle_batch(oracle, lengths, table, q_bits, kpool, vpool, hq, hkv, hd, rows, block_tokens=64):
    out = np.zeros((len(lengths), rows, hq * hd), np.float32)
    kf = clori_b200.bf16_bits_to_f32(kpool).reshape(-1, hkv * hd)
    vf = clori_b200.bf16_bits_to_f32(vpool).reshape(-1, hkv * hd)
    for s, length in enumerate(lengths):
        idx = np.array([oracle.block_row(table[s], block_tokens, r) for r in range(length)])
        out[s] = oracle.gqa_attention(clori_b200.bf16_bits_to_f32(q_bits[s]), kf[idx], vf[idx],
                                      length - rows, hq, hkv, hd, threads=8)
    return out


@pytest.mark.parametrize("rows,out_dtype", [(1, abi.DTYPE_F32), (4, abi.DTYPE_BF16), (8, abi.DTYPE_F32)])
def test_block_table_decode_and_verify_bf16(backend, oracle, rows, out_dtype):
    # BASELINE config 2 scaled down in token counts only: 40/8 heads, hd 128,
    # 64-token blocks, table = random permutation of a shared pool.
    hq, hkv, hd = 40, 8, 128
    lengths, table, q, kpool, vpool = workloads.batched_decode_bf16(
        seed=1, sessions=12, low=9, high=700, query_heads=hq, kv_heads=hkv, head_dim=hd, rows=rows)
    lengths[0], lengths[1], lengths[2] = max(rows, 9), 64, 65  # ragged edges
    table, pool_blocks = workloads.block_table(lengths, 64, seed=1)
    kpool, vpool = kpool[:pool_blocks + 3], vpool[:pool_blocks + 3]
    if kpool.shape[0] < pool_blocks:
        pytest.skip("pool smaller than table")
    r = clori_b200.attention_requirement(rows, int(lengths.max()), 0, hq, hkv, hd, dtype=abi.DTYPE_BF16,
                                         output_dtype=out_dtype,
                                         numeric_contract=abi.NUMERIC_BF16_F32_ACCUMULATE)
    tq = backend.tensor("q", q)
    tk, tv = backend.tensor("kpool", kpool), backend.tensor("vpool", vpool)
    tl = backend.tensor("lens", lengths)
    tt = backend.tensor("table", table)
    out = backend.alloc("o", out_dtype, (len(lengths), rows, hq * hd))
    rc, facts = backend.attention_batch_execute(r, tq, tk, tv, tl, out, block_table=tt,
                                                block_tokens=64, max_blocks_per_session=table.shape[1])
    assert rc == 0 and facts.kernel_launches >= 1
    got = out.read()
    if out_dtype == abi.DTYPE_BF16:
        got = clori_b200.bf16_bits_to_f32(got)
    ref = oracle_batch(oracle, lengths, table, q, kpool, vpool, hq, hkv, hd, rows)
    tol = 2e-3 if out_dtype == abi.DTYPE_F32 else 2e-3 + 2.0 ** -8 * np.abs(ref)
    assert np.all(np.abs(got - ref) <= tol)
    assert cosine(got, ref) >= 0.9999


def test_block_table_entry_outside_pool_is_refused(backend):
    hq, hkv, hd = 8, 2, 128
    lengths, table, q, kpool, vpool = workloads.batched_decode_bf16(
        seed=3, sessions=3, low=100, high=200, query_heads=hq, kv_heads=hkv, head_dim=hd)
    table = table.copy()
    table[1, 0] = kpool.shape[0] + 7
    r = clori_b200.attention_requirement(1, int(lengths.max()), 0, hq, hkv, hd, dtype=abi.DTYPE_BF16,
                                         output_dtype=abi.DTYPE_F32,
                                         numeric_contract=abi.NUMERIC_BF16_F32_ACCUMULATE)
    t = [backend.tensor(n, a) for n, a in (("q", q), ("k", kpool), ("v", vpool), ("l", lengths), ("t", table))]
    out = backend.alloc("o", abi.DTYPE_F32, (3, 1, hq * hd))
    rc, _ = backend.attention_batch_execute(r, t[0], t[1], t[2], t[3], out, block_table=t[4],
                                            block_tokens=64, max_blocks_per_session=table.shape[1],
                                            check=False)
    assert rc == abi.YVEX_ERR_FORMAT


def test_contiguous_sessions_f32(backend, oracle):
    hq, hkv, hd, rows, cap = 8, 2, 64, 2, 300
    rng = np.random.default_rng(31)
    lengths = np.array([300, 2, 150, 64], np.int32)
    q = rng.standard_normal((4, rows, hq * hd)).astype(np.float32)
    k = rng.standard_normal((4, cap, hkv * hd)).astype(np.float32)
    v = rng.standard_normal((4, cap, hkv * hd)).astype(np.float32)
    r = clori_b200.attention_requirement(rows, cap, 0, hq, hkv, hd)
    t = [backend.tensor(n, a) for n, a in (("q", q), ("k", k), ("v", v), ("l", lengths))]
    out = backend.alloc("o", abi.DTYPE_F32, (4, rows, hq * hd))
    rc, _ = backend.attention_batch_execute(r, t[0], t[1], t[2], t[3], out,
                                            kv_session_stride=cap * hkv * hd)
    assert rc == 0
    got = out.read()
    for s, length in enumerate(lengths):
        ref = oracle.gqa_attention(q[s], k[s, :length], v[s, :length], length - rows, hq, hkv, hd)
        assert np.all(np.abs(got[s] - ref) < 2e-4 * (1 + np.abs(ref)))


def test_batch_refusals(backend):
    hq, hkv, hd = 8, 2, 128
    lengths, table, q, kpool, vpool = workloads.batched_decode_bf16(
        seed=5, sessions=2, low=70, high=90, query_heads=hq, kv_heads=hkv, head_dim=hd)
    t = [backend.tensor(n, a) for n, a in (("q", q), ("k", kpool), ("v", vpool), ("l", lengths), ("t", table))]
    out = backend.alloc("o", abi.DTYPE_F32, (2, 1, hq * hd))

    def call(**changes):
        r = clori_b200.attention_requirement(1, int(lengths.max()), 0, hq, hkv, hd, dtype=abi.DTYPE_BF16,
                                             output_dtype=abi.DTYPE_F32,
                                             numeric_contract=abi.NUMERIC_BF16_F32_ACCUMULATE)
        for key, value in changes.items():
            setattr(r, key, value)
        rc, _ = backend.attention_batch_execute(r, t[0], t[1], t[2], t[3], out, block_table=t[4],
                                                block_tokens=64, max_blocks_per_session=table.shape[1],
                                                check=False)
        return rc
    assert call() == 0
    assert call(query_tokens=10**6) == abi.YVEX_ERR_INVALID_ARG  # more rows than KV tokens
    assert call(query_heads=7) == abi.YVEX_ERR_INVALID_ARG
    assert call(numeric_contract=abi.NUMERIC_EXACT_F32) == abi.YVEX_ERR_UNSUPPORTED
    assert call(deterministic=0) == abi.YVEX_ERR_UNSUPPORTED
    assert call(key_value_tokens=10**6) == abi.YVEX_ERR_INVALID_ARG  # table too short
