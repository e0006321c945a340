"""The tensor-core decode/verify kernel (bf16, head_dim 128) against the CPU
oracle and against the general kernel, over the KV layouts it must read:
token-major rows, interleaved [K|V] rows, head-major blocks, block tables with
64- and 128-token blocks, ragged lengths around every tile and split edge.
Tolerance: max-abs <= 2e-3 and cosine >= 0.9999 (bf16 operands)."""
import numpy as np
import pytest

import clori_b200
from clori_b200 import abi
from gqa_shim import run_problem

pytestmark = pytest.mark.gpu
HD = 128


def bf16(rng, shape, scale=1.0):
    return clori_b200.f32_to_bf16_bits(rng.standard_normal(shape, dtype=np.float32) * np.float32(scale))


def widen(bits):
    return clori_b200.bf16_bits_to_f32(bits)


def check(got, ref):
    assert np.abs(got - ref).max() <= 2e-3, float(np.abs(got - ref).max())
    a, b = got.astype(np.float64).ravel(), ref.astype(np.float64).ravel()
    assert a @ b / np.sqrt((a @ a) * (b @ b)) >= 0.9999


@pytest.mark.parametrize("rows,hq,hkv", [(1, 40, 8), (4, 32, 8), (8, 40, 8), (1, 8, 8), (3, 16, 1)])
@pytest.mark.parametrize("chunk", [None, 64, 256])
def test_contiguous_token_major(backend, oracle, rows, hq, hkv, chunk):
    rng = np.random.Generator(np.random.PCG64(rows * 100 + hq))
    lengths = [rows, 63, 64, 65, 127, 129, 700, 1023, 1024, 1025]
    lengths = [max(n, rows) for n in lengths]
    cap = 1100
    width = hkv * HD
    q = bf16(rng, (len(lengths), rows, hq * HD))
    k = bf16(rng, (len(lengths), cap, width))
    v = bf16(rng, (len(lengths), cap, width))
    kw = dict(q=backend.tensor("q", q), k=backend.tensor("k", k), v=backend.tensor("v", v),
              lengths=lengths, rows=rows, hq=hq, hkv=hkv, hd=HD, dtype=abi.DTYPE_BF16,
              k_token_stride=width, v_token_stride=width, k_head_stride=HD, v_head_stride=HD,
              k_outer_stride=cap * width, v_outer_stride=cap * width, kv_max=cap, chunk_tokens=chunk)
    got, status, launches, plan = run_problem(backend, **kw)
    general, status_g, _, _ = run_problem(backend, force_general=True, **kw)
    assert status == 0 and status_g == 0
    for s, n in enumerate(lengths):
        ref = oracle.gqa_attention(widen(q[s]), widen(k[s, :n]), widen(v[s, :n]), n - rows, hq, hkv, HD, threads=8)
        check(got[s], ref)
        check(general[s], ref)


def test_interleaved_kv_rows_and_full_mask(backend, oracle):
    # The reference's session layout: one row per token holding [K heads | V heads].
    rng = np.random.Generator(np.random.PCG64(7))
    hq, hkv, rows, n = 32, 8, 2, 300
    width = hkv * HD
    q = bf16(rng, (1, rows, hq * HD))
    kv = bf16(rng, (n, 2 * width))
    tkv = backend.tensor("kv", kv)
    for causal in (True, False):
        got, status, _, _ = run_problem(
            backend, q=backend.tensor("q", q), k=tkv, v=tkv, v_offset_elems=width, lengths=[n], rows=rows,
            hq=hq, hkv=hkv, hd=HD, dtype=abi.DTYPE_BF16, causal=causal, k_token_stride=2 * width,
            v_token_stride=2 * width, k_head_stride=HD, v_head_stride=HD, k_outer_stride=0, v_outer_stride=0)
        assert status == 0
        ref = oracle.gqa_attention(widen(q[0]), widen(kv[:, :width]), widen(kv[:, width:]),
                                   n - rows if causal else 0, hq, hkv, HD, causal=causal, threads=8)
        check(got[0], ref)


@pytest.mark.parametrize("block_tokens,head_major", [(64, False), (64, True), (128, False), (128, True)])
def test_block_table_layouts(backend, oracle, block_tokens, head_major):
    rng = np.random.Generator(np.random.PCG64(block_tokens + head_major))
    hq, hkv, rows = 40, 8, 1
    lengths = np.array([1, 64, 65, 500, 2049, 130, 4000], np.int32)
    blocks = (lengths + block_tokens - 1) // block_tokens
    pool_blocks = int(blocks.sum()) + 2
    order = rng.permutation(pool_blocks).astype(np.int32)
    table = np.full((len(lengths), int(blocks.max())), -1, np.int32)
    cursor = 0
    for s, nb in enumerate(blocks):
        table[s, :nb] = order[cursor:cursor + nb]
        cursor += nb
    # logical pool [block][token][head][dim]; the device copy may be head-major.
    kpool = bf16(rng, (pool_blocks, block_tokens, hkv, HD))
    vpool = bf16(rng, (pool_blocks, block_tokens, hkv, HD))
    if head_major:
        kdev, vdev = kpool.transpose(0, 2, 1, 3).copy(), vpool.transpose(0, 2, 1, 3).copy()
        token_stride, head_stride = HD, block_tokens * HD
    else:
        kdev, vdev = kpool, vpool
        token_stride, head_stride = hkv * HD, HD
    q = bf16(rng, (len(lengths), rows, hq * HD))
    got, status, _, _ = run_problem(
        backend, q=backend.tensor("q", q), k=backend.tensor("k", kdev), v=backend.tensor("v", vdev),
        lengths=lengths, rows=rows, hq=hq, hkv=hkv, hd=HD, dtype=abi.DTYPE_BF16, table=table,
        block_tokens=block_tokens, pool_blocks=pool_blocks, k_token_stride=token_stride,
        v_token_stride=token_stride, k_head_stride=head_stride, v_head_stride=head_stride,
        k_outer_stride=block_tokens * hkv * HD, v_outer_stride=block_tokens * hkv * HD)
    assert status == 0
    kflat, vflat = kpool.reshape(-1, hkv * HD), vpool.reshape(-1, hkv * HD)
    for s, n in enumerate(lengths):
        idx = np.array([oracle.block_row(table[s], block_tokens, r) for r in range(n)])
        ref = oracle.gqa_attention(widen(q[s]), widen(kflat[idx]), widen(vflat[idx]), n - rows, hq, hkv, HD, threads=8)
        check(got[s], ref)


def test_unused_rows_of_the_last_block_may_hold_nan(backend, oracle):
    # Rows of a pool block beyond the session's length are never read as data:
    # NaN and Inf bit patterns there must not reach the output.
    rng = np.random.Generator(np.random.PCG64(99))
    hq, hkv, n = 8, 2, 70
    kpool = bf16(rng, (2, 64, hkv * HD))
    vpool = bf16(rng, (2, 64, hkv * HD))
    kpool[1, 6:] = 0x7FC0  # NaN
    vpool[1, 6:] = 0x7F80  # +Inf
    table = np.array([[0, 1]], np.int32)
    q = bf16(rng, (1, 1, hq * HD))
    for general in (False, True):
        got, status, _, _ = run_problem(
            backend, q=backend.tensor("q", q), k=backend.tensor("k", kpool), v=backend.tensor("v", vpool),
            lengths=[n], rows=1, hq=hq, hkv=hkv, hd=HD, dtype=abi.DTYPE_BF16, table=table, pool_blocks=2,
            k_token_stride=hkv * HD, v_token_stride=hkv * HD, k_head_stride=HD, v_head_stride=HD,
            k_outer_stride=64 * hkv * HD, v_outer_stride=64 * hkv * HD, force_general=general)
        assert status == 0
        flat_k, flat_v = kpool.reshape(-1, hkv * HD)[:n], vpool.reshape(-1, hkv * HD)[:n]
        ref = oracle.gqa_attention(widen(q[0]), widen(flat_k), widen(flat_v), n - 1, hq, hkv, HD)
        check(got[0], ref)


def test_peaked_attention_keeps_value_precision(backend, oracle):
    # One key dominates: the output must equal that value row to far better
    # than bf16 precision of the probabilities (P is carried as head + tail).
    rng = np.random.Generator(np.random.PCG64(5))
    hq, hkv, n = 8, 2, 257
    q = bf16(rng, (1, 1, hq * HD))
    k = bf16(rng, (n, hkv * HD), 0.05)
    v = bf16(rng, (n, hkv * HD), 3.0)
    qf = widen(q)[0, 0].reshape(hq, HD)
    for h in range(hkv):  # make token 100 align with the mean query of each group
        k.reshape(n, hkv, HD)[100, h] = clori_b200.f32_to_bf16_bits(qf[h * 4:(h + 1) * 4].mean(axis=0) * 4)
    got, status, _, _ = run_problem(
        backend, q=backend.tensor("q", q), k=backend.tensor("k", k), v=backend.tensor("v", v), lengths=[n],
        rows=1, hq=hq, hkv=hkv, hd=HD, dtype=abi.DTYPE_BF16, k_token_stride=hkv * HD,
        v_token_stride=hkv * HD, k_head_stride=HD, v_head_stride=HD, k_outer_stride=0, v_outer_stride=0)
    ref = oracle.gqa_attention(widen(q[0]), widen(k), widen(v), n - 1, hq, hkv, HD)
    assert status == 0
    assert np.abs(got[0] - ref).max() <= 2e-4


def test_sequence_sharded_partials_combine_to_the_whole(backend, oracle):
    # KV sequence split into 4 contiguous shards (as on 4 GPUs): each shard emits
    # (o, m, l) per (row, head) with its absolute base position; the LSE combine
    # of the gathered partials equals attention over the whole sequence.
    import ctypes as C
    rng = np.random.Generator(np.random.PCG64(21))
    hq, hkv, rows, n, shards = 32, 8, 4, 2048 + 130, 4
    width = hkv * HD
    q = bf16(rng, (1, rows, hq * HD))
    k, v = bf16(rng, (n, width)), bf16(rng, (n, width))
    bounds = [0, 576, 1152, 1728, n]
    parts = []
    for g in range(shards):
        lo, hi = bounds[g], bounds[g + 1]
        out, status, _, _ = run_problem(
            backend, q=backend.tensor("q", q), k=backend.tensor("k", k[lo:hi]), v=backend.tensor("v", v[lo:hi]),
            lengths=[hi - lo], rows=rows, hq=hq, hkv=hkv, hd=HD, dtype=abi.DTYPE_BF16, k_token_stride=width,
            v_token_stride=width, k_head_stride=HD, v_head_stride=HD, k_outer_stride=0, v_outer_stride=0,
            query_start=[n - rows], position_base=lo, partial_output=True)
        assert status == 0
        parts.append(out.reshape(rows * hq, HD + 2))
    gathered = np.stack(parts, axis=1)  # [items][shards][hd+2]
    tparts = backend.tensor("gathered", np.ascontiguousarray(gathered))
    out = backend.alloc("out", abi.DTYPE_F32, (rows, hq * HD))
    status = backend.tensor("st", np.zeros(1, np.int32))
    rc = backend.lib.yvx_cuda_lse_combine(tparts.data_ptr, rows * hq, shards, HD, out.data_ptr,
                                          abi.DTYPE_F32, status.data_ptr, backend.stream)
    assert rc == 0 and backend.lib.yvx_cuda_stream_synchronize(backend.stream) == 0
    out.struct.is_written = 1
    ref = oracle.gqa_attention(widen(q[0]), widen(k), widen(v), n - rows, hq, hkv, HD, threads=8)
    check(out.read(), ref)
    assert int(status.read()[0]) == 0
