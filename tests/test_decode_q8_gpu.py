"""Decode / speculative verify over a Q8_0 KV cache on a B200 against the CPU
oracle: KV dequantised with the reference's Q8_0 codec (x = f16(d) * int8),
then the reference's CPU attention. Tolerance: max-abs <= 2e-3, cosine >= 0.9999.
Also checks the device pack kernel against the layout definition byte for byte."""
import ctypes as C

import numpy as np
import pytest

import clori_b200
from clori_b200 import abi, q8_records, workloads

pytestmark = pytest.mark.gpu
HD = 128


def dequant(oracle, rows, tokens, width):
    return oracle.q8_0_decode_rows(rows, tokens * width).reshape(tokens, width)


def device_pack(backend, k_rows, v_rows, hkv, table, pool_blocks):
    records = backend.alloc("records", abi.DTYPE_I8, (pool_blocks, hkv, q8_records.RECORD_BYTES))
    assert backend.lib.yvx_cuda_memset_async(records.data_ptr, 0, records.nbytes, backend.stream) == 0
    tk, tv = backend.tensor("krows", k_rows.view(np.int8)), backend.tensor("vrows", v_rows.view(np.int8))
    ids = backend.tensor("ids", table) if table is not None else None
    rc = backend.lib.yvx_cuda_q8_kv_pack(tk.data_ptr, tv.data_ptr, k_rows.shape[0], hkv, records.data_ptr,
                                         ids.data_ptr if ids else None, hkv * q8_records.RECORD_BYTES,
                                         q8_records.RECORD_BYTES, 0, backend.stream)
    assert rc == 0 and backend.lib.yvx_cuda_stream_synchronize(backend.stream) == 0
    records.struct.is_written = 1
    return records


def cosine(a, b):
    a, b = a.astype(np.float64).ravel(), b.astype(np.float64).ravel()
    return float(a @ b / np.sqrt((a @ a) * (b @ b)))


def test_pack_kernel_matches_layout_definition(backend, oracle):
    k_rows, v_rows = workloads.q8_0_kv(seed=3, kv_tokens=200, kv_heads=8)
    table = np.array([3, 1, 0, 5], np.int32)
    records = device_pack(backend, k_rows, v_rows, 8, table, 6)
    want = q8_records.pack_records(k_rows, v_rows, 8, table, 6)
    assert np.array_equal(records.read(np.uint8), want)


@pytest.mark.parametrize("rows,tokens", [(4, 5000), (1, 64), (1, 65), (8, 1000), (2, 63)])
def test_single_session_verify_rows(backend, oracle, rows, tokens):
    # BASELINE config 4 scaled down in KV length only: 32 query / 8 KV heads,
    # int8 lanes uniform in [-127,127], f16 scales ~ U(0.002, 0.02).
    hq, hkv = 32, 8
    k_rows, v_rows = workloads.q8_0_kv(seed=3, kv_tokens=tokens, kv_heads=hkv)
    q = workloads.verify_queries_bf16(seed=3, rows=rows, query_heads=hq)
    records = device_pack(backend, k_rows, v_rows, hkv, None, (tokens + 63) // 64)
    r = clori_b200.attention_requirement(rows, tokens, 0, hq, hkv, HD, dtype=abi.DTYPE_Q8_0,
                                         query_dtype=abi.DTYPE_BF16, output_dtype=abi.DTYPE_F32,
                                         numeric_contract=abi.NUMERIC_Q8_0_KV_F32_ACCUMULATE)
    out = backend.alloc("o", abi.DTYPE_F32, (1, rows, hq * HD))
    rc, facts = backend.attention_batch_execute(r, backend.tensor("q", q[None]), records, records,
                                                backend.tensor("l", np.array([tokens], np.int32)), out)
    assert rc == 0
    kf, vf = dequant(oracle, k_rows, tokens, hkv * HD), dequant(oracle, v_rows, tokens, hkv * HD)
    ref = oracle.gqa_attention(clori_b200.bf16_bits_to_f32(q), kf, vf, tokens - rows, hq, hkv, HD, threads=8)
    got = out.read()[0]
    assert np.abs(got - ref).max() <= 2e-3
    assert cosine(got, ref) >= 0.9999


def test_block_table_batch_with_garbage_in_unused_slots(backend, oracle):
    hq, hkv, rows = 40, 8, 1
    rng = np.random.default_rng(8)
    lengths = np.array([70, 64, 300, 1], np.int32)
    blocks = (lengths + 63) // 64
    pool_blocks = int(blocks.sum()) + 1
    order = rng.permutation(pool_blocks).astype(np.int32)
    table = np.full((len(lengths), int(blocks.max())), -1, np.int32)
    pool = np.zeros((pool_blocks, hkv, q8_records.RECORD_BYTES), np.uint8)
    cursor, host_kv = 0, []
    for s, n in enumerate(lengths):
        table[s, :blocks[s]] = order[cursor:cursor + blocks[s]]
        cursor += blocks[s]
        k_rows, v_rows = workloads.q8_0_kv(seed=20 + s, kv_tokens=int(n), kv_heads=hkv)
        host_kv.append((k_rows, v_rows))
        # unused slots of the session's last block: NaN / Inf scale patterns and noise
        noise = rng.integers(0, 256, size=(pool_blocks, hkv, q8_records.RECORD_BYTES)).astype(np.uint8)
        packed = q8_records.pack_records(k_rows, v_rows, hkv, table[s], pool_blocks)
        used = q8_records.pack_records(np.full_like(k_rows, 255), np.full_like(v_rows, 255), hkv, table[s], pool_blocks) != 0
        for j in table[s, :blocks[s]]:
            pool[j] = np.where(used[j], packed[j], noise[j])
            _, _, ks, vs = q8_records.record_offsets()
            tail = int(n) - (int(n) - 1) // 64 * 64 if j == table[s, blocks[s] - 1] else 64
            for off in (ks[tail:], vs[tail:]):
                pool[j][:, off.ravel()] = 0x00
                pool[j][:, off.ravel() + 1] = 0x7C  # +Inf in f16
    q = clori_b200.f32_to_bf16_bits(rng.standard_normal((len(lengths), rows, hq * HD)).astype(np.float32))
    r = clori_b200.attention_requirement(rows, int(lengths.max()), 0, hq, hkv, HD, dtype=abi.DTYPE_Q8_0,
                                         query_dtype=abi.DTYPE_BF16, output_dtype=abi.DTYPE_BF16,
                                         numeric_contract=abi.NUMERIC_Q8_0_KV_F32_ACCUMULATE)
    records = backend.tensor("records", pool.view(np.int8))
    out = backend.alloc("o", abi.DTYPE_BF16, (len(lengths), rows, hq * HD))
    rc, _ = backend.attention_batch_execute(r, backend.tensor("q", q), records, records,
                                            backend.tensor("l", lengths), out,
                                            block_table=backend.tensor("t", table), block_tokens=64,
                                            max_blocks_per_session=table.shape[1])
    assert rc == 0
    got = clori_b200.bf16_bits_to_f32(out.read())
    for s, n in enumerate(lengths):
        kf = dequant(oracle, host_kv[s][0], int(n), hkv * HD)
        vf = dequant(oracle, host_kv[s][1], int(n), hkv * HD)
        ref = oracle.gqa_attention(clori_b200.bf16_bits_to_f32(q[s]), kf, vf, int(n) - rows, hq, hkv, HD)
        assert np.all(np.abs(got[s] - ref) <= 2e-3 + 2.0 ** -8 * np.abs(ref))
        assert cosine(got[s], ref) >= 0.9999


def test_q8_contract_refusals(backend):
    hq, hkv = 32, 8
    records = backend.tensor("records", np.zeros((1, hkv, q8_records.RECORD_BYTES), np.int8))
    q = backend.tensor("q", np.zeros((1, 1, hq * HD), np.uint16))
    lens = backend.tensor("l", np.array([10], np.int32))
    out = backend.alloc("o", abi.DTYPE_F32, (1, 1, hq * HD))

    def call(**changes):
        r = clori_b200.attention_requirement(1, 10, 0, hq, hkv, HD, dtype=abi.DTYPE_Q8_0,
                                             query_dtype=abi.DTYPE_BF16, output_dtype=abi.DTYPE_F32,
                                             numeric_contract=abi.NUMERIC_Q8_0_KV_F32_ACCUMULATE)
        for k, v in changes.items():
            setattr(r, k, v)
        return backend.attention_batch_execute(r, q, records, records, lens, out, check=False)[0]
    assert call() == 0
    assert call(head_dimension=64) in (abi.YVEX_ERR_UNSUPPORTED, abi.YVEX_ERR_INVALID_ARG)
    assert call(query_dtype=abi.DTYPE_F32) == abi.YVEX_ERR_UNSUPPORTED
    assert call(key_value_tokens=100) == abi.YVEX_ERR_FORMAT  # records smaller than declared


def test_sequence_sharded_q8_partials_combine_to_the_whole(backend, oracle):
    # The KV sequence split into 3 block-aligned shards (as on 3 GPUs): each shard
    # emits (o, m, l) with its absolute base position, the gathered [shard][item]
    # buffer is folded by the strided LSE combine, and the result equals attention
    # over the whole sequence.
    hq, hkv, rows, tokens, shards = 32, 8, 4, 64 * 23 + 17, 3
    k_rows, v_rows = workloads.q8_0_kv(seed=9, kv_tokens=tokens, kv_heads=hkv)
    q = workloads.verify_queries_bf16(seed=9, rows=rows, query_heads=hq)
    blocks = (tokens + 63) // 64
    records = device_pack(backend, k_rows, v_rows, hkv, None, blocks)
    tq = backend.tensor("q", q)
    status = backend.tensor("status", np.zeros(1, np.int32))
    items = rows * hq
    gathered = backend.alloc("gathered", abi.DTYPE_F32, (shards, items, HD + 2))
    lib = backend.lib
    record = q8_records.RECORD_BYTES
    for g in range(shards):
        lo, hi = abi.u64(), abi.u64()
        assert lib.yvex_b200_kv_sequence_shard(tokens, shards, g, 64, C.byref(lo), C.byref(hi))
        p = abi.GqaProblem()
        p.sessions, p.query_rows, p.query_heads, p.kv_heads, p.head_dim = 1, rows, hq, hkv, HD
        p.causal, p.scale = 1, 1.0 / np.sqrt(HD)
        p.query_dtype, p.kv_dtype, p.output_dtype = abi.DTYPE_BF16, abi.DTYPE_Q8_0, abi.DTYPE_F32
        p.query, p.query_row_stride, p.query_session_stride = tq.data_ptr, hq * HD, rows * hq * HD
        p.key = records.data_ptr + (lo.value // 64) * hkv * record
        p.key_head_stride, p.key_block_stride, p.block_tokens = record, hkv * record, 64
        p.kv_tokens_uniform = p.kv_tokens_max = hi.value - lo.value
        p.query_start_uniform, p.kv_position_base = tokens - rows, lo.value
        p.partial_output = gathered.data_ptr + g * items * (HD + 2) * 4
        p.chunk_tokens, p.max_splits = 256, (hi.value - lo.value + 255) // 256
        scratch = backend.alloc("scratch", abi.DTYPE_F32, (1,), max(lib.yvx_cuda_gqa_partials_bytes(C.byref(p)), 16))
        p.partials, p.status = scratch.data_ptr, status.data_ptr
        n = C.c_uint()
        assert lib.yvx_cuda_gqa_attention(C.byref(p), backend.stream, C.byref(n)) == 0
    out = backend.alloc("out", abi.DTYPE_F32, (rows, hq * HD))
    rc = lib.yvx_cuda_lse_combine_strided(gathered.data_ptr, items, shards, HD, HD + 2, items * (HD + 2),
                                          out.data_ptr, abi.DTYPE_F32, status.data_ptr, backend.stream)
    assert rc == 0 and lib.yvx_cuda_stream_synchronize(backend.stream) == 0
    out.struct.is_written = 1
    assert int(status.read()[0]) == 0
    kf, vf = dequant(oracle, k_rows, tokens, hkv * HD), dequant(oracle, v_rows, tokens, hkv * HD)
    ref = oracle.gqa_attention(clori_b200.bf16_bits_to_f32(q), kf, vf, tokens - rows, hq, hkv, HD, threads=8)
    got = out.read()
    assert np.abs(got - ref).max() <= 2e-3
    assert cosine(got, ref) >= 0.9999


@pytest.mark.parametrize("tokens,chunk", [(64 * 23 + 17, 256), (8192, 512), (8192, 64), (100, 0)])
def test_one_launch_step_folds_and_exchanges_in_the_kernel_tail(backend, oracle, tokens, chunk):
    # The whole step (attention, fold of the splits, exchange, fold of the ranks) in ONE
    # cooperative launch, here with a single rank: the exchange area is this GPU's own, so every
    # wait is satisfied by the launch itself. Three epochs over the same area; the result equals
    # the CPU attention and repeats bit for bit.
    hq, hkv, rows = 32, 8, 4
    k_rows, v_rows = workloads.q8_0_kv(seed=10, kv_tokens=tokens, kv_heads=hkv)
    q = workloads.verify_queries_bf16(seed=10, rows=rows, query_heads=hq)
    blocks = (tokens + 63) // 64
    records = device_pack(backend, k_rows, v_rows, hkv, None, blocks)
    tq = backend.tensor("q", q)
    status = backend.tensor("status", np.zeros(1, np.int32))
    lib, items, record = backend.lib, rows * hq, q8_records.RECORD_BYTES
    area_bytes = lib.yvx_cuda_lse_exchange_bytes(1, items, HD)
    counter_offset = lib.yvx_cuda_lse_exchange_counter_offset(1, items, HD)
    area = backend.tensor("area", np.zeros(area_bytes // 4, np.int32))
    gather = backend.tensor("gather", np.array([area.data_ptr], np.int64), dtype=abi.DTYPE_I64)
    arrivals = backend.tensor("arrivals", np.array([area.data_ptr + counter_offset], np.int64), dtype=abi.DTYPE_I64)
    mine = backend.alloc("mine", abi.DTYPE_F32, (items, HD + 2))
    out = backend.alloc("out", abi.DTYPE_F32, (rows, hq * HD))
    p = abi.GqaProblem()
    p.sessions, p.query_rows, p.query_heads, p.kv_heads, p.head_dim = 1, rows, hq, hkv, HD
    p.causal, p.scale = 1, 1.0 / np.sqrt(HD)
    p.query_dtype, p.kv_dtype, p.output_dtype = abi.DTYPE_BF16, abi.DTYPE_Q8_0, abi.DTYPE_F32
    p.query, p.query_row_stride, p.query_session_stride = tq.data_ptr, hq * HD, rows * hq * HD
    p.key = records.data_ptr
    p.key_head_stride, p.key_block_stride, p.block_tokens = record, hkv * record, 64
    p.kv_tokens_uniform = p.kv_tokens_max = tokens
    p.query_start_uniform = tokens - rows
    p.partial_output, p.output = mine.data_ptr, out.data_ptr
    lib.yvx_cuda_gqa_plan_splits(C.byref(p), backend.sm_count)
    if chunk:
        p.chunk_tokens, p.max_splits = chunk, (tokens + chunk - 1) // chunk
    scratch = backend.alloc("scratch", abi.DTYPE_F32, (1,), max(lib.yvx_cuda_gqa_partials_bytes(C.byref(p)), 16))
    p.partials, p.status = scratch.data_ptr, status.data_ptr
    x = abi.LseExchange()
    x.ranks, x.rank, x.gather, x.arrivals, x.one_launch = 1, 0, gather.data_ptr, arrivals.data_ptr, 1
    results = []
    for epoch in (1, 2, 3):
        x.epoch = epoch
        n = C.c_uint()
        rc = lib.yvx_cuda_gqa_attention_exchange(C.byref(p), C.byref(x), backend.stream, C.byref(n))
        assert rc == 0, lib.yvx_cuda_last_error_text()
        assert lib.yvx_cuda_stream_synchronize(backend.stream) == 0, lib.yvx_cuda_last_error_text()
        # 8192 tokens in 64-token splits are 1024 CTAs, more than are resident at once: that plan
        # silently takes the two-launch path; every other case here is a single launch
        assert n.value == (2 if chunk == 64 else 1)
        out.struct.is_written = 1
        results.append(out.read().copy())
        assert int(status.read()[0]) == 0
    assert np.array_equal(results[0], results[1]) and np.array_equal(results[0], results[2])
    kf, vf = dequant(oracle, k_rows, tokens, hkv * HD), dequant(oracle, v_rows, tokens, hkv * HD)
    ref = oracle.gqa_attention(clori_b200.bf16_bits_to_f32(q), kf, vf, tokens - rows, hq, hkv, HD, threads=8)
    assert np.abs(results[0] - ref).max() <= 2e-3 and cosine(results[0], ref) >= 0.9999
    counters = area.read()[counter_offset // 4: counter_offset // 4 + items]
    assert counters.tolist() == [3] * items
    if chunk == 64:
        return
    # an epoch the tickets cannot reach runs into the bounded wait instead of hanging
    x.epoch = 9
    rc = lib.yvx_cuda_gqa_attention_exchange(C.byref(p), C.byref(x), backend.stream, C.byref(n))
    assert rc == 0 and lib.yvx_cuda_stream_synchronize(backend.stream) == 0
    assert int(status.read()[0]) == 3
