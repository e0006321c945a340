"""A pooled session serialised to the reference's state-bank layout ([values, positions,
auxiliary] at 8-byte aligned offsets; values = F32 rows [row][K heads | V heads], positions
u64) and restored into another pool: every byte of the bank against a host-built
expectation, and the restored pool rows against the originals. Bit-exact."""
import ctypes as C

import numpy as np
import pytest

import clori_b200
from clori_b200 import abi

pytestmark = pytest.mark.gpu


def test_pool_session_round_trips_through_the_reference_bank_layout(backend, library):
    rng = np.random.default_rng(31)
    sessions, kv_heads, hd, block, capacity = 3, 2, 64, 16, 100
    lengths = np.array([100, 37, 64], np.int32)
    width = kv_heads * hd
    blocks_per = (capacity + block - 1) // block
    pool_blocks = sessions * blocks_per + 5
    table = rng.permutation(pool_blocks)[:sessions * blocks_per].astype(np.int32).reshape(sessions, blocks_per)
    kpool = clori_b200.f32_to_bf16_bits(rng.standard_normal((pool_blocks, block, width)).astype(np.float32))
    vpool = clori_b200.f32_to_bf16_bits(rng.standard_normal((pool_blocks, block, width)).astype(np.float32))
    component = (abi.KvBankComponent * 1)(abi.KvBankComponent(1, capacity, 2 * width + 6, 0, 0))   # a padded row
    span, total = (abi.KvBankSpan * 1)(), abi.u64()
    assert library.yvex_b200_kv_bank_layout(component, 1, span, C.byref(total)) == 1
    bank_bytes = (total.value + 255) & ~255
    bank = backend.tensor("bank", np.full(sessions * bank_bytes, 0xAB, np.uint8).view(np.int8), dtype=abi.DTYPE_I8)
    t = dict(k=backend.tensor("k", kpool, dtype=abi.DTYPE_BF16), v=backend.tensor("v", vpool, dtype=abi.DTYPE_BF16),
             table=backend.tensor("table", table), lens=backend.tensor("lens", lengths),
             status=backend.tensor("status", np.zeros(1, np.int32)))

    def args(kp, vp, tab):
        a = abi.KvBankArgs()
        a.sessions, a.kv_heads, a.head_dim, a.kv_tokens, a.row_capacity = sessions, kv_heads, hd, t["lens"].data_ptr, capacity
        a.bank, a.bank_session_bytes = bank.data_ptr, bank_bytes
        a.values_offset, a.positions_offset, a.value_width = span[0].offset[0], span[0].offset[1], 2 * width + 6
        a.position_base = 1000
        a.key_pool, a.value_pool, a.block_table = kp.data_ptr, vp.data_ptr, tab.data_ptr
        a.block_tokens, a.block_table_stride, a.pool_blocks = block, blocks_per, pool_blocks
        a.pool_token_stride, a.pool_head_stride, a.pool_block_stride = width, hd, block * width
        a.status = t["status"].data_ptr
        return a

    a = args(t["k"], t["v"], t["table"])
    assert library.yvx_cuda_kv_bank_transfer(C.byref(a), 1, backend.stream) == 0, library.yvx_cuda_last_error_text()
    assert library.yvx_cuda_stream_synchronize(backend.stream) == 0
    bank.struct.is_written = 1
    got = bank.read().view(np.uint8).reshape(sessions, bank_bytes)
    f = clori_b200.bf16_bits_to_f32
    for s in range(sessions):
        expect = np.full(bank_bytes, 0xAB, np.uint8)
        values = expect[span[0].offset[0]:span[0].offset[0] + span[0].bytes[0]].view(np.float32).reshape(capacity, 2 * width + 6)
        positions = expect[span[0].offset[1]:span[0].offset[1] + span[0].bytes[1]].view(np.uint64)
        for row in range(lengths[s]):
            blk, within = table[s, row // block], row % block
            values[row, :width], values[row, width:2 * width] = f(kpool[blk, within]), f(vpool[blk, within])
            positions[row] = 1000 + row
        assert np.array_equal(got[s], expect), s          # rows beyond the length and the padding are untouched
    # restore into empty pools behind another table
    table2 = rng.permutation(pool_blocks)[:sessions * blocks_per].astype(np.int32).reshape(sessions, blocks_per)
    k2 = backend.tensor("k2", np.zeros_like(kpool), dtype=abi.DTYPE_BF16)
    v2 = backend.tensor("v2", np.zeros_like(vpool), dtype=abi.DTYPE_BF16)
    tab2 = backend.tensor("table2", table2)
    b = args(k2, v2, tab2)
    assert library.yvx_cuda_kv_bank_transfer(C.byref(b), 0, backend.stream) == 0
    assert library.yvx_cuda_stream_synchronize(backend.stream) == 0
    k2.struct.is_written = v2.struct.is_written = 1
    rk, rv = k2.read(np.uint16).reshape(kpool.shape), v2.read(np.uint16).reshape(vpool.shape)
    for s in range(sessions):
        for row in range(lengths[s]):
            src, dst = (table[s, row // block], row % block), (table2[s, row // block], row % block)
            assert np.array_equal(rk[dst], kpool[src]) and np.array_equal(rv[dst], vpool[src])
    assert int(t["status"].read()[0]) == 0
    # a bank value bf16 cannot hold is reported when it is restored
    poisoned = bank.read().view(np.uint8).copy()
    poisoned[span[0].offset[0]:span[0].offset[0] + 4] = np.array([0.3], np.float32).view(np.uint8)
    bank.write(poisoned.view(np.int8))
    assert library.yvx_cuda_kv_bank_transfer(C.byref(b), 0, backend.stream) == 0
    assert library.yvx_cuda_stream_synchronize(backend.stream) == 0
    assert int(t["status"].read()[0]) == 2
