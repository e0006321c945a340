"""The pooled KV path end to end on a B200: the block pool hands out blocks, the
append operator rotates and writes new rows through the pool's table, a forked
session shares its parent's prefix and copies the shared partial block on its
first write, rejected candidate rows disappear, and batched attention over the
pool equals the CPU oracle on each session's logical rows (bf16 operands:
max-abs <= 2e-3, cosine >= 0.9999)."""
import ctypes as C

import numpy as np
import pytest

import clori_b200
from clori_b200 import abi

pytestmark = pytest.mark.gpu
HQ, HKV, HD, BLOCK = 8, 2, 128, 64
WIDTH = HKV * HD


class Harness:
    def __init__(self, backend, oracle, blocks=16, sessions=4, per=6):
        self.b, self.lib, self.oracle = backend, backend.lib, oracle
        self.blocks, self.per = blocks, per
        self.pool = self.lib.yvex_b200_kv_pool_create(blocks, BLOCK, sessions, per)
        self.kp = backend.tensor("kp", np.zeros((blocks, BLOCK, WIDTH), np.uint16), dtype=abi.DTYPE_BF16)
        self.vp = backend.tensor("vp", np.zeros((blocks, BLOCK, WIDTH), np.uint16), dtype=abi.DTYPE_BF16)
        self.logical = {}          # session -> (k rows, v rows) as the oracle sees them (bf16-valued f32)
        self.rng = np.random.default_rng(21)

    def table(self, session):
        row = self.lib.yvex_b200_kv_pool_table(self.pool, session)
        return np.array([row[i] for i in range(self.per)], np.int32)

    def append(self, session, rows, accept=None):
        """Reserve `rows` candidates, perform the copy-on-write if asked, append, commit `accept`."""
        lib, b = self.lib, self.b
        copy = abi.KvCopy()
        assert lib.yvex_b200_kv_pool_reserve(self.pool, session, rows, C.byref(copy)) == 0
        if copy.needed:
            nbytes = copy.rows * WIDTH * 2
            for pool in (self.kp, self.vp):
                assert lib.yvx_cuda_copy_async(pool.data_ptr + copy.destination_block * BLOCK * WIDTH * 2,
                                               pool.data_ptr + copy.source_block * BLOCK * WIDTH * 2,
                                               nbytes, b.stream) == 0
        start = int(lib.yvex_b200_kv_pool_committed(self.pool, session))
        k = self.rng.standard_normal((1, rows, WIDTH)).astype(np.float32)
        v = clori_b200.bf16_bits_to_f32(clori_b200.f32_to_bf16_bits(
            self.rng.standard_normal((1, rows, WIDTH)).astype(np.float32)))
        cos, sin = self.oracle.rope_tables(start, rows, HD, 1.0e6)
        t = dict(k=b.tensor("k", k), v=b.tensor("v", v), cos=b.tensor("cos", cos[None]), sin=b.tensor("sin", sin[None]),
                 table=b.tensor("table", self.table(session)[None]))
        r = abi.KvAppendRequest()
        r.session_count, r.token_count = 1, rows
        r.query_heads, r.key_value_heads, r.head_dimension, r.rotary_dimension = 0, HKV, HD, HD
        r.bf16_staged_products = 1
        cast = lambda x: C.cast(x.ptr, C.c_void_p)
        r.key, r.value, r.cosines, r.sines = cast(t["k"]), cast(t["v"]), cast(t["cos"]), cast(t["sin"])
        r.max_kv_tokens = start
        r.key_pool, r.value_pool, r.block_table = cast(self.kp), cast(self.vp), cast(t["table"])
        r.block_tokens, r.max_blocks_per_session, r.pool_blocks = BLOCK, self.per, self.blocks
        facts, err = abi.OperationFacts(), abi.Error()
        rc = lib.yvex_b200_kv_append_rotary_execute(b.handle, C.byref(r), C.byref(facts), C.byref(err))
        assert rc == 0, err.message
        accept = rows if accept is None else accept
        assert lib.yvex_b200_kv_pool_commit(self.pool, session, accept) == 0
        k_rot = self.oracle.rotary_half(k[0], cos, sin, HKV, HD, HD, True)
        old_k, old_v = self.logical.get(session, (np.zeros((0, WIDTH), np.float32),) * 2)
        self.logical[session] = (np.concatenate([old_k, k_rot[:accept]]), np.concatenate([old_v, v[0, :accept]]))
        return copy

    def fork(self, parent):
        child = C.c_uint()
        assert self.lib.yvex_b200_kv_pool_session_fork(self.pool, parent, C.byref(child)) == 0
        self.logical[child.value] = tuple(a.copy() for a in self.logical[parent])
        return child.value

    def check_attention(self, sessions):
        b = self.b
        lengths = np.array([len(self.logical[s][0]) for s in sessions], np.int32)
        q = clori_b200.f32_to_bf16_bits(self.rng.standard_normal((len(sessions), 1, HQ * HD)).astype(np.float32))
        table = np.stack([self.table(s) for s in sessions])
        r = clori_b200.attention_requirement(1, int(lengths.max()), 0, HQ, HKV, HD, dtype=abi.DTYPE_BF16,
                                             output_dtype=abi.DTYPE_F32,
                                             numeric_contract=abi.NUMERIC_BF16_F32_ACCUMULATE)
        out = b.alloc("o", abi.DTYPE_F32, (len(sessions), 1, HQ * HD))
        rc, _ = b.attention_batch_execute(r, b.tensor("q", q), self.kp, self.vp, b.tensor("lens", lengths), out,
                                          block_table=b.tensor("t", table), block_tokens=BLOCK,
                                          max_blocks_per_session=self.per)
        assert rc == 0
        got = out.read()
        for i, s in enumerate(sessions):
            k, v = self.logical[s]
            ref = self.oracle.gqa_attention(clori_b200.bf16_bits_to_f32(q[i]), k, v, len(k) - 1, HQ, HKV, HD, threads=4)
            assert np.abs(got[i] - ref).max() <= 2e-3
            a, c = got[i].astype(np.float64).ravel(), ref.astype(np.float64).ravel()
            assert a @ c / np.sqrt((a @ a) * (c @ c)) >= 0.9999


def test_append_fork_copy_on_write_and_rejection(backend, oracle):
    h = Harness(backend, oracle)
    a = C.c_uint()
    assert h.lib.yvex_b200_kv_pool_session_open(h.pool, C.byref(a)) == 0
    a = a.value
    assert h.append(a, 150).needed == 0                  # prefill-sized append: 3 blocks, the last partial
    h.check_attention([a])
    child = h.fork(a)                                    # shares all three blocks
    assert h.table(child).tolist() == h.table(a).tolist()
    copy = h.append(child, 5)                            # first write: private copy of the 22 shared rows
    assert copy.needed == 1 and copy.rows == 150 % BLOCK
    assert h.table(child)[2] != h.table(a)[2] and h.table(child)[:2].tolist() == h.table(a)[:2].tolist()
    assert h.append(a, 3).needed == 0                    # the parent is the only holder again: in place
    h.check_attention([a, child])
    # speculative verify: 8 candidates appended, 2 accepted; the rest must not be visible
    h.append(child, 8, accept=2)
    h.append(child, 70)                                  # crosses into a new block
    h.check_attention([child, a])
    assert int(h.lib.yvex_b200_kv_pool_committed(h.pool, child)) == 150 + 5 + 2 + 70
    h.lib.yvex_b200_kv_pool_destroy(h.pool)
