"""Block-pool bookkeeping (host only): allocation order, shared prefixes after a
fork, copy-on-write of a shared partial block, candidate rows that are rejected,
exhaustion of the pool, the table and the session slots. Index work: exact."""
import ctypes as C

import numpy as np
import pytest

from clori_b200 import abi

OK, INVALID, BOUNDS, NOMEM = 0, abi.YVEX_ERR_INVALID_ARG, -7, -2


@pytest.fixture()
def pool(library):
    handle = library.yvex_b200_kv_pool_create(8, 4, 3, 4)   # 8 blocks of 4 rows, 3 sessions, 4 blocks each
    assert handle
    yield library, handle
    library.yvex_b200_kv_pool_destroy(handle)


def table(lib, handle, session, n=4):
    row = lib.yvex_b200_kv_pool_table(handle, session)
    return [row[i] for i in range(n)]


def test_reserve_commit_and_rejected_candidates(pool):
    lib, h = pool
    s, copy = C.c_uint(), abi.KvCopy()
    assert lib.yvex_b200_kv_pool_session_open(h, C.byref(s)) == OK and s.value == 0
    assert lib.yvex_b200_kv_pool_reserve(h, 0, 6, C.byref(copy)) == OK and copy.needed == 0
    assert table(lib, h, 0) == [0, 1, -1, -1] and lib.yvex_b200_kv_pool_free_blocks(h) == 6
    assert lib.yvex_b200_kv_pool_reserved(h, 0) == 6 and lib.yvex_b200_kv_pool_committed(h, 0) == 0
    # speculative verify: 6 candidates, 3 accepted -> the second block goes back
    assert lib.yvex_b200_kv_pool_commit(h, 0, 3) == OK
    assert lib.yvex_b200_kv_pool_committed(h, 0) == 3 and table(lib, h, 0) == [0, -1, -1, -1]
    assert lib.yvex_b200_kv_pool_free_blocks(h) == 7
    assert lib.yvex_b200_kv_pool_commit(h, 0, 1) == BOUNDS          # nothing reserved any more
    # a second reserve continues in the partial block and takes the freed block again
    assert lib.yvex_b200_kv_pool_reserve(h, 0, 2, C.byref(copy)) == OK and copy.needed == 0
    assert table(lib, h, 0) == [0, 1, -1, -1]
    # reserving again without a commit drops the earlier candidates first
    assert lib.yvex_b200_kv_pool_reserve(h, 0, 1, C.byref(copy)) == OK
    assert table(lib, h, 0) == [0, -1, -1, -1] and lib.yvex_b200_kv_pool_reserved(h, 0) == 4


def test_fork_shares_blocks_and_copies_on_write(pool):
    lib, h = pool
    a, b, copy = C.c_uint(), C.c_uint(), abi.KvCopy()
    assert lib.yvex_b200_kv_pool_session_open(h, C.byref(a)) == OK
    assert lib.yvex_b200_kv_pool_reserve(h, a.value, 6, C.byref(copy)) == OK
    assert lib.yvex_b200_kv_pool_commit(h, a.value, 6) == OK
    assert lib.yvex_b200_kv_pool_session_fork(h, a.value, C.byref(b)) == OK
    assert table(lib, h, b.value) == table(lib, h, a.value) == [0, 1, -1, -1]
    assert lib.yvex_b200_kv_pool_committed(h, b.value) == 6
    assert [lib.yvex_b200_kv_pool_block_refcount(h, i) for i in range(3)] == [2, 2, 0]
    assert lib.yvex_b200_kv_pool_free_blocks(h) == 6
    # the child writes row 6: block 1 is shared and partial -> private copy of its 2 rows
    assert lib.yvex_b200_kv_pool_reserve(h, b.value, 1, C.byref(copy)) == OK
    assert (copy.needed, copy.source_block, copy.destination_block, copy.rows) == (1, 1, 2, 2)
    assert table(lib, h, b.value) == [0, 2, -1, -1] and table(lib, h, a.value) == [0, 1, -1, -1]
    assert [lib.yvex_b200_kv_pool_block_refcount(h, i) for i in range(3)] == [2, 1, 1]
    # the parent is now the only holder of block 1 and writes in place
    assert lib.yvex_b200_kv_pool_reserve(h, a.value, 1, C.byref(copy)) == OK and copy.needed == 0
    # closing the parent keeps the shared block alive for the child
    assert lib.yvex_b200_kv_pool_session_close(h, a.value) == OK
    assert lib.yvex_b200_kv_pool_block_refcount(h, 0) == 1 and lib.yvex_b200_kv_pool_block_refcount(h, 1) == 0
    assert lib.yvex_b200_kv_pool_free_blocks(h) == 6
    # a fork at a block boundary needs no copy
    assert lib.yvex_b200_kv_pool_commit(h, b.value, 1) == OK
    assert lib.yvex_b200_kv_pool_reserve(h, b.value, 1, C.byref(copy)) == OK
    assert lib.yvex_b200_kv_pool_commit(h, b.value, 1) == OK and lib.yvex_b200_kv_pool_committed(h, b.value) == 8
    c = C.c_uint()
    assert lib.yvex_b200_kv_pool_session_fork(h, b.value, C.byref(c)) == OK
    assert lib.yvex_b200_kv_pool_reserve(h, c.value, 1, C.byref(copy)) == OK and copy.needed == 0


def test_exhaustion_and_bad_arguments(pool):
    lib, h = pool
    s, copy = [C.c_uint() for _ in range(4)], abi.KvCopy()
    for i in range(3):
        assert lib.yvex_b200_kv_pool_session_open(h, C.byref(s[i])) == OK
    assert lib.yvex_b200_kv_pool_session_open(h, C.byref(s[3])) == BOUNDS          # session slots
    assert lib.yvex_b200_kv_pool_reserve(h, 0, 17, C.byref(copy)) == BOUNDS        # 5 blocks > table row
    assert lib.yvex_b200_kv_pool_reserve(h, 0, 16, C.byref(copy)) == OK
    assert lib.yvex_b200_kv_pool_reserve(h, 1, 16, C.byref(copy)) == OK
    assert lib.yvex_b200_kv_pool_free_blocks(h) == 0
    assert lib.yvex_b200_kv_pool_reserve(h, 2, 1, C.byref(copy)) == NOMEM          # pool full
    assert lib.yvex_b200_kv_pool_commit(h, 0, 0) == OK                             # reject everything
    assert lib.yvex_b200_kv_pool_free_blocks(h) == 4
    assert lib.yvex_b200_kv_pool_reserve(h, 2, 1, C.byref(copy)) == OK
    assert lib.yvex_b200_kv_pool_reserve(h, 7, 1, C.byref(copy)) == INVALID
    assert lib.yvex_b200_kv_pool_reserve(h, 0, 0, C.byref(copy)) == INVALID
    assert lib.yvex_b200_kv_pool_session_close(h, 2) == OK
    assert lib.yvex_b200_kv_pool_session_close(h, 2) == INVALID
    assert not lib.yvex_b200_kv_pool_create(0, 4, 1, 1)


def test_refused_reserve_forgets_the_candidates_it_released(pool):
    # A reserve that runs out of blocks has already released the session's old candidate
    # blocks; the reserved range must go with them, or a later commit would accept rows
    # whose table entries are -1.
    lib, h = pool
    a, b, copy = C.c_uint(), C.c_uint(), abi.KvCopy()
    assert lib.yvex_b200_kv_pool_session_open(h, C.byref(a)) == OK
    assert lib.yvex_b200_kv_pool_session_open(h, C.byref(b)) == OK
    assert lib.yvex_b200_kv_pool_reserve(h, a.value, 16, C.byref(copy)) == OK      # 4 of 8 blocks
    assert lib.yvex_b200_kv_pool_commit(h, a.value, 16) == OK
    assert lib.yvex_b200_kv_pool_reserve(h, b.value, 8, C.byref(copy)) == OK       # 2 candidate blocks
    free_before = lib.yvex_b200_kv_pool_free_blocks(h)
    assert lib.yvex_b200_kv_pool_session_open(h, C.byref(C.c_uint())) == OK
    assert lib.yvex_b200_kv_pool_reserve(h, 2, 8, C.byref(copy)) == OK             # takes the last 2 blocks
    assert lib.yvex_b200_kv_pool_free_blocks(h) == free_before - 2 == 0
    assert lib.yvex_b200_kv_pool_reserve(h, b.value, 16, C.byref(copy)) == NOMEM   # old candidates released, 4 needed
    assert lib.yvex_b200_kv_pool_commit(h, b.value, 1) == BOUNDS                   # nothing is reserved any more
    assert lib.yvex_b200_kv_pool_committed(h, b.value) == 0
    assert lib.yvex_b200_kv_pool_reserve(h, b.value, 8, C.byref(copy)) == OK       # the released blocks serve again
    assert lib.yvex_b200_kv_pool_commit(h, b.value, 8) == OK


def test_random_walk_keeps_every_row_addressable_and_counts_balanced(library):
    lib = library
    rng = np.random.default_rng(5)
    blocks, bt, sessions, per = 64, 8, 6, 12
    h = lib.yvex_b200_kv_pool_create(blocks, bt, sessions, per)
    live, copy = {}, abi.KvCopy()
    for step in range(2000):
        action = rng.integers(0, 5)
        if action == 0 and len(live) < sessions:
            s = C.c_uint()
            if live and rng.integers(0, 2):
                parent = int(rng.choice(list(live)))
                if lib.yvex_b200_kv_pool_session_fork(h, parent, C.byref(s)) == OK:
                    live[s.value] = live[parent]
            elif lib.yvex_b200_kv_pool_session_open(h, C.byref(s)) == OK:
                live[s.value] = 0
        elif action == 1 and live:
            s = int(rng.choice(list(live)))
            assert lib.yvex_b200_kv_pool_session_close(h, s) == OK
            del live[s]
        elif live:
            s = int(rng.choice(list(live)))
            n = int(rng.integers(1, 9))
            rc = lib.yvex_b200_kv_pool_reserve(h, s, n, C.byref(copy))
            if rc == OK:
                accepted = int(rng.integers(0, n + 1))
                assert lib.yvex_b200_kv_pool_commit(h, s, accepted) == OK
                live[s] += accepted
            else:
                assert rc in (BOUNDS, NOMEM)
        # invariants: every committed row has a block; references add up
        counts = np.zeros(blocks, np.int64)
        for s, rows in live.items():
            assert lib.yvex_b200_kv_pool_committed(h, s) == rows
            row = lib.yvex_b200_kv_pool_table(h, s)
            used = (rows + bt - 1) // bt
            for j in range(per):
                assert (row[j] >= 0) == (j < used)
                if row[j] >= 0:
                    counts[row[j]] += 1
        assert [lib.yvex_b200_kv_pool_block_refcount(h, i) for i in range(blocks)] == counts.tolist()
        assert lib.yvex_b200_kv_pool_free_blocks(h) == int((counts == 0).sum())
    lib.yvex_b200_kv_pool_destroy(h)
