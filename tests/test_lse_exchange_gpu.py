"""The cross-GPU fold of split-attention partials, with all ranks played by one
cooperative launch on one GPU (blocks that wait on one another must be
co-resident, so the ranks are never separate launches here): every rank ends up
with the fold of all ranks' rows in rank order, over several epochs reusing the
double-buffered area and the ever-growing arrival counters."""
import ctypes as C

import numpy as np
import pytest

from clori_b200 import abi

pytestmark = pytest.mark.gpu


def fold(rows):
    """rows [ranks, items, hd+2] -> [items, hd] in float64 (reference)."""
    hd = rows.shape[2] - 2
    m, l = rows[:, :, hd].astype(np.float64), rows[:, :, hd + 1].astype(np.float64)
    mm = m.max(axis=0)
    w = np.where(np.isinf(m), 0.0, l * np.exp(m - mm))
    return (rows[:, :, :hd].astype(np.float64) * w[:, :, None]).sum(axis=0) / w.sum(axis=0)[:, None]


@pytest.mark.parametrize("tagged", [0, 1])
@pytest.mark.parametrize("ranks,items,hd", [(2, 16, 128), (4, 128, 128), (8, 40, 64)])
def test_emulated_ranks_fold_each_others_rows(backend, ranks, items, hd, tagged):
    lib, rng = backend.lib, np.random.default_rng(ranks * 100 + items)
    area_bytes = lib.yvx_cuda_lse_exchange_bytes(ranks, items, hd)
    counter_offset = lib.yvx_cuda_lse_exchange_counter_offset(ranks, items, hd)
    areas = [backend.tensor(f"area{r}", np.zeros(area_bytes // 4, np.int32)) for r in range(ranks)]
    gather = backend.tensor("gather", np.array([a.data_ptr for a in areas], np.int64), dtype=abi.DTYPE_I64)
    arrivals = backend.tensor("arrivals", np.array([a.data_ptr + counter_offset for a in areas], np.int64),
                              dtype=abi.DTYPE_I64)
    status = backend.tensor("status", np.zeros(1, np.int32))
    out = backend.alloc("out", abi.DTYPE_F32, (ranks, items, hd))
    for epoch in (1, 2, 3):
        rows = rng.standard_normal((ranks, items, hd + 2)).astype(np.float32)
        rows[:, :, hd + 1] = rng.uniform(0.5, 50.0, (ranks, items)).astype(np.float32)   # l > 0
        if epoch == 2:
            rows[0, :, hd], rows[0, :, hd + 1] = -np.inf, 0.0                            # an empty shard
        t = backend.tensor("rows", rows)
        rc = lib.yvx_cuda_lse_exchange_emulated_form(t.data_ptr, ranks, items, hd, gather.data_ptr, arrivals.data_ptr,
                                                     epoch, out.data_ptr, status.data_ptr, backend.stream, tagged, -1)
        assert rc == 0, lib.yvx_cuda_last_error_text()
        assert lib.yvx_cuda_stream_synchronize(backend.stream) == 0, lib.yvx_cuda_last_error_text()
        out.struct.is_written = 1
        got, ref = out.read(), fold(rows)
        assert int(status.read()[0]) == 0
        for r in range(ranks):
            assert np.abs(got[r] - ref).max() <= 1e-5 * (1.0 + np.abs(ref).max())
            assert np.array_equal(got[r], got[0])          # every rank computes the same bits
    counters = areas[0].read()[counter_offset // 4: counter_offset // 4 + items]
    # the tagged form has no arrival counters on its path
    assert counters.tolist() == ([0] * items if tagged else [3 * ranks] * items)


def test_a_missing_rank_runs_into_the_bounded_wait(backend):
    # Two ranks are launched but the counters are told to expect a third epoch's worth:
    # epoch 2 on fresh counters can never be reached, the wait gives up and reports it.
    lib = backend.lib
    ranks, items, hd = 2, 4, 64
    area_bytes = lib.yvx_cuda_lse_exchange_bytes(ranks, items, hd)
    counter_offset = lib.yvx_cuda_lse_exchange_counter_offset(ranks, items, hd)
    areas = [backend.tensor(f"area{r}", np.zeros(area_bytes // 4, np.int32)) for r in range(ranks)]
    gather = backend.tensor("gather", np.array([a.data_ptr for a in areas], np.int64), dtype=abi.DTYPE_I64)
    arrivals = backend.tensor("arrivals", np.array([a.data_ptr + counter_offset for a in areas], np.int64),
                              dtype=abi.DTYPE_I64)
    status = backend.tensor("status", np.zeros(1, np.int32))
    out = backend.alloc("out", abi.DTYPE_F32, (ranks, items, hd))
    rows = backend.tensor("rows", np.ones((ranks, items, hd + 2), np.float32))
    rc = lib.yvx_cuda_lse_exchange_emulated(rows.data_ptr, ranks, items, hd, gather.data_ptr, arrivals.data_ptr,
                                            2, out.data_ptr, status.data_ptr, backend.stream)
    assert rc == 0
    assert lib.yvx_cuda_stream_synchronize(backend.stream) == 0
    assert int(status.read()[0]) == 3


def test_a_rank_that_never_publishes_runs_the_tagged_waits_out(backend):
    lib = backend.lib
    ranks, items, hd = 3, 4, 64
    area_bytes = lib.yvx_cuda_lse_exchange_bytes(ranks, items, hd)
    counter_offset = lib.yvx_cuda_lse_exchange_counter_offset(ranks, items, hd)
    areas = [backend.tensor(f"area{r}", np.zeros(area_bytes // 4, np.int32)) for r in range(ranks)]
    gather = backend.tensor("gather", np.array([a.data_ptr for a in areas], np.int64), dtype=abi.DTYPE_I64)
    arrivals = backend.tensor("arrivals", np.array([a.data_ptr + counter_offset for a in areas], np.int64),
                              dtype=abi.DTYPE_I64)
    status = backend.tensor("status", np.zeros(1, np.int32))
    out = backend.alloc("out", abi.DTYPE_F32, (ranks, items, hd))
    rows = backend.tensor("rows", np.ones((ranks, items, hd + 2), np.float32))
    rc = lib.yvx_cuda_lse_exchange_emulated_form(rows.data_ptr, ranks, items, hd, gather.data_ptr, arrivals.data_ptr,
                                                 1, out.data_ptr, status.data_ptr, backend.stream, 1, 1)
    assert rc == 0
    assert lib.yvx_cuda_stream_synchronize(backend.stream) == 0
    assert int(status.read()[0]) == 3
