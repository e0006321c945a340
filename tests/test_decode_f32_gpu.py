"""The bulk-staged F32 decode / verify kernel (head_dim 128, at most 8 query
vectors per KV head) against the CPU oracle and against the general kernel,
under the exact-F32 contract's tolerance 2e-4 * (1 + |ref|): ragged lengths
around every 16-token sub-chunk and 112-token chunk edge, one to eight vectors,
token-major and interleaved [K | V] rows, causal verify rows and the full mask."""
import numpy as np
import pytest

from clori_b200 import abi
from gqa_shim import run_problem

pytestmark = pytest.mark.gpu
HD = 128


def close(got, ref):
    return np.all(np.abs(got - ref) <= 2e-4 * (1.0 + np.abs(ref)))


@pytest.mark.parametrize("rows,hq,hkv", [(1, 32, 8), (1, 8, 8), (2, 16, 4), (4, 4, 2), (1, 16, 2), (8, 3, 3)])
@pytest.mark.parametrize("chunk", [None, 16, 96])
def test_token_major_rows(backend, oracle, rows, hq, hkv, chunk):
    rng = np.random.Generator(np.random.PCG64(rows * 1000 + hq * 10 + hkv))
    lengths = [max(n, rows) for n in (1, 15, 16, 17, 111, 112, 113, 225, 1000, 2049)]
    cap, width = 2100, hkv * HD
    q = rng.standard_normal((len(lengths), rows, hq * HD), dtype=np.float32)
    k = rng.standard_normal((len(lengths), cap, width), dtype=np.float32)
    v = rng.standard_normal((len(lengths), cap, width), dtype=np.float32)
    kw = dict(q=backend.tensor("q", q), k=backend.tensor("k", k), v=backend.tensor("v", v),
              lengths=lengths, rows=rows, hq=hq, hkv=hkv, hd=HD, dtype=abi.DTYPE_F32,
              k_token_stride=width, v_token_stride=width, k_head_stride=HD, v_head_stride=HD,
              k_outer_stride=cap * width, v_outer_stride=cap * width, kv_max=cap, chunk_tokens=chunk)
    got, status, launches, plan = run_problem(backend, **kw)
    general, status_g, _, _ = run_problem(backend, force_general=True, **kw)
    assert status == 0 and status_g == 0
    if chunk is None:
        assert plan[0] % 16 == 0 and plan[0] <= 112      # the bulk kernel's own plan
    for s, n in enumerate(lengths):
        ref = oracle.gqa_attention(q[s], k[s, :n], v[s, :n], n - rows, hq, hkv, HD, threads=8)
        assert close(got[s], ref) and close(general[s], ref)


def test_interleaved_rows_full_mask_and_repeats(backend, oracle):
    # the reference's session layout: one row per token holding [K heads | V heads]
    rng = np.random.Generator(np.random.PCG64(11))
    hq, hkv, rows, n = 32, 8, 1, 4096
    width = hkv * HD
    q = rng.standard_normal((1, rows, hq * HD), dtype=np.float32)
    kv = rng.standard_normal((1, n, 2 * width), dtype=np.float32)
    t = backend.tensor("kv", kv)
    kw = dict(q=backend.tensor("q", q), k=t, v=t, lengths=[n], rows=rows, hq=hq, hkv=hkv, hd=HD,
              dtype=abi.DTYPE_F32, causal=False, k_token_stride=2 * width, v_token_stride=2 * width,
              k_head_stride=HD, v_head_stride=HD, k_outer_stride=n * 2 * width, v_outer_stride=n * 2 * width,
              v_offset_elems=width, query_start=[0])
    first, status, launches, plan = run_problem(backend, **kw)
    again, _, _, _ = run_problem(backend, **kw)
    assert status == 0 and launches == 2 and plan[0] == 112
    assert np.array_equal(first, again)                   # deterministic split and merge order
    ref = oracle.gqa_attention(q[0], kv[0, :, :width], kv[0, :, width:], 0, hq, hkv, HD, causal=False, threads=8)
    assert close(first[0], ref)


def test_rows_past_the_length_may_hold_nan(backend, oracle):
    rng = np.random.Generator(np.random.PCG64(12))
    hq, hkv, n, cap = 8, 2, 100, 128
    width = hkv * HD
    q = rng.standard_normal((1, 1, hq * HD), dtype=np.float32)
    k = rng.standard_normal((1, cap, width), dtype=np.float32)
    v = rng.standard_normal((1, cap, width), dtype=np.float32)
    k[0, n:], v[0, n:] = np.nan, np.nan
    got, status, _, _ = run_problem(
        backend, q=backend.tensor("q", q), k=backend.tensor("k", k), v=backend.tensor("v", v), lengths=[n],
        rows=1, hq=hq, hkv=hkv, hd=HD, dtype=abi.DTYPE_F32, k_token_stride=width, v_token_stride=width,
        k_head_stride=HD, v_head_stride=HD, k_outer_stride=cap * width, v_outer_stride=cap * width, kv_max=cap)
    ref = oracle.gqa_attention(q[0], k[0, :n], v[0, :n], n - 1, hq, hkv, HD, threads=4)
    assert status == 0 and close(got[0], ref)


def test_calls_can_be_captured_into_a_graph_and_replayed(backend, oracle):
    """Split attention + dependent-launched combine inside a stream capture: the replayed
    graph produces the same bits as the direct call."""
    import ctypes as C
    rng = np.random.Generator(np.random.PCG64(13))
    hq, hkv, n = 32, 8, 1500
    width = hkv * HD
    q = rng.standard_normal((1, 1, hq * HD), dtype=np.float32)
    k = rng.standard_normal((1, n, width), dtype=np.float32)
    v = rng.standard_normal((1, n, width), dtype=np.float32)
    kw = dict(q=backend.tensor("q", q), k=backend.tensor("k", k), v=backend.tensor("v", v), lengths=[n], rows=1,
              hq=hq, hkv=hkv, hd=HD, dtype=abi.DTYPE_F32, k_token_stride=width, v_token_stride=width,
              k_head_stride=HD, v_head_stride=HD, k_outer_stride=n * width, v_outer_stride=n * width)
    direct, status, _, _ = run_problem(backend, **kw)
    assert status == 0
    lib = backend.lib
    captured = {}

    def capture_entry(problem, stream, launches):
        assert lib.yvx_cuda_graph_capture_begin(stream) == 0, lib.yvx_cuda_last_error_text()
        rc = lib.yvx_cuda_gqa_attention(problem, stream, launches)
        graph = C.c_void_p()
        assert lib.yvx_cuda_graph_capture_end(stream, C.byref(graph)) == 0, lib.yvx_cuda_last_error_text()
        for _ in range(2):
            assert lib.yvx_cuda_graph_launch(graph, stream) == 0
        captured["graph"] = graph
        return rc

    lib.capture_entry = capture_entry
    replayed, status, launches, _ = run_problem(backend, entry="capture_entry", **kw)
    assert status == 0 and launches == 2
    assert np.array_equal(replayed, direct)
    assert lib.yvx_cuda_graph_destroy(captured["graph"]) == 0
    del lib.capture_entry


@pytest.mark.parametrize("rows,hq,hkv,n", [(1, 32, 8, 4096), (2, 8, 2, 1500), (1, 40, 8, 333), (2, 16, 4, 112), (8, 2, 2, 25000)])
def test_single_launch_fold_by_the_last_cta(backend, oracle, rows, hq, hkv, n):
    """With arrival tickets the kernel folds its own splits: one launch, the same numbers as the
    two-launch path to rounding, identical repeats, and the tickets back at zero."""
    rng = np.random.Generator(np.random.PCG64(14 + n))
    width = hkv * HD
    q = rng.standard_normal((1, rows, hq * HD), dtype=np.float32)
    k = rng.standard_normal((1, n, width), dtype=np.float32)
    v = rng.standard_normal((1, n, width), dtype=np.float32)
    kw = dict(q=backend.tensor("q", q), k=backend.tensor("k", k), v=backend.tensor("v", v), lengths=[n], rows=rows,
              hq=hq, hkv=hkv, hd=HD, dtype=abi.DTYPE_F32, k_token_stride=width, v_token_stride=width,
              k_head_stride=HD, v_head_stride=HD, k_outer_stride=n * width, v_outer_stride=n * width)
    two, status, launches, plan = run_problem(backend, **kw)
    assert status == 0 and launches == (2 if plan[1] > 1 else 1)
    tickets = backend.tensor("tickets", np.zeros(2 * hkv, np.int32))
    one, status, launches, _ = run_problem(backend, tickets=tickets, **kw)
    again, _, _, _ = run_problem(backend, tickets=tickets, **kw)
    assert status == 0 and launches == 1
    assert np.array_equal(one, again)
    assert np.abs(one - two).max() <= 1e-6
    assert not tickets.read().any()
    ref = oracle.gqa_attention(q[0], k[0], v[0], n - rows, hq, hkv, HD, threads=8)
    assert close(one[0], ref)
