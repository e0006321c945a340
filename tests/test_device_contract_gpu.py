"""Device-side contract checks: values the host cannot see (session lengths stored in
device memory) and launch shapes just beyond the old grid limit. Nothing here reads or
writes out of range: the kernels record status 2 and treat the offending session as
empty, which is what makes these cases safe to run."""
import ctypes as C

import numpy as np
import pytest

import clori_b200
from clori_b200 import abi
from gqa_shim import run_problem
from test_kv_append_gpu import append

pytestmark = pytest.mark.gpu
HD = 128


def _bf16_case(backend, lengths, stored, rows=1, hq=40, hkv=8, seed=5):
    """KV sized for `lengths`; the device array of lengths holds `stored` instead."""
    rng = np.random.Generator(np.random.PCG64(seed))
    cap, width = max(lengths), hkv * HD
    bits = lambda shape: clori_b200.f32_to_bf16_bits(rng.standard_normal(shape, dtype=np.float32))
    q, k, v = bits((len(lengths), rows, hq * HD)), bits((len(lengths), cap, width)), bits((len(lengths), cap, width))
    return dict(q=backend.tensor("q", q), k=backend.tensor("k", k), v=backend.tensor("v", v),
                lengths=stored, rows=rows, hq=hq, hkv=hkv, hd=HD, dtype=abi.DTYPE_BF16,
                k_token_stride=width, v_token_stride=width, k_head_stride=HD, v_head_stride=HD,
                k_outer_stride=cap * width, v_outer_stride=cap * width, kv_max=cap)


@pytest.mark.parametrize("force_general", [False, True])
@pytest.mark.parametrize("bad", [2049, -1, -2147483648])
def test_stored_length_beyond_the_admitted_maximum_is_status_2(backend, oracle, force_general, bad):
    lengths = [2048, 1500, 2048]
    case = _bf16_case(backend, lengths, [2048, bad, 2048])     # the helper uploads them as int32
    out, status, _, plan = run_problem(backend, force_general=force_general, **case)
    assert status == 2
    assert plan[1] > 1, "the split scratch and the combine's part count must be in play"
    # the sessions with admitted lengths are unaffected
    f = clori_b200.bf16_bits_to_f32
    host = {n: case[n].read() for n in ("q", "k", "v")}
    for s in (0, 2):
        ref = oracle.gqa_attention(f(host["q"][s]), f(host["k"][s]), f(host["v"][s]), lengths[s] - 1, 40, 8, HD, threads=4)
        assert np.abs(out[s] - ref).max() <= 2e-3


def test_f32_prefill_with_more_row_tiles_than_grid_y_admits(backend, oracle):
    # 16 heads x ceil(33000 / 8) row tiles = 66000 (head, tile) pairs, over the 65535 that
    # fit grid.y; a narrow head keeps the causal arithmetic small.
    heads, hd, tokens = 16, 16, 33000
    rng = np.random.default_rng(8)
    q = rng.standard_normal((tokens, heads * hd)).astype(np.float32)
    k = rng.standard_normal((tokens, heads * hd)).astype(np.float32)
    v = rng.standard_normal((tokens, heads * hd)).astype(np.float32)
    r = clori_b200.attention_requirement(tokens, tokens, 0, heads, heads, hd)
    out = backend.alloc("o", abi.DTYPE_F32, (tokens, heads * hd))
    tensors = [backend.tensor(n, a) for n, a in (("q", q), ("k", k), ("v", v))]
    rc, facts = backend.attention_execute(r, *tensors, out)
    assert rc == abi.YVEX_OK
    got = out.read()
    for first in (0, 16379, tokens - 48):
        rows = slice(first, first + 48)
        ref = oracle.gqa_f32_reference(q[rows], k, v, first, heads, heads, hd, True)
        assert np.all(np.abs(got[rows] - ref) <= 2e-4 * (1 + np.abs(ref)))
    # and the backend is still usable afterwards
    rc, _ = backend.attention_execute(r, *tensors, out)
    assert rc == abi.YVEX_OK


def test_more_sessions_than_grid_z_admits_is_refused_before_the_launch(backend):
    p = abi.GqaProblem()
    p.sessions, p.query_rows, p.query_heads, p.kv_heads, p.head_dim = 70000, 1, 8, 8, 64
    p.chunk_tokens, p.max_splits, p.kv_tokens_uniform, p.kv_tokens_max = 64, 1, 1, 1
    dummy = backend.alloc("d", abi.DTYPE_F32, (64,))
    for name in ("query", "key", "value", "output", "status"):
        setattr(p, name, dummy.data_ptr)
    p.query_dtype = p.kv_dtype = p.output_dtype = abi.DTYPE_F32
    n = C.c_uint()
    assert backend.lib.yvx_cuda_gqa_attention(C.byref(p), backend.stream, C.byref(n)) == abi.YVEX_ERR_BOUNDS
    assert b"launch limits" in backend.lib.yvx_cuda_last_error_text()
    assert backend.lib.yvx_cuda_stream_synchronize(backend.stream) == 0


@pytest.mark.parametrize("bad", [5, -1])
def test_append_beyond_the_row_capacity_writes_nothing(backend, bad):
    # two sessions with room for 4 rows each; session 1's stored length points past its rows
    sessions, tokens, kv_heads, hd, cap = 2, 1, 2, 16, 4
    rng = np.random.default_rng(3)
    k = rng.standard_normal((sessions, tokens, kv_heads * hd)).astype(np.float32)
    v = rng.standard_normal((sessions, tokens, kv_heads * hd)).astype(np.float32)
    cos = np.ones((sessions, tokens, hd), np.float32)
    sin = np.zeros((sessions, tokens, hd), np.float32)
    state = np.full((sessions, cap, 2 * kv_heads * hd), 7.0, np.float32)
    result = append(backend, None, k, v, cos, sin, 0, kv_heads, hd, hd, False,
                    kv_tokens=np.array([1, bad]), state=state, row_capacity=cap)
    assert result["status"] == 2
    got = result["state"]
    assert np.array_equal(got[0, 1], np.concatenate([k[0, 0], v[0, 0]]))      # the good session landed
    assert np.all(got[1] == 7.0) and np.all(got[0, [0, 2, 3]] == 7.0)         # nothing else was touched
