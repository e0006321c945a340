"""The attention entry point for callers that cannot allocate device memory.

Some users of the library run attention where cudaMalloc is off limits: the
device was handed to their own pool allocator, or the step is latency-critical
and an allocation would synchronise the device, or they are a plug-in that only
receives its inputs and outputs. yvx_cuda_gqa_attention_static_scratch serves
them by keeping the split-KV partials in a fixed array inside the library.

This file is named to be collected last: if it fails, every other test has
already run. It passes alone in a fresh process and after the other tests,
because the entry point looks the array up on its first call per device.
"""
import numpy as np
import pytest

import clori_b200
from clori_b200 import abi
from gqa_shim import run_problem

pytestmark = pytest.mark.gpu
HD = 128


def _case(backend, seed, lengths, rows, hq, hkv):
    rng = np.random.Generator(np.random.PCG64(seed))
    cap, width = max(lengths), hkv * HD
    bits = lambda shape: clori_b200.f32_to_bf16_bits(rng.standard_normal(shape, dtype=np.float32))
    q, k, v = bits((len(lengths), rows, hq * HD)), bits((len(lengths), cap, width)), bits((len(lengths), cap, width))
    return dict(q=backend.tensor("q", q), k=backend.tensor("k", k), v=backend.tensor("v", v),
                lengths=lengths, rows=rows, hq=hq, hkv=hkv, hd=HD, dtype=abi.DTYPE_BF16,
                k_token_stride=width, v_token_stride=width, k_head_stride=HD, v_head_stride=HD,
                k_outer_stride=cap * width, v_outer_stride=cap * width, kv_max=cap)


def _oracle_session(oracle, case, host, s):
    """CPU attention of session s of a case over its first lengths[s] rows."""
    f = clori_b200.bf16_bits_to_f32
    n = case["lengths"][s]
    return oracle.gqa_attention(f(host["q"][s]), f(host["k"][s, :n]), f(host["v"][s, :n]), n - case["rows"],
                                case["hq"], case["hkv"], HD, threads=4)


def test_static_scratch_entry_equals_the_regular_entry_twice_in_a_row(backend, oracle):
    # Two different problems back to back through the shared array: the second
    # call sees the first call's bytes in the scratch and must not be affected.
    first = _case(backend, 1, [4096, 700, 65, 3000], 1, 40, 8)
    second = _case(backend, 2, [900, 2500], 4, 32, 8)
    for case in (first, second):
        want, status_w, launches_w, plan = run_problem(backend, **case)
        got, status_g, launches_g, _ = run_problem(
            backend, entry="yvx_cuda_gqa_attention_static_scratch", own_scratch=False, **case)
        assert plan[1] > 1, "the case must exercise the split scratch"
        assert status_w == 0 and status_g == 0 and launches_g == launches_w == 2
        # Same kernels, same split plan: the outputs are identical, which is
        # inside the 2e-3 max-abs tolerance the bf16 parity tests use.
        assert np.abs(got - want).max() <= 2e-3
        assert np.array_equal(got, want)
        # and against the CPU attention itself (bf16 operands: 2e-3 max-abs), on the two
        # shortest sessions of the case
        host = {name: case[name].read() for name in ("q", "k", "v")}
        for s in np.argsort(case["lengths"])[:2]:
            ref = _oracle_session(oracle, case, host, int(s))
            assert np.abs(got[s] - ref).max() <= 2e-3


def test_static_scratch_entry_refuses_problems_beyond_its_capacity(backend):
    capacity = backend.lib.yvx_cuda_gqa_static_scratch_capacity()
    assert capacity == 16 << 20
    big = _case(backend, 3, [2048] * 40, 8, 40, 8)  # 40*8*40 items x 32 splits of 64 tokens
    got, rc, _, plan = run_problem(backend, entry="yvx_cuda_gqa_attention_static_scratch",
                                   own_scratch=False, chunk_tokens=64, **big)
    needed = 40 * 8 * 40 * plan[1] * (HD + 2) * 4
    assert needed > capacity
    assert got is None and rc == abi.YVEX_ERR_BOUNDS
    assert b"built-in array" in backend.lib.yvx_cuda_last_error_text()
