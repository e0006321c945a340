"""The CPU attention on a sample of every benchmark configuration at its FULL size.

The whole output of a full-size configuration would take the CPU checker minutes to
hours, so each test runs the configuration once on the device exactly as the benchmark
does (same generators, same entry points: the functions of bench.py) and compares a
sample that the CPU finishes in seconds: whole sessions of the batched decode, one
KV-head group of the long quantised verify, a band of causal prefill rows, eight heads
of a latent-decode session. Bars: max-abs <= 2e-3 for bf16 / Q8_0 operands (the prefill
writes bf16, so half a bf16 ulp of the value is added), 2e-4 * (1 + |ref|) for F32."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bench  # noqa: E402
from clori_b200 import abi  # noqa: E402

pytestmark = pytest.mark.gpu
THREADS = min(os.cpu_count() or 1, 16)


def test_decode_f32_config_against_cpu(backend, oracle):
    result, sample = bench.bench_decode_f32(backend.lib, backend, abi, 6545.0, 3)
    assert result["status_word"] == 0
    error, _ = bench.check_decode_f32(oracle, sample, THREADS)
    assert error <= 2e-4 * (1.0 + float(np.abs(sample["o"]).max()))


def test_batched_decode_config_sessions_against_cpu(oracle):
    w = bench.Workload(0, bench.SEED)
    w.step()
    w.backend.sync()
    w.out.struct.is_written = 1
    got = w.cl.bf16_bits_to_f32(w.out.read())
    shortest = [int(s) for s in np.argsort(w.lengths)[:3]]
    for s in shortest + [int(np.argsort(w.lengths)[len(w.lengths) // 2])]:
        q, k, v = w.host_session(s)
        ref = oracle.gqa_attention(q, k, v, k.shape[0] - 1, bench.QUERY_HEADS, bench.KV_HEADS, bench.HEAD_DIM,
                                   threads=THREADS)
        half_ulp = np.abs(ref) * 2.0 ** -8
        assert np.all(np.abs(got[s, 0] - ref[0]) <= 2e-3 + half_ulp[0])
    w.backend.close()


def test_prefill_config_rows_against_cpu(backend, oracle):
    result, sample = bench.bench_prefill(backend.lib, backend, abi, 1)
    assert result["status_word"] == 0
    error, _ = bench.check_prefill(oracle, sample, THREADS)
    assert error <= 2e-3 + 2.0 ** -8


def test_verify_q8_config_head_group_against_cpu(backend, oracle):
    result, sample = bench.bench_verify_q8(backend.lib, backend, abi, 6545.0, 2)
    assert result["status_word"] == 0
    error, _ = bench.check_verify_q8(oracle, sample, THREADS)
    assert error <= 2e-3


def test_latent_decode_config_heads_against_cpu(backend):
    result, sample = bench.bench_mla(backend.lib, backend, abi, 6545.0, 2)
    assert result["status_word"] == 0
    error, _ = bench.check_mla(sample)
    assert error <= 2e-3
