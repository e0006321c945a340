"""Prefill attention on the tcgen05/TMEM kernel (bf16, head_dim 128) against
the CPU oracle and the general kernel. Tolerance for bf16 operands: max-abs
<= 2e-3 and cosine >= 0.9999 (values ~ N(0, 0.5^2) after RoPE as in the
benchmark configuration; the bf16 output adds half a bf16 ulp)."""
import numpy as np
import pytest

import clori_b200
from clori_b200 import abi, workloads
from gqa_shim import run_problem

pytestmark = pytest.mark.gpu
HD = 128


def widen(bits):
    return clori_b200.bf16_bits_to_f32(bits)


def cosine(a, b):
    a, b = a.astype(np.float64).ravel(), b.astype(np.float64).ravel()
    return float(a @ b / np.sqrt((a @ a) * (b @ b)))


def run(backend, q, k, v, rows, lengths, hq, hkv, causal=True, out_dtype=abi.DTYPE_F32, general=False,
        query_start=None):
    cap = k.shape[1]
    width = hkv * HD
    out, status, launches, _ = run_problem(
        backend, q=backend.tensor("q", q), k=backend.tensor("k", k), v=backend.tensor("v", v),
        lengths=lengths, rows=rows, hq=hq, hkv=hkv, hd=HD, dtype=abi.DTYPE_BF16, out_dtype=out_dtype,
        causal=causal, k_token_stride=width, v_token_stride=width, k_head_stride=HD, v_head_stride=HD,
        k_outer_stride=cap * width, v_outer_stride=cap * width, kv_max=cap, force_general=general,
        query_start=query_start)
    assert status == 0
    if out_dtype == abi.DTYPE_BF16:
        out = widen(out)
    return out, launches


@pytest.mark.parametrize("tokens,hq,hkv,batch", [(128, 2, 1, 1), (300, 4, 2, 2), (129, 5, 1, 1), (1024, 8, 2, 1)])
def test_causal_prefill_matches_oracle(backend, oracle, tokens, hq, hkv, batch):
    q, k, v = workloads.prefill_bf16(seed=2, batch=batch, tokens=tokens, query_heads=hq, kv_heads=hkv)
    got, launches = run(backend, q, k, v, tokens, [tokens] * batch, hq, hkv)
    assert launches == 1
    for b in range(batch):
        ref = oracle.gqa_attention(widen(q[b]), widen(k[b]), widen(v[b]), 0, hq, hkv, HD, threads=8)
        assert np.abs(got[b] - ref).max() <= 2e-3, float(np.abs(got[b] - ref).max())
        assert cosine(got[b], ref) >= 0.9999


def test_chunked_prefill_and_full_mask_and_bf16_output(backend, oracle):
    # 200 new query rows over 500 cached tokens (query_start = 300), then the
    # same tensors without a mask, output published as bf16.
    hq, hkv = 4, 2
    q, _, _ = workloads.prefill_bf16(seed=3, batch=1, tokens=200, query_heads=hq, kv_heads=hkv)
    _, k, v = workloads.prefill_bf16(seed=4, batch=1, tokens=500, query_heads=hq, kv_heads=hkv)
    got, _ = run(backend, q, k, v, 200, [500], hq, hkv)
    ref = oracle.gqa_attention(widen(q[0]), widen(k[0]), widen(v[0]), 300, hq, hkv, HD, threads=8)
    assert np.abs(got[0] - ref).max() <= 2e-3 and cosine(got[0], ref) >= 0.9999
    got, _ = run(backend, q, k, v, 200, [500], hq, hkv, causal=False, out_dtype=abi.DTYPE_BF16)
    ref = oracle.gqa_attention(widen(q[0]), widen(k[0]), widen(v[0]), 0, hq, hkv, HD, causal=False, threads=8)
    assert np.all(np.abs(got[0] - ref) <= 2e-3 + 2.0 ** -8 * np.abs(ref)) and cosine(got[0], ref) >= 0.9999


def test_prefill_agrees_with_general_kernel_and_repeats_bit_for_bit(backend):
    hq, hkv, tokens = 10, 2, 700
    q, k, v = workloads.prefill_bf16(seed=5, batch=2, tokens=tokens, query_heads=hq, kv_heads=hkv)
    a, _ = run(backend, q, k, v, tokens, [tokens] * 2, hq, hkv)
    b, _ = run(backend, q, k, v, tokens, [tokens] * 2, hq, hkv)
    g, _ = run(backend, q, k, v, tokens, [tokens] * 2, hq, hkv, general=True)
    assert a.tobytes() == b.tobytes()
    assert np.abs(a - g).max() <= 2e-3


def test_peaked_rows_survive_the_lazy_rescale(backend, oracle):
    # Scores that jump by far more than 2^8 between tiles force the O rescale path.
    rng = np.random.Generator(np.random.PCG64(11))
    hq, hkv, tokens = 2, 1, 512
    q = clori_b200.f32_to_bf16_bits(rng.standard_normal((1, tokens, hq * HD), dtype=np.float32))
    k = clori_b200.f32_to_bf16_bits(rng.standard_normal((1, tokens, hkv * HD), dtype=np.float32) * np.float32(0.2))
    v = clori_b200.f32_to_bf16_bits(rng.standard_normal((1, tokens, hkv * HD), dtype=np.float32))
    kf = widen(k)
    qf = widen(q)[0].reshape(tokens, hq, HD)
    for t in (140, 270, 400):  # late keys aligned with the query direction of head 0: huge scores
        kf[0, t] = qf[500, 0] * 3.0
    k = clori_b200.f32_to_bf16_bits(kf)
    got, _ = run(backend, q, k, v, tokens, [tokens], hq, hkv)
    ref = oracle.gqa_attention(widen(q[0]), widen(k[0]), widen(v[0]), 0, hq, hkv, HD, threads=8)
    assert np.abs(got[0] - ref).max() <= 4e-3
    assert cosine(got[0], ref) >= 0.9999
