"""Parity of the exact-attention operator (F32 contract) on a B200, through the
C-ABI, against the CPU oracle and the golden fixtures. The cases follow the
reference's own CUDA tests (tests/unit/cuda/quant_qtype.c:1998-2970,
tests/unit/cuda/ops.c:536-625) with the tolerances written there."""
import os

import numpy as np
import pytest

import clori_b200
from clori_b200 import abi, workloads

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def run(backend, q, k, v, query_start, hq, hkv, hd, causal=True, tq=None, tkv=None, **strides):
    tq = q.shape[0] if tq is None else tq
    tkv = k.shape[0] if tkv is None else tkv
    r = clori_b200.attention_requirement(tq, tkv, query_start, hq, hkv, hd, causal=causal, **strides)
    tq_, tk_, tv_ = backend.tensor("q", q), backend.tensor("k", k), backend.tensor("v", v)
    out = backend.alloc("o", abi.DTYPE_F32, (tq, hq * hd))
    rc, facts = backend.attention_execute(r, tq_, tk_, tv_, out)
    assert rc == abi.YVEX_OK
    return out.read(), facts


def test_tiny_gqa_closed_form(backend):
    # quant_qtype.c:2019-2136
    q = np.array([[1, 0, 1, 0], [1, 0, 1, 0]], np.float32)
    k = np.array([[1, 0], [0, 1]], np.float32)
    v = np.array([[2, 4], [6, 8]], np.float32)
    r = clori_b200.attention_requirement(2, 2, 0, 2, 1, 2)
    rc, nbytes = backend.attention_workspace_required(r)
    assert rc == 0 and nbytes == 0
    out, facts = run(backend, q, k, v, 0, 2, 1, 2)
    assert facts.kernel_launches == 1 and facts.device_synchronizations == 1
    assert np.array_equal(out[0], [2, 4, 2, 4])
    p = np.exp(np.float32(1.0) / np.sqrt(np.float32(2.0)))
    e0, e1 = (p * 2 + 6) / (p + 1), (p * 4 + 8) / (p + 1)
    assert np.all(np.abs(out[1] - [e0, e1, e0, e1]) < 1e-6)
    full, _ = run(backend, q, k, v, 0, 2, 1, 2, causal=False)
    assert np.all(np.abs(full - [[e0, e1, e0, e1]] * 2) < 1e-6)


def _pattern(count, mul, add, mod, shift, div):
    index = np.arange(count, dtype=np.uint64)
    return (((index * mul + add) % mod).astype(np.int64) - shift).astype(np.float32) / np.float32(div)


def test_small_mha_pattern(backend, oracle):
    # quant_qtype.c:2283-2341: 5 tokens, 1 head, hd 128, 2e-5.
    n = 5 * 128
    q = _pattern(n, 3, 0, 19, 9, 8).reshape(5, 128)
    k = _pattern(n, 5, 2, 23, 11, 9).reshape(5, 128)
    v = _pattern(n, 7, 1, 29, 14, 10).reshape(5, 128)
    for causal in (True, False):
        out, _ = run(backend, q, k, v, 0, 1, 1, 128, causal=causal)
        ref = oracle.gqa_f32_reference(q, k, v, 0, 1, 1, 128, causal)
        assert np.all(np.abs(out - ref) < 2e-5)


def test_qwen_geometry_and_cached_decode(backend, oracle):
    # quant_qtype.c:2393-2555: 24 query / 4 KV heads, hd 256, 2e-4*(1+|ref|).
    hq, hkv, hd = 24, 4, 256
    q = _pattern(3 * hq * hd, 3, 0, 29, 14, 32).reshape(3, hq * hd)
    k = _pattern(3 * hkv * hd, 5, 1, 31, 15, 32).reshape(3, hkv * hd)
    v = _pattern(3 * hkv * hd, 7, 2, 37, 18, 16).reshape(3, hkv * hd)
    for causal in (False, True):
        out, facts = run(backend, q, k, v, 0, hq, hkv, hd, causal=causal)
        ref = oracle.gqa_f32_reference(q, k, v, 0, hq, hkv, hd, causal)
        assert facts.kernel_launches == 1
        assert np.all(np.abs(out - ref) < 2e-4 * (1 + np.abs(ref)))
    q1 = _pattern(hq * hd, 11, 0, 43, 21, 32).reshape(1, hq * hd)
    k = _pattern(3 * hkv * hd, 13, 1, 47, 23, 32).reshape(3, hkv * hd)
    v = _pattern(3 * hkv * hd, 17, 2, 53, 26, 16).reshape(3, hkv * hd)
    out, _ = run(backend, q1, k, v, 2, hq, hkv, hd)
    ref = oracle.gqa_f32_reference(q1, k, v, 2, hq, hkv, hd, True)
    assert np.all(np.abs(out - ref) < 2e-4 * (1 + np.abs(ref)))
    r = clori_b200.attention_requirement(1, 3, 3, hq, hkv, hd)
    t = [backend.tensor("x", a) for a in (q1, k, v)]
    o = backend.alloc("o", abi.DTYPE_F32, (1, hq * hd))
    rc, _ = backend.attention_execute(r, *t, o, check=False)
    assert rc == abi.YVEX_ERR_INVALID_ARG
    rc, _ = backend.attention_workspace_required(
        clori_b200.attention_requirement(3, 3, 0, hq, hkv, hd + 1), check=False)
    assert rc == abi.YVEX_ERR_UNSUPPORTED


def test_strided_interleaved_kv_views(backend, oracle):
    # quant_qtype.c:2557-2680: [Q|gate] rows and interleaved [K|V] rows.
    hq, hkv, hd, tq, tkv = 24, 4, 256, 2, 4
    qw, kvw = hq * hd, hkv * hd
    q = _pattern(tq * qw, 19, 3, 59, 29, 32).reshape(tq, qw)
    k = _pattern(tkv * kvw, 23, 5, 61, 30, 32).reshape(tkv, kvw)
    v = _pattern(tkv * kvw, 29, 7, 67, 33, 16).reshape(tkv, kvw)
    q_inter = np.zeros((tq - 1) * 2 * qw + qw, np.float32)
    for t in range(tq):
        q_inter[t * 2 * qw:t * 2 * qw + qw] = q[t]
    kv_inter = np.concatenate([k, v], axis=1).reshape(-1)
    q_store, kv_store = backend.tensor("q", q_inter), backend.tensor("kv", kv_inter)
    out = backend.alloc("o", abi.DTYPE_F32, (tq, qw))
    q_view = q_store.f32_subview(0, q_inter.size)
    k_view = kv_store.f32_subview(0, kv_inter.size - kvw)
    v_view = kv_store.f32_subview(kvw, kv_inter.size - kvw)
    assert q_view and k_view and v_view
    r = clori_b200.attention_requirement(tq, tkv, tkv - tq, hq, hkv, hd, query_token_stride=2 * qw,
                                         key_token_stride=2 * kvw, value_token_stride=2 * kvw)
    rc, facts = backend.attention_execute(r, q_view, k_view, v_view, out)
    assert rc == 0 and facts.kernel_launches == 1
    ref = oracle.gqa_f32_reference(q, k, v, tkv - tq, hq, hkv, hd, True)
    assert np.all(np.abs(out.read() - ref) < 2e-4 * (1 + np.abs(ref)))
    r.value_token_stride = kvw - 1
    rc, _ = backend.attention_execute(r, q_view, k_view, v_view, out, check=False)
    assert rc == abi.YVEX_ERR_INVALID_ARG
    # a view whose byte count disagrees with the strides is a format error
    r.value_token_stride = 2 * kvw
    short = kv_store.f32_subview(kvw, kv_inter.size - kvw - 1)
    rc, _ = backend.attention_execute(r, q_view, k_view, short, out, check=False)
    assert rc == abi.YVEX_ERR_FORMAT


def test_tile_sized_mha_repeats_bit_for_bit_and_rejects_nan(backend, oracle):
    # quant_qtype.c:2717-2866: 257 x 128, bf16-valued inputs, 2e-3*(1+|ref|),
    # byte-identical repeat, NaN in Q or V is a format error, bf16 output is
    # refused by the F32 contract.
    rng = np.random.default_rng(17)
    n, hd = 257, 128
    q, k, v = (clori_b200.bf16_bits_to_f32(clori_b200.f32_to_bf16_bits(
        rng.standard_normal((n, hd)).astype(np.float32))) for _ in range(3))
    a, _ = run(backend, q, k, v, 0, 1, 1, hd)
    b, _ = run(backend, q, k, v, 0, 1, 1, hd)
    assert a.tobytes() == b.tobytes()
    ref = oracle.gqa_attention(q, k, v, 0, 1, 1, hd)
    assert np.all(np.abs(a - ref) < 2e-3 * (1 + np.abs(ref)))      # the reference's bar for this path
    for poisoned in ("q", "v"):
        qq, vv = q.copy(), v.copy()
        (qq if poisoned == "q" else vv)[3, 5] = np.nan
        r = clori_b200.attention_requirement(n, n, 0, 1, 1, hd)
        t = [backend.tensor("x", x) for x in (qq, k, vv)]
        o = backend.alloc("o", abi.DTYPE_F32, (n, hd))
        rc, _ = backend.attention_execute(r, *t, o, check=False)
        assert rc == abi.YVEX_ERR_FORMAT
    r = clori_b200.attention_requirement(n, n, 0, 1, 1, hd, output_dtype=abi.DTYPE_BF16)
    t = [backend.tensor("x", x) for x in (q, k, v)]
    o = backend.alloc("o", abi.DTYPE_F32, (n, hd))
    rc, _ = backend.attention_execute(r, *t, o, check=False)
    assert rc == abi.YVEX_ERR_UNSUPPORTED


def test_uniform_value_analytic_oracle_at_long_lengths(backend):
    # quant_qtype.c:2868-2970: when every V row is the same vector the output is
    # that vector for any scores; lengths chosen there: 65 (2 heads), 5757.
    rng = np.random.default_rng(23)
    for tokens, heads in ((65, 2), (5757, 1)):
        hd = 128
        q = rng.standard_normal((tokens, heads * hd)).astype(np.float32)
        k = rng.standard_normal((tokens, heads * hd)).astype(np.float32)
        row = rng.standard_normal(heads * hd).astype(np.float32)
        v = np.tile(row, (tokens, 1))
        out, _ = run(backend, q, k, v, 0, heads, heads, hd)
        assert np.all(np.abs(out - row[None, :]) < 2e-5 * (1 + np.abs(row[None, :])))


def test_golden_fixtures_from_the_reference_cpu(backend):
    g = np.load(os.path.join(GOLDEN, "gqa_attention.npz"))
    for i in range(int(g["count"])):
        tq, tkv, qs, hq, hkv, hd, causal = (int(x) for x in g[f"meta{i}"])
        out, _ = run(backend, g[f"q{i}"], g[f"k{i}"], g[f"v{i}"], qs, hq, hkv, hd, causal=bool(causal))
        ref = g[f"out{i}"]
        assert np.all(np.abs(out - ref) < 2e-4 * (1 + np.abs(ref))), i


def test_config1_decode_f32_against_oracle(backend, oracle):
    # BASELINE config 1, full size: 1 token, 32/8 heads, hd 128, KV 4096, seed 0.
    q, k, v = workloads.decode_f32(seed=0)
    out, facts = run(backend, q, k, v, 4095, 32, 8, 128)
    ref = oracle.gqa_attention(q, k, v, 4095, 32, 8, 128, threads=8)
    assert facts.kernel_launches == 1  # one launch: the last CTA of every KV head folds the splits
    assert np.abs(out - ref).max() <= 2e-4
    assert np.all(np.abs(out - ref) < 2e-4 * (1 + np.abs(ref)))
    cos = float((out * ref).sum() / np.sqrt((out * out).sum() * (ref * ref).sum()))
    assert cos >= 0.9999


@pytest.mark.parametrize("tq,tkv,hq,hkv,hd,causal", [
    (1, 1, 4, 2, 64, True), (1, 63, 4, 4, 32, True), (1, 64, 8, 2, 128, True),
    (1, 65, 8, 2, 128, True), (4, 1000, 32, 8, 128, True), (8, 777, 10, 2, 96, True),
    (7, 7, 3, 1, 200, True), (16, 300, 6, 2, 16, False), (130, 130, 4, 2, 64, True),
    (2, 9000, 5, 5, 128, True), (3, 129, 40, 8, 128, True),
])
def test_random_shapes_against_oracle(backend, oracle, tq, tkv, hq, hkv, hd, causal):
    rng = np.random.default_rng(tq * 1000 + tkv)
    q = rng.standard_normal((tq, hq * hd)).astype(np.float32)
    k = rng.standard_normal((tkv, hkv * hd)).astype(np.float32)
    v = rng.standard_normal((tkv, hkv * hd)).astype(np.float32)
    qs = tkv - tq if causal else 0
    out, _ = run(backend, q, k, v, qs, hq, hkv, hd, causal=causal)
    ref = oracle.gqa_attention(q, k, v, qs, hq, hkv, hd, causal=causal, threads=8)
    assert np.all(np.abs(out - ref) < 2e-4 * (1 + np.abs(ref)))


def test_op_attention_primitive(backend, oracle):
    # tests/unit/cuda/ops.c:536-625 sequence of calls and refusals, 1e-4.
    g = np.load(os.path.join(GOLDEN, "op_attention.npz"))
    for i in range(int(g["count"])):
        seq, hd, position, causal = (int(x) for x in g[f"meta{i}"])
        q = backend.tensor("q", g[f"q{i}"])
        k = backend.tensor("k", g[f"k{i}"])
        v = backend.tensor("v", g[f"v{i}"])
        s = backend.alloc("s", abi.DTYPE_F32, (seq,))
        p = backend.alloc("p", abi.DTYPE_F32, (seq,))
        o = backend.alloc("o", abi.DTYPE_F32, (hd,))
        scale = float(g[f"scale{i}"])
        assert backend.op_attention(q, k, v, seq, position, scale, causal, s, p, o) == 0
        assert np.all(np.abs(o.read() - g[f"out{i}"]) < 1e-4)
        assert np.all(np.abs(s.read() - g[f"scores{i}"]) < 1e-4)
        assert np.all(np.abs(p.read() - g[f"probs{i}"]) < 1e-5)
        assert backend.op_attention(q, k, v, seq, seq, scale, 1, s, p, o, check=False) == abi.YVEX_ERR_BOUNDS
        assert backend.op_attention(q, k, v, 0, 0, scale, 1, s, p, o, check=False) != 0
        assert backend.op_attention(q, k, v, seq, 0, float("nan"), 1, s, p, o, check=False) == abi.YVEX_ERR_INVALID_ARG
    q = backend.tensor("q", np.array([0.1, 0.2, 0.3, 0.4], np.float32))
    k = backend.tensor("k", np.array([[0.2, 0.1, 0.0, 0.3], [0.4, 0.3, 0.2, 0.1], [0.1, 0.5, 0.3, 0.2]], np.float32))
    vals = np.array([[1, 2, 3, 4], [10, 20, 30, 40], [5, 6, 7, 8]], np.float32)
    v = backend.tensor("v", vals)
    s, p = backend.alloc("s", abi.DTYPE_F32, (3,)), backend.alloc("p", abi.DTYPE_F32, (3,))
    o = backend.alloc("o", abi.DTYPE_F32, (4,))
    assert backend.op_attention(q, k, v, 3, 0, 0.5, 1, s, p, o) == 0
    assert np.all(np.abs(o.read() - vals[0]) < 1e-4)


def _bf16_valued(rng, shape, scale=1.0):
    x = rng.standard_normal(shape).astype(np.float32) * np.float32(scale)
    return clori_b200.bf16_bits_to_f32(clori_b200.f32_to_bf16_bits(x))


@pytest.mark.parametrize("tokens,hq,hkv,causal", [(257, 1, 1, True), (300, 40, 8, True), (513, 4, 4, False),
                                                  (1030, 8, 2, True)])
def test_prefill_sized_f32_problems_run_on_the_tensor_cores(backend, oracle, tokens, hq, hkv, causal):
    # quant_qtype.c:2717-2866: inputs that bf16 holds exactly, 2e-3 * (1 + |ref|), identical repeats
    rng = np.random.default_rng(tokens)
    q, k, v = (_bf16_valued(rng, (tokens, h * 128), 0.5) for h in (hq, hkv, hkv))
    out, facts = run(backend, q, k, v, 0, hq, hkv, 128, causal=causal)
    assert facts.kernel_launches >= 5           # three staging launches, the gated pair
    rows = np.r_[0:40, tokens - 40:tokens]
    for first in (0, tokens - 40):
        ref = oracle.gqa_f32_reference(q[first:first + 40], k, v, first, hq, hkv, 128, causal)
        assert np.all(np.abs(out[first:first + 40] - ref) <= 2e-3 * (1 + np.abs(ref)))
    again, _ = run(backend, q, k, v, 0, hq, hkv, 128, causal=causal)
    assert np.array_equal(out.view(np.uint32), again.view(np.uint32))
    # one lane that bf16 cannot hold: found on the device, the exact kernel answers (2e-4)
    k2 = k.copy()
    k2[tokens // 2, 5] = np.float32(0.3)
    exact, _ = run(backend, q, k2, v, 0, hq, hkv, 128, causal=causal)
    for first in (0, tokens - 40):
        ref = oracle.gqa_f32_reference(q[first:first + 40], k2, v, first, hq, hkv, 128, causal)
        assert np.all(np.abs(exact[first:first + 40] - ref) <= 2e-4 * (1 + np.abs(ref)))
    assert rows.size == 80


def test_prefill_sized_f32_problem_with_a_nan_is_refused(backend):
    rng = np.random.default_rng(5)
    q, k, v = (_bf16_valued(rng, (300, h * 128)) for h in (8, 2, 2))
    v[17, 3] = np.nan
    r = clori_b200.attention_requirement(300, 300, 0, 8, 2, 128)
    out = backend.alloc("o", abi.DTYPE_F32, (300, 8 * 128))
    with pytest.raises(clori_b200.YvexError) as refusal:
        backend.attention_execute(r, backend.tensor("q", q), backend.tensor("k", k), backend.tensor("v", v), out)
    assert refusal.value.code == abi.YVEX_ERR_FORMAT
