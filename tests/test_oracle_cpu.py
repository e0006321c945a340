"""The CPU oracle against the reference: golden fixtures generated from the
reference's compiled CPU code, the reference's own known-answer vectors, and
(where oracle/_ref exists) the reference's code run side by side."""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _load(name):
    return np.load(os.path.join(GOLDEN, name))


def test_primitive_matches_golden_bit_for_bit(oracle):
    g = _load("op_attention.npz")
    for i in range(int(g["count"])):
        seq, hd, position, causal = (int(x) for x in g[f"meta{i}"])
        rc, out, scores, probs = oracle.op_attention(g[f"q{i}"], g[f"k{i}"], g[f"v{i}"], position,
                                                     float(g[f"scale{i}"]), causal)
        assert rc == 0
        assert np.array_equal(out, g[f"out{i}"])
        assert np.array_equal(scores, g[f"scores{i}"])
        assert np.array_equal(probs, g[f"probs{i}"])


def test_gqa_matches_golden_bit_for_bit(oracle):
    g = _load("gqa_attention.npz")
    for i in range(int(g["count"])):
        tq, tkv, qs, hq, hkv, hd, causal = (int(x) for x in g[f"meta{i}"])
        out = oracle.gqa_attention(g[f"q{i}"], g[f"k{i}"], g[f"v{i}"], qs, hq, hkv, hd,
                                   causal=bool(causal), threads=2)
        assert np.array_equal(out, g[f"out{i}"]), i


def test_codecs_match_golden(oracle):
    g = _load("codecs.npz")
    values = g["values"]
    assert [oracle.bf16_encode(x) for x in values] == list(g["bf16"])
    assert [oracle.f16_encode(x) for x in values] == list(g["f16"])
    decoded = np.array([oracle.f16_decode(b) for b in range(65536)], np.float32)
    assert np.array_equal(decoded.view(np.uint32), g["f16_decode_all"].view(np.uint32))
    for src, enc, dec in zip(g["q8_source"], g["q8_encoded"], g["q8_decoded"]):
        assert np.array_equal(oracle.q8_0_encode_block(src), enc)
        assert np.array_equal(oracle.q8_0_decode_block(enc), dec)


def test_bf16_known_answers_from_reference_tests(oracle):
    # tests/reference/deepseek_attention.c external vectors: bf16 bits and the
    # float they round from / widen to.
    assert oracle.bf16_decode(0x3F80) == 1.0
    assert oracle.bf16_decode(0x3F82) == 1.015625
    assert oracle.bf16_encode(1.00390625) == 0x3F80  # tie rounds to even
    assert oracle.bf16_encode(1.01171875) == 0x3F82
    assert oracle.bf16_encode(-0.0) == 0x8000


def test_q8_0_rejects_negative_scale(oracle):
    block = np.zeros(34, np.uint8)
    block[:2] = np.array([-1.0], np.float16).view(np.uint8)
    assert oracle.q8_0_decode_block(block) is None


def test_cpu_primitive_expectations_of_reference_unit_test(oracle):
    # tests/unit/backend_ops.c:444-531: position 0 returns V[0]; the full prefix
    # mixes; an out-of-range position is a bounds error (-7).
    q = np.array([0.1, 0.2, 0.3, 0.4], np.float32)
    k = np.array([[0.2, 0.1, 0.0, 0.3], [0.4, 0.3, 0.2, 0.1], [0.1, 0.5, 0.3, 0.2]], np.float32)
    v = np.array([[1, 2, 3, 4], [10, 20, 30, 40], [5, 6, 7, 8]], np.float32)
    rc, out, _, _ = oracle.op_attention(q, k, v, 0, 0.5, 1)
    assert rc == 0 and np.allclose(out, v[0], atol=1e-6)
    rc, out, _, probs = oracle.op_attention(q, k, v, 2, 0.5, 1)
    assert rc == 0 and abs(out[0] - v[0, 0]) > 1e-4 and abs(probs.sum() - 1.0) < 1e-6
    rc, _, _, _ = oracle.op_attention(q, k, v, 3, 0.5, 1)
    assert rc == -7


def test_tiny_gqa_closed_form_of_reference_cuda_test(oracle):
    # tests/unit/cuda/quant_qtype.c:2019-2136: 2 query heads on 1 KV head, hd 2.
    q = np.array([[1, 0, 1, 0], [1, 0, 1, 0]], np.float32)
    k = np.array([[1, 0], [0, 1]], np.float32)
    v = np.array([[2, 4], [6, 8]], np.float32)
    out = oracle.gqa_attention(q, k, v, 0, 2, 1, 2, causal=True)
    p = np.exp(np.float32(1.0) / np.sqrt(np.float32(2.0)))
    e0, e1 = (p * 2 + 6) / (p + 1), (p * 4 + 8) / (p + 1)
    assert np.array_equal(out[0], [2, 4, 2, 4])
    assert np.allclose(out[1], [e0, e1, e0, e1], atol=1e-6)
    full = oracle.gqa_attention(q, k, v, 0, 2, 1, 2, causal=False)
    assert np.allclose(full, [[e0, e1, e0, e1]] * 2, atol=1e-6)


def test_double_oracle_agrees_with_float_scalar_oracle(oracle):
    # The float oracle the reference's CUDA tests use (quant_qtype.c:2343-2391)
    # and the CPU primitive must agree within the tests' own tolerance.
    rng = np.random.default_rng(5)
    q = rng.standard_normal((3, 24 * 256)).astype(np.float32) / 4
    k = rng.standard_normal((3, 4 * 256)).astype(np.float32) / 4
    v = rng.standard_normal((3, 4 * 256)).astype(np.float32)
    a = oracle.gqa_attention(q, k, v, 0, 24, 4, 256, causal=True)
    b = oracle.gqa_f32_reference(q, k, v, 0, 24, 4, 256, True)
    assert np.all(np.abs(a - b) < 2e-4 * (1 + np.abs(b)))


def test_strided_views_equal_packed(oracle):
    rng = np.random.default_rng(6)
    hq, hkv, hd, tq, tkv = 6, 2, 32, 2, 9
    q = rng.standard_normal((tq, hq * hd)).astype(np.float32)
    k = rng.standard_normal((tkv, hkv * hd)).astype(np.float32)
    v = rng.standard_normal((tkv, hkv * hd)).astype(np.float32)
    packed = oracle.gqa_attention(q, k, v, tkv - tq, hq, hkv, hd)
    kv = np.concatenate([k, v], axis=1)  # interleaved [K|V] rows
    flat = kv.reshape(-1)
    strided = oracle.gqa_attention(q, flat, flat[hkv * hd:], tkv - tq, hq, hkv, hd,
                                   k_stride=2 * hkv * hd, v_stride=2 * hkv * hd,
                                   query_tokens=tq, kv_tokens=tkv)
    assert np.array_equal(packed, strided)


def test_sink_reduction_known_answer(oracle):
    # tests/reference/deepseek_attention.c:2724-2726, check :2928-2940: sink
    # logit 0, logits {0, ln 2}, values {1,2},{3,4} -> {1.75, 2.5}. Logits are
    # realised as q.row/sqrt(hd) with a one-hot query on an extra lane pair.
    hd = 4
    q = np.zeros((1, hd), np.float32)
    q[0, 2] = 1.0
    rows = np.array([[1, 2, 0, 0], [3, 4, np.log(2.0) * 2.0, 0]], np.float32)
    out = oracle.latent_reduce(q, rows, np.zeros(1, np.float32), query_start=1, heads=1,
                               head_dim=hd, round_bf16=False)
    assert np.allclose(out[0, :2], [1.75, 2.5], atol=1e-6)


def test_latent_reduce_is_shared_row_attention(oracle):
    # With the sink far below every score the latent reduce is ordinary
    # attention whose keys equal its values (tests/unit/deepseek_attention.c:593
    # uses -100 for the same purpose).
    rng = np.random.default_rng(7)
    heads, hd, rows_n = 4, 64, 20
    q = rng.standard_normal((2, heads * hd)).astype(np.float32)
    rows = rng.standard_normal((rows_n, hd)).astype(np.float32)
    out = oracle.latent_reduce(q, rows, np.full(heads, -100.0, np.float32), query_start=18,
                               heads=heads, head_dim=hd, round_bf16=False)
    ref = oracle.gqa_attention(q, rows, rows, 18, heads, 1, hd)
    assert np.allclose(out, ref, atol=2e-6)


def test_block_rows(oracle):
    table = np.array([5, 2, 9], np.int32)
    assert oracle.block_row(table, 64, 0) == 320
    assert oracle.block_row(table, 64, 63) == 383
    assert oracle.block_row(table, 64, 64) == 128
    assert oracle.block_row(table, 64, 130) == 9 * 64 + 2
    pool = np.arange(10 * 64 * 3, dtype=np.uint16).reshape(640, 3)
    got = oracle.block_gather_u16(pool, table, 64, 150)
    want = np.stack([pool[oracle.block_row(table, 64, r)] for r in range(150)])
    assert np.array_equal(got, want)


def test_page_touch(oracle):
    assert oracle.page_touch(0, 1, 16) == (0, 0)
    assert oracle.page_touch(15, 2, 16) == (0, 1)
    assert oracle.page_touch(16 * 7, 16, 16) == (7, 7)
    assert oracle.page_touch(5, 0, 16) is None


def test_oracle_equals_reference_code_on_random_inputs(oracle, reference):
    rng = np.random.default_rng(11)
    for tq, tkv, hq, hkv, hd, causal in [(1, 300, 8, 2, 128, True), (3, 33, 4, 4, 96, True),
                                         (2, 40, 10, 5, 64, False)]:
        q = rng.standard_normal((tq, hq * hd)).astype(np.float32)
        k = rng.standard_normal((tkv, hkv * hd)).astype(np.float32)
        v = rng.standard_normal((tkv, hkv * hd)).astype(np.float32)
        qs = tkv - tq if causal else 0
        a = oracle.gqa_attention(q, k, v, qs, hq, hkv, hd, causal=causal, threads=2)
        b = reference.gqa_attention(q, k, v, qs, hq, hkv, hd, causal=causal, threads=2)
        assert np.array_equal(a, b)
    xs = rng.standard_normal(3000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 9, 3000).astype(np.float32)
    for x in xs:
        assert oracle.bf16_encode(x) == reference.bf16_encode(x)
        assert oracle.f16_encode(x) == reference.f16_encode(x)
    for _ in range(20):
        block = rng.standard_normal(32).astype(np.float32) * 5
        assert np.array_equal(oracle.q8_0_encode_block(block), reference.q8_0_encode_block(block))


def test_mla_restatement_matches_dense_recomputation(oracle):
    # No reference counterpart exists for the split-rope variant; the
    # restatement is checked against a plain numpy float64 evaluation.
    from clori_b200 import bf16_bits_to_f32, workloads
    qn, qr, w, lat, rk = workloads.mla_decode_bf16(seed=4, batch=1, heads=3, nope_dim=16,
                                                   latent_dim=32, rope_dim=8, context=50)
    scale = 1.0 / np.sqrt(24.0)
    out = oracle.mla_decode(qn[0], qr[0], w, lat[0], rk[0], scale)
    f = lambda b: bf16_bits_to_f32(b).astype(np.float64)
    q_lat = np.einsum("hi,hic->hc", f(qn[0]), f(w))
    from clori_b200 import f32_to_bf16_bits
    q_lat = f(f32_to_bf16_bits(q_lat.astype(np.float32)))
    s = (q_lat @ f(lat[0]).T + f(qr[0]) @ f(rk[0]).T) * scale
    p = np.exp(s - s.max(axis=1, keepdims=True))
    p /= p.sum(axis=1, keepdims=True)
    assert np.allclose(out, p @ f(lat[0]), atol=1e-6)


def test_full_latent_reduce_restatement_cross_checks(oracle):
    # Window-only class with a window wider than the history is plain shared-row
    # attention with a sink: it must equal the simpler restatement, and the sink
    # known-answer vector of the reference must come out of it too.
    import ctypes as C
    from clori_b200 import abi
    rng = np.random.default_rng(12)
    heads, hd, rows_n, tokens = 3, 32, 20, 2
    q = rng.standard_normal((tokens, heads * hd)).astype(np.float32)
    rows = rng.standard_normal((rows_n, hd)).astype(np.float32)
    sinks = rng.standard_normal(heads).astype(np.float32)
    positions = np.arange(rows_n, dtype=np.uint64)
    zeros = np.zeros(4, np.uint64)
    a = abi.LatentReduceArgs()
    a.query, a.local, a.local_positions = q.ctypes.data, rows.ctypes.data, positions.ctypes.data
    a.initial_local_count, a.local_stride = rows_n - tokens, hd
    a.compressed = a.compressed_positions = a.selected = a.selected_count = zeros.ctypes.data
    a.sinks, a.query_heads, a.head_dim = sinks.ctypes.data, heads, hd
    a.sliding_window, a.ratio, a.attention_class = 128, 0, 0
    a.phase_start_position, a.token_count = rows_n - tokens, tokens
    full = oracle.latent_reduce_full(a, tokens, heads, hd)
    simple = oracle.latent_reduce(q, rows, sinks, query_start=rows_n - tokens, heads=heads, head_dim=hd)
    assert np.array_equal(full, simple)
    # a window of 4 hides the older rows
    a.sliding_window = 4
    windowed = oracle.latent_reduce_full(a, tokens, heads, hd)
    visible = oracle.latent_reduce(q[1:], rows[rows_n - 4:], sinks, query_start=3, heads=heads, head_dim=hd)
    assert np.array_equal(windowed[1:], visible)


def test_rotary_half_known_answers_of_the_reference(oracle):
    # bf16-staged products: tests/unit/cuda/quant_qtype.c:1989-2062
    rb = lambda x: float(oracle.bf16_round(np.array([x], np.float32))[1][0])
    values = np.array([[-1.34375, -2.0625, 3.0, 4.0]], np.float32)
    cos = np.full((1, 2), 0.63671875, np.float32)
    sin = np.full((1, 2), 0.546875, np.float32)
    got = oracle.rotary_half(values, cos, sin, 1, 4, 2, staged=True)
    first = rb(rb(np.float32(-1.34375) * np.float32(0.63671875)) - rb(np.float32(-2.0625) * np.float32(0.546875)))
    second = rb(rb(np.float32(-2.0625) * np.float32(0.63671875)) + rb(np.float32(-1.34375) * np.float32(0.546875)))
    assert got.tolist() == [[first, second, 3.0, 4.0]]
    # plain single precision: tests/unit/cuda/quant_qtype.c:3057-3104
    values = np.array([[1.0, 2.0, 7.0, 8.0]], np.float32)
    got = oracle.rotary_half(values, np.full((1, 2), 0.75, np.float32), np.full((1, 2), 0.5, np.float32),
                             2, 2, 2, staged=False)
    assert got.tolist() == [[-0.25, 2.0, 1.25, 9.5]]


def test_rope_tables_follow_the_decoder_convention(oracle):
    # src/runtime/decoder.c:1080-1094: pair = coordinate mod width/2, bf16-rounded cos/sin
    cos, sin = oracle.rope_tables(3, 2, 8, 1.0e6)
    assert cos.shape == (2, 8) and np.array_equal(cos[:, :4], cos[:, 4:]) and np.array_equal(sin[:, :4], sin[:, 4:])
    angle = 4.0 * (1.0e6 ** (-2.0 * 1 / 8.0))
    assert cos[1, 1] == oracle.bf16_round(np.array([np.cos(angle)], np.float32))[1][0]
    assert sin[1, 5] == oracle.bf16_round(np.array([np.sin(angle)], np.float32))[1][0]
    assert cos[0, 0] == oracle.bf16_round(np.array([np.cos(3.0)], np.float32))[1][0]


def test_full_attention_known_answer_of_the_reference(oracle):
    # tests/unit/minimax_h3.c:641-681
    qkv = np.array([[1, 0, 1, 0, 1, 2], [0, 1, 0, 1, 3, 4]], np.float32)
    selected = np.exp(np.float32(1.0) / np.sqrt(np.float32(2.0)))
    first = (selected * 1.0 + 3.0) / (selected + 1.0)
    out = oracle.full_attention_f32(qkv, 1, 2)
    assert abs(out[0, 0] - first) < 1e-6 and abs(out[0, 1] - (first + 1.0)) < 1e-6
