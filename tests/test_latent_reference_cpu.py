"""Pins the CPU restatement of the shared-latent attention stage to the reference's
own compiled CPU code (src/graph/core.c, attention.c, numeric.c built into
oracle/_ref) and to the golden fixtures that code produced: the output rotation and
its frequencies, the ranked top-k, the sparse index selection and the whole reduce
of a phase (selection, two passes, publication, inverse rotation, publication).
Everything here is bit-exact."""
import ctypes as C
import os

import numpy as np
import pytest

import clori_b200
from latent_cases import bf16_valued, build, host_args
from oracle.binding import PositionPolicy, indexer_struct

u64 = np.uint64
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "latent_attention.npz")
PLAIN = (10000, 0, 0, 0, 0)
YARN = (10000, 16, 65536, 32, 1)      # theta, factor, original context, beta_fast, beta_slow


def test_rotation_known_answer_of_the_reference(oracle):
    # tests/reference/deepseek_attention.c:2690-2695: width 6, 2 rotated lanes, position 1, theta 10000
    freq = oracle.rope_frequencies(PositionPolicy(*PLAIN), 2)
    x = np.array([10, 20, 30, 40, 1, 2], np.float32)
    forward = oracle.rope_apply(x, 2, 1, freq, False)
    inverse = oracle.rope_apply(x, 2, 1, freq, True)
    assert np.abs(forward - np.array([10, 20, 30, 40, -1.1426396369934082, 1.922075629234314], np.float32)).max() <= 1e-6
    assert np.abs(inverse - np.array([10, 20, 30, 40, 2.2232441902160645, 0.23913362622261047], np.float32)).max() <= 1e-6


@pytest.mark.parametrize("policy", [PLAIN, YARN])
def test_rotation_equals_the_reference(oracle, reference, policy):
    rng = np.random.default_rng(3)
    pol = PositionPolicy(*policy)
    for width, rope, position in [(512, 64, 0), (512, 64, 1), (512, 64, 131071), (64, 16, 999983), (6, 2, 7), (9, 5, 3)]:
        x = bf16_valued(rng, width)
        freq = oracle.rope_frequencies(pol, rope)
        for inverse in (False, True):
            got, ref = oracle.rope_apply(x, rope, position, freq, inverse), reference.rope_apply(x, rope, position, pol, inverse)
            assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))


def test_topk_equals_the_reference(oracle, reference):
    rng = np.random.default_rng(4)
    for count, k in [(1, 1), (7, 3), (600, 512), (600, 700), (2048, 512)]:
        scores = rng.integers(-6, 6, count).astype(np.float32) / 4          # many ties
        scores[rng.integers(0, count, 3)] = -0.0
        ordinals = rng.permutation(count * 4)[:count].astype(u64)
        assert np.array_equal(oracle.topk_select(scores, ordinals, k), reference.topk_select(scores, ordinals, k))
    assert oracle.topk_select(np.array([1, np.nan], np.float32), np.array([0, 1], u64), 1) is None
    assert reference.topk_select(np.array([1, np.nan], np.float32), np.array([0, 1], u64), 1) is None
    assert oracle.topk_select(np.array([1, 2], np.float32), np.array([5, 5], u64), 1) is None
    assert reference.topk_select(np.array([1, 2], np.float32), np.array([5, 5], u64), 1) is None


def select_all(oracle, case):
    """Fills case['selected'] from the restated selection; returns the indexer struct."""
    ix = indexer_struct(case["index_keys"][:max(case["compressed_rows"], 0)].reshape(case["compressed_rows"], -1),
                        case["compressed_positions"][:case["compressed_rows"]], case["index_query"],
                        case["index_weights"], case["index_heads"], case["index_dim"], case["topk"], case["ratio"])
    for t in range(case["tokens"]):
        picked, valid, _ = oracle.csa_select(ix, t, case["start"] + t)
        case["selected_count"][t] = len(picked)
        case["selected"][t, :len(picked)] = picked
    return ix


CASES = [  # heads, hd, class, tokens, start, topk, index heads, index dim, rope dims
    (4, 64, 0, 3, 300, 8, 0, 0, 16),
    (4, 64, 2, 2, 1023, 8, 0, 0, 16),
    (4, 64, 1, 3, 301, 8, 4, 32, 16),
    (8, 128, 1, 2, 90, 64, 4, 32, 32),     # fewer candidates than k
    (6, 512, 1, 2, 2301, 512, 64, 128, 64),  # the reference configuration's widths, 575 candidates for 512
]


@pytest.mark.parametrize("case_id", range(len(CASES)))
@pytest.mark.parametrize("policy", [PLAIN, YARN])
def test_whole_reduce_equals_the_reference(oracle, reference, case_id, policy):
    heads, hd, cls, tokens, start, topk, ih, idim, rope = CASES[case_id]
    rng = np.random.default_rng(100 + case_id)
    case = build(rng, heads, hd, 128, cls, tokens, start, topk=topk, index_heads=ih, index_dim=idim, rope_dims=rope)
    pol = PositionPolicy(*policy)
    freq = oracle.rope_frequencies(pol, rope)
    ix = select_all(oracle, case) if cls == 1 else None
    got = oracle.latent_reduce_full(host_args(case, frequency=freq), tokens, heads, hd)
    ref = reference.latent_reduce_chunk(host_args(case, frequency=freq), case["compressed_rows"], pol, ix, tokens, heads, hd)
    assert got is not None and ref is not None
    out, counts, positions = ref
    assert np.array_equal(got.view(np.uint32), out.view(np.uint32))
    if cls == 1:
        assert np.array_equal(counts, case["selected_count"])
        for t in range(tokens):
            n = int(counts[t])
            assert np.array_equal(positions[t, :n], case["compressed_positions"][case["selected"][t, :n]])
            picked, valid = reference.csa_select(ix, t, start + t)
            assert np.array_equal(picked, case["selected"][t, :n]) and valid == (start + t + 1) // 4


def test_restatement_against_the_golden_fixtures(oracle):
    g = np.load(GOLDEN)
    for i in range(int(g["count"])):
        heads, hd, cls, tokens, start, topk, ih, idim, rope = (int(x) for x in g[f"meta{i}"])
        case = {k[:-len(str(i)) - 1]: g[k] for k in g.files if k.endswith(f"_{i}")}
        for name in ("query", "local", "compressed", "index_keys", "index_query", "index_weights"):
            if name in case:
                case[name] = clori_b200.bf16_bits_to_f32(case[name])
        case.update(heads=heads, hd=hd, cls=cls, tokens=tokens, start=start, topk=topk, window=128,
                    ratio={0: 0, 1: 4, 2: 128}[cls], initial=min(start, 127), rope_dims=rope,
                    index_heads=ih, index_dim=idim, compressed_rows=int(g[f"rows{i}"]),
                    selected=np.zeros((tokens, topk), u64), selected_count=np.zeros(tokens, u64))
        freq = oracle.rope_frequencies(PositionPolicy(*(int(x) for x in g[f"policy{i}"])), rope)
        assert np.array_equal(freq, g[f"frequency{i}"])
        if cls == 1:
            select_all(oracle, case)
            assert np.array_equal(case["selected_count"], g[f"counts{i}"])
            for t in range(tokens):
                n = int(case["selected_count"][t])
                assert np.array_equal(case["compressed_positions"][case["selected"][t, :n]], g[f"positions{i}"][t, :n])
        got = oracle.latent_reduce_full(host_args(case, frequency=freq), tokens, heads, hd)
        assert np.array_equal(got.view(np.uint32), g[f"out{i}"].view(np.uint32))
