"""The CPU checker of the rolling compressor: bit-equal to the reference's own compiled
code on random inputs, equal to the reference-made fixtures, and right on cases whose
answer is known in closed form."""
import os

import numpy as np
import pytest

import clori_b200
from compressor_cases import CASES, build
from oracle.binding import PositionPolicy, compressor_initial_state

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "compressor.npz")


def feed(run, chunks, case, **kw):
    kv, score = case["state"]
    rows, positions, start = [], [], 0
    for n in chunks:
        got = run(start, case["token_kv"][start:start + n], case["token_score"][start:start + n], kv, score, **kw)
        assert got is not None
        rows.append(got[0]), positions.append(got[1])
        kv, score, start = got[2], got[3], start + n
    return np.concatenate(rows), np.concatenate(positions), kv, score


def test_checker_equals_the_reference_fixtures(oracle):
    g = np.load(GOLDEN)
    for i in range(int(g["count"])):
        kind, ratio, hd, overlap, rope = (int(x) for x in g[f"meta{i}"])
        f32 = lambda name: clori_b200.bf16_bits_to_f32(g[f"{name}_{i}"])
        case = dict(token_kv=f32("token_kv"), token_score=f32("token_score"),
                    state=compressor_initial_state(ratio, hd, overlap))
        run = lambda start, tk, ts, kv, sc: oracle.compressor_chunk(
            ratio, hd, overlap, start, tk, ts, f32("ape"), kv, sc, f32("norm"), float(g["epsilon"]), rope,
            g[f"frequency{i}"])
        rows, positions, kv, score = feed(run, g[f"chunks{i}"], case)
        assert np.array_equal(rows.view(np.uint32), clori_b200.bf16_bits_to_f32(g[f"rows{i}"]).view(np.uint32))
        assert np.array_equal(positions, g[f"positions{i}"])
        assert np.array_equal(kv.view(np.uint32), g[f"state_kv{i}"].view(np.uint32))
        assert np.array_equal(score.view(np.uint32), g[f"state_score{i}"].view(np.uint32))
        # one chunk or many: the same rows and the same state
        whole = feed(run, [int(g[f"chunks{i}"].sum())], case)
        assert np.array_equal(whole[0], rows) and np.array_equal(whole[2], kv) and np.array_equal(whole[3], score)


@pytest.mark.parametrize("case_index", range(len(CASES)))
@pytest.mark.parametrize("published", [False, True])
def test_checker_equals_reference_code_on_random_inputs(oracle, reference, case_index, published):
    kind, ratio, hd, overlap, rope, policy, chunks = CASES[case_index]
    case = build(77 + case_index, ratio, hd, overlap, chunks)
    pol = PositionPolicy(*policy)
    freq = oracle.rope_frequencies(pol, rope)
    norm = case["norm"] if published else None
    mine = feed(lambda start, tk, ts, kv, sc: oracle.compressor_chunk(
        ratio, hd, overlap, start, tk, ts, case["ape"], kv, sc, norm, 1e-6, rope, freq), chunks, case)
    theirs = feed(lambda start, tk, ts, kv, sc: reference.compressor_chunk(
        kind, ratio, hd, overlap, start, tk, ts, case["ape"], kv, sc, norm, 1e-6, rope, pol), chunks, case)
    for a, b in zip(mine, theirs):
        assert a.shape == b.shape and np.array_equal(a.view(np.uint8), b.view(np.uint8))


def test_known_answers(oracle):
    # equal scores: the emitted lane is the plain mean of the group's values
    ratio, hd = 4, 8
    kv0, sc0 = compressor_initial_state(ratio, hd, 0)
    tk = np.arange(ratio * hd, dtype=np.float32).reshape(ratio, hd)
    rows, positions, kv, score = oracle.compressor_chunk(ratio, hd, 0, 0, tk, np.zeros_like(tk),
                                                        np.zeros((ratio, hd), np.float32), kv0, sc0)
    assert np.array_equal(rows[0], tk.mean(axis=0)) and list(positions) == [0]
    assert np.array_equal(kv, tk)                    # without a second half the ring keeps its rows
    # a dominant score picks its row; the position row is added to the score
    ape = np.zeros((ratio, hd), np.float32)
    ape[2] = 200.0
    rows = oracle.compressor_chunk(ratio, hd, 0, 0, tk, np.zeros_like(tk), ape, kv0, sc0)[0]
    assert np.array_equal(rows[0], tk[2])
    # two halves: the first emission sees only the current half (the previous half is at minus infinity),
    # the second mixes lanes [0, hd) of the first group with lanes [hd, 2 hd) of the second
    kv0, sc0 = compressor_initial_state(ratio, hd, 1)
    tk = np.arange(2 * ratio * 2 * hd, dtype=np.float32).reshape(2 * ratio, 2 * hd)
    rows, positions, kv, score = oracle.compressor_chunk(ratio, hd, 1, 0, tk, np.zeros_like(tk),
                                                        np.zeros((ratio, 2 * hd), np.float32), kv0, sc0)
    assert list(positions) == [0, 4]
    assert np.array_equal(rows[0], tk[:ratio, hd:].mean(axis=0))
    assert np.array_equal(rows[1], np.concatenate([tk[:ratio, :hd], tk[ratio:, hd:]]).mean(axis=0))
    assert np.array_equal(kv[:ratio], tk[ratio:]) and np.array_equal(kv[ratio:], tk[ratio:])


def test_refusals(oracle):
    ratio, hd = 4, 8
    kv0, sc0 = compressor_initial_state(ratio, hd, 0)
    tk = np.ones((ratio, hd), np.float32)
    ape = np.zeros((ratio, hd), np.float32)
    bad = tk.copy()
    bad[1, 3] = np.nan
    assert oracle.compressor_chunk(ratio, hd, 0, 0, bad, tk, ape, kv0, sc0) is None
    assert oracle.compressor_chunk(ratio, hd, 0, 0, tk, bad, ape, kv0, sc0) is None
    assert oracle.compressor_chunk(ratio, hd, 0, 0, tk, tk, ape, kv0, sc0, np.ones(hd, np.float32), 0.0) is None
    # no tokens: nothing emitted, the state is handed through
    got = oracle.compressor_chunk(ratio, hd, 0, 0, np.zeros((0, hd), np.float32), np.zeros((0, hd), np.float32),
                                  ape, kv0, sc0)
    assert got is not None and len(got[1]) == 0 and np.array_equal(got[2], kv0)
