"""The CPU checker of the publication chain of projected rows: bit-equal to the reference's
own compiled functions applied in the reference's order, and to the reference-made fixtures."""
import os

import numpy as np
import pytest

from oracle.binding import PositionPolicy
from publish_cases import CASES, POLICY, build

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "rows_publish.npz")


def same_bits(a, b):
    return a is not None and b is not None and a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_checker_equals_the_reference_fixtures(oracle):
    g = np.load(GOLDEN)
    for i, (name, width, rpt, tokens, start, chain) in enumerate(CASES):
        freq = g[f"frequency{i}"] if chain.get("rope_dims") else None
        got = oracle.rows_publish(g[f"in{i}"], rpt, start, norm_weights=g[f"weights{i}"], rope_frequency=freq, **chain)
        assert same_bits(got, g[f"out{i}"]), name


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_checker_equals_reference_code(oracle, reference, case):
    name, width, rpt, tokens, start, chain = case
    pol = PositionPolicy(*POLICY)
    x, w = build(61 + width, width, rpt * tokens)
    freq = oracle.rope_frequencies(pol, chain["rope_dims"]) if chain.get("rope_dims") else None
    assert same_bits(oracle.rows_publish(x, rpt, start, norm_weights=w, rope_frequency=freq, **chain),
                     reference.rows_publish(x, rpt, start, policy=pol, norm_weights=w, **chain))


def test_known_answers_and_refusals(oracle):
    # unit norm of a constant row is 1 in every lane (epsilon aside), published as bf16
    x = np.full((2, 64), 3.0, np.float32)
    y = oracle.rows_publish(x, 1, 0, norm_mode=1, epsilon=1e-6)
    assert np.all(y == 1.0)
    # rotation at position 0 is the identity; rows_per_token spreads positions over rows
    freq = np.full(8, 0.5, np.float64)
    x = np.arange(4 * 32, dtype=np.float32).reshape(4, 32)
    y = oracle.rows_publish(x, 2, 0, rope_dims=16, rope_frequency=freq)
    assert np.array_equal(y[:2], x[:2]) and not np.array_equal(y[2:, 16:], x[2:, 16:])
    assert np.array_equal(y[2:, :16], x[2:, :16])
    # refusals: a non-finite lane, a zero epsilon, an activation width that is not whole blocks
    bad = x.copy()
    bad[1, 3] = np.nan
    assert oracle.rows_publish(bad, 1, 0, norm_mode=1) is None
    assert oracle.rows_publish(x, 1, 0, norm_mode=1, epsilon=0.0) is None
    assert oracle.rows_publish(x, 1, 0, quantization=8, activation_count=24, block_width=16) is None
