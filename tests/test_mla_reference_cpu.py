"""Pins the CPU restatement of the split-rope latent decode (latent 512 + rope key 64,
absorbed up-projection) to the reference's own compiled CPU reduce
(yvex_attention_reduce_chunk, src/graph/core.c:608-701). The decode is a shared-row
K == V attention over rows [latent | rope key] of width 576, which the reference
computes as its window class with every row visible and sinks at -100
(tests/unit/deepseek_attention.c:593); the first 512 output lanes are the mix of latent
rows. The reference publishes bf16 (round to nearest even) of a single-precision
accumulation where the restatement returns the double-precision mix unrounded, so the
two agree to half a bf16 ulp of the published value (2^(exponent - 8), at most 2^-8
relative) plus the accumulation noise (3e-6 absolute)."""
import os

import numpy as np
import pytest

import clori_b200
from clori_b200 import workloads

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "mla_decode.npz")
SCALE = 1.0 / np.sqrt(192.0)
f = clori_b200.bf16_bits_to_f32


def published_close(restated, published):
    magnitude = np.abs(published).astype(np.float64)
    half_ulp = np.where(magnitude > 0, 2.0 ** (np.floor(np.log2(np.maximum(magnitude, 1e-300))) - 8), 0.0)
    bound = half_ulp + 3e-6
    return bool(np.all(np.abs(restated.astype(np.float64) - published) <= bound))


def golden_lengths(sessions, context):
    lengths = [context] * sessions
    if sessions > 1:
        lengths[1] = max(1, context - 37)
    return lengths


@pytest.mark.parametrize("seed,context", [(4, 17), (5, 300), (6, 1500)])
def test_restatement_equals_reference_reduce_on_the_embedding(oracle, reference, seed, context):
    qn, qr, w, lat, rk = workloads.mla_decode_bf16(seed=seed, batch=1, context=context)
    restated, absorbed = oracle.mla_decode(qn[0], qr[0], w, lat[0], rk[0], SCALE, with_absorbed=True)
    published = reference.mla_decode_embedded(absorbed, f(qr[0]), f(lat[0]), f(rk[0]))
    assert published is not None
    assert np.array_equal(f(clori_b200.f32_to_bf16_bits(published)), published)
    assert published_close(restated, published)


def test_restatement_equals_reference_made_fixtures(oracle):
    g = np.load(GOLDEN)
    for i in range(int(g["count"])):
        seed, sessions, context = (int(x) for x in g[f"meta{i}"])
        qn, qr, w, lat, rk = workloads.mla_decode_bf16(seed=seed, batch=sessions, context=context)
        for s, n in enumerate(golden_lengths(sessions, context)):
            restated, absorbed = oracle.mla_decode(qn[s], qr[s], w, lat[s, :n], rk[s, :n], SCALE,
                                                   with_absorbed=True)
            assert np.array_equal(clori_b200.f32_to_bf16_bits(absorbed), g[f"absorbed{i}_{s}"])
            assert published_close(restated, f(g[f"out{i}_{s}"]))


def test_sink_mass_and_scale_fold_are_negligible(oracle, reference):
    # the embedding's two approximations, measured: sinks at -100 add exp(-100 - max) to the
    # denominator, and sqrt(576/192) enters the query as one float multiply per lane.
    qn, qr, w, lat, rk = workloads.mla_decode_bf16(seed=9, batch=1, context=64)
    restated, absorbed = oracle.mla_decode(qn[0], qr[0], w, lat[0], rk[0], SCALE, with_absorbed=True)
    a = reference.mla_decode_embedded(absorbed, f(qr[0]), f(lat[0]), f(rk[0]))
    b = reference.mla_decode_embedded(absorbed, f(qr[0]), f(lat[0]), f(rk[0]), softmax_dim=576)
    plain = oracle.mla_decode(qn[0], qr[0], w, lat[0], rk[0], 1.0 / np.sqrt(576.0))
    assert published_close(restated, a) and published_close(plain, b)
