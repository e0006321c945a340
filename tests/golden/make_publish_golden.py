"""Generates tests/golden/rows_publish.npz from the REFERENCE's own compiled CPU code (its
yvex_attention_rms_norm / _unit_rms_norm, _compute_round, _rope_apply and _activation_apply in
the order its chunk executor applies them, built into oracle/_ref/libyvex_ref.so):

    python tests/golden/make_publish_golden.py

Each case stores its seeded rows, norm weights, the frequencies of the position policy and the
rows the reference published.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
from oracle.binding import Oracle, PositionPolicy, Reference, build_oracle  # noqa: E402
from publish_cases import CASES, POLICY, build  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    build_oracle()
    ref, oracle = Reference(), Oracle()
    pol = PositionPolicy(*POLICY)
    out = {"count": np.int64(len(CASES))}
    for i, (name, width, rpt, tokens, start, chain) in enumerate(CASES):
        x, w = build(20261128 + i, width, rpt * tokens)
        y = ref.rows_publish(x, rpt, start, policy=pol, norm_weights=w, **chain)
        assert y is not None, name
        out[f"in{i}"], out[f"weights{i}"], out[f"out{i}"] = x, w, y
        if chain.get("rope_dims"):
            out[f"frequency{i}"] = oracle.rope_frequencies(pol, chain["rope_dims"])
    np.savez_compressed(os.path.join(HERE, "rows_publish.npz"), **out)
    print("wrote", os.path.join(HERE, "rows_publish.npz"))


if __name__ == "__main__":
    main()
