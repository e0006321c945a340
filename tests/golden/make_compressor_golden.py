"""Generates tests/golden/compressor.npz from the REFERENCE's own compiled CPU code
(yvex_attention_rolling_state_step_cpu once per token and, on each emission, its
yvex_attention_compute_round / yvex_attention_rms_norm / yvex_attention_rope_apply,
built into oracle/_ref/libyvex_ref.so from the reference sources):

    python tests/golden/make_compressor_golden.py

Each case feeds its chunks one after another from position 0 and stores the seeded
inputs (bf16-valued arrays as bf16 bits), the frequencies of its position policy, and
what the reference computed: every published row with its position and the state
after the last chunk.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import clori_b200  # noqa: E402
from compressor_cases import CASES, build  # noqa: E402
from oracle.binding import Oracle, PositionPolicy, Reference, build_oracle  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
EPSILON = 1e-6


def main():
    build_oracle()
    ref, oracle = Reference(), Oracle()
    out = {"count": np.int64(len(CASES)), "epsilon": np.float64(EPSILON)}
    for i, (kind, ratio, hd, overlap, rope, policy, chunks) in enumerate(CASES):
        case = build(20261126 + i, ratio, hd, overlap, chunks)
        pol = PositionPolicy(*policy)
        kv, score = case["state"]
        rows, positions, start = [], [], 0
        for n in chunks:
            got = ref.compressor_chunk(kind, ratio, hd, overlap, start, case["token_kv"][start:start + n],
                                       case["token_score"][start:start + n], case["ape"], kv, score,
                                       case["norm"], EPSILON, rope, pol)
            assert got is not None
            rows.append(got[0]), positions.append(got[1])
            kv, score, start = got[2], got[3], start + n
        out[f"meta{i}"] = np.array([kind, ratio, hd, overlap, rope], np.int64)
        out[f"policy{i}"] = np.array(policy, np.int64)
        out[f"chunks{i}"] = np.array(chunks, np.int64)
        out[f"frequency{i}"] = oracle.rope_frequencies(pol, rope)
        for name in ("token_kv", "token_score", "ape", "norm"):
            out[f"{name}_{i}"] = clori_b200.f32_to_bf16_bits(case[name])
        out[f"rows{i}"] = clori_b200.f32_to_bf16_bits(np.concatenate(rows))   # published rows are bf16 values
        assert np.array_equal(clori_b200.bf16_bits_to_f32(out[f"rows{i}"]), np.concatenate(rows))
        out[f"positions{i}"] = np.concatenate(positions)
        out[f"state_kv{i}"], out[f"state_score{i}"] = kv, score
    np.savez_compressed(os.path.join(HERE, "compressor.npz"), **out)
    print("wrote", os.path.join(HERE, "compressor.npz"))


if __name__ == "__main__":
    main()
