"""Generates tests/golden/latent_attention.npz from the REFERENCE's own compiled CPU
code (yvex_attention_reduce_chunk and what it calls, built into
oracle/_ref/libyvex_ref.so from the reference sources):

    python tests/golden/make_latent_golden.py

Each case stores its seeded inputs (bf16-valued arrays as bf16 bits), the position
policy with the frequencies it yields, and what the reference computed: the
published output of the phase and, for the sparse class, how many rows each token
selected and their positions in ranked order.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import clori_b200  # noqa: E402
from latent_cases import build, host_args  # noqa: E402
from oracle.binding import Oracle, PositionPolicy, Reference, build_oracle, indexer_struct  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = [  # heads, hd, class, tokens, start, topk, index heads, index dim, rope dims, policy
    (4, 64, 0, 3, 300, 8, 0, 0, 16, (10000, 0, 0, 0, 0)),
    (4, 64, 2, 2, 1023, 8, 0, 0, 16, (10000, 16, 65536, 32, 1)),
    (4, 64, 1, 3, 301, 8, 4, 32, 16, (10000, 16, 65536, 32, 1)),
    (8, 128, 1, 2, 90, 64, 4, 32, 32, (10000, 0, 0, 0, 0)),
    (4, 512, 1, 1, 2301, 512, 64, 128, 64, (10000, 16, 65536, 32, 1)),
]


def main():
    build_oracle()
    ref, oracle = Reference(), Oracle()
    out = {"count": np.int64(len(CASES))}
    for i, (heads, hd, cls, tokens, start, topk, ih, idim, rope, policy) in enumerate(CASES):
        rng = np.random.Generator(np.random.PCG64(20261125 + i))
        case = build(rng, heads, hd, 128, cls, tokens, start, topk=topk, index_heads=ih, index_dim=idim,
                     rope_dims=rope)
        pol = PositionPolicy(*policy)
        # the frequencies are inputs of the restatement's rotation; the reference derives its own
        freq = oracle.rope_frequencies(pol, rope)
        ix = None
        if cls == 1:
            ix = indexer_struct(case["index_keys"][:case["compressed_rows"]],
                                case["compressed_positions"][:case["compressed_rows"]], case["index_query"],
                                case["index_weights"], ih, idim, topk, case["ratio"])
        result = ref.latent_reduce_chunk(host_args(case, frequency=freq), case["compressed_rows"], pol, ix,
                                         tokens, heads, hd)
        assert result is not None
        published, counts, positions = result
        out[f"meta{i}"] = np.array([heads, hd, cls, tokens, start, topk, ih, idim, rope], np.int64)
        out[f"policy{i}"] = np.array(policy, np.int64)
        out[f"frequency{i}"] = freq
        out[f"rows{i}"] = np.int64(case["compressed_rows"])
        out[f"out{i}"], out[f"counts{i}"], out[f"positions{i}"] = published, counts, positions
        for name in ("query", "local", "compressed", "index_keys", "index_query", "index_weights"):
            if name in case:
                out[f"{name}_{i}"] = clori_b200.f32_to_bf16_bits(case[name])
        for name in ("local_positions", "compressed_positions", "sinks"):
            out[f"{name}_{i}"] = case[name]
    np.savez_compressed(os.path.join(HERE, "latent_attention.npz"), **out)
    print("written", os.path.join(HERE, "latent_attention.npz"))


if __name__ == "__main__":
    main()
