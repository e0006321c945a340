"""Seeded rows for the tests of the publication chain of projected rows: the three uses the
reference makes of it, and chains without some of their steps."""
import numpy as np

from latent_cases import bf16_valued

POLICY = (10000, 16, 65536, 32, 1)
# name, width, rows per token, tokens, start position, chain
CASES = [
    ("query_heads", 512, 64, 3, 1000, dict(norm_mode=1, rope_dims=64)),
    ("local_rows", 512, 1, 40, 70000, dict(norm_mode=2, rope_dims=64, quantization=8, activation_count=448,
                                           block_width=64)),
    ("index_queries", 128, 64, 3, 999983, dict(rope_dims=64, quantization=4, activation_count=128, block_width=32,
                                               hadamard=1)),
    ("query_low_norm", 1024, 1, 9, 0, dict(norm_mode=2)),
    ("narrow_heads", 192, 4, 5, 12, dict(norm_mode=1, rope_dims=32, quantization=8, activation_count=128,
                                         block_width=32)),
]


def build(seed, width, rows):
    rng = np.random.Generator(np.random.PCG64(seed))
    return bf16_valued(rng, (rows, width)), bf16_valued(rng, (width,), 0.25) + np.float32(1.0)
