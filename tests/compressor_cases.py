"""Seeded inputs for the rolling-compressor tests: bf16-valued projected rows (the
projection stage publishes bf16-representable values), position rows, norm weights,
and the state a session starts from."""
import numpy as np

import clori_b200

from latent_cases import bf16_valued
from oracle.binding import compressor_initial_state

# kind (1 main rows, 2 index rows), ratio, head_dim, overlap, rope dims, position policy,
# chunk lengths fed one after another from position 0
CASES = [
    (1, 4, 512, 1, 64, (10000, 16, 65536, 32, 1), (3, 1, 9, 8)),      # sparse class, main rows
    (2, 4, 128, 1, 64, (10000, 0, 0, 0, 0), (5, 4, 1, 1, 1, 1, 7)),   # sparse class, index rows
    (1, 128, 64, 0, 16, (10000, 16, 65536, 32, 1), (100, 28, 1, 130, 255)),  # dense compressed class
    (1, 8, 96, 0, 32, (10000, 0, 0, 0, 0), (8, 16, 3)),               # chunks that end on a boundary
]


def rounded(x):
    return clori_b200.bf16_bits_to_f32(clori_b200.f32_to_bf16_bits(x))


def build(seed, ratio, head_dim, overlap, chunks):
    rng = np.random.Generator(np.random.PCG64(seed))
    width = head_dim * (2 if overlap else 1)
    total = int(sum(chunks))
    return dict(token_kv=bf16_valued(rng, (total, width)), token_score=bf16_valued(rng, (total, width), 2.0),
                ape=bf16_valued(rng, (ratio, width), 0.5), norm=rounded(bf16_valued(rng, (head_dim,), 0.25) + np.float32(1.0)),
                state=compressor_initial_state(ratio, head_dim, overlap))
