"""Seeded rows for the activation fake-quantisation tests: magnitudes from subnormal to
huge, signed zeros, exact half-way values of both number formats, and blocks that are
entirely tiny (the scale floor)."""
import numpy as np

# quantisation, block width, Hadamard transform, lanes per row
CASES = [(8, 64, 0, 448), (4, 32, 1, 128), (8, 64, 0, 64), (4, 32, 1, 96), (4, 32, 0, 512), (8, 64, 1, 512),
         (8, 128, 0, 128), (4, 16, 1, 48)]


def rows(seed, count, n=24):
    rng = np.random.Generator(np.random.PCG64(seed))
    x = rng.standard_normal((n, count)).astype(np.float32)
    x[1] *= np.float32(1e-3)
    x[2] *= np.float32(300.0)
    x[3] *= np.float32(1e-30)
    x[4] *= np.float32(1e20)
    x[5] = np.round(x[5] * 4) / 4                 # quarters: FP4 half-way points
    x[6] = np.round(x[6] * 16) / 16 * 28          # multiples of 1.75: FP8 half-way points after scaling
    x[7, : count // 2] = 0.0
    x[7, 1] = -0.0
    x[8] = 0.0                                    # the scale floor
    x[9] *= np.float32(1e-42)                     # subnormal lanes
    x[10, 0] = np.float32(3.0e38)
    return x
