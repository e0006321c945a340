"""The CPU checker of the activation fake quantisation: bit-equal to the reference's own
compiled code on seeded rows, equal to the reference-made fixtures, right on known answers."""
import os

import numpy as np
import pytest

from activation_cases import CASES, rows

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "activation_quant.npz")


def same_bits(a, b):
    return a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_checker_equals_the_reference_fixtures(oracle):
    g = np.load(GOLDEN)
    for i in range(int(g["count"])):
        quantization, block, hadamard, count = (int(x) for x in g[f"meta{i}"])
        assert same_bits(oracle.activation_quant(g[f"in{i}"], quantization, block, hadamard), g[f"out{i}"])


@pytest.mark.parametrize("case", CASES)
def test_checker_equals_reference_code(oracle, reference, case):
    quantization, block, hadamard, count = case
    x = rows(41 + count, count, n=64)
    assert same_bits(oracle.activation_quant(x, quantization, block, hadamard),
                     reference.activation_quant(x, quantization, block, hadamard))


def test_known_answers(oracle):
    # FP4: amax 6 -> scale 1; values on the grid survive, half-way values go to the even code
    x = np.array([[6.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -5.0, 0.0, -0.0, 1.0, 3.0, 4.0, 0.5]], np.float32)
    y = oracle.activation_quant(x, 4, 16, 0)
    assert np.array_equal(y[0], np.array([6, 0, 1, 1, 2, 2, 4, 4, -0.0, -4, 0, -0.0, 1, 3, 4, 0.5], np.float32))
    assert np.signbit(y[0, 8]) and np.signbit(y[0, 11]) and not np.signbit(y[0, 10])
    # FP8: amax 448 -> scale 1; 17 lies half-way between 16 and 18 (codes with mantissa 0 and 1): even code
    x = np.zeros((1, 64), np.float32)
    x[0, :6] = [448.0, 17.0, 19.0, 0.001, 1.0, -240.0]
    y = oracle.activation_quant(x, 8, 64, 0)
    assert list(y[0, :6]) == [448.0, 16.0, 20.0, 2.0 ** -9, 1.0, -240.0]   # 0.001 -> one step of 2^-9
    # a power-of-two amax/limit keeps its scale; anything above moves to the next power of two
    x = np.zeros((1, 64), np.float32)
    x[0, 0], x[0, 1] = 448.0 * 2, 2.0
    assert oracle.activation_quant(x, 8, 64, 0)[0, 1] == 2.0
    x[0, 0] = np.nextafter(np.float32(896.0), np.float32(1e9))
    y = oracle.activation_quant(x, 8, 64, 0)
    assert y[0, 0] == 896.0 and y[0, 1] == 2.0      # scale 4: 224.00002 -> 224, 0.5 -> 0.5
    # Hadamard of a unit impulse: every lane 1/sqrt(n); of a constant: n/sqrt(n) in lane 0
    x = np.zeros((1, 32), np.float32)
    x[0, 0] = 1.0
    y = oracle.activation_quant(x, 4, 32, 1)
    assert np.all(y[0] == y[0, 0]) and abs(float(y[0, 0]) - 32 ** -0.5) < 0.05
    # refusals: a row that is not a whole number of blocks, a non-finite lane
    assert oracle.activation_quant(np.ones((1, 100), np.float32), 8, 64, 0) is None
    bad = np.ones((1, 64), np.float32)
    bad[0, 5] = np.inf
    assert oracle.activation_quant(bad, 8, 64, 0) is None and oracle.activation_quant(bad, 4, 32, 1) is None
