"""Generates tests/golden/activation_quant.npz from the REFERENCE's own compiled CPU code
(yvex_attention_activation_apply, built into oracle/_ref/libyvex_ref.so from the reference
sources):

    python tests/golden/make_activation_golden.py

Each case stores its seeded rows and the rows the reference made of them.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
from activation_cases import CASES, rows  # noqa: E402
from oracle.binding import Reference, build_oracle  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    build_oracle()
    ref = Reference()
    out = {"count": np.int64(len(CASES))}
    for i, (quantization, block, hadamard, count) in enumerate(CASES):
        x = rows(20261127 + i, count)
        y = ref.activation_quant(x, quantization, block, hadamard)
        assert y is not None
        out[f"meta{i}"] = np.array([quantization, block, hadamard, count], np.int64)
        out[f"in{i}"], out[f"out{i}"] = x, y
    np.savez_compressed(os.path.join(HERE, "activation_quant.npz"), **out)
    print("wrote", os.path.join(HERE, "activation_quant.npz"))


if __name__ == "__main__":
    main()
