"""Generates tests/golden/*.npz from the REFERENCE's own compiled CPU code.

Run in a container where the reference tree is mounted (it builds
oracle/_ref/libyvex_ref.so from the reference sources and calls only that):

    python tests/golden/make_golden.py

The fixtures are small seeded input/output pairs of yvex_backend_op_attention
(looped per head for grouped-query cases) and of the bf16 / f16 / Q8_0 codecs.
The oracle restatement and the CUDA path are both tested against them.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle.binding import Reference, build_oracle  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    build_oracle()
    ref = Reference()
    rng = np.random.Generator(np.random.PCG64(20261125))

    # --- primitive: one head, one query ----------------------------------
    prim = {}
    for i, (seq, hd, position, causal, scale) in enumerate(
            [(3, 4, 2, 1, 0.5), (17, 64, 9, 1, 0.125), (40, 128, 39, 1, 0.0883883), (33, 96, 0, 0, 0.1)]):
        q = rng.standard_normal(hd, dtype=np.float32)
        k = rng.standard_normal((seq, hd), dtype=np.float32)
        v = rng.standard_normal((seq, hd), dtype=np.float32)
        rc, out, scores, probs = ref.op_attention(q, k, v, position, scale, causal)
        assert rc == 0
        prim.update({f"q{i}": q, f"k{i}": k, f"v{i}": v, f"out{i}": out, f"scores{i}": scores,
                     f"probs{i}": probs,
                     f"meta{i}": np.array([seq, hd, position, causal], np.int64),
                     f"scale{i}": np.float32(scale)})
    prim["count"] = np.int64(4)
    np.savez_compressed(os.path.join(HERE, "op_attention.npz"), **prim)

    # --- grouped-query cases: (Tq, Tkv, qstart, Hq, Hkv, hd, causal) -------
    gqa = {}
    cases = [(1, 96, 95, 8, 2, 128, 1), (4, 70, 66, 8, 2, 128, 1), (5, 5, 0, 4, 4, 64, 1),
             (3, 50, 10, 6, 3, 32, 0), (2, 70, 68, 40, 8, 128, 1), (8, 100, 92, 10, 2, 128, 1),
             (1, 40, 39, 24, 4, 256, 1)]
    for i, (tq, tkv, qs, hq, hkv, hd, causal) in enumerate(cases):
        q = rng.standard_normal((tq, hq * hd), dtype=np.float32)
        k = rng.standard_normal((tkv, hkv * hd), dtype=np.float32)
        v = rng.standard_normal((tkv, hkv * hd), dtype=np.float32)
        out = ref.gqa_attention(q, k, v, qs, hq, hkv, hd, causal=bool(causal), threads=4)
        gqa.update({f"q{i}": q, f"k{i}": k, f"v{i}": v, f"out{i}": out,
                    f"meta{i}": np.array([tq, tkv, qs, hq, hkv, hd, causal], np.int64)})
    gqa["count"] = np.int64(len(cases))
    np.savez_compressed(os.path.join(HERE, "gqa_attention.npz"), **gqa)

    # --- codecs -------------------------------------------------------------
    values = np.concatenate([
        rng.standard_normal(2000, dtype=np.float32) * np.float32(10.0) ** rng.integers(-12, 12, 2000).astype(np.float32),
        np.array([0.0, -0.0, 1.0, -1.0, 65504.0, 65520.0, 1e-8, 5.96e-8, 6.1e-5, np.inf, -np.inf,
                  np.nan, 1.00390625, 1.01171875, 3.3895314e38], np.float32)])
    bf16 = np.array([ref.bf16_encode(x) for x in values], np.uint16)
    f16 = np.array([ref.f16_encode(x) for x in values], np.uint16)
    f16_all = np.array([ref.f16_decode(b) for b in range(65536)], np.float32)
    blocks = rng.standard_normal((64, 32), dtype=np.float32) * np.float32(3.0)
    blocks[0] = 0.0
    q8 = np.stack([ref.q8_0_encode_block(b) for b in blocks])
    q8_dec = np.stack([ref.q8_0_decode_block(e) for e in q8])
    np.savez_compressed(os.path.join(HERE, "codecs.npz"), values=values, bf16=bf16, f16=f16,
                        f16_decode_all=f16_all, q8_source=blocks, q8_encoded=q8, q8_decoded=q8_dec)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
