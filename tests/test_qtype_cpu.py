"""Pins the CPU restatement of the encoded-row decode and row dot (the arithmetic of the
attention job's projections) to the reference's own compiled yvex_quant_decode_block and
yvex_quant_cpu_dot (src/gguf/quant_block.c:780-832, src/gguf/quant_compute.c:116-181).
Bit-exact."""
import numpy as np
import pytest

from clori_b200 import abi

QTYPES = [abi.QTYPE_F32, abi.QTYPE_F16, abi.QTYPE_BF16, abi.QTYPE_Q8_0]


@pytest.mark.parametrize("qtype", QTYPES)
def test_decode_and_dot_equal_the_reference(oracle, reference, qtype):
    rng = np.random.default_rng(20 + qtype)
    for width in (32, 96, 1024):
        values = rng.standard_normal((5, width)).astype(np.float32) * np.float32(10.0) ** rng.integers(-3, 3, (5, 1)).astype(np.float32)
        encoded = oracle.qtype_encode_rows(values, qtype)
        decoded = oracle.qtype_decode_rows(encoded, qtype, width)
        vectors = rng.standard_normal((3, width)).astype(np.float32)
        products = oracle.qtype_matvec(encoded, qtype, width, vectors, round_bf16=False)
        rounded = oracle.qtype_matvec(encoded, qtype, width, vectors, round_bf16=True)
        for r in range(5):
            assert np.array_equal(decoded[r].view(np.uint32), reference.qtype_decode_row(encoded[r], qtype, width).view(np.uint32))
            for t in range(3):
                want = np.float32(reference.qtype_dot(encoded[r], qtype, vectors[t]))
                assert products[t, r].view(np.uint32) == want.view(np.uint32)
                assert rounded[t, r] == oracle.bf16_round(np.array([want], np.float32))[1][0]


def test_refusals_follow_the_reference(oracle, reference):
    width = 64
    encoded = oracle.qtype_encode_rows(np.ones((1, width), np.float32), abi.QTYPE_Q8_0)
    bad = encoded.copy()
    bad[0, 0:2] = np.array([0x00, 0xBC], np.uint8)          # f16 -1.0: a negative block scale
    vector = np.ones(width, np.float32)
    assert reference.qtype_dot(bad[0], abi.QTYPE_Q8_0, vector) is None
    assert oracle.qtype_matvec(bad, abi.QTYPE_Q8_0, width, vector[None]) is None
    inf = oracle.qtype_encode_rows(np.full((1, width), np.inf, np.float32), abi.QTYPE_F32)
    assert reference.qtype_dot(inf[0], abi.QTYPE_F32, vector) is None
    assert oracle.qtype_matvec(inf, abi.QTYPE_F32, width, vector[None]) is None
    # a row width that is not a multiple of the block
    assert oracle.lib.yvx_oracle_qtype_row_bytes(abi.QTYPE_Q8_0, 40) == 0
