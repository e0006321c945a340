"""Full (non-causal) attention over interleaved [row][head][Q | K | V][width] rows
(the reference's yvex_graph_full_attention_f32, src/graph/numeric.c:1771-1826) through
the plain-pointer entry: the layout is pure strides (query_head_stride = key_head_stride
= value_head_stride = 3 * width). Checked against the CPU restatement and the reference's
known answer (tests/unit/minimax_h3.c:641-681, tolerance 1e-6 there)."""
import numpy as np
import pytest

from clori_b200 import abi
from gqa_shim import run_problem

pytestmark = pytest.mark.gpu


def run_interleaved(backend, qkv, heads, width):
    rows = qkv.shape[0]
    t = backend.tensor("qkv", qkv)
    stride = 3 * heads * width
    out, status, launches, _ = run_problem(
        backend, q=t, k=t, v=t, lengths=[rows], rows=rows, hq=heads, hkv=heads, hd=width,
        dtype=abi.DTYPE_F32, causal=False, k_token_stride=stride, v_token_stride=stride,
        k_head_stride=3 * width, v_head_stride=3 * width, k_outer_stride=rows * stride,
        v_outer_stride=rows * stride, k_offset_elems=width, v_offset_elems=2 * width,
        q_row_stride=stride, q_head_stride=3 * width, query_start=[0])
    assert status == 0
    return out.reshape(rows, heads * width)


def test_known_answer_of_the_reference(backend, oracle):
    qkv = np.array([[1, 0, 1, 0, 1, 2], [0, 1, 0, 1, 3, 4]], np.float32)
    selected = np.exp(np.float32(1.0) / np.sqrt(np.float32(2.0)))
    first = (selected * 1.0 + 3.0) / (selected + 1.0)
    got = run_interleaved(backend, qkv, 1, 2)
    assert abs(got[0, 0] - first) < 1e-6 and abs(got[0, 1] - (first + 1.0)) < 1e-6
    ref = oracle.full_attention_f32(qkv, 1, 2)
    assert abs(ref[0, 0] - first) < 1e-6 and np.abs(got - ref).max() < 1e-6


@pytest.mark.parametrize("rows,heads,width", [(7, 3, 16), (200, 4, 64), (333, 2, 128)])
def test_matches_the_restatement(backend, oracle, rows, heads, width):
    rng = np.random.default_rng(rows + heads + width)
    qkv = rng.standard_normal((rows, heads * 3 * width)).astype(np.float32)
    got = run_interleaved(backend, qkv, heads, width)
    ref = oracle.full_attention_f32(qkv, heads, width)
    assert ref is not None
    assert np.all(np.abs(got - ref) <= 2e-5 * (1.0 + np.abs(ref)))
