"""The tensor-core projection (tcgen05 GEMM over BF16 weight rows) against the CPU twin of the
reference's projection (exact products summed in double, narrowed, published as bf16): a published
value may differ by one bf16 step where the exact sum sits an F32 rounding away from a tie; the
unpublished F32 sums agree to F32 accumulation accuracy."""
import ctypes as C

import numpy as np
import pytest

from clori_b200 import abi
import job_cases

pytestmark = pytest.mark.gpu


def bf16_step(x):
    """The spacing of bf16 values at |x| (8 significant bits)."""
    return np.exp2(np.floor(np.log2(np.maximum(np.abs(x), 1e-30))) - 7.0)


@pytest.mark.parametrize("tokens,rows,width,groups", [(128, 128, 64, 1), (300, 200, 1024, 1), (130, 96, 320, 3),
                                                      (1000, 520, 4096, 1), (64, 136, 72, 2)])
def test_gemm_matches_the_cpu_projection(backend, oracle, tokens, rows, width, groups):
    rng = np.random.default_rng(tokens + rows + width)
    values = job_cases.bf16_valued(rng, (rows * groups + 5, width), 1.0 / np.sqrt(width))
    encoded = oracle.qtype_encode_rows(values, abi.QTYPE_BF16)
    stride = groups * width + 6
    x = job_cases.bf16_valued(rng, (tokens, stride))
    first_row = 5
    w, xi = backend.tensor("w", encoded.view(np.int8), dtype=abi.DTYPE_I8), backend.tensor("x", x)
    out = backend.alloc("y", abi.DTYPE_F32, (tokens, groups * rows + 3))
    status = backend.tensor("status", np.zeros(1, np.int32))
    staging = backend.alloc("staging", abi.DTYPE_I8,
                            (backend.lib.yvx_cuda_bf16_gemm_staging_bytes(tokens, groups, width),))
    for rounded in (0, 1):
        a = abi.GemmArgs()
        a.weights, a.first_row, a.rows, a.width = w.data_ptr, first_row, rows, width
        a.input, a.tokens, a.input_stride = xi.data_ptr, tokens, stride
        a.output, a.output_stride, a.groups, a.round_bf16 = out.data_ptr, groups * rows + 3, groups, rounded
        a.staging, a.status = staging.data_ptr, status.data_ptr
        assert backend.lib.yvx_cuda_bf16_gemm(C.byref(a), backend.stream) == 0, backend.lib.yvx_cuda_last_error_text()
        assert backend.lib.yvx_cuda_stream_synchronize(backend.stream) == 0, backend.lib.yvx_cuda_last_error_text()
        out.struct.is_written = 1
        got = out.read()[:, :groups * rows]
        want = np.concatenate([oracle.qtype_matvec(encoded, abi.QTYPE_BF16, width,
                                                   np.ascontiguousarray(x[:, k * width:(k + 1) * width]),
                                                   first_row + k * rows, rows, bool(rounded)) for k in range(groups)], axis=1)
        assert int(status.read()[0]) == 0
        # F32 accumulation error of a sum of `width` exact products
        scale = np.sqrt(width) * np.abs(values).max() * np.abs(x).max()
        if rounded:
            differing = got != want
            # one bf16 step of the larger value, plus the accumulation error for sums near zero
            assert np.all(np.abs(got - want) <= bf16_step(np.maximum(np.abs(got), np.abs(want))) * 1.0001 + 2e-6 * scale)
            assert differing.mean() <= 0.01, differing.mean()
        else:
            assert np.abs(got - want).max() <= 2e-6 * scale + 1e-6 * np.abs(want).max()


def test_gemm_refuses_activations_bf16_cannot_hold(backend, oracle):
    rng = np.random.default_rng(5)
    tokens, rows, width = 128, 128, 64
    encoded = oracle.qtype_encode_rows(job_cases.bf16_valued(rng, (rows, width)), abi.QTYPE_BF16)
    x = job_cases.bf16_valued(rng, (tokens, width))
    x[7, 9] = np.float32(1.0) + np.float32(2.0 ** -12)
    w, xi = backend.tensor("w", encoded.view(np.int8), dtype=abi.DTYPE_I8), backend.tensor("x", x)
    out = backend.alloc("y", abi.DTYPE_F32, (tokens, rows))
    status = backend.tensor("status", np.zeros(1, np.int32))
    staging = backend.alloc("staging", abi.DTYPE_I8, (backend.lib.yvx_cuda_bf16_gemm_staging_bytes(tokens, 1, width),))
    a = abi.GemmArgs()
    a.weights, a.rows, a.width, a.input, a.tokens, a.input_stride = w.data_ptr, rows, width, xi.data_ptr, tokens, width
    a.output, a.output_stride, a.groups, a.round_bf16 = out.data_ptr, rows, 1, 1
    a.staging, a.status = staging.data_ptr, status.data_ptr
    assert backend.lib.yvx_cuda_bf16_gemm(C.byref(a), backend.stream) == 0
    assert backend.lib.yvx_cuda_stream_synchronize(backend.stream) == 0
    assert int(status.read()[0]) == 2
    a.width = 60          # not a multiple of 8
    assert backend.lib.yvx_cuda_bf16_gemm(C.byref(a), backend.stream) == abi.YVEX_ERR_BOUNDS
