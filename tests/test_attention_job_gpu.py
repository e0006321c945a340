"""yvex_backend_attention_execute (the reference's encoded-attention job, schema 3) on a
B200 against the phase evaluated on the CPU in the order of the reference's CPU twin
(src/graph/attention_execute.c:452-1122), stage by stage through the job's output spans.

Bars. Projections accumulate exact products in double on both sides, so published rows
are bit-equal wherever no norm is involved; behind a norm (device sqrt and a tree-reduced
sum of squares against libm and a serial sum) at most 1 lane in 100 differs, by one bf16
ulp; the reduce carries the reference's CPU-vs-device tolerance (5e-4 absolute and
relative, src/graph/attention.c:919-920) plus one bf16 ulp; the output projections
inherit those differences through two rounded products: 2^-6 relative to the largest
output of the row plus 5e-4."""
import ctypes as C

import numpy as np
import pytest

from clori_b200 import abi
import job_cases

pytestmark = pytest.mark.gpu
CASES = [(abi.ATTENTION_SWA, 3, 40, 0), (abi.ATTENTION_SWA, 2, 0, 0), (abi.ATTENTION_CSA, 6, 37, 0),
         (abi.ATTENTION_CSA, 1, 3, 0), (abi.ATTENTION_CSA, 9, 0, 0), (abi.ATTENTION_HCA, 5, 252, 0),
         (abi.ATTENTION_HCA, 1, 700, 0), (abi.ATTENTION_CSA, 4, 64, 1)]


def ulp_lanes(got, want):
    """(lanes that differ, lanes that differ by more than one bf16 ulp)."""
    a, b = got.astype(np.float64).ravel(), want.astype(np.float64).ravel()
    ulp = np.where(b != 0, 2.0 ** (np.floor(np.log2(np.maximum(np.abs(b), 1e-300))) - 7), 2.0 ** -133)
    differ = a != b
    return int(differ.sum()), int((np.abs(a - b) > ulp * 1.0001).sum())


@pytest.mark.parametrize("cls,tokens,start,visible", CASES)
def test_job_matches_the_cpu_evaluation(backend, oracle, cls, tokens, start, visible):
    job = job_cases.build(oracle, cls, tokens, start, seed=100 + cls * 10 + tokens, block_visible=visible)
    want = job_cases.evaluate(oracle, job)
    rc, out, got, failure, err = job_cases.run(backend, job)
    assert rc == 0, (err.where, err.message, failure.stage)
    assert failure.code == abi.JOB_FAILURE_NONE and out.tokens_executed == tokens
    assert out.kernel_launches >= 10 and out.h2d_bytes > 0 and out.d2h_bytes > 0 and out.device_synchronizations == 1
    # projections without a norm in front of them: bit-equal
    assert np.array_equal(got["core_input"], want["core_input"])
    for name in ("index_weights",):
        if name in got:
            assert np.array_equal(got[name], want[name]), name
    # behind a norm: one bf16 ulp on at most 1 lane in 100
    for name in ("q_low", "query", "raw_kv", "index_query", "compressed_kv", "indexer_kv"):
        if name in got:
            differ, beyond = ulp_lanes(got[name], want[name])
            assert beyond == 0 and differ <= max(1, got[name].size // 100), (name, differ, beyond)
    for name in ("compressed_positions", "indexer_positions", "valid_candidate_counts"):
        if name in got:
            assert np.array_equal(got[name], want[name]), name
    for name in ("main_kv_state", "main_score_state", "indexer_kv_state", "indexer_score_state"):
        if name in got:
            assert np.array_equal(got[name].view(np.uint32), want[name].view(np.uint32)), name
    exact_inputs = all(np.array_equal(got[n], want[n]) for n in ("q_low", "query", "raw_kv", "index_query", "indexer_kv")
                       if n in got)
    if "topk_counts" in got:
        assert np.array_equal(got["topk_counts"], want["topk_counts"])
        if exact_inputs:   # the ranking is an integer problem once its inputs are equal
            assert np.array_equal(got["topk_positions"], want["topk_positions"])
        assert out.topk_count == want["topk_counts"].max() and out.valid_candidate_count == want["valid_candidate_counts"].max()
    a, b = got["attention_values"].astype(np.float64), want["attention_values"].astype(np.float64)
    bound = 5e-4 + 5e-4 * np.maximum(np.abs(a), np.abs(b)) + 2.0 ** -7 * np.abs(b) * (1.0 if exact_inputs else 4.0)
    assert np.all(np.abs(a - b) <= bound), float((np.abs(a - b) - bound).max())
    a, b = got["output"].astype(np.float64), want["output"].astype(np.float64)
    assert np.all(np.abs(a - b) <= 5e-4 + 2.0 ** -6 * np.abs(b).max(axis=1, keepdims=True))
    assert np.isfinite(got["output"]).all()


def test_job_through_device_tensors_and_without_evidence_spans(backend, oracle):
    job = job_cases.build(oracle, abi.ATTENTION_CSA, 5, 21, seed=7)
    want = job_cases.evaluate(oracle, job)
    g = job.geometry
    packed = np.ascontiguousarray(job.input[:, :g["hidden"]])
    device_in = backend.tensor("in", packed)
    device_out = backend.alloc("out", abi.DTYPE_F32, (5, g["hidden"]))
    job.struct.input = None
    job.struct.device_input = C.pointer(device_in.struct)
    job.struct.device_output = C.pointer(device_out.struct)
    rc, out, got, failure, err = job_cases.run(backend, job, want=())
    assert rc == 0, (err.where, err.message)
    result = device_out.read()
    a, b = result.astype(np.float64), want["output"].astype(np.float64)
    assert np.all(np.abs(a - b) <= 5e-4 + 2.0 ** -6 * np.abs(b).max(axis=1, keepdims=True))
    assert np.array_equal(device_in.read(), packed)          # the caller's input is not rounded in place
    assert out.d2d_bytes >= 2 * packed.nbytes
    # the same job again: the weights are resident now, so far fewer bytes go up
    first_upload = out.h2d_bytes
    rc, out, _, _, _ = job_cases.run(backend, job, want=())
    assert rc == 0 and out.h2d_bytes < first_upload // 4


def test_job_reads_resident_weights_and_state_where_the_runtime_keeps_them(backend, oracle, library):
    # The runtime's side of src/backend/residency.c: one device arena mirroring a host range
    # of weights, and a resolver from host state ranges to device copies.
    job = job_cases.build(oracle, abi.ATTENTION_CSA, 4, 45, seed=11)
    want = job_cases.evaluate(oracle, job)
    rc, plain, uploaded, _, err = job_cases.run(backend, job, want=("output",))
    assert rc == 0 and plain.device_state_staged == 0
    a, b = uploaded["output"].astype(np.float64), want["output"].astype(np.float64)
    assert np.all(np.abs(a - b) <= 5e-4 + 2.0 ** -6 * np.abs(b).max(axis=1, keepdims=True))
    # weights: pack every encoded weight into one host arena, mirror it on the device
    encoded = [job.weights[slot][0] for slot in sorted(job.weights)]
    offsets = np.cumsum([0] + [(e.nbytes + 255) & ~255 for e in encoded])
    arena = np.zeros(int(offsets[-1]), np.uint8)
    for slot, e, at in zip(sorted(job.weights), encoded, offsets):
        arena[at:at + e.nbytes] = e.reshape(-1)
        job.struct.weights[slot].encoded = arena.ctypes.data + int(at)
    mirror = backend.tensor("weights", arena.view(np.int8), dtype=abi.DTYPE_I8)
    err = abi.Error()
    assert library.yvex_backend_resident_attach(backend.handle, arena.ctypes.data, arena.nbytes, C.byref(mirror.struct), 1,
                                                C.byref(err)) == 0, err.message
    assert library.yvex_backend_resident_attach(backend.handle, arena.ctypes.data, arena.nbytes, C.byref(mirror.struct), 1,
                                                C.byref(err)) == abi.YVEX_ERR_STATE
    address = abi.u64()
    assert library.yvex_backend_resident_resolve(backend.handle, arena.ctypes.data + 300, 10, C.byref(address)) == 1
    assert address.value == mirror.data_ptr + 300
    assert library.yvex_backend_resident_resolve(backend.handle, arena.ctypes.data + arena.nbytes - 4, 10, C.byref(address)) == 0
    # state: device copies of the histories and rolling states, found by host address
    state = {}
    for array in (job.local, job.local_positions, job.compressed, job.compressed_positions, job.indexer):
        state[array.ctypes.data] = (array.nbytes, backend.tensor("s", array.view(np.int8).reshape(-1), dtype=abi.DTYPE_I8))
    for kv, score, _, _, _ in job.rolling.values():
        for array in (kv, score):
            state[array.ctypes.data] = (array.nbytes, backend.tensor("s", array.view(np.int8).reshape(-1), dtype=abi.DTYPE_I8))
    calls = {"hit": 0, "miss": 0}

    def resolve(_context, host, nbytes, out):
        for base, (size, tensor) in state.items():
            if base <= host and host + nbytes <= base + size:
                out[0] = tensor.data_ptr + (host - base)
                calls["hit"] += 1
                return 1
        calls["miss"] += 1
        return 0
    callback = abi.STATE_RESOLVE_FN(resolve)
    marker = C.c_int(1)
    assert library.yvex_backend_state_residency_attach(backend.handle, C.byref(marker), callback, 5, C.byref(err)) == 0
    assert library.yvex_backend_state_residency_validate_generation(backend.handle, 4, C.byref(err)) == abi.YVEX_ERR_STATE
    assert library.yvex_backend_state_residency_validate_generation(backend.handle, 6, C.byref(err)) == 0
    rc, resident, got, _, err = job_cases.run(backend, job, want=("output",))
    assert rc == 0, (err.where, err.message)
    assert np.array_equal(got["output"], uploaded["output"])      # same numbers either way
    assert calls["hit"] >= 8 and resident.device_state_staged == 1 and resident.device_state_staged_bytes > 0
    assert resident.h2d_bytes < plain.h2d_bytes // 10           # only the new tokens' input goes over the bus
    library.yvex_backend_state_residency_detach(backend.handle)
    assert library.yvex_backend_resident_detach(backend.handle, C.byref(err)) == 0
    assert library.yvex_backend_resident_resolve(backend.handle, arena.ctypes.data, 10, C.byref(address)) == 0


def test_typed_refusals(backend, oracle):
    def refused(mutate, code, status, stage=None):
        job = job_cases.build(oracle, abi.ATTENTION_CSA, 2, 9, seed=3)
        mutate(job.struct)
        rc, out, _, failure, err = job_cases.run(backend, job, want=("output",))
        assert rc == status and failure.code == code, (rc, failure.code, failure.stage)
        if stage:
            assert failure.stage == stage
        assert err.code == status

    def schema(j): j.schema = 2
    def envelope(j): j.operation_scope = abi.ATTENTION_SCOPE_ENVELOPE
    def qtype(j): j.weights[abi.WEIGHT_Q_B].qtype = 10          # Q2_K: no device projection here
    def missing(j): j.weights[abi.WEIGHT_OUT_A].present = 0
    def geometry(j): j.weights[abi.WEIGHT_KV].row_count += 1
    def position(j): j.main_rolling.cursor = (j.main_rolling.cursor + 1) % 4
    def paired(j): j.indexer_count += 1
    def checkpoints(j): j.retain_prefix_checkpoints = 1
    def budget(j): j.max_device_bytes = 4096
    refused(schema, abi.JOB_FAILURE_INVALID_ARGUMENT, abi.YVEX_ERR_INVALID_ARG)
    refused(envelope, abi.JOB_FAILURE_CAPABILITY, abi.YVEX_ERR_UNSUPPORTED, b"cuda.attention.mhc_pre")
    refused(qtype, abi.JOB_FAILURE_CAPABILITY, abi.YVEX_ERR_UNSUPPORTED, b"cuda.attention.q_b")
    refused(missing, abi.JOB_FAILURE_INVALID_ARGUMENT, abi.YVEX_ERR_INVALID_ARG, b"cuda.attention.output_a")
    refused(geometry, abi.JOB_FAILURE_INVALID_ARGUMENT, abi.YVEX_ERR_FORMAT, b"cuda.attention.kv")
    refused(position, abi.JOB_FAILURE_INVALID_ARGUMENT, abi.YVEX_ERR_STATE, b"cuda.attention.main_rolling")
    refused(paired, abi.JOB_FAILURE_INVALID_ARGUMENT, abi.YVEX_ERR_FORMAT, b"cuda.attention.topk")
    refused(checkpoints, abi.JOB_FAILURE_CAPABILITY, abi.YVEX_ERR_UNSUPPORTED)
    refused(budget, abi.JOB_FAILURE_BUDGET, abi.YVEX_ERR_BOUNDS, b"cuda.attention.alloc.budget")
    # a span too small for what the phase publishes
    job = job_cases.build(oracle, abi.ATTENTION_SWA, 2, 9, seed=3)
    out, arrays = job_cases.spans(job, want=("output",))
    out.output.capacity -= 1
    failure, err = abi.AttentionJobFailure(), abi.Error()
    rc = backend.lib.yvex_backend_attention_execute(backend.handle, C.byref(job.struct), C.byref(out), C.byref(failure), C.byref(err))
    assert rc == abi.YVEX_ERR_BOUNDS and failure.code == abi.JOB_FAILURE_COPY
    # a non-finite input is a numeric failure found on the device, and the backend stays usable
    job = job_cases.build(oracle, abi.ATTENTION_SWA, 2, 9, seed=3)
    job.input[1, 5] = np.inf
    rc, out, _, failure, err = job_cases.run(backend, job, want=("output",))
    assert rc == abi.YVEX_ERR_FORMAT and failure.code == abi.JOB_FAILURE_NUMERIC
    job = job_cases.build(oracle, abi.ATTENTION_SWA, 2, 9, seed=3)
    rc, _, _, _, _ = job_cases.run(backend, job, want=("output",))
    assert rc == 0


def test_cancellation_between_the_phases_of_the_transaction(backend, oracle):
    # The predicate is polled on the host between the phases; the n-th poll cancels.
    stages = []
    for cancel_at in range(1, 7):
        polls = {"n": 0}

        def requested(_context, polls=polls, cancel_at=cancel_at):
            polls["n"] += 1
            return 1 if polls["n"] >= cancel_at else 0
        callback = abi.CANCELLED_FN(requested)
        cancellation = abi.JobCancellation(callback, None)
        job = job_cases.build(oracle, abi.ATTENTION_CSA, 3, 13, seed=5)
        job.struct.cancellation = C.pointer(cancellation)
        rc, out, got, failure, err = job_cases.run(backend, job, want=("output",))
        assert rc == abi.YVEX_ERR_CANCELLED and failure.code == abi.JOB_FAILURE_CANCELLED, cancel_at
        assert failure.stage.startswith(b"cuda.attention.cancel.")
        stages.append(failure.stage)
    assert stages[0] == b"cuda.attention.cancel.before_dispatch" and stages[-1] == b"cuda.attention.cancel.publish"
    assert b"cuda.attention.cancel.after_allocation" in stages and b"cuda.attention.cancel.before_commit" in stages
    # a predicate that never fires lets the job through, and a cancelled backend is not poisoned
    callback = abi.CANCELLED_FN(lambda _context: 0)
    cancellation = abi.JobCancellation(callback, None)
    job = job_cases.build(oracle, abi.ATTENTION_CSA, 3, 13, seed=5)
    job.struct.cancellation = C.pointer(cancellation)
    rc, _, _, _, _ = job_cases.run(backend, job, want=("output",))
    assert rc == 0


def test_capability_query_is_truthful(backend, library, monkeypatch):
    result, err = abi.CapabilityResult(), abi.Error()
    supported = {abi.VARIANT_TENSOR_ALLOC, abi.VARIANT_TENSOR_ZERO, abi.VARIANT_TENSOR_WRITE, abi.VARIANT_TENSOR_READ,
                 abi.VARIANT_TENSOR_COPY, abi.VARIANT_ATTENTION_CAUSAL_F32, abi.VARIANT_ATTENTION_NONCAUSAL_F32,
                 abi.VARIANT_QTYPE_ROW_DOT, abi.VARIANT_ATTENTION_ENCODED}
    for variant in range(abi.VARIANT_COUNT):
        assert library.yvex_backend_query_capability(backend.handle, variant, C.byref(result), C.byref(err)) == 0
        assert result.backend_kind == abi.BACKEND_KIND_CUDA and result.variant == variant
        if variant in supported:
            assert result.state == abi.CAPABILITY_SUPPORTED and result.reason == 0 and result.function_available == 1
        else:
            assert result.state == abi.CAPABILITY_UNSUPPORTED and result.function_available == 0
            assert library.yvex_backend_capability_reason_name(result.reason) == b"variant-unsupported"
    assert library.yvex_backend_operation_variant_name(abi.VARIANT_ATTENTION_ENCODED) == b"encoded-attention"
    assert library.yvex_backend_query_capability(backend.handle, abi.VARIANT_COUNT, C.byref(result), C.byref(err)) == abi.YVEX_ERR_INVALID_ARG
    # after a failed launch (host-side hook: the GPU is not touched) every variant reads FAILED
    import clori_b200
    other = clori_b200.Backend(0)
    monkeypatch.setenv("YVEX_B200_TEST_LAUNCH_FAILURE", "cuda.attention")
    job = job_cases.build(__import__("oracle.binding", fromlist=["Oracle"]).Oracle(), abi.ATTENTION_SWA, 1, 5, seed=2)
    rc, _, _, failure, _ = job_cases.run(other, job, want=("output",))
    assert rc == abi.YVEX_ERR_BACKEND
    monkeypatch.delenv("YVEX_B200_TEST_LAUNCH_FAILURE")
    assert library.yvex_backend_query_capability(other.handle, abi.VARIANT_ATTENTION_ENCODED, C.byref(result), C.byref(err)) == 0
    assert result.state == abi.CAPABILITY_FAILED
    assert library.yvex_backend_capability_reason_name(result.reason) == b"launch-failed"
    rc, _, _, failure, _ = job_cases.run(other, job, want=("output",))
    assert rc == abi.YVEX_ERR_BACKEND and failure.code == abi.JOB_FAILURE_CAPABILITY       # sticky
    other.close()


@pytest.mark.parametrize("qtype", [abi.QTYPE_F32, abi.QTYPE_F16, abi.QTYPE_BF16, abi.QTYPE_Q8_0])
def test_projection_kernel_is_bit_equal_to_the_cpu_dot(backend, oracle, qtype):
    rng = np.random.default_rng(60 + qtype)
    # the last three reach the streaming kernel with 1, 2 and 4 rows per warp (row counts against the SM count)
    for rows, width, tokens, groups in ((40, 96, 1, 1), (130, 1024, 5, 1), (64, 4096, 3, 1), (24, 256, 6, 4),
                                        (5000, 1280, 1, 1), (9601, 512, 2, 1), (1300, 2304, 1, 8)):
        values = job_cases.bf16_valued(rng, (rows * groups, width), 1.0 / np.sqrt(width))
        encoded = oracle.qtype_encode_rows(values, qtype)
        stride = groups * width + 8
        x = job_cases.bf16_valued(rng, (tokens, stride))
        w, xi = backend.tensor("w", encoded.view(np.int8), dtype=abi.DTYPE_I8), backend.tensor("x", x)
        out = backend.alloc("y", abi.DTYPE_F32, (tokens, groups * rows + 3))
        status = backend.tensor("status", np.zeros(1, np.int32))
        for rounded in (0, 1):
            a = abi.MatvecArgs()
            a.weights, a.qtype, a.rows, a.width, a.row_bytes = w.data_ptr, qtype, rows, width, encoded.shape[1]
            a.input, a.tokens, a.input_stride = xi.data_ptr, tokens, stride
            a.output, a.output_stride, a.groups, a.round_bf16, a.status = out.data_ptr, groups * rows + 3, groups, rounded, status.data_ptr
            assert backend.lib.yvx_cuda_qtype_matvec(C.byref(a), backend.stream) == 0, backend.lib.yvx_cuda_last_error_text()
            assert backend.lib.yvx_cuda_stream_synchronize(backend.stream) == 0
            out.struct.is_written = 1
            got = out.read()[:, :groups * rows]
            want = np.concatenate([oracle.qtype_matvec(encoded, qtype, width, np.ascontiguousarray(x[:, k * width:(k + 1) * width]),
                                                       k * rows, rows, bool(rounded)) for k in range(groups)], axis=1)
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (rows, width, tokens, groups, rounded)
        assert int(status.read()[0]) == 0
    a.qtype = 10
    assert backend.lib.yvx_cuda_qtype_matvec(C.byref(a), backend.stream) == abi.YVEX_ERR_UNSUPPORTED


@pytest.mark.parametrize("qtype", [abi.QTYPE_F16, abi.QTYPE_BF16])
def test_projection_kernel_keeps_subnormal_weights_and_reports_infinite_ones(backend, oracle, qtype):
    """16-bit weights are placed into doubles bit field by bit field: zeros, subnormals and the
    largest finite values must come out exactly, an infinite weight must raise the status word."""
    rng = np.random.default_rng(70 + qtype)
    rows, width = 64, 512
    values = job_cases.bf16_valued(rng, (rows, width), 1.0 / np.sqrt(width))
    tiny = 2.0 ** -24 if qtype == abi.QTYPE_F16 else 2.0 ** -133      # subnormal in the encoding
    values[::3, ::5] = tiny * rng.integers(1, 64, values[::3, ::5].shape)
    values[1::7, 3::11] = 0.0
    values[5, 7] = -0.0
    values[2::9, 1::13] = 32768.0 if qtype == abi.QTYPE_F16 else 2.0 ** 120
    encoded = oracle.qtype_encode_rows(values, qtype)
    decoded = oracle.qtype_decode_rows(encoded, qtype, width)
    special = np.zeros(values.shape, bool)
    special[::3, ::5] = special[1::7, 3::11] = special[2::9, 1::13] = True
    assert np.array_equal(decoded[special], values[special])        # the planted values are exactly representable
    assert np.signbit(decoded[5, 7]) and decoded[5, 7] == 0.0
    x = job_cases.bf16_valued(rng, (3, width))
    x[:, ::17] *= 2.0 ** -30
    w, xi = backend.tensor("w", encoded.view(np.int8), dtype=abi.DTYPE_I8), backend.tensor("x", x)
    out = backend.alloc("y", abi.DTYPE_F32, (3, rows))
    status = backend.tensor("status", np.zeros(1, np.int32))
    a = abi.MatvecArgs()
    a.weights, a.qtype, a.rows, a.width, a.row_bytes = w.data_ptr, qtype, rows, width, encoded.shape[1]
    a.input, a.tokens, a.input_stride = xi.data_ptr, 3, width
    a.output, a.output_stride, a.groups, a.round_bf16, a.status = out.data_ptr, rows, 1, 0, status.data_ptr
    assert backend.lib.yvx_cuda_qtype_matvec(C.byref(a), backend.stream) == 0
    assert backend.lib.yvx_cuda_stream_synchronize(backend.stream) == 0
    out.struct.is_written = 1
    want = oracle.qtype_matvec(encoded, qtype, width, x, 0, rows, False)
    assert np.array_equal(out.read().view(np.uint32), want.view(np.uint32))
    assert int(status.read()[0]) == 0
    # one infinite weight: the CPU dot refuses, the kernel raises the non-finite status
    bad = encoded.copy()
    bad.view(np.uint16)[9, 100] = 0x7c00 if qtype == abi.QTYPE_F16 else 0x7f80
    assert oracle.qtype_matvec(bad, qtype, width, x, 0, rows, False) is None
    w2 = backend.tensor("w2", bad.view(np.int8), dtype=abi.DTYPE_I8)
    a.weights = w2.data_ptr
    assert backend.lib.yvx_cuda_qtype_matvec(C.byref(a), backend.stream) == 0
    assert backend.lib.yvx_cuda_stream_synchronize(backend.stream) == 0
    assert int(status.read()[0]) == 1


def test_job_with_tensor_core_projections_stays_within_a_bf16_step(backend, oracle, library):
    """Opted in, jobs of enough tokens run q_a, q_b, kv, out_a and out_b (BF16 weights) through the tcgen05 GEMM:
    published rows may move by one bf16 step against the exact projections, the state stays bit-equal."""
    cls, tokens, start = abi.ATTENTION_CSA, 9, 0
    qtypes = {slot: abi.QTYPE_BF16 for slot in (abi.WEIGHT_Q_A, abi.WEIGHT_Q_B, abi.WEIGHT_KV, abi.WEIGHT_OUT_A,
                                                abi.WEIGHT_OUT_B)}
    job = job_cases.build(oracle, cls, tokens, start, seed=333, qtypes=qtypes)
    rc, out0, exact, failure, err = job_cases.run(backend, job)
    assert rc == 0, (err.where, err.message, failure.stage)
    error = abi.Error()
    library.yvex_b200_backend_projection_gemm.argtypes = [C.c_void_p, C.c_ulonglong, C.POINTER(abi.Error)]
    assert library.yvex_b200_backend_projection_gemm(backend.handle, 4, C.byref(error)) == 0
    rc, out1, got, failure, err = job_cases.run(backend, job)
    assert library.yvex_b200_backend_projection_gemm(backend.handle, 0, C.byref(error)) == 0
    assert rc == 0, (err.where, err.message, failure.stage)
    assert out1.kernel_launches > out0.kernel_launches          # a staging launch per GEMM
    for name in ("q_low", "query", "raw_kv"):
        differ, beyond = ulp_lanes(got[name], exact[name])
        assert beyond == 0 and differ <= max(2, got[name].size // 50), (name, differ, beyond)
    for name in ("main_kv_state", "main_score_state", "indexer_kv_state", "indexer_score_state"):
        if name in got:
            assert np.array_equal(got[name].view(np.uint32), exact[name].view(np.uint32)), name
    scale = np.abs(exact["output"]).max(axis=-1, keepdims=True)
    assert np.all(np.abs(got["output"] - exact["output"]) <= 2.0 ** -6 * scale + 5e-4)
