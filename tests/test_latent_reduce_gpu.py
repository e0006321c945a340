"""The shared-latent reduce stage on a B200 against its CPU restatement, over the
reference's three attention classes (window only; window + selected compressed
rows, ratio 4; window + all compressed rows, ratio 128), decode and multi-token
phases, plus the reference's sink known-answer vector. The published value is the
quotient rounded to bf16, so the comparison allows one bf16 ulp on top of the
reference's CPU-vs-CUDA publication tolerance (5e-4 absolute and relative,
src/graph/attention.c:919-920)."""
import ctypes as C

import numpy as np
import pytest

import clori_b200
from clori_b200 import abi
from latent_cases import bf16_valued, build, host_args  # noqa: F401

pytestmark = pytest.mark.gpu
u64 = np.uint64


def run_gpu(backend, case, block_visible=0, workspace=True):
    t = {}
    for name in ("query", "local", "compressed", "sinks"):
        t[name] = backend.tensor(name, case[name])
    for name in ("local_positions", "compressed_positions", "selected", "selected_count"):
        t[name] = backend.tensor(name, case[name].view(np.int64), dtype=abi.DTYPE_I64)
    out = backend.alloc("out", abi.DTYPE_F32, (case["tokens"], case["heads"] * case["hd"]))
    status = backend.tensor("status", np.zeros(1, np.int32))
    a = host_args(case, block_visible)
    for name in ("query", "local", "local_positions", "compressed", "compressed_positions", "selected",
                 "selected_count", "sinks"):
        setattr(a, name, t[name].data_ptr)
    a.out, a.status = out.data_ptr, status.data_ptr
    if workspace:  # lets the library split the candidate list over CTAs (second launch folds)
        nbytes = int(backend.lib.yvx_cuda_latent_reduce_workspace_bytes(C.byref(a)))
        if nbytes:
            a.workspace = backend.alloc("work", abi.DTYPE_I8, (nbytes,)).data_ptr
    launches = C.c_uint()
    rc = backend.lib.yvx_cuda_latent_reduce_launches(C.byref(a), backend.stream, C.byref(launches))
    assert rc == 0, backend.lib.yvx_cuda_last_error_text()
    assert launches.value == (2 if a.workspace else 1)
    run_gpu.launches = launches.value
    assert backend.lib.yvx_cuda_stream_synchronize(backend.stream) == 0
    out.struct.is_written = 1
    return out.read(), int(status.read()[0])


def close(got, ref):
    return np.all(np.abs(got - ref) <= 5e-4 + (5e-4 + 2.0 ** -7) * np.maximum(np.abs(got), np.abs(ref)))


@pytest.mark.parametrize("cls", [0, 1, 2])
@pytest.mark.parametrize("tokens,start", [(1, 0), (1, 700), (5, 130), (3, 1023)])
def test_reduce_matches_restatement(backend, oracle, cls, tokens, start):
    rng = np.random.default_rng(cls * 100 + tokens + start)
    case = build(rng, heads=16, hd=512, window=128, attention_class=cls, tokens=tokens, start=start)
    got, status = run_gpu(backend, case)
    ref = oracle.latent_reduce_full(host_args(case), tokens, 16, 512)
    assert status == 0 and ref is not None
    assert close(got, ref)
    # the published values are bf16-representable
    assert np.array_equal(got, clori_b200.bf16_bits_to_f32(clori_b200.f32_to_bf16_bits(got)))


@pytest.mark.parametrize("cls", [0, 1, 2])
def test_split_and_single_launch_agree(backend, oracle, cls):
    rng = np.random.default_rng(77 + cls)
    case = build(rng, heads=16, hd=512, window=128, attention_class=cls, tokens=2, start=5000)
    split, status = run_gpu(backend, case)
    assert status == 0 and run_gpu.launches == 2
    single, status = run_gpu(backend, case, workspace=False)
    assert status == 0 and run_gpu.launches == 1
    ref = oracle.latent_reduce_full(host_args(case), 2, 16, 512)
    assert close(split, ref) and close(single, ref) and close(split, single)
    again, _ = run_gpu(backend, case)
    assert np.array_equal(again, split)       # the split plan is deterministic


def test_long_phase_needs_no_split(backend, oracle):
    rng = np.random.default_rng(78)
    case = build(rng, heads=16, hd=128, window=128, attention_class=2, tokens=200, start=900)
    got, status = run_gpu(backend, case)
    assert status == 0 and run_gpu.launches == 1
    assert close(got, oracle.latent_reduce_full(host_args(case), 200, 16, 128))


def test_candidate_block_visible_and_small_head(backend, oracle):
    rng = np.random.default_rng(5)
    case = build(rng, heads=10, hd=64, window=128, attention_class=0, tokens=4, start=40)
    got, status = run_gpu(backend, case, block_visible=1)
    ref = oracle.latent_reduce_full(host_args(case, 1), 4, 10, 64)
    assert status == 0 and close(got, ref)


def test_sink_known_answer_of_the_reference(backend):
    # tests/reference/deepseek_attention.c:2724-2726,2928-2940: sink logit 0, logits
    # {0, ln 2}, values {1,2},{3,4} -> {1.75, 2.5} (both exactly representable in bf16).
    hd = 4
    case = dict(query=np.array([[0, 0, 1, 0]], np.float32),
                local=np.array([[1, 2, 0, 0], [3, 4, np.log(2.0) * 2.0, 0]], np.float32),
                local_positions=np.array([0, 1], u64), initial=1, compressed=np.zeros((1, hd), np.float32),
                compressed_positions=np.zeros(1, u64), selected=np.zeros((1, 1), u64),
                selected_count=np.zeros(1, u64), topk=1, sinks=np.zeros(1, np.float32), heads=1, hd=hd,
                window=128, ratio=0, cls=0, start=1, tokens=1)
    got, status = run_gpu(backend, case)
    assert status == 0
    assert abs(got[0, 0] - 1.75) <= 2.0 ** -7 and abs(got[0, 1] - 2.5) <= 2.0 ** -6


def test_contract_and_nonfinite_refusals(backend):
    rng = np.random.default_rng(9)
    case = build(rng, heads=8, hd=128, window=128, attention_class=0, tokens=1, start=10)
    case["ratio"] = 4  # class 0 requires ratio 0
    a = host_args(case)
    a.out = a.status = 1
    assert backend.lib.yvx_cuda_latent_reduce(C.byref(a), backend.stream) == abi.YVEX_ERR_INVALID_ARG
    case = build(rng, heads=8, hd=128, window=128, attention_class=0, tokens=1, start=10)
    case["local"][3, 7] = np.inf
    _, status = run_gpu(backend, case)
    assert status == 1
