"""Latent-compressed (MLA-style) decode on a B200 against the CPU restatement and
against fixtures the reference's own compiled reduce produced (the decode is a
shared-row K == V attention over [latent | rope key] rows, which
yvex_attention_reduce_chunk, src/graph/core.c:608-701, computes). bf16 operands:
max-abs <= 2e-3, cosine >= 0.9999; the reference publishes bf16, so half a bf16 ulp
of the published value is added where its fixtures are the comparand."""
import ctypes as C
import os

import numpy as np
import pytest

import clori_b200
from clori_b200 import abi, workloads

pytestmark = pytest.mark.gpu


def run_mla(backend, q_nope, q_rope, w_uk, latent, rope_key, lengths, scale, chunk=None, sm_count=None):
    lib = backend.lib
    sessions, heads, nope = q_nope.shape
    cap, dc = latent.shape[1], latent.shape[2]
    dr = q_rope.shape[2]
    p = abi.MlaProblem()
    p.sessions, p.heads, p.nope_dim, p.latent_dim, p.rope_dim, p.scale = sessions, heads, nope, dc, dr, scale
    t = {n: backend.tensor(n, a) for n, a in (("qn", q_nope), ("qr", q_rope), ("w", w_uk), ("lat", latent),
                                              ("rk", rope_key))}
    p.q_nope, p.q_rope, p.w_uk = t["qn"].data_ptr, t["qr"].data_ptr, t["w"].data_ptr
    p.latent, p.rope_key = t["lat"].data_ptr, t["rk"].data_ptr
    p.latent_session_stride, p.rope_session_stride = cap * dc, cap * dr
    if isinstance(lengths, int):    # every session has this many tokens, and the host knows it
        p.kv_tokens, p.kv_tokens_uniform, p.kv_tokens_max = None, lengths, cap
    else:
        lens = backend.tensor("lens", np.asarray(lengths, np.int32))
        p.kv_tokens, p.kv_tokens_max = lens.data_ptr, cap
    lib.yvx_cuda_mla_plan(C.byref(p), sm_count or backend.sm_count)
    if chunk:   # more (and shorter) splits than the planner would choose
        p.chunk_tokens, p.max_splits = chunk, (cap + chunk - 1) // chunk
    q_abs = backend.alloc("qabs", abi.DTYPE_BF16, (sessions, heads, dc + dr))
    parts = backend.alloc("parts", abi.DTYPE_F32, (1,), lib.yvx_cuda_mla_partials_bytes(C.byref(p)))
    out = backend.alloc("out", abi.DTYPE_F32, (sessions, heads, dc))
    status = backend.tensor("status", np.zeros(1, np.int32))
    p.q_absorbed, p.partials, p.output, p.status = q_abs.data_ptr, parts.data_ptr, out.data_ptr, status.data_ptr
    launches = C.c_uint()
    rc = lib.yvx_cuda_mla_decode(C.byref(p), backend.stream, None, C.byref(launches))
    assert rc == 0, lib.yvx_cuda_last_error_text()
    assert lib.yvx_cuda_stream_synchronize(backend.stream) == 0, lib.yvx_cuda_last_error_text()
    out.struct.is_written = 1
    q_abs.struct.is_written = 1
    plan = (p.chunk_tokens, p.max_splits, p.balanced_pairs) if p.balanced_pairs else (p.chunk_tokens, p.max_splits)
    return out.read(), q_abs.read(), int(status.read()[0]), launches.value, plan


def cosine(a, b):
    a, b = a.astype(np.float64).ravel(), b.astype(np.float64).ravel()
    return float(a @ b / np.sqrt((a @ a) * (b @ b)))


@pytest.fixture(params=["paired", "independent", "quad"])
def form(request, monkeypatch):
    """The forms of the attention kernel: a cluster of two CTAs that computes every score tile once and
    exchanges the weights, two independent CTAs that both compute it, and a cluster of four CTAs with a
    quarter of the latent columns each."""
    monkeypatch.delenv("YVEX_B200_MLA_INDEPENDENT", raising=False)
    monkeypatch.delenv("YVEX_B200_MLA_FORM", raising=False)
    if request.param == "independent":
        monkeypatch.setenv("YVEX_B200_MLA_INDEPENDENT", "1")
    if request.param == "quad":
        monkeypatch.setenv("YVEX_B200_MLA_FORM", "quad")
    return request.param


@pytest.mark.parametrize("sessions,context", [(1, 32), (2, 100), (3, 700)])
def test_mla_decode_matches_restatement(backend, oracle, sessions, context, form):
    qn, qr, w, lat, rk = workloads.mla_decode_bf16(seed=4, batch=sessions, context=context)
    lengths = [context] * sessions
    if sessions > 1:
        lengths[1] = max(1, context - 37)  # ragged: a length that is not a tile multiple
    scale = 1.0 / np.sqrt(192.0)
    out, q_abs, status, launches, plan = run_mla(backend, qn, qr, w, lat, rk, lengths, scale)
    assert status == 0 and launches == (2 if form == "quad" and plan[1] == 1 else 3)   # one item per session: no fold
    for s in range(sessions):
        n = lengths[s]
        ref = oracle.mla_decode(qn[s], qr[s], w, lat[s, :n], rk[s, :n], scale)
        assert np.abs(out[s] - ref).max() <= 2e-3, float(np.abs(out[s] - ref).max())
        assert cosine(out[s], ref) >= 0.9999
    # the absorbed query: bf16 of an f32-accumulated product, within one bf16 ulp of the f64 one
    f = clori_b200.bf16_bits_to_f32
    exact = np.einsum("bhi,hic->bhc", f(qn).astype(np.float64), f(w).astype(np.float64))
    got = f(q_abs[:, :, :512]).astype(np.float64)
    assert np.all(np.abs(got - exact) <= 2.0 ** -8 * np.abs(exact) + 1e-6)
    assert np.array_equal(q_abs[:, :, 512:], qr)


def test_mla_decode_folds_many_splits_of_ragged_sessions(backend, oracle, form):
    """Six splits of 128 tokens, of which a session fills six, three or one (the rest write empty partial rows):
    the fold of the partial rows gives the same bits every time."""
    context = 700
    qn, qr, w, lat, rk = workloads.mla_decode_bf16(seed=12, batch=3, context=context)
    lengths = [context, 300, 64]
    scale = 1.0 / np.sqrt(192.0)
    out, _, status, _, plan = run_mla(backend, qn, qr, w, lat, rk, lengths, scale, chunk=128)
    assert status == 0 and plan == (128, 6)
    for _ in range(3):
        again, _, status, _, _ = run_mla(backend, qn, qr, w, lat, rk, lengths, scale, chunk=128)
        assert status == 0 and np.array_equal(again.view(np.uint32), out.view(np.uint32))
    for s in range(3):
        n = lengths[s]
        ref = oracle.mla_decode(qn[s], qr[s], w, lat[s, :n], rk[s, :n], scale)
        assert np.abs(out[s] - ref).max() <= 2e-3, float(np.abs(out[s] - ref).max())
        assert cosine(out[s], ref) >= 0.9999


@pytest.mark.parametrize("sms,pieces", [(4, 1), (10, 2), (14, 2), (30, 3), (40, 4)])
def test_mla_decode_balanced_runs_across_sessions(backend, oracle, monkeypatch, sms, pieces):
    """Uniform lengths under the balanced plan: the three sessions' tiles laid end to end are cut into one run
    per pair of SMs (the plan is made for 4 to 40 SMs: one run holds two whole sessions, one holds nothing), so a pair finishes one session and starts the
    next (its barriers begin again) and a session is cut into up to four items; same bits every time."""
    monkeypatch.delenv("YVEX_B200_MLA_INDEPENDENT", raising=False)
    monkeypatch.delenv("YVEX_B200_MLA_FORM", raising=False)
    monkeypatch.setenv("YVEX_B200_MLA_PLAN", "balanced")
    context = 700
    qn, qr, w, lat, rk = workloads.mla_decode_bf16(seed=21, batch=3, context=context)
    scale = 1.0 / np.sqrt(192.0)
    out, _, status, _, plan = run_mla(backend, qn, qr, w, lat, rk, context, scale, sm_count=sms)
    assert status == 0 and plan == (704, pieces, sms // 2)
    for _ in range(3):
        again, _, status, _, _ = run_mla(backend, qn, qr, w, lat, rk, context, scale, sm_count=sms)
        assert status == 0 and np.array_equal(again.view(np.uint32), out.view(np.uint32))
    for s in range(3):
        ref = oracle.mla_decode(qn[s], qr[s], w, lat[s], rk[s], scale)
        assert np.abs(out[s] - ref).max() <= 2e-3, float(np.abs(out[s] - ref).max())
        assert cosine(out[s], ref) >= 0.9999


@pytest.mark.parametrize("context", [64, 129, 1000, 2500])
def test_mla_decode_with_maxima_that_grow_along_the_sequence(backend, oracle, context, form):
    """Later rows score higher and higher, so the running maximum grows again and again: every path that
    rescales the accumulator runs (in the paired form also the adoption of the peer's maximum and weights
    that were scaled with a maximum the accumulator has already left behind)."""
    qn, qr, w, lat, rk = workloads.mla_decode_bf16(seed=9, batch=2, context=context)
    f, bits = clori_b200.bf16_bits_to_f32, clori_b200.f32_to_bf16_bits
    ramp = (1.0 + 6.0 * (np.arange(context, dtype=np.float32) / context) ** 2)[None, :, None]
    lat, rk = bits(f(lat) * ramp), bits(f(rk) * ramp)
    lengths = [context, max(1, context - 21)]
    scale = 1.0 / np.sqrt(192.0)
    out, _, status, _, _ = run_mla(backend, qn, qr, w, lat, rk, lengths, scale)
    assert status == 0
    # the same bits every time: what a CTA adopts from its peer does not depend on when the message arrives
    for _ in range(3):
        again, _, status, _, _ = run_mla(backend, qn, qr, w, lat, rk, lengths, scale)
        assert status == 0 and np.array_equal(again.view(np.uint32), out.view(np.uint32))
    for s in range(2):
        n = lengths[s]
        ref = oracle.mla_decode(qn[s], qr[s], w, lat[s, :n], rk[s, :n], scale)
        bar = 2e-3 * max(1.0, float(np.abs(ref).max()))
        assert np.abs(out[s] - ref).max() <= bar, (float(np.abs(out[s] - ref).max()), bar)
        assert cosine(out[s], ref) >= 0.9999


def test_mla_decode_matches_reference_made_fixtures(backend, form):
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "mla_decode.npz"))
    f = clori_b200.bf16_bits_to_f32
    scale = 1.0 / np.sqrt(192.0)
    for i in range(int(g["count"])):
        seed, sessions, context = (int(x) for x in g[f"meta{i}"])
        qn, qr, w, lat, rk = workloads.mla_decode_bf16(seed=seed, batch=sessions, context=context)
        lengths = [context] * sessions
        if sessions > 1:
            lengths[1] = max(1, context - 37)
        out, q_abs, status, _, _ = run_mla(backend, qn, qr, w, lat, rk, lengths, scale)
        assert status == 0
        for s in range(sessions):
            published = f(g[f"out{i}_{s}"]).astype(np.float64)
            magnitude = np.abs(published)
            half_ulp = np.where(magnitude > 0, 2.0 ** (np.floor(np.log2(np.maximum(magnitude, 1e-300))) - 8), 0.0)
            assert np.all(np.abs(out[s] - published) <= 2e-3 + half_ulp), float(np.abs(out[s] - published).max())
            assert cosine(out[s], published) >= 0.9999
            # the device's absorbed query against the one the fixture was computed from:
            # f32 accumulation on the device, f64 in the restatement, both rounded to bf16
            got, want = f(q_abs[s, :, :512]), f(g[f"absorbed{i}_{s}"])
            assert np.all(np.abs(got - want) <= 2.0 ** -7 * np.abs(want) + 1e-6)


def test_mla_refuses_other_geometries(backend):
    p = abi.MlaProblem()
    p.sessions, p.heads, p.nope_dim, p.latent_dim, p.rope_dim = 1, 64, 128, 512, 64
    p.kv_tokens_max, p.chunk_tokens, p.max_splits = 64, 32, 2
    dummy = backend.alloc("d", abi.DTYPE_F32, (64,))
    for f in ("q_nope", "q_rope", "w_uk", "latent", "rope_key", "q_absorbed", "partials", "output", "status"):
        setattr(p, f, dummy.data_ptr)
    n = C.c_uint()
    assert backend.lib.yvx_cuda_mla_decode(C.byref(p), backend.stream, None, C.byref(n)) == abi.YVEX_ERR_UNSUPPORTED
