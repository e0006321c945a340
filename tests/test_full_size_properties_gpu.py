"""Size-independent properties at the full sizes of the benchmark configurations,
where the CPU checker would take minutes: exact homogeneity in V (doubling every
value doubles every output bit for bit: products, f32 sums and the final
rounding all commute with a power of two), uniform values (softmax weights sum
to one, so the output is the constant, wherever masks and block tables put the
boundaries), the first causal row (sees one token: output = that value row), and
invariance to the split size."""
import ctypes as C
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import clori_b200  # noqa: E402
from clori_b200 import abi  # noqa: E402

pytestmark = pytest.mark.gpu
UNIFORM_BYTE = 0x3F                       # bf16 0x3F3F
UNIFORM_BF16 = float(clori_b200.bf16_bits_to_f32(np.array([0x3F3F], np.uint16))[0])


def _alloc(lib, nbytes):
    p = C.c_void_p()
    assert lib.yvx_cuda_malloc(C.byref(p), nbytes) == 0, lib.yvx_cuda_last_error_text()
    return p


def _download(lib, stream, ptr, array):
    assert lib.yvx_cuda_download_async(array.ctypes.data, ptr, array.nbytes, stream) == 0
    assert lib.yvx_cuda_stream_synchronize(stream) == 0, lib.yvx_cuda_last_error_text()
    return array


def test_batched_block_table_decode_at_full_size():
    import bench
    w = bench.Workload(0, bench.SEED)
    lib, s = w.lib, w.backend.stream
    elems = w.pool_blocks * bench.BLOCK_TOKENS * bench.KV_HEADS * bench.HEAD_DIM

    def run():
        w.step()
        w.backend.sync()
        w.out.struct.is_written = 1
        return clori_b200.bf16_bits_to_f32(w.out.read())

    lib.yvx_cuda_fill_normal(w.vpool.data_ptr, abi.DTYPE_BF16, elems, 4242, 0.5, s)
    once = run()
    lib.yvx_cuda_fill_normal(w.vpool.data_ptr, abi.DTYPE_BF16, elems, 4242, 1.0, s)
    twice = run()
    assert np.isfinite(once).all() and np.abs(once).max() > 0
    assert np.array_equal(twice, 2.0 * once)
    lib.yvx_cuda_memset_async(w.vpool.data_ptr, UNIFORM_BYTE, elems * 2, s)
    flat = run()
    assert np.abs(flat - UNIFORM_BF16).max() <= UNIFORM_BF16 * 2.0 ** -7
    w.backend.close()


def test_causal_prefill_at_full_size(backend):
    lib, s = backend.lib, backend.stream
    batch, tokens, hq, hkv, hd = 2, 8192, 40, 8, 128
    qn, kn = batch * tokens * hq * hd, batch * tokens * hkv * hd
    q, k, v, out, status = _alloc(lib, qn * 2), _alloc(lib, kn * 2), _alloc(lib, kn * 2), _alloc(lib, qn * 2), _alloc(lib, 4)
    lib.yvx_cuda_fill_normal(q, abi.DTYPE_BF16, qn, 301, 0.5, s)
    lib.yvx_cuda_fill_normal(k, abi.DTYPE_BF16, kn, 302, 0.5, s)
    lib.yvx_cuda_memset_async(status, 0, 4, s)
    p = abi.GqaProblem()
    p.sessions, p.query_rows, p.query_heads, p.kv_heads, p.head_dim = batch, tokens, hq, hkv, hd
    p.causal, p.scale = 1, 1.0 / np.sqrt(hd)
    p.query_dtype = p.kv_dtype = p.output_dtype = abi.DTYPE_BF16
    p.query, p.query_row_stride, p.query_session_stride, p.output = q, hq * hd, tokens * hq * hd, out
    p.key, p.value = k, v
    p.key_token_stride = p.value_token_stride = hkv * hd
    p.key_head_stride = p.value_head_stride = hd
    p.key_session_stride = p.value_session_stride = tokens * hkv * hd
    p.kv_tokens_uniform = p.kv_tokens_max = tokens
    lib.yvx_cuda_gqa_plan_splits(C.byref(p), backend.sm_count)
    scratch = _alloc(lib, max(lib.yvx_cuda_gqa_partials_bytes(C.byref(p)), 16))
    p.partials, p.status = scratch, status

    def run():
        n = C.c_uint()
        assert lib.yvx_cuda_gqa_attention(C.byref(p), s, C.byref(n)) == 0, lib.yvx_cuda_last_error_text()
        bits = _download(lib, s, out, np.empty((batch, tokens, hq, hd), np.uint16))
        return clori_b200.bf16_bits_to_f32(bits)

    lib.yvx_cuda_fill_normal(v, abi.DTYPE_BF16, kn, 303, 0.5, s)
    once = run()
    v_host = clori_b200.bf16_bits_to_f32(_download(lib, s, v, np.empty((batch, tokens, hkv, hd), np.uint16)))
    # row 0 sees token 0 only
    for head in range(hq):
        assert np.array_equal(once[:, 0, head], v_host[:, 0, head // (hq // hkv)])
    lib.yvx_cuda_fill_normal(v, abi.DTYPE_BF16, kn, 303, 1.0, s)
    twice = run()
    assert np.isfinite(once).all() and np.array_equal(twice, 2.0 * once)
    lib.yvx_cuda_memset_async(v, UNIFORM_BYTE, kn * 2, s)
    flat = run()
    assert np.abs(flat - UNIFORM_BF16).max() <= UNIFORM_BF16 * 2.0 ** -7
    st = _download(lib, s, status, np.zeros(1, np.int32))
    assert st[0] == 0
    for ptr in (q, k, v, out, status, scratch):
        lib.yvx_cuda_free(ptr)


def test_q8_verify_at_full_size(backend):
    lib, s = backend.lib, backend.stream
    hq, hkv, hd, tokens, rows = 32, 8, 128, 131072, 4
    record = lib.yvx_cuda_q8_record_bytes()
    blocks = tokens // 64
    pool_bytes = blocks * hkv * record
    records, q, status = _alloc(lib, pool_bytes), _alloc(lib, rows * hq * hd * 2), _alloc(lib, 4)
    out = _alloc(lib, rows * hq * hd * 4)
    lib.yvx_cuda_fill_normal(q, abi.DTYPE_BF16, rows * hq * hd, 202, 1.0, s)
    lib.yvx_cuda_memset_async(status, 0, 4, s)
    p = abi.GqaProblem()
    p.sessions, p.query_rows, p.query_heads, p.kv_heads, p.head_dim = 1, rows, hq, hkv, hd
    p.causal, p.scale = 1, 1.0 / np.sqrt(hd)
    p.query_dtype, p.kv_dtype, p.output_dtype = abi.DTYPE_BF16, abi.DTYPE_Q8_0, abi.DTYPE_F32
    p.query, p.query_row_stride, p.query_session_stride, p.output = q, hq * hd, rows * hq * hd, out
    p.key = records
    p.key_head_stride, p.key_block_stride, p.block_tokens = record, hkv * record, 64
    p.kv_tokens_uniform = p.kv_tokens_max = tokens
    p.query_start_from_end = 1
    p.status = status

    def run(chunk):
        lib.yvx_cuda_gqa_plan_splits(C.byref(p), backend.sm_count)
        if chunk:
            p.chunk_tokens, p.max_splits = chunk, (tokens + chunk - 1) // chunk
        scratch = _alloc(lib, max(lib.yvx_cuda_gqa_partials_bytes(C.byref(p)), 16))
        p.partials = scratch
        n = C.c_uint()
        assert lib.yvx_cuda_gqa_attention(C.byref(p), s, C.byref(n)) == 0, lib.yvx_cuda_last_error_text()
        got = _download(lib, s, out, np.empty((rows, hq * hd), np.float32)).copy()
        lib.yvx_cuda_free(scratch)
        return got

    # invariance to the split size on seeded records
    lib.yvx_cuda_fill_q8_records(records, blocks * hkv, 201, 0.002, 0.02, s)
    planned, fine = run(0), run(1024)
    assert np.isfinite(planned).all() and np.abs(planned - fine).max() <= 1e-5
    # every byte 0x2C: stored lanes 0x2C = 44 - 128, scales f16 0x2C2C -> every K row equal, every value -84 * scale
    lib.yvx_cuda_memset_async(records, 0x2C, pool_bytes, s)
    scale = float(np.array([0x2C2C], np.uint16).view(np.float16)[0])
    flat = run(0)
    assert np.abs(flat - (-84.0) * scale).max() <= 84.0 * scale * 2.0 ** -9
    st = _download(lib, s, status, np.zeros(1, np.int32))
    assert st[0] == 0
    for ptr in (records, q, out, status):
        lib.yvx_cuda_free(ptr)


def test_latent_decode_at_full_size(backend):
    lib, s = backend.lib, backend.stream
    sessions, heads, nope, dc, dr, context = 32, 128, 128, 512, 64, 16384
    sizes = {"q_nope": sessions * heads * nope, "q_rope": sessions * heads * dr, "w_uk": heads * nope * dc,
             "latent": sessions * context * dc, "rope_key": sessions * context * dr}
    bufs = {name: _alloc(lib, n * 2) for name, n in sizes.items()}
    for i, (name, n) in enumerate(sizes.items()):
        sigma = 1.0 / np.sqrt(dc) if name == "w_uk" else 1.0
        lib.yvx_cuda_fill_normal(bufs[name], abi.DTYPE_BF16, n, 401 + i, sigma, s)
    p = abi.MlaProblem()
    p.sessions, p.heads, p.nope_dim, p.latent_dim, p.rope_dim = sessions, heads, nope, dc, dr
    p.scale = 1.0 / np.sqrt(192.0)
    p.q_nope, p.q_rope, p.w_uk = bufs["q_nope"], bufs["q_rope"], bufs["w_uk"]
    p.latent, p.rope_key = bufs["latent"], bufs["rope_key"]
    p.latent_session_stride, p.rope_session_stride = context * dc, context * dr
    p.kv_tokens_uniform = p.kv_tokens_max = context
    out, status = _alloc(lib, sessions * heads * dc * 4), _alloc(lib, 4)
    lib.yvx_cuda_memset_async(status, 0, 4, s)
    p.output, p.status = out, status

    def run(chunk):
        lib.yvx_cuda_mla_plan(C.byref(p), backend.sm_count)
        if chunk:
            p.chunk_tokens, p.max_splits = chunk, (context + chunk - 1) // chunk
        q_abs = _alloc(lib, lib.yvx_cuda_mla_absorbed_bytes(C.byref(p)))
        parts = _alloc(lib, lib.yvx_cuda_mla_partials_bytes(C.byref(p)))
        p.q_absorbed, p.partials = q_abs, parts
        n = C.c_uint()
        assert lib.yvx_cuda_mla_decode(C.byref(p), s, None, C.byref(n)) == 0, lib.yvx_cuda_last_error_text()
        got = _download(lib, s, out, np.empty((sessions, heads, dc), np.float32)).copy()
        lib.yvx_cuda_free(q_abs)
        lib.yvx_cuda_free(parts)
        return got

    planned, fine = run(0), run(1984)
    assert np.isfinite(planned).all() and np.abs(planned - fine).max() <= 2e-3
    # a constant latent row: every output dim is that constant
    lib.yvx_cuda_memset_async(bufs["latent"], UNIFORM_BYTE, sizes["latent"] * 2, s)
    flat = run(0)
    assert np.abs(flat - UNIFORM_BF16).max() <= UNIFORM_BF16 * 2.0 ** -7
    st = _download(lib, s, status, np.zeros(1, np.int32))
    assert st[0] == 0
    for ptr in list(bufs.values()) + [out, status]:
        lib.yvx_cuda_free(ptr)
