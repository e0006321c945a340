"""Test helper: drives yvx_cuda_gqa_attention (the plain-pointer shim) directly
so that tests can pick the general or the specialised kernel and lay KV out in
ways the operator-level request does not express."""
import ctypes as C

import numpy as np

from clori_b200 import abi


def run_problem(backend, *, q, k, v, lengths, rows, hq, hkv, hd, dtype, out_dtype=abi.DTYPE_F32,
                causal=True, table=None, block_tokens=64, pool_blocks=0,
                k_token_stride, v_token_stride, k_head_stride, v_head_stride,
                k_outer_stride, v_outer_stride, v_offset_elems=0, kv_max=None,
                force_general=False, chunk_tokens=None, query_start=None, position_base=0,
                partial_output=False, entry="yvx_cuda_gqa_attention", own_scratch=True,
                k_offset_elems=0, q_row_stride=None, q_head_stride=0, tickets=None):
    """q: device Tensor [sessions, rows, hq*hd]; k, v: device Tensors holding the
    cache in any layout described by the strides (elements). Returns the output
    array (or the (o, m, l) partials) and the launch count."""
    lib = backend.lib
    sessions = len(lengths)
    p = abi.GqaProblem()
    p.sessions, p.query_rows, p.query_heads, p.kv_heads, p.head_dim = sessions, rows, hq, hkv, hd
    p.causal, p.scale = int(causal), 1.0 / np.sqrt(hd)
    p.query_dtype = p.kv_dtype = dtype
    p.output_dtype = out_dtype
    p.query, p.query_row_stride = q.data_ptr, q_row_stride or hq * hd
    p.query_session_stride, p.query_head_stride = rows * p.query_row_stride, q_head_stride
    esize = abi.DTYPE_BYTES[dtype]
    p.key, p.value = k.data_ptr + k_offset_elems * esize, v.data_ptr + v_offset_elems * esize
    p.key_token_stride, p.value_token_stride = k_token_stride, v_token_stride
    p.key_head_stride, p.value_head_stride = k_head_stride, v_head_stride
    lens = backend.tensor("lens", np.asarray(lengths, np.int32))
    p.kv_tokens = lens.data_ptr
    p.kv_tokens_max = int(kv_max if kv_max is not None else max(lengths))
    if table is not None:
        t = backend.tensor("table", np.asarray(table, np.int32))
        p.block_table, p.block_tokens, p.block_table_stride = t.data_ptr, block_tokens, table.shape[1]
        p.pool_blocks = pool_blocks
        p.key_block_stride, p.value_block_stride = k_outer_stride, v_outer_stride
    else:
        p.key_session_stride, p.value_session_stride = k_outer_stride, v_outer_stride
    if query_start is None:
        p.query_start_from_end = 1
    else:
        qs = backend.tensor("qs", np.asarray(query_start, np.int32))
        p.query_start = qs.data_ptr
    p.kv_position_base = position_base
    p.force_general = int(force_general)
    if tickets is not None:
        p.tickets = tickets.data_ptr
    lib.yvx_cuda_gqa_plan_splits(C.byref(p), backend.sm_count)
    if chunk_tokens:
        p.chunk_tokens = chunk_tokens
        p.max_splits = (p.kv_tokens_max + chunk_tokens - 1) // chunk_tokens
    status = backend.tensor("status", np.zeros(1, np.int32))
    p.status = status.data_ptr
    if own_scratch:
        scratch = backend.alloc("partials", abi.DTYPE_F32, (1,),
                                max(lib.yvx_cuda_gqa_partials_bytes(C.byref(p)), 16))
        p.partials = scratch.data_ptr
    if partial_output:
        out = backend.alloc("parts", abi.DTYPE_F32, (sessions, rows, hq, hd + 2))
        p.partial_output = out.data_ptr
    else:
        out = backend.alloc("out", out_dtype, (sessions, rows, hq * hd))
        p.output = out.data_ptr
    launches = C.c_uint()
    rc = getattr(lib, entry)(C.byref(p), backend.stream, C.byref(launches))
    if rc != 0 and entry != "yvx_cuda_gqa_attention":
        return None, rc, 0, (p.chunk_tokens, p.max_splits)
    assert rc == 0, lib.yvx_cuda_last_error_text()
    assert lib.yvx_cuda_stream_synchronize(backend.stream) == 0, lib.yvx_cuda_last_error_text()
    out.struct.is_written = 1
    return out.read(), int(status.read()[0]), launches.value, (p.chunk_tokens, p.max_splits)
