"""Python view of the operator interface in include/yvex_b200/attention.h.

Names and argument meaning follow the reference's C interface
(include/yvex/backend.h, include/yvex/internal/transformer.h:245-294); every
method is one call through the C-ABI and returns the reference's status codes
(raised as YvexError when non-zero unless `check=False`).
"""
import ctypes as C

import numpy as np

from . import abi


class YvexError(RuntimeError):
    def __init__(self, code, where, message):
        super().__init__(f"{abi.load().yvex_status_name(code).decode()} ({code}) at {where}: {message}")
        self.code, self.where, self.message = code, where, message


def _raise(err):
    raise YvexError(err.code, err.where.decode(errors="replace"), err.message.decode(errors="replace"))


def f32_to_bf16_bits(x):
    """Round-to-nearest-even bf16 bits of a float32 array (NaNs quieted)."""
    x = np.ascontiguousarray(x, np.float32)
    bits = x.view(np.uint32)
    high = bits >> 16
    low = bits & 0xFFFF
    nan = ((bits & 0x7F800000) == 0x7F800000) & ((bits & 0x007FFFFF) != 0)
    up = (low > 0x8000) | ((low == 0x8000) & ((high & 1) == 1))
    out = np.where(nan, high | 0x40, high + up.astype(np.uint32))
    return out.astype(np.uint16)


def bf16_bits_to_f32(bits):
    return (np.ascontiguousarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def attention_requirement(query_tokens, key_value_tokens, query_start, query_heads,
                          key_value_heads, head_dimension, causal=True, dtype=abi.DTYPE_F32,
                          output_dtype=None, numeric_contract=abi.NUMERIC_EXACT_F32,
                          query_token_stride=0, key_token_stride=0, value_token_stride=0,
                          query_dtype=None):
    r = abi.AttentionRequirement()
    r.query_tokens, r.key_value_tokens, r.query_start = query_tokens, key_value_tokens, query_start
    r.query_heads, r.key_value_heads, r.head_dimension = query_heads, key_value_heads, head_dimension
    r.query_token_stride, r.key_token_stride, r.value_token_stride = (
        query_token_stride, key_token_stride, value_token_stride)
    r.query_dtype = dtype if query_dtype is None else query_dtype
    r.key_dtype = r.value_dtype = dtype
    r.output_dtype = dtype if output_dtype is None else output_dtype
    r.layout = abi.LAYOUT_TOKEN_HEAD_DIM
    r.mask = abi.MASK_CAUSAL if causal else abi.MASK_FULL
    r.numeric_contract = numeric_contract
    r.deterministic = 1
    return r


_NP_DTYPES = {abi.DTYPE_F32: np.float32, abi.DTYPE_BF16: np.uint16, abi.DTYPE_F16: np.uint16,
              abi.DTYPE_I32: np.int32, abi.DTYPE_I8: np.int8, abi.DTYPE_I64: np.int64,
              abi.DTYPE_F64: np.float64}


class Tensor:
    """A yvex_device_tensor owned by (or wrapped into) a Backend."""

    def __init__(self, backend, pointer, shape, dtype):
        self.backend, self.ptr, self.shape, self.dtype = backend, pointer, tuple(shape), dtype

    @property
    def struct(self):
        return self.ptr.contents

    @property
    def data_ptr(self):
        return self.ptr.contents.data

    @property
    def nbytes(self):
        return self.ptr.contents.bytes

    def write(self, array):
        array = np.ascontiguousarray(array)
        assert array.nbytes <= self.nbytes, (array.nbytes, self.nbytes)
        err = abi.Error()
        rc = self.backend.lib.yvex_backend_tensor_write(
            self.backend.handle, self.ptr, array.ctypes.data_as(C.c_void_p), array.nbytes, C.byref(err))
        if rc:
            _raise(err)
        return self

    def read(self, np_dtype=None, shape=None):
        np_dtype = np_dtype or _NP_DTYPES[self.dtype]
        out = np.empty(self.nbytes // np.dtype(np_dtype).itemsize, np_dtype)
        err = abi.Error()
        rc = self.backend.lib.yvex_backend_tensor_read(
            self.backend.handle, self.ptr, out.ctypes.data_as(C.c_void_p), out.nbytes, C.byref(err))
        if rc:
            _raise(err)
        return out.reshape(shape or self.shape)

    def f32_subview(self, offset, count):
        view = abi.DeviceTensor()
        ok = self.backend.lib.yvex_backend_tensor_f32_subview(self.ptr, offset, count, C.byref(view))
        if not ok:
            return None
        return Tensor(self.backend, C.pointer(view), (count,), abi.DTYPE_F32)

    def release(self):
        if self.ptr is not None:
            err = abi.Error()
            handle = self.ptr
            rc = self.backend.lib.yvex_backend_tensor_release(self.backend.handle, C.byref(handle), C.byref(err))
            self.ptr = None
            if rc:
                _raise(err)


class Backend:
    """yvex_backend on one B200 (yvex_backend_open with kind CUDA)."""

    def __init__(self, device=0, kind=abi.BACKEND_KIND_CUDA):
        self.lib = abi.load()
        self.handle = C.c_void_p()
        options = abi.BackendOptions(kind, str(device).encode(), 0)
        err = abi.Error()
        rc = self.lib.yvex_backend_open(C.byref(self.handle), C.byref(options), C.byref(err))
        if rc:
            _raise(err)
        self.device = device
        self._tensors = []

    # -- tensors -------------------------------------------------------------
    def _desc(self, name, dtype, shape, nbytes=None):
        desc = abi.TensorDesc()
        desc.name = name.encode()
        desc.dtype = dtype
        shape = tuple(int(d) for d in shape)
        if len(shape) > abi.MAX_DIMS:  # the ABI holds four dims: fold the leading ones
            shape = (int(np.prod(shape[:len(shape) - abi.MAX_DIMS + 1])),) + shape[len(shape) - abi.MAX_DIMS + 1:]
        desc.rank = len(shape)
        for i, d in enumerate(shape):
            desc.dims[i] = int(d)
        desc.bytes = int(nbytes if nbytes is not None else int(np.prod(shape)) * abi.DTYPE_BYTES[dtype])
        return desc

    def alloc(self, name, dtype, shape, nbytes=None):
        desc = self._desc(name, dtype, shape, nbytes)
        ptr = C.POINTER(abi.DeviceTensor)()
        err = abi.Error()
        rc = self.lib.yvex_backend_tensor_alloc(self.handle, C.byref(desc), C.byref(ptr), C.byref(err))
        if rc:
            _raise(err)
        t = Tensor(self, ptr, shape, dtype)
        self._tensors.append(t)
        return t

    def wrap(self, name, dtype, shape, device_pointer, nbytes=None):
        desc = self._desc(name, dtype, shape, nbytes)
        ptr = C.POINTER(abi.DeviceTensor)()
        err = abi.Error()
        rc = self.lib.yvex_b200_tensor_wrap(self.handle, C.byref(desc), C.c_void_p(device_pointer),
                                            C.byref(ptr), C.byref(err))
        if rc:
            _raise(err)
        t = Tensor(self, ptr, shape, dtype)
        self._tensors.append(t)
        return t

    def tensor(self, name, array, dtype=None):
        """Allocate a tensor shaped like `array` and upload it."""
        array = np.ascontiguousarray(array)
        if dtype is None:
            dtype = {np.dtype(np.float32): abi.DTYPE_F32, np.dtype(np.uint16): abi.DTYPE_BF16,
                     np.dtype(np.int32): abi.DTYPE_I32, np.dtype(np.int8): abi.DTYPE_I8,
                     np.dtype(np.int64): abi.DTYPE_I64, np.dtype(np.float64): abi.DTYPE_F64}[array.dtype]
        return self.alloc(name, dtype, array.shape, array.nbytes).write(array)

    # -- operators -----------------------------------------------------------
    def attention_workspace_required(self, requirement, check=True):
        ops = self.lib.yvex_b200_transformer_operations_get(self.handle)
        nbytes = abi.u64(2**64 - 1)
        err = abi.Error()
        rc = ops.contents.attention_workspace_required(C.byref(requirement), C.byref(nbytes), C.byref(err))
        if rc and check:
            _raise(err)
        return rc, nbytes.value

    def attention_execute(self, requirement, query, key, value, output, check=True):
        """operations->attention_execute(backend, request, facts, err)."""
        ops = self.lib.yvex_b200_transformer_operations_get(self.handle)
        request = abi.AttentionRequest()
        request.requirement = requirement
        request.query = query.ptr if query is not None else None
        request.key = key.ptr if key is not None else None
        request.value = value.ptr if value is not None else None
        request.output = output.ptr if output is not None else None
        facts = abi.OperationFacts()
        err = abi.Error()
        rc = ops.contents.attention_execute(self.handle, C.byref(request), C.byref(facts), C.byref(err))
        if rc and check:
            _raise(err)
        return rc, facts

    def attention_batch_execute(self, requirement, query, key, value, kv_tokens, output,
                                block_table=None, block_tokens=0, max_blocks_per_session=0,
                                kv_session_stride=0, kv_block_stride=0, kv_head_stride=0,
                                check=True):
        request = abi.BatchRequest()
        request.requirement = requirement
        request.session_count = kv_tokens.shape[0]
        request.kv_layout = abi.KV_BLOCK_TABLE if block_table is not None else abi.KV_CONTIGUOUS
        request.query, request.key, request.value = query.ptr, key.ptr, value.ptr
        request.kv_tokens = kv_tokens.ptr
        request.block_table = block_table.ptr if block_table is not None else None
        request.block_tokens = block_tokens
        request.max_blocks_per_session = max_blocks_per_session
        request.kv_session_stride = kv_session_stride
        request.kv_block_stride = kv_block_stride
        request.kv_head_stride = kv_head_stride
        request.output = output.ptr
        facts = abi.OperationFacts()
        err = abi.Error()
        rc = self.lib.yvex_b200_attention_batch_execute(self.handle, C.byref(request), C.byref(facts), C.byref(err))
        if rc and check:
            _raise(err)
        return rc, facts

    def op_attention(self, query, keys, values, seq_len, position, scale, causal, scores,
                     probabilities, out, check=True):
        err = abi.Error()
        rc = self.lib.yvex_backend_op_attention(
            self.handle, query.ptr, keys.ptr, values.ptr, seq_len, position, scale, int(causal),
            scores.ptr, probabilities.ptr, out.ptr, C.byref(err))
        if rc and check:
            _raise(err)
        return rc

    def kv_append_rotary(self, key, value, cosines, sines, *, kv_heads, head_dim, rotary_dim, max_kv_tokens,
                         query=None, query_heads=0, kv_tokens=None, token_position=None, staged=True,
                         state_values=None, state_positions=None, state_capacity=0, state_row_stride=0,
                         key_pool=None, value_pool=None, block_table=None, block_tokens=0, check=True):
        """yvex_b200_kv_append_rotary_execute: key/value [sessions, tokens, kv_heads*head_dim] F32 tensors."""
        cast = lambda t: C.cast(t.ptr, C.c_void_p) if t is not None else None
        r = abi.KvAppendRequest()
        r.session_count, r.token_count = key.shape[0], key.shape[1]
        r.query_heads, r.key_value_heads, r.head_dimension, r.rotary_dimension = query_heads, kv_heads, head_dim, rotary_dim
        r.bf16_staged_products = int(staged)
        r.query, r.key, r.value, r.cosines, r.sines = cast(query), cast(key), cast(value), cast(cosines), cast(sines)
        r.kv_tokens, r.max_kv_tokens, r.token_position = cast(kv_tokens), max_kv_tokens, cast(token_position)
        r.state_values, r.state_positions = cast(state_values), cast(state_positions)
        r.state_capacity, r.state_row_stride = state_capacity, state_row_stride
        r.key_pool, r.value_pool, r.block_table = cast(key_pool), cast(value_pool), cast(block_table)
        if block_table is not None:
            r.block_tokens, r.max_blocks_per_session = block_tokens, block_table.shape[1]
            r.pool_blocks = key_pool.shape[0]
        facts, err = abi.OperationFacts(), abi.Error()
        rc = self.lib.yvex_b200_kv_append_rotary_execute(self.handle, C.byref(r), C.byref(facts), C.byref(err))
        if rc and check:
            _raise(err)
        return rc, facts

    def mla_decode(self, q_nope, q_rope, w_uk, latent, rope_key, output, *, max_kv_tokens, scale,
                   kv_tokens=None, check=True):
        """yvex_b200_mla_decode_execute: bf16 tensors [sessions, 128, 128 | 64], [128, 128, 512],
        caches [sessions, capacity, 512 | 64]; output F32 [sessions, 128, 512]."""
        cast = lambda t: C.cast(t.ptr, C.c_void_p) if t is not None else None
        r = abi.MlaDecodeRequest()
        r.session_count, r.heads, r.nope_dimension = q_nope.shape[0], q_nope.shape[1], q_nope.shape[2]
        r.latent_dimension, r.rope_dimension = latent.shape[2], rope_key.shape[2]
        r.context_capacity, r.max_kv_tokens, r.scale = latent.shape[1], max_kv_tokens, scale
        r.q_nope, r.q_rope, r.w_uk = cast(q_nope), cast(q_rope), cast(w_uk)
        r.latent, r.rope_key, r.kv_tokens, r.output = cast(latent), cast(rope_key), cast(kv_tokens), cast(output)
        facts, err = abi.OperationFacts(), abi.Error()
        rc = self.lib.yvex_b200_mla_decode_execute(self.handle, C.byref(r), C.byref(facts), C.byref(err))
        if rc and check:
            _raise(err)
        return rc, facts

    def _latent_stage(self, function, request, fields, check):
        """Fill a latent-stage request from keyword fields (Tensors become pointers) and call it.
        Returns (rc, facts, failure, request)."""
        for name, value in fields.items():
            setattr(request, name, C.cast(value.ptr, C.c_void_p) if isinstance(value, Tensor) else value)
        failure, facts, err = abi.AttentionFailure(), abi.OperationFacts(), abi.Error()
        rc = function(self.handle, C.byref(request), C.byref(failure), C.byref(facts), C.byref(err))
        if rc and check:
            _raise(err)
        return rc, facts, failure, request

    def attention_publish(self, values, *, check=True, **fields):
        """yvex_b200_attention_publish_execute over an F32 [rows, width] tensor in place. Fields as in
        yvex_b200_attention_publish_request (rows_per_token, token_position, norm_mode, norm_weights,
        rms_norm_epsilon, rope_dimension, rope_frequency, activation_*); rows / row_stride / width
        default to the tensor's shape."""
        fields = {"rows": values.shape[0], "row_stride": values.shape[1], "width": values.shape[1],
                  "rows_per_token": 1, **fields}
        return self._latent_stage(self.lib.yvex_b200_attention_publish_execute, abi.AttentionPublishRequest(),
                                  {"values": values, **fields}, check)[:3]

    def attention_activation(self, values, *, quantization, block_width, hadamard=False, count=None, check=True):
        """yvex_b200_attention_activation_execute over the first `count` lanes of every row, in place."""
        fields = {"values": values, "rows": values.shape[0], "row_stride": values.shape[1],
                  "count": values.shape[1] if count is None else count, "quantization": quantization,
                  "block_width": block_width, "hadamard": int(hadamard)}
        return self._latent_stage(self.lib.yvex_b200_attention_activation_execute,
                                  abi.AttentionActivationRequest(), fields, check)[:3]

    def attention_compress(self, *, check=True, **fields):
        """yvex_b200_attention_compress_execute; fields as in yvex_b200_attention_compress_request.
        Returns (rc, facts, failure, emitted rows)."""
        rc, facts, failure, request = self._latent_stage(self.lib.yvex_b200_attention_compress_execute,
                                                         abi.AttentionCompressRequest(), fields, check)
        return rc, facts, failure, int(request.emitted)

    def attention_select(self, *, check=True, **fields):
        """yvex_b200_attention_select_execute; fields as in yvex_b200_attention_select_request."""
        return self._latent_stage(self.lib.yvex_b200_attention_select_execute, abi.AttentionSelectRequest(),
                                  fields, check)[:3]

    def attention_reduce(self, *, check=True, **fields):
        """yvex_b200_attention_reduce_execute; fields as in yvex_b200_attention_reduce_request."""
        return self._latent_stage(self.lib.yvex_b200_attention_reduce_execute, abi.AttentionReduceRequest(),
                                  fields, check)[:3]

    # -- lifecycle -----------------------------------------------------------
    def bind_stream(self, stream, synchronous=True):
        err = abi.Error()
        rc = self.lib.yvex_b200_backend_bind_stream(self.handle, C.c_void_p(stream), int(synchronous), C.byref(err))
        if rc:
            _raise(err)

    @property
    def stream(self):
        return self.lib.yvex_b200_backend_stream(self.handle)

    @property
    def sm_count(self):
        return self.lib.yvex_b200_backend_sm_count(self.handle)

    def sync(self, check=True):
        err = abi.Error()
        rc = self.lib.yvex_backend_sync(self.handle, C.byref(err))
        if rc and check:
            _raise(err)
        return rc

    def close(self):
        if self.handle:
            for t in self._tensors:
                if t.ptr is not None:
                    t.release()
            self._tensors = []
            err = abi.Error()
            rc = self.lib.yvex_backend_close_checked(C.byref(self.handle), C.byref(err))
            if rc:
                _raise(err)
            self.handle = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class KvPool:
    """Host-side block bookkeeping of the pooled KV layout (yvex_b200_kv_pool_*)."""

    def __init__(self, blocks, block_tokens, max_sessions, max_blocks_per_session):
        self.lib = abi.load()
        self.per = max_blocks_per_session
        self.handle = self.lib.yvex_b200_kv_pool_create(blocks, block_tokens, max_sessions, max_blocks_per_session)
        if not self.handle:
            raise ValueError("bad block pool geometry")

    def _check(self, rc):
        if rc:
            raise YvexError(rc, "b200.kv.pool", abi.load().yvex_status_name(rc).decode())

    def open(self):
        s = C.c_uint()
        self._check(self.lib.yvex_b200_kv_pool_session_open(self.handle, C.byref(s)))
        return s.value

    def fork(self, parent):
        s = C.c_uint()
        self._check(self.lib.yvex_b200_kv_pool_session_fork(self.handle, parent, C.byref(s)))
        return s.value

    def close_session(self, session):
        self._check(self.lib.yvex_b200_kv_pool_session_close(self.handle, session))

    def reserve(self, session, rows):
        """Returns None, or (source_block, destination_block, rows) to copy for K and V before appending."""
        copy = abi.KvCopy()
        self._check(self.lib.yvex_b200_kv_pool_reserve(self.handle, session, rows, C.byref(copy)))
        return (copy.source_block, copy.destination_block, copy.rows) if copy.needed else None

    def commit(self, session, accepted):
        self._check(self.lib.yvex_b200_kv_pool_commit(self.handle, session, accepted))

    def table(self, session):
        row = self.lib.yvex_b200_kv_pool_table(self.handle, session)
        return np.array([row[i] for i in range(self.per)], np.int32)

    def committed(self, session):
        return int(self.lib.yvex_b200_kv_pool_committed(self.handle, session))

    def free_blocks(self):
        return int(self.lib.yvex_b200_kv_pool_free_blocks(self.handle))

    def destroy(self):
        if self.handle:
            self.lib.yvex_b200_kv_pool_destroy(self.handle)
            self.handle = None
