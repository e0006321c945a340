"""TEST INFRASTRUCTURE ONLY: ctypes bindings of the CPU checkers.

`Oracle` wraps libyvx_oracle.so (the C restatement, always buildable).
`Reference` wraps _ref/libyvex_ref.so (the reference's own CPU code; exists
only where it was built from the reference tree) and exposes the same methods
for the functions both provide, so tests can run either against the other.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libyvx_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libyvex_ref.so")

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_u64 = C.c_ulonglong
_u64p = np.ctypeslib.ndpointer(np.uint64, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")


class PositionPolicy(C.Structure):
    """yvx_oracle_position_policy."""
    _fields_ = [(name, _u64) for name in ("theta", "scaling_factor", "original_context", "beta_fast", "beta_slow")]


class Indexer(C.Structure):
    """yvx_oracle_indexer (host pointers)."""
    _fields_ = [("keys", C.c_void_p), ("positions", C.c_void_p), ("rows", _u64), ("key_stride", _u64),
                ("query", C.c_void_p), ("weights", C.c_void_p), ("heads", _u64), ("head_dim", _u64),
                ("topk", _u64), ("ratio", _u64)]


def indexer_struct(keys, positions, query, weights, heads, head_dim, topk, ratio):
    """The arrays must stay alive while the struct is in use; they are attached to it."""
    ix = Indexer()
    ix.arrays = [np.ascontiguousarray(keys, np.float32), np.ascontiguousarray(positions, np.uint64),
                 np.ascontiguousarray(query, np.float32), np.ascontiguousarray(weights, np.float32)]
    ix.keys, ix.positions, ix.query, ix.weights = (a.ctypes.data for a in ix.arrays)
    ix.rows, ix.key_stride = ix.arrays[0].shape
    ix.heads, ix.head_dim, ix.topk, ix.ratio = heads, head_dim, topk, ratio
    return ix


class CompressorArgs(C.Structure):
    """yvx_oracle_compressor_args (host pointers here, device pointers in the library)."""
    _fields_ = [("ratio", _u64), ("head_dim", _u64), ("overlap", C.c_int), ("start_position", _u64),
                ("token_count", _u64), ("token_kv", C.c_void_p), ("token_score", C.c_void_p),
                ("token_stride", _u64), ("ape", C.c_void_p), ("state_kv", C.c_void_p),
                ("state_score", C.c_void_p), ("after_kv", C.c_void_p), ("after_score", C.c_void_p),
                ("compressed", C.c_void_p), ("compressed_stride", _u64), ("positions", C.c_void_p),
                ("norm_weights", C.c_void_p), ("epsilon", C.c_double), ("rope_dims", _u64),
                ("rope_frequency", C.c_void_p), ("device_status", C.c_void_p)]


def compressor_initial_state(ratio, head_dim, overlap):
    """The state before any token: zeros, and with two halves the previous half's
    scores at minus infinity (src/graph/attention.c:540-551)."""
    width, slots = head_dim * (2 if overlap else 1), ratio * (2 if overlap else 1)
    kv, score = np.zeros((slots, width), np.float32), np.zeros((slots, width), np.float32)
    if overlap:
        score[:ratio, :head_dim] = -np.inf
    return kv, score


def _compressor_call(call, ratio, head_dim, overlap, start, token_kv, token_score, ape, state_kv,
                     state_score, norm_weights, epsilon, rope_dims, rope_frequency):
    token_kv = np.ascontiguousarray(token_kv, np.float32)
    token_score = np.ascontiguousarray(token_score, np.float32)
    ape = np.ascontiguousarray(ape, np.float32)
    state_kv = np.ascontiguousarray(state_kv, np.float32)
    state_score = np.ascontiguousarray(state_score, np.float32)
    tokens = token_kv.shape[0]
    capacity = max(1, tokens // ratio + 1)
    after_kv, after_score = np.zeros_like(state_kv), np.zeros_like(state_score)
    compressed = np.zeros((capacity, head_dim), np.float32)
    positions = np.zeros(capacity, np.uint64)
    a = CompressorArgs()
    a.ratio, a.head_dim, a.overlap, a.start_position, a.token_count = ratio, head_dim, int(overlap), start, tokens
    a.token_kv, a.token_score = token_kv.ctypes.data, token_score.ctypes.data
    a.token_stride = token_kv.shape[1] if tokens else head_dim * 2
    a.ape, a.state_kv, a.state_score = ape.ctypes.data, state_kv.ctypes.data, state_score.ctypes.data
    a.after_kv, a.after_score = after_kv.ctypes.data, after_score.ctypes.data
    a.compressed, a.compressed_stride, a.positions = compressed.ctypes.data, head_dim, positions.ctypes.data
    keep = [token_kv, token_score, ape, state_kv, state_score]
    if norm_weights is not None:
        keep.append(np.ascontiguousarray(norm_weights, np.float32))
        a.norm_weights, a.epsilon, a.rope_dims = keep[-1].ctypes.data, float(epsilon), rope_dims
        if rope_dims and rope_frequency is not None:
            keep.append(np.ascontiguousarray(rope_frequency, np.float64))
            a.rope_frequency = keep[-1].ctypes.data
    emitted = _u64()
    ok = call(a, emitted)
    if ok != 1:
        return None
    n = emitted.value
    return compressed[:n].copy(), positions[:n].copy(), after_kv, after_score


class PublishArgs(C.Structure):
    """yvx_oracle_publish_args (host pointers here, device pointers in the library)."""
    _fields_ = [("values", C.c_void_p), ("rows", _u64), ("rows_per_token", _u64), ("row_stride", _u64),
                ("width", _u64), ("norm_mode", C.c_int), ("norm_weights", C.c_void_p), ("epsilon", C.c_double),
                ("rope_dims", _u64), ("rope_frequency", C.c_void_p), ("start_position", _u64),
                ("quantization", C.c_uint), ("activation_count", _u64), ("block_width", _u64),
                ("hadamard", C.c_int), ("device_status", C.c_void_p)]


def _publish_call(call, rows, rows_per_token, start, norm_mode=0, norm_weights=None, epsilon=1e-6, rope_dims=0,
                  rope_frequency=None, quantization=0, activation_count=0, block_width=0, hadamard=0):
    out = np.ascontiguousarray(rows, np.float32).copy()
    a = PublishArgs()
    a.values, a.rows, a.rows_per_token, a.row_stride, a.width = out.ctypes.data, out.shape[0], rows_per_token, \
        out.shape[1], out.shape[1]
    keep = []
    a.norm_mode, a.epsilon = norm_mode, float(epsilon)
    if norm_weights is not None:
        keep.append(np.ascontiguousarray(norm_weights, np.float32))
        a.norm_weights = keep[-1].ctypes.data
    a.rope_dims, a.start_position = rope_dims, start
    if rope_frequency is not None:
        keep.append(np.ascontiguousarray(rope_frequency, np.float64))
        a.rope_frequency = keep[-1].ctypes.data
    a.quantization, a.activation_count, a.block_width, a.hadamard = quantization, activation_count, block_width, \
        int(hadamard)
    return out if call(a) == 1 else None


def _activation_call(function, rows, quantization, block_width, hadamard):
    function.argtypes = [_f32p, _u64, C.c_uint, _u64, C.c_int]
    out = np.ascontiguousarray(rows, np.float32).copy()
    for row in out.reshape(-1, out.shape[-1]):
        if function(row, row.size, quantization, block_width, int(hadamard)) != 1:
            return None
    return out


def reference_tree():
    """Where the reference's sources lie: the YVEX_REFERENCE_TREE environment variable,
    else a checkout named `reference` beside this repository; None when neither exists."""
    candidates = [os.environ.get("YVEX_REFERENCE_TREE"),
                  os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for tree in candidates:
        if tree and os.path.isdir(os.path.join(tree, "src", "backend")):
            return tree
    return None


def build_oracle(tree=None):
    """Compile the restatement, and the reference build when its tree exists."""
    subprocess.run(["make", "-s", "-C", HERE, "oracle"], check=True)
    reference_tree_path = tree or reference_tree()
    if reference_tree_path:
        subprocess.run(["make", "-s", "-C", HERE, "ref", f"REF={reference_tree_path}"], check=True)
        import shutil
        nvcc = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
        if os.path.exists(nvcc):
            # the reference's CUDA attention kernels as a cubin (timed by bench.py as "reference_gpu")
            subprocess.run(["make", "-s", "-C", HERE, "ref_cuda", f"REF={reference_tree_path}", f"NVCC={nvcc}"],
                           check=True)


REFERENCE_CUBIN = os.path.join(HERE, "_ref", "transformer_kernels.sm_100.cubin")


class _Gqa:
    """Shared wrappers; subclasses set self.lib and self.prefix."""

    def _bind_common(self):
        p = self.prefix
        lib = self.lib
        getattr(lib, p + "bf16_decode").restype = C.c_float
        getattr(lib, p + "bf16_decode").argtypes = [C.c_ushort]
        getattr(lib, p + "bf16_encode").restype = C.c_ushort
        getattr(lib, p + "bf16_encode").argtypes = [C.c_float]
        getattr(lib, p + "f16_decode").restype = C.c_float
        getattr(lib, p + "f16_decode").argtypes = [C.c_ushort]
        getattr(lib, p + "f16_encode").restype = C.c_ushort
        getattr(lib, p + "f16_encode").argtypes = [C.c_float]
        getattr(lib, p + "q8_0_encode_block").argtypes = [_f32p, _u8p]
        getattr(lib, p + "q8_0_decode_block").argtypes = [_u8p, _f32p]
        getattr(lib, p + "op_attention").argtypes = [
            _f32p, _f32p, _f32p, _u64, _u64, C.c_float, C.c_int, _u64, _f32p, _f32p, _f32p]
        getattr(lib, p + "gqa_attention").argtypes = [
            _f32p, _f32p, _f32p, _f32p, _u64, _u64, _u64, _u64, _u64, _u64, _u64, _u64, _u64,
            C.c_float, C.c_int, C.c_uint]

    def bf16_encode(self, x):
        return int(getattr(self.lib, self.prefix + "bf16_encode")(float(np.float32(x))))

    def bf16_decode(self, bits):
        return float(getattr(self.lib, self.prefix + "bf16_decode")(int(bits)))

    def f16_encode(self, x):
        return int(getattr(self.lib, self.prefix + "f16_encode")(float(np.float32(x))))

    def f16_decode(self, bits):
        return float(getattr(self.lib, self.prefix + "f16_decode")(int(bits)))

    def q8_0_encode_block(self, values):
        values = np.ascontiguousarray(values, np.float32)
        assert values.shape == (32,)
        out = np.zeros(34, np.uint8)
        ok = getattr(self.lib, self.prefix + "q8_0_encode_block")(values, out)
        return out if ok else None

    def q8_0_decode_block(self, encoded):
        encoded = np.ascontiguousarray(encoded, np.uint8)
        out = np.zeros(32, np.float32)
        ok = getattr(self.lib, self.prefix + "q8_0_decode_block")(encoded, out)
        return out if ok else None

    def op_attention(self, q, k, v, position, scale, causal):
        q = np.ascontiguousarray(q, np.float32)
        k = np.ascontiguousarray(k, np.float32)
        v = np.ascontiguousarray(v, np.float32)
        seq, hd = k.shape
        scores = np.zeros(seq, np.float32)
        probs = np.zeros(seq, np.float32)
        out = np.zeros(hd, np.float32)
        rc = getattr(self.lib, self.prefix + "op_attention")(
            q, k, v, seq, position, scale, int(causal), hd, scores, probs, out)
        return rc, out, scores, probs

    def gqa_attention(self, q, k, v, query_start, query_heads, kv_heads, head_dim,
                      causal=True, scale=None, threads=1,
                      q_stride=0, k_stride=0, v_stride=0,
                      query_tokens=None, kv_tokens=None):
        """q [Tq, Hq*hd] (or strided flat), k/v [Tkv, Hkv*hd]; returns [Tq, Hq*hd]."""
        q = np.ascontiguousarray(q, np.float32)
        k = np.ascontiguousarray(k, np.float32)
        v = np.ascontiguousarray(v, np.float32)
        tq = query_tokens if query_tokens is not None else q.shape[0]
        tkv = kv_tokens if kv_tokens is not None else k.shape[0]
        if scale is None:
            scale = 1.0 / np.sqrt(np.float32(head_dim))
        out = np.zeros((tq, query_heads * head_dim), np.float32)
        rc = getattr(self.lib, self.prefix + "gqa_attention")(
            q.reshape(-1), k.reshape(-1), v.reshape(-1), out.reshape(-1), tq, tkv,
            query_start, query_heads, kv_heads, head_dim, q_stride, k_stride, v_stride,
            float(scale), int(causal), threads)
        if rc != 0:
            raise RuntimeError(f"{self.prefix}gqa_attention failed: {rc}")
        return out


class Oracle(_Gqa):
    prefix = "yvx_oracle_"

    def __init__(self):
        if not os.path.exists(ORACLE_SO):
            build_oracle()
        self.lib = C.CDLL(ORACLE_SO)
        self._bind_common()
        lib = self.lib
        lib.yvx_oracle_exp.restype = C.c_double
        lib.yvx_oracle_exp.argtypes = [C.c_double]
        lib.yvx_oracle_bf16_decode_array.argtypes = [_u16p, _f32p, C.c_size_t]
        lib.yvx_oracle_bf16_encode_array.argtypes = [_f32p, _u16p, C.c_size_t]
        lib.yvx_oracle_q8_0_decode_rows.argtypes = [_u8p, _f32p, C.c_size_t]
        lib.yvx_oracle_gqa_f32_reference.restype = None
        lib.yvx_oracle_gqa_f32_reference.argtypes = [
            _f32p, _f32p, _f32p, _f32p, _u64, _u64, _u64, _u64, _u64, _u64, C.c_int]
        lib.yvx_oracle_block_row.restype = _u64
        lib.yvx_oracle_block_row.argtypes = [_i32p, _u64, _u64]
        lib.yvx_oracle_block_gather_u16.restype = None
        lib.yvx_oracle_block_gather_u16.argtypes = [_u16p, _i32p, _u64, _u64, _u64, _u16p]
        lib.yvx_oracle_page_touch.argtypes = [_u64, _u64, _u64, C.POINTER(_u64), C.POINTER(_u64)]
        lib.yvx_oracle_latent_reduce.argtypes = [
            _f32p, _f32p, _f32p, _f32p, _u64, _u64, _u64, _u64, _u64, _u64, C.c_int]
        lib.yvx_oracle_latent_reduce_full.argtypes = [C.c_void_p, _f32p]
        lib.yvx_oracle_mla_decode.argtypes = [
            _u16p, _u16p, _u16p, _u16p, _u16p, _f32p, _u64, _u64, _u64, _u64, _u64,
            C.c_float, C.c_void_p]

    def rotary_half(self, values, cosines, sines, heads, head_dim, rotary_dim, staged):
        """values [tokens, heads*head_dim] float32; returns the rotated copy."""
        out = np.ascontiguousarray(values, np.float32).copy()
        cos = np.ascontiguousarray(cosines, np.float32)
        sin = np.ascontiguousarray(sines, np.float32)
        self.lib.yvx_oracle_rotary_half.argtypes = [_f32p, _f32p, _f32p, _u64, _u64, _u64, _u64, C.c_int]
        ok = self.lib.yvx_oracle_rotary_half(out.reshape(-1), cos.reshape(-1), sin.reshape(-1), out.shape[0],
                                             heads, head_dim, rotary_dim, int(staged))
        assert ok == 1
        return out

    def full_attention_f32(self, qkv, heads, head_width):
        """qkv [rows, heads*3*head_width] float32 -> [rows, heads*head_width]."""
        qkv = np.ascontiguousarray(qkv, np.float32)
        rows = qkv.shape[0]
        out = np.empty((rows, heads * head_width), np.float32)
        scratch = np.empty(rows, np.float32)
        self.lib.yvx_oracle_full_attention_f32.argtypes = [_f32p, _u64, _u64, _u64, _f32p, _f32p]
        ok = self.lib.yvx_oracle_full_attention_f32(qkv.reshape(-1), rows, heads, head_width, out.reshape(-1), scratch)
        return out if ok == 1 else None

    def rope_tables(self, token_start, tokens, width, theta):
        cos = np.empty((tokens, width), np.float32)
        sin = np.empty((tokens, width), np.float32)
        self.lib.yvx_oracle_rope_tables.argtypes = [_u64, _u64, _u64, C.c_double, _f32p, _f32p]
        ok = self.lib.yvx_oracle_rope_tables(token_start, tokens, width, float(theta),
                                             cos.reshape(-1), sin.reshape(-1))
        assert ok == 1
        return cos, sin

    def rope_frequencies(self, policy, rope_dims):
        out = np.zeros(rope_dims // 2, np.float64)
        self.lib.yvx_oracle_rope_frequencies.argtypes = [C.c_void_p, _u64, _f64p]
        assert self.lib.yvx_oracle_rope_frequencies(C.addressof(policy), rope_dims, out) == 1
        return out

    def rope_apply(self, values, rope_dims, position, frequency, inverse):
        out = np.ascontiguousarray(values, np.float32).copy()
        self.lib.yvx_oracle_rope_apply.argtypes = [_f32p, _u64, _u64, _u64, _f64p, C.c_int]
        ok = self.lib.yvx_oracle_rope_apply(out, out.size, rope_dims, position,
                                            np.ascontiguousarray(frequency, np.float64), int(inverse))
        return out if ok == 1 else None

    def topk_select(self, scores, ordinals, k):
        scores = np.ascontiguousarray(scores, np.float32)
        ordinals = np.ascontiguousarray(ordinals, np.uint64)
        out, n = np.zeros(max(len(scores), 1), np.uint64), _u64()
        self.lib.yvx_oracle_topk_select.argtypes = [_f32p, _u64p, _u64, _u64, _u64p, C.POINTER(_u64)]
        ok = self.lib.yvx_oracle_topk_select(scores, ordinals, len(scores), k, out, C.byref(n))
        return out[:n.value].copy() if ok == 1 else None

    def csa_select(self, indexer, token, query_position):
        """-> (selected row indices in ranked order, valid candidate count, float score per row)."""
        out, n, valid = np.zeros(max(indexer.rows, 1), np.uint64), _u64(), _u64()
        scores = np.zeros(max(indexer.rows, 1), np.float32)
        self.lib.yvx_oracle_csa_select.argtypes = [C.c_void_p, _u64, _u64, _u64p, C.POINTER(_u64),
                                                   C.POINTER(_u64), _f32p]
        ok = self.lib.yvx_oracle_csa_select(C.addressof(indexer), token, query_position, out, C.byref(n),
                                            C.byref(valid), scores)
        return (out[:n.value].copy(), valid.value, scores[:indexer.rows]) if ok == 1 else None

    def exp(self, x):
        return float(self.lib.yvx_oracle_exp(float(x)))

    def bf16_round(self, x):
        """float32 array -> (uint16 bits, float32 values after bf16 rounding)."""
        x = np.ascontiguousarray(x, np.float32)
        bits = np.zeros(x.shape, np.uint16)
        self.lib.yvx_oracle_bf16_encode_array(x.reshape(-1), bits.reshape(-1), x.size)
        return bits, self.bf16_widen(bits)

    def bf16_widen(self, bits):
        bits = np.ascontiguousarray(bits, np.uint16)
        out = np.zeros(bits.shape, np.float32)
        self.lib.yvx_oracle_bf16_decode_array(bits.reshape(-1), out.reshape(-1), bits.size)
        return out

    def q8_0_encode_rows(self, values):
        """float32 [..., n] with n % 32 == 0 -> uint8 [..., n/32*34] GGUF Q8_0 rows."""
        values = np.ascontiguousarray(values, np.float32)
        blocks = values.reshape(-1, 32)
        out = np.zeros((blocks.shape[0], 34), np.uint8)
        for i in range(blocks.shape[0]):
            enc = self.q8_0_encode_block(blocks[i])
            assert enc is not None
            out[i] = enc
        return out.reshape(values.shape[:-1] + (values.shape[-1] // 32 * 34,))

    def q8_0_decode_rows(self, encoded, elements):
        encoded = np.ascontiguousarray(encoded, np.uint8).reshape(-1)
        out = np.zeros(elements, np.float32)
        ok = self.lib.yvx_oracle_q8_0_decode_rows(encoded, out, elements)
        return out if ok else None

    def gqa_f32_reference(self, q, k, v, query_start, query_heads, kv_heads, head_dim, causal):
        q = np.ascontiguousarray(q, np.float32)
        k = np.ascontiguousarray(k, np.float32)
        v = np.ascontiguousarray(v, np.float32)
        out = np.zeros((q.shape[0], query_heads * head_dim), np.float32)
        self.lib.yvx_oracle_gqa_f32_reference(
            q.reshape(-1), k.reshape(-1), v.reshape(-1), out.reshape(-1), q.shape[0],
            k.shape[0], query_start, query_heads, kv_heads, head_dim, int(causal))
        return out

    def block_row(self, table, block_tokens, row):
        table = np.ascontiguousarray(table, np.int32)
        return int(self.lib.yvx_oracle_block_row(table, block_tokens, row))

    def block_gather_u16(self, pool, table, block_tokens, rows):
        pool = np.ascontiguousarray(pool, np.uint16)
        table = np.ascontiguousarray(table, np.int32)
        width = pool.shape[-1]
        out = np.zeros((rows, width), np.uint16)
        self.lib.yvx_oracle_block_gather_u16(pool.reshape(-1), table, block_tokens, rows,
                                             width, out.reshape(-1))
        return out

    def page_touch(self, start, count, page_elements):
        first, last = _u64(), _u64()
        ok = self.lib.yvx_oracle_page_touch(start, count, page_elements,
                                            C.byref(first), C.byref(last))
        return (first.value, last.value) if ok else None

    def latent_reduce(self, q, rows, sinks, query_start, heads, head_dim, round_bf16=True):
        q = np.ascontiguousarray(q, np.float32)
        rows = np.ascontiguousarray(rows, np.float32)
        sinks = np.ascontiguousarray(sinks, np.float32)
        out = np.zeros_like(q)
        ok = self.lib.yvx_oracle_latent_reduce(
            q.reshape(-1), rows.reshape(-1), sinks, out.reshape(-1), q.shape[0],
            rows.shape[0], query_start, heads, head_dim, rows.shape[1], int(round_bf16))
        return out if ok else None

    def latent_reduce_full(self, args_struct, tokens, heads, head_dim):
        """args_struct: a ctypes struct whose leading fields are yvx_oracle_latent_args
        (host pointers). Returns float32 [tokens, heads*head_dim] or None."""
        out = np.zeros((tokens, heads * head_dim), np.float32)
        ok = self.lib.yvx_oracle_latent_reduce_full(C.addressof(args_struct), out.reshape(-1))
        return out if ok else None

    def compressor_chunk(self, ratio, head_dim, overlap, start, token_kv, token_score, ape, state_kv,
                         state_score, norm_weights=None, epsilon=1e-6, rope_dims=0, rope_frequency=None):
        """Rolling compressor over a chunk -> (compressed [emitted, head_dim], positions,
        after_kv, after_score) or None on a refusal."""
        self.lib.yvx_oracle_compressor_chunk.argtypes = [C.c_void_p, C.POINTER(_u64)]
        return _compressor_call(
            lambda a, n: self.lib.yvx_oracle_compressor_chunk(C.addressof(a), C.byref(n)),
            ratio, head_dim, overlap, start, token_kv, token_score, ape, state_kv, state_score,
            norm_weights, epsilon, rope_dims, rope_frequency)

    def rows_publish(self, rows, rows_per_token, start, **chain):
        """Norm / rotation / activation chain over float32 [rows, width] -> new array, or None.
        chain: norm_mode, norm_weights, epsilon, rope_dims, rope_frequency, quantization,
        activation_count, block_width, hadamard."""
        self.lib.yvx_oracle_rows_publish.argtypes = [C.c_void_p]
        return _publish_call(lambda a: self.lib.yvx_oracle_rows_publish(C.addressof(a)), rows, rows_per_token,
                             start, **chain)

    def activation_quant(self, rows, quantization, block_width, hadamard):
        """Fake quantisation of every row of a float32 [rows, count] array -> new array, or None."""
        return _activation_call(self.lib.yvx_oracle_activation_quant, rows, quantization, block_width, hadamard)

    def qtype_encode_rows(self, values, qtype):
        """float32 [rows, width] -> encoded uint8 [rows, row_bytes] (F32 0, F16 1, Q8_0 8, BF16 30)."""
        values = np.ascontiguousarray(values, np.float32)
        rows = values.shape[0]
        if qtype == 0:
            return values.view(np.uint8).reshape(rows, -1).copy()
        if qtype == 1:
            return values.astype(np.float16).view(np.uint8).reshape(rows, -1).copy()
        if qtype == 30:
            return self.bf16_round_bits(values).view(np.uint8).reshape(rows, -1).copy()
        if qtype == 8:
            return self.q8_0_encode_rows(values).reshape(rows, -1)
        raise ValueError(qtype)

    def bf16_round_bits(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.zeros(x.shape, np.uint16)
        self.lib.yvx_oracle_bf16_encode_array(x.reshape(-1), out.reshape(-1), x.size)
        return out

    def qtype_decode_rows(self, encoded, qtype, width, first_row=0, rows=None):
        """Encoded uint8 [all rows, row_bytes] -> float32 [rows, width]."""
        encoded = np.ascontiguousarray(encoded, np.uint8)
        rows = encoded.shape[0] - first_row if rows is None else rows
        out = np.zeros((rows, width), np.float32)
        self.lib.yvx_oracle_qtype_decode_row.argtypes = [C.c_uint, C.c_void_p, _u64, _f32p]
        for r in range(rows):
            assert self.lib.yvx_oracle_qtype_decode_row(qtype, encoded[first_row + r].ctypes.data, width, out[r]) == 1
        return out

    def qtype_matvec(self, encoded, qtype, width, inputs, first_row=0, rows=None, round_bf16=True):
        """inputs float32 [tokens, >= width] -> float32 [tokens, rows]; None on a refusal."""
        encoded = np.ascontiguousarray(encoded, np.uint8)
        inputs = np.ascontiguousarray(inputs, np.float32)
        rows = encoded.shape[0] - first_row if rows is None else rows
        out = np.zeros((inputs.shape[0], rows), np.float32)
        self.lib.yvx_oracle_qtype_matvec.argtypes = [C.c_uint, C.c_void_p, _u64, _u64, _u64, _f32p, _u64, _u64,
                                                     _f32p, _u64, C.c_int]
        ok = self.lib.yvx_oracle_qtype_matvec(qtype, encoded.ctypes.data, first_row, rows, width,
                                              inputs.reshape(-1), inputs.shape[0], inputs.shape[1],
                                              out.reshape(-1), rows, int(round_bf16))
        return out if ok == 1 else None

    def mla_decode(self, q_nope, q_rope, w_uk, latent, rope_key, scale, with_absorbed=False):
        """bf16 bit arrays: q_nope [H,dn], q_rope [H,dr], w_uk [H,dn,dc],
        latent [L,dc], rope_key [L,dr] -> float32 [H,dc]; with_absorbed also returns the
        absorbed query float32 [H,dc] (bf16-valued)."""
        heads, nope = q_nope.shape
        context, dc = latent.shape
        dr = q_rope.shape[1]
        out = np.zeros((heads, dc), np.float32)
        absorbed = np.zeros((heads, dc), np.float32) if with_absorbed else None
        ok = self.lib.yvx_oracle_mla_decode(
            np.ascontiguousarray(q_nope, np.uint16).reshape(-1),
            np.ascontiguousarray(q_rope, np.uint16).reshape(-1),
            np.ascontiguousarray(w_uk, np.uint16).reshape(-1),
            np.ascontiguousarray(latent, np.uint16).reshape(-1),
            np.ascontiguousarray(rope_key, np.uint16).reshape(-1),
            out.reshape(-1), heads, nope, dc, dr, context, float(scale),
            absorbed.ctypes.data if absorbed is not None else None)
        if not ok:
            return None
        return (out, absorbed) if absorbed is not None else out


class Reference(_Gqa):
    prefix = "yvx_ref_"

    def __init__(self):
        if not os.path.exists(REF_SO):
            raise FileNotFoundError(REF_SO)
        self.lib = C.CDLL(REF_SO)
        self._bind_common()

    def rope_apply(self, values, rope_dims, position, policy, inverse):
        out = np.ascontiguousarray(values, np.float32).copy()
        self.lib.yvx_ref_rope_apply.argtypes = [_f32p, _u64, _u64, _u64, C.c_void_p, C.c_int]
        ok = self.lib.yvx_ref_rope_apply(out, out.size, rope_dims, position, C.addressof(policy), int(inverse))
        return out if ok == 1 else None

    def topk_select(self, scores, ordinals, k):
        scores = np.ascontiguousarray(scores, np.float32)
        ordinals = np.ascontiguousarray(ordinals, np.uint64)
        out, n = np.zeros(max(len(scores), 1), np.uint64), _u64()
        self.lib.yvx_ref_topk_select.argtypes = [_f32p, _u64p, _u64, _u64, _u64p, C.POINTER(_u64)]
        ok = self.lib.yvx_ref_topk_select(scores, ordinals, len(scores), k, out, C.byref(n))
        return out[:n.value].copy() if ok == 1 else None

    def csa_select(self, indexer, token, query_position):
        out, n, valid = np.zeros(max(indexer.rows, 1), np.uint64), _u64(), _u64()
        self.lib.yvx_ref_csa_select.argtypes = [C.c_void_p, _u64, _u64, _u64p, C.POINTER(_u64), C.POINTER(_u64)]
        ok = self.lib.yvx_ref_csa_select(C.addressof(indexer), token, query_position, out, C.byref(n),
                                         C.byref(valid))
        return (out[:n.value].copy(), valid.value) if ok == 1 else None

    def latent_reduce_chunk(self, args_struct, compressed_rows, policy, indexer, tokens, heads, head_dim):
        """The reference's whole CPU reduce of a phase (selection, two passes, publication,
        inverse rotation, publication) -> (out [tokens, heads*head_dim], per-token selected
        counts, per-token selected positions) or None when the reference refuses."""
        out = np.zeros((tokens, heads * head_dim), np.float32)
        topk = int(indexer.topk) if indexer is not None else 1
        counts, positions = np.zeros(tokens, np.uint64), np.zeros((tokens, topk), np.uint64)
        self.lib.yvx_ref_latent_reduce_chunk.argtypes = [C.c_void_p, _u64, C.c_void_p, C.c_void_p, _f32p,
                                                         _u64p, _u64p]
        ok = self.lib.yvx_ref_latent_reduce_chunk(
            C.addressof(args_struct), compressed_rows, C.addressof(policy),
            C.addressof(indexer) if indexer is not None else None, out.reshape(-1),
            counts, positions.reshape(-1))
        return (out, counts, positions) if ok == 1 else None


    def qtype_dot(self, encoded_row, qtype, vector):
        """The reference's yvex_quant_cpu_dot of one encoded row with one vector -> float or None."""
        encoded_row = np.ascontiguousarray(encoded_row, np.uint8)
        vector = np.ascontiguousarray(vector, np.float32)
        out = C.c_float()
        self.lib.yvx_ref_qtype_dot.argtypes = [C.c_uint, C.c_void_p, _u64, _f32p, _u64, C.POINTER(C.c_float)]
        ok = self.lib.yvx_ref_qtype_dot(qtype, encoded_row.ctypes.data, encoded_row.size, vector, vector.size,
                                        C.byref(out))
        return float(out.value) if ok == 1 else None

    def qtype_decode_row(self, encoded_row, qtype, width):
        encoded_row = np.ascontiguousarray(encoded_row, np.uint8)
        out = np.zeros(width, np.float32)
        self.lib.yvx_ref_qtype_decode_row.argtypes = [C.c_uint, C.c_void_p, _u64, _f32p]
        return out if self.lib.yvx_ref_qtype_decode_row(qtype, encoded_row.ctypes.data, width, out) == 1 else None

    def mla_decode_embedded(self, q_absorbed, q_rope, latent, rope_key, softmax_dim=192):
        """The split-rope latent decode of one session computed by the reference's own
        yvex_attention_reduce_chunk (src/graph/core.c:608-701). The decode is a shared-row
        K == V attention in disguise: history rows are [latent | rope_key] (width dc + dr),
        the query of a head is [absorbed query | rope query], every row is visible (window
        class, window wider than the history, one new token at the last position) and the
        sinks sit at -100 as tests/unit/deepseek_attention.c:593 has them, which leaves no
        sink mass in single precision. The reference fixes the softmax scale at
        1/sqrt(row width); sqrt(row width / softmax_dim) is folded into the query. The
        reference's inverse output rotation touches only the trailing dr lanes, which are
        dropped: the first dc lanes are the bf16-published mix of latent rows.

        q_absorbed float32 [H, dc] (bf16-valued), q_rope / latent / rope_key float32
        -> float32 [H, dc], or None when the reference refuses."""
        from clori_b200 import abi
        heads, dc = q_absorbed.shape
        context, dr = rope_key.shape
        width = dc + dr
        rows = np.ascontiguousarray(np.concatenate([latent, rope_key], axis=1), np.float32)
        fold = np.float32(np.sqrt(float(width) / float(softmax_dim)))
        query = np.ascontiguousarray(
            (np.concatenate([q_absorbed, q_rope], axis=1).astype(np.float32) * fold).reshape(1, heads * width))
        positions = np.arange(context, dtype=np.uint64)
        sinks = np.full(heads, -100.0, np.float32)
        nothing_u64, nothing_f32 = np.zeros(1, np.uint64), np.zeros(width, np.float32)
        a = abi.LatentReduceArgs()
        a.query, a.local, a.local_positions = query.ctypes.data, rows.ctypes.data, positions.ctypes.data
        a.initial_local_count, a.local_stride = context - 1, width
        a.compressed, a.compressed_positions, a.compressed_stride = nothing_f32.ctypes.data, nothing_u64.ctypes.data, width
        a.selected, a.selected_count, a.topk_capacity = nothing_u64.ctypes.data, nothing_u64.ctypes.data, 1
        a.sinks, a.query_heads, a.head_dim = sinks.ctypes.data, heads, width
        a.sliding_window, a.ratio, a.attention_class = context + 1, 0, 0
        a.phase_start_position, a.token_count, a.candidate_block_visible = context - 1, 1, 0
        a.rope_dims = dr
        result = self.latent_reduce_chunk(a, 0, PositionPolicy(10000, 0, 0, 0, 0), None, 1, heads, width)
        if result is None:
            return None
        return np.ascontiguousarray(result[0].reshape(heads, width)[:, :dc])

    def compressor_chunk(self, kind, ratio, head_dim, overlap, start, token_kv, token_score, ape,
                         state_kv, state_score, norm_weights=None, epsilon=1e-6, rope_dims=0, policy=None):
        """The reference's own transition per token and publication chain per emission.
        kind: 1 main rows, 2 index rows."""
        self.lib.yvx_ref_compressor_chunk.argtypes = [C.c_void_p, C.c_uint, C.c_void_p, C.POINTER(_u64)]
        return _compressor_call(
            lambda a, n: self.lib.yvx_ref_compressor_chunk(
                C.addressof(a), kind, C.addressof(policy) if policy is not None else None, C.byref(n)),
            ratio, head_dim, overlap, start, token_kv, token_score, ape, state_kv, state_score,
            norm_weights, epsilon, rope_dims, None)


    def rows_publish(self, rows, rows_per_token, start, policy=None, **chain):
        """The reference's own functions in its order; the rotation takes the policy, not frequencies."""
        chain.pop("rope_frequency", None)
        self.lib.yvx_ref_rows_publish.argtypes = [C.c_void_p, C.c_void_p]
        return _publish_call(lambda a: self.lib.yvx_ref_rows_publish(
            C.addressof(a), C.addressof(policy) if policy is not None else None), rows, rows_per_token, start, **chain)

    def activation_quant(self, rows, quantization, block_width, hadamard):
        return _activation_call(self.lib.yvx_ref_activation_quant, rows, quantization, block_width, hadamard)


def reference_available():
    return os.path.exists(REF_SO)
