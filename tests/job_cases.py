"""Seeded encoded-attention jobs (yvex_backend_attention_job, schema 3) and their CPU
evaluation, shared by the GPU parity tests of yvex_backend_attention_execute.

`build` lays out one phase: weights in a mix of the admitted encodings, the history of the
session (local window rows, compressed rows, index rows, rolling compressor states) and the
new tokens' inputs. `evaluate` runs the phase on the CPU in the order of the reference's CPU
twin (src/graph/attention_execute.c:452-1122): each step is a function of the CPU checker
that is bit-equal to the reference's compiled function of that step."""
import ctypes as C

import numpy as np

import clori_b200
from clori_b200 import abi
from oracle.binding import PositionPolicy, compressor_initial_state, indexer_struct

u64 = np.uint64
GEOMETRY = dict(hidden=256, q_rank=128, heads=4, hd=128, rope=64, window=16, groups=2, out_rank=64,
                index_heads=4, index_dim=128, topk=8)
POLICY = (10000, 16, 65536, 32, 1)        # theta, factor, original context, beta_fast, beta_slow
KV_ACTIVATION = dict(required=1, block_width=64, quantization=8, hadamard=0)       # FP8, blocks of 64
INDEX_ACTIVATION = dict(required=1, block_width=32, quantization=4, hadamard=1)    # transform + FP4


def bf16_valued(rng, shape, scale=1.0):
    x = rng.standard_normal(shape).astype(np.float32) * np.float32(scale)
    return clori_b200.bf16_bits_to_f32(clori_b200.f32_to_bf16_bits(x))


class Job:
    """Owns every host array a job points at (the job holds raw pointers)."""

    def __init__(self):
        self.struct = abi.AttentionJob()
        self.keep = []
        self.weights = {}                  # slot -> (float32 values [rows, width], qtype, encoded uint8)

    def array(self, a):
        self.keep.append(a)
        return a.ctypes.data


def build(oracle, attention_class, tokens, start, seed, block_visible=0, qtypes=None, geometry=None):
    g = dict(GEOMETRY, **(geometry or {}))
    rng = np.random.Generator(np.random.PCG64(seed))
    ratio = {abi.ATTENTION_SWA: 0, abi.ATTENTION_CSA: 4, abi.ATTENTION_HCA: 128}[attention_class]
    job = Job()
    j = job.struct
    j.schema, j.phase = abi.ATTENTION_JOB_SCHEMA, abi.ATTENTION_PHASE_PREFILL if tokens > 1 else abi.ATTENTION_PHASE_DECODE
    j.attention_class, j.compute_contract = attention_class, abi.ATTENTION_COMPUTE_BF16_F32_RNE_V1
    j.operation_scope = abi.ATTENTION_SCOPE_CORE
    j.token_position, j.token_count, j.input_stride = start, tokens, g["hidden"] + 8
    j.hidden_width, j.q_rank, j.query_heads, j.head_dimension, j.kv_width = g["hidden"], g["q_rank"], g["heads"], g["hd"], g["hd"]
    j.sliding_window, j.compression_ratio = g["window"], ratio
    j.output_groups, j.output_rank = g["groups"], g["out_rank"]
    j.output_group_input_width = g["heads"] * g["hd"] // g["groups"]
    j.rms_epsilon = 1e-6
    (j.position.theta, j.position.scaling_factor, j.position.original_context, j.position.beta_fast,
     j.position.beta_slow) = POLICY
    j.position.rope_dimensions = g["rope"]
    for name, spec in (("attention_kv_activation", KV_ACTIVATION), ("compressor_activation", KV_ACTIVATION),
                       ("compressor_rotated_activation", INDEX_ACTIVATION), ("indexer_query_activation", INDEX_ACTIVATION)):
        a = getattr(j, name)
        a.required, a.block_width, a.quantization, a.hadamard = (spec[k] for k in ("required", "block_width", "quantization", "hadamard"))
    j.candidate_block_visible = block_visible
    j.max_device_bytes = 1 << 30
    query_width, low_width = g["heads"] * g["hd"], g["groups"] * g["out_rank"]
    chosen = {abi.WEIGHT_Q_A: abi.QTYPE_BF16, abi.WEIGHT_Q_B: abi.QTYPE_Q8_0, abi.WEIGHT_KV: abi.QTYPE_F32,
              abi.WEIGHT_OUT_A: abi.QTYPE_F16, abi.WEIGHT_OUT_B: abi.QTYPE_BF16, abi.WEIGHT_MAIN_KV: abi.QTYPE_BF16,
              abi.WEIGHT_MAIN_GATE: abi.QTYPE_Q8_0, abi.WEIGHT_INDEX_KV: abi.QTYPE_F16, abi.WEIGHT_INDEX_GATE: abi.QTYPE_BF16,
              abi.WEIGHT_INDEX_Q: abi.QTYPE_BF16, abi.WEIGHT_INDEX_PROJECTION: abi.QTYPE_Q8_0}
    chosen.update(qtypes or {})

    def weight(slot, rows, width, scale=None, values=None):
        qtype = chosen.get(slot, abi.QTYPE_F32)
        if values is None:
            values = rng.standard_normal((rows, width)).astype(np.float32) * np.float32(scale if scale else 1.0 / np.sqrt(width))
        encoded = oracle.qtype_encode_rows(values, qtype)
        w = j.weights[slot]
        w.encoded, w.encoded_bytes = job.array(encoded), encoded.nbytes
        w.row_bytes, w.row_width, w.row_count, w.qtype, w.present = encoded.shape[1], width, rows, qtype, 1
        job.weights[slot] = (encoded, qtype, width)

    weight(abi.WEIGHT_Q_A, g["q_rank"], g["hidden"])
    weight(abi.WEIGHT_Q_A_NORM, 1, g["q_rank"], values=1.0 + 0.1 * rng.standard_normal((1, g["q_rank"])).astype(np.float32))
    weight(abi.WEIGHT_Q_B, query_width, g["q_rank"])
    weight(abi.WEIGHT_KV, g["hd"], g["hidden"])
    weight(abi.WEIGHT_KV_NORM, 1, g["hd"], values=1.0 + 0.1 * rng.standard_normal((1, g["hd"])).astype(np.float32))
    weight(abi.WEIGHT_SINKS, 1, g["heads"], values=rng.standard_normal((1, g["heads"])).astype(np.float32))
    weight(abi.WEIGHT_OUT_A, low_width, j.output_group_input_width)
    weight(abi.WEIGHT_OUT_B, g["hidden"], low_width)
    # inputs and the local history: positions [start - history, start)
    job.input = bf16_valued(rng, (tokens, j.input_stride)) + np.float32(0.001)      # not bf16-valued: the job rounds
    j.input = job.array(job.input)
    history = min(start, g["window"] - 1)
    job.local_stride = g["hd"] + 16
    job.local = bf16_valued(rng, (max(history, 1), job.local_stride))
    job.local_positions = np.arange(start - history, start, dtype=u64) if history else np.zeros(1, u64)
    j.local_kv, j.local_positions = job.array(job.local), job.array(job.local_positions)
    j.local_count, j.local_stride = history, job.local_stride
    job.history = history
    if ratio:
        rows = start // ratio
        job.compressed = bf16_valued(rng, (max(rows, 1), g["hd"]))
        job.compressed_positions = (np.arange(max(rows, 1), dtype=u64) * u64(ratio))
        j.compressed_kv, j.compressed_positions = job.array(job.compressed), job.array(job.compressed_positions)
        j.compressed_count, j.compressed_stride = rows, g["hd"]
        job.compressed_rows = rows
        overlap = 1 if attention_class == abi.ATTENTION_CSA else 0
        job.rolling = {}
        kinds = [("main_rolling", g["hd"], abi.WEIGHT_MAIN_KV)]
        if attention_class == abi.ATTENTION_CSA:
            j.indexer_heads, j.indexer_head_dimension, j.indexer_topk = g["index_heads"], g["index_dim"], g["topk"]
            job.indexer = bf16_valued(rng, (max(rows, 1), g["index_dim"]))
            j.indexer_kv, j.indexer_positions = job.array(job.indexer), job.array(job.compressed_positions)
            j.indexer_count, j.indexer_stride = rows, g["index_dim"]
            kinds.append(("indexer_rolling", g["index_dim"], abi.WEIGHT_INDEX_KV))
            weight(abi.WEIGHT_INDEX_Q, g["index_heads"] * g["index_dim"], g["q_rank"])
            weight(abi.WEIGHT_INDEX_PROJECTION, g["index_heads"], g["hidden"])
        for name, head_dim, base in kinds:
            r = getattr(j, name)
            width, slots = head_dim * (2 if overlap else 1), ratio * (2 if overlap else 1)
            kv, score = compressor_initial_state(ratio, head_dim, overlap)
            if start:   # a state that has consumed `start` tokens: seeded values where the record is live
                kv = rng.standard_normal(kv.shape).astype(np.float32)
                score = rng.standard_normal(score.shape).astype(np.float32)
            r.present, r.overlap, r.next_token_position, r.ratio, r.head_dimension = 1, overlap, start, ratio, head_dim
            r.state_width, r.state_slots = width, slots
            r.cursor = r.current_fill = start % ratio
            r.previous_fill = ratio if overlap and start >= ratio else 0
            r.kv_state, r.score_state = job.array(kv), job.array(score)
            r.kv_state_capacity = r.score_state_capacity = kv.size
            job.rolling[name] = (kv, score, head_dim, overlap, base)
            weight(base, width, g["hidden"])
            weight(base + 1, width, g["hidden"])
            weight(base + 2, ratio, width, scale=0.5)
            weight(base + 3, 1, head_dim, values=1.0 + 0.1 * rng.standard_normal((1, head_dim)).astype(np.float32))
    job.geometry, job.ratio, job.tokens, job.start, job.cls = g, ratio, tokens, start, attention_class
    return job


def spans(job, want=("core_input", "q_low", "query", "raw_kv", "attention_values", "output", "compressed_kv",
                     "compressed_positions", "indexer_kv", "indexer_positions", "index_query", "index_weights",
                     "topk_counts", "topk_positions", "valid_candidate_counts", "main_kv_state", "main_score_state",
                     "indexer_kv_state", "indexer_score_state")):
    """An output struct with a host array behind every requested span -> (struct, {name: array})."""
    g, t, j = job.geometry, job.tokens, job.struct
    new = (job.start + t) // job.ratio - job.start // job.ratio if job.ratio else 0
    main = j.main_rolling.state_slots * j.main_rolling.state_width
    index = j.indexer_rolling.state_slots * j.indexer_rolling.state_width
    shapes = {"core_input": (t, g["hidden"]), "q_low": (t, g["q_rank"]), "query": (t, g["heads"] * g["hd"]),
              "raw_kv": (t, g["hd"]), "attention_values": (t, g["heads"] * g["hd"]), "output": (t, g["hidden"]),
              "compressed_kv": (new, g["hd"]), "indexer_kv": (new, g["index_dim"]),
              "index_query": (t, g["index_heads"] * g["index_dim"]), "index_weights": (t, g["index_heads"]),
              "main_kv_state": (main,), "main_score_state": (main,), "indexer_kv_state": (index,),
              "indexer_score_state": (index,)}
    ushapes = {"compressed_positions": (new,), "indexer_positions": (new,), "topk_counts": (t,),
               "topk_positions": (t, g["topk"]), "valid_candidate_counts": (t,)}
    out, arrays = abi.AttentionJobOutput(), {}
    sparse, compressed = job.cls == abi.ATTENTION_CSA, job.cls != abi.ATTENTION_SWA
    for name in want:
        shape = shapes.get(name) or ushapes[name]
        needs_sparse = name in ("indexer_kv", "indexer_positions", "index_query", "index_weights", "topk_counts",
                                "topk_positions", "valid_candidate_counts", "indexer_kv_state", "indexer_score_state")
        needs_compressed = name in ("compressed_kv", "compressed_positions", "main_kv_state", "main_score_state")
        if (needs_sparse and not sparse) or (needs_compressed and not compressed) or not np.prod(shape):
            continue
        arrays[name] = np.full(shape, np.nan, np.float32) if name in shapes else np.zeros(shape, u64)
        span = getattr(out, name)
        span.data, span.capacity = arrays[name].ctypes.data, arrays[name].size
    return out, arrays


def evaluate(oracle, job):
    """The phase on the CPU -> {name: array} with the names of the output spans."""
    g, j, t, start, ratio = job.geometry, job.struct, job.tokens, job.start, job.ratio
    hd, rope, heads = g["hd"], g["rope"], g["heads"]
    frequency = oracle.rope_frequencies(PositionPolicy(*POLICY), rope)

    def matvec(slot, inputs, round_bf16=True, first_row=0, rows=None):
        encoded, qtype, width = job.weights[slot]
        out = oracle.qtype_matvec(encoded, qtype, width, np.ascontiguousarray(inputs[:, :width]), first_row, rows, round_bf16)
        assert out is not None
        return out

    def decode(slot):
        encoded, qtype, width = job.weights[slot]
        return oracle.qtype_decode_rows(encoded, qtype, width)

    r = {}
    core = oracle.bf16_round(job.input[:, :g["hidden"]])[1]
    r["core_input"] = core
    q_low = matvec(abi.WEIGHT_Q_A, core)
    q_low = oracle.rows_publish(q_low, 1, start, norm_mode=2, norm_weights=decode(abi.WEIGHT_Q_A_NORM)[0], epsilon=j.rms_epsilon)
    r["q_low"] = q_low
    query = matvec(abi.WEIGHT_Q_B, q_low)
    query = oracle.rows_publish(query.reshape(t * heads, hd), heads, start, norm_mode=1, epsilon=j.rms_epsilon,
                                rope_dims=rope, rope_frequency=frequency).reshape(t, heads * hd)
    r["query"] = query
    raw = matvec(abi.WEIGHT_KV, core)
    raw = oracle.rows_publish(raw, 1, start, norm_mode=2, norm_weights=decode(abi.WEIGHT_KV_NORM)[0], epsilon=j.rms_epsilon,
                              rope_dims=rope, rope_frequency=frequency, quantization=KV_ACTIVATION["quantization"],
                              activation_count=hd - rope, block_width=KV_ACTIVATION["block_width"])
    r["raw_kv"] = raw
    sinks = decode(abi.WEIGHT_SINKS).reshape(-1)
    new = (start + t) // ratio - start // ratio if ratio else 0
    compressed, compressed_positions = None, None
    if ratio:
        emitted = {}
        for name, (kv, score, head_dim, overlap, base) in job.rolling.items():
            token_kv, token_score = matvec(base, core, False), matvec(base + 1, core, False)
            rows, positions, after_kv, after_score = oracle.compressor_chunk(
                ratio, head_dim, overlap, start, token_kv, token_score, decode(base + 2), kv, score,
                norm_weights=decode(base + 3)[0], epsilon=j.rms_epsilon, rope_dims=rope, rope_frequency=frequency)
            if len(rows):
                if name == "main_rolling":
                    rows[:, :head_dim - rope] = oracle.activation_quant(rows[:, :head_dim - rope], KV_ACTIVATION["quantization"],
                                                                        KV_ACTIVATION["block_width"], 0)
                else:
                    rows = oracle.activation_quant(rows, INDEX_ACTIVATION["quantization"], INDEX_ACTIVATION["block_width"], 1)
            emitted[name] = (rows, positions, after_kv, after_score)
        rows, positions, after_kv, after_score = emitted["main_rolling"]
        assert len(rows) == new
        r["compressed_kv"], r["compressed_positions"] = rows, positions
        r["main_kv_state"], r["main_score_state"] = after_kv.reshape(-1), after_score.reshape(-1)
        compressed = np.concatenate([job.compressed[:job.compressed_rows], rows]) if new else job.compressed[:max(job.compressed_rows, 1)]
        compressed_positions = np.concatenate([job.compressed_positions[:job.compressed_rows], positions]).astype(u64) \
            if new else job.compressed_positions
    selected = np.zeros((t, g["topk"]), u64)
    selected_count = np.zeros(t, u64)
    if job.cls == abi.ATTENTION_CSA:
        rows, positions, after_kv, after_score = emitted["indexer_rolling"]
        r["indexer_kv"], r["indexer_positions"] = rows, positions
        r["indexer_kv_state"], r["indexer_score_state"] = after_kv.reshape(-1), after_score.reshape(-1)
        index_query = matvec(abi.WEIGHT_INDEX_Q, q_low)
        index_query = oracle.rows_publish(index_query.reshape(t * g["index_heads"], g["index_dim"]), g["index_heads"], start,
                                          rope_dims=rope, rope_frequency=frequency, quantization=INDEX_ACTIVATION["quantization"],
                                          activation_count=g["index_dim"], block_width=INDEX_ACTIVATION["block_width"],
                                          hadamard=1).reshape(t, -1)
        index_weights = matvec(abi.WEIGHT_INDEX_PROJECTION, core)
        r["index_query"], r["index_weights"] = index_query, index_weights
        total = job.compressed_rows + new
        r["topk_counts"], r["valid_candidate_counts"] = np.zeros(t, u64), np.zeros(t, u64)
        r["topk_positions"] = np.zeros((t, g["topk"]), u64)
        if total:
            keys = np.concatenate([job.indexer[:job.compressed_rows], rows]) if new else job.indexer[:job.compressed_rows]
            ix = indexer_struct(keys, compressed_positions[:total], index_query, index_weights, g["index_heads"],
                                g["index_dim"], g["topk"], ratio)
            for token in range(t):
                chosen, valid, _ = oracle.csa_select(ix, token, start + token)
                selected_count[token] = len(chosen)
                selected[token, :len(chosen)] = chosen
                r["topk_counts"][token], r["valid_candidate_counts"][token] = len(chosen), valid
                r["topk_positions"][token, :len(chosen)] = compressed_positions[chosen]
    # the reduce over the whole local window: history rows then the phase's own rows
    local = np.zeros((job.history + t, job.local_stride), np.float32)
    local[:job.history] = job.local[:job.history]
    local[job.history:, :hd] = raw
    local_positions = np.concatenate([job.local_positions[:job.history], np.arange(start, start + t, dtype=u64)]).astype(u64)
    a = abi.LatentReduceArgs()
    keep = [np.ascontiguousarray(query), local, local_positions, sinks.astype(np.float32), selected, selected_count, frequency]
    if compressed is None:
        compressed, compressed_positions = np.zeros((1, hd), np.float32), np.zeros(1, u64)
    keep += [np.ascontiguousarray(compressed, np.float32), np.ascontiguousarray(compressed_positions, u64)]
    a.query, a.local, a.local_positions = keep[0].ctypes.data, local.ctypes.data, local_positions.ctypes.data
    a.initial_local_count, a.local_stride = job.history, job.local_stride
    a.compressed, a.compressed_positions, a.compressed_stride = keep[7].ctypes.data, keep[8].ctypes.data, hd
    a.selected, a.selected_count, a.topk_capacity = selected.ctypes.data, selected_count.ctypes.data, g["topk"]
    a.sinks, a.query_heads, a.head_dim = keep[3].ctypes.data, heads, hd
    a.sliding_window, a.ratio, a.attention_class = g["window"], ratio, job.cls
    a.phase_start_position, a.token_count, a.candidate_block_visible = start, t, j.candidate_block_visible
    a.rope_dims, a.rope_frequency = rope, frequency.ctypes.data
    attention = oracle.latent_reduce_full(a, t, heads, hd)
    assert attention is not None
    r["attention_values"] = attention
    group_width = j.output_group_input_width
    low = np.concatenate([matvec(abi.WEIGHT_OUT_A, np.ascontiguousarray(attention[:, k * group_width:(k + 1) * group_width]),
                                 True, k * g["out_rank"], g["out_rank"]) for k in range(g["groups"])], axis=1)
    r["output"] = matvec(abi.WEIGHT_OUT_B, low)
    return r


def run(backend, job, want=None):
    """yvex_backend_attention_execute -> (rc, output struct, {span: array}, failure, error)."""
    out, arrays = spans(job) if want is None else spans(job, want)
    failure, err = abi.AttentionJobFailure(), abi.Error()
    rc = backend.lib.yvex_backend_attention_execute(backend.handle, C.byref(job.struct), C.byref(out), C.byref(failure),
                                                    C.byref(err))
    return rc, out, arrays, failure, err
