"""Seeded cases for the shared-latent attention stage (reduce, index selection,
output rotation), shared by the CPU pin tests, the GPU parity tests and the script
that writes the golden fixtures. Values are bf16-representable, positions follow
the reference's layout (compressed row i covers positions [i*ratio, (i+1)*ratio))."""
import numpy as np

import clori_b200
from clori_b200 import abi

u64 = np.uint64


def bf16_valued(rng, shape, scale=1.0):
    x = rng.standard_normal(shape).astype(np.float32) * np.float32(scale)
    return clori_b200.bf16_bits_to_f32(clori_b200.f32_to_bf16_bits(x))


def build(rng, heads, hd, window, attention_class, tokens, start, topk=8, index_heads=0, index_dim=0,
          rope_dims=0):
    """One phase: `tokens` new rows at position `start`. With index_heads > 0 (class 1)
    the case also carries the index keys, queries and weights the selection needs; the
    `selected` lists are then to be filled from a selection, not drawn at random."""
    ratio = {0: 0, 1: 4, 2: 128}[attention_class]
    history = min(start, window - 1)
    local_positions = np.arange(start - history, start + tokens, dtype=u64)
    local = bf16_valued(rng, (len(local_positions), hd + 16))  # padded stride
    last = start + tokens - 1
    n_comp = (last + 1) // ratio if ratio else 0
    comp = bf16_valued(rng, (max(n_comp, 1), hd))
    comp_pos = (np.arange(max(n_comp, 1), dtype=u64) * u64(max(ratio, 1)))
    selected = np.zeros((tokens, topk), u64)
    selected_count = np.zeros(tokens, u64)
    case = dict(query=bf16_valued(rng, (tokens, heads * hd)), local=local, local_positions=local_positions,
                initial=history, compressed=comp, compressed_positions=comp_pos, compressed_rows=n_comp,
                selected=selected, selected_count=selected_count, topk=topk,
                sinks=rng.standard_normal(heads).astype(np.float32), heads=heads, hd=hd, window=window,
                ratio=ratio, cls=attention_class, start=start, tokens=tokens, rope_dims=rope_dims)
    if attention_class == 1 and not index_heads:
        for t in range(tokens):
            visible = (start + t + 1) // ratio
            k = min(topk, visible)
            selected_count[t] = k
            if k:
                selected[t, :k] = rng.choice(visible, size=k, replace=False).astype(u64)
    if index_heads:
        case.update(index_keys=bf16_valued(rng, (max(n_comp, 1), index_dim)),
                    index_query=bf16_valued(rng, (tokens, index_heads * index_dim)),
                    index_weights=bf16_valued(rng, (tokens, index_heads), 0.5),
                    index_heads=index_heads, index_dim=index_dim)
    return case


def host_args(case, block_visible=0, frequency=None):
    a = abi.LatentReduceArgs()
    ptr = lambda x: x.ctypes.data
    a.query, a.local, a.local_positions = ptr(case["query"]), ptr(case["local"]), ptr(case["local_positions"])
    a.initial_local_count, a.local_stride = case["initial"], case["local"].shape[1]
    a.compressed, a.compressed_positions, a.compressed_stride = ptr(case["compressed"]), ptr(case["compressed_positions"]), case["hd"]
    a.selected, a.selected_count, a.topk_capacity = ptr(case["selected"]), ptr(case["selected_count"]), case["topk"]
    a.sinks, a.query_heads, a.head_dim = ptr(case["sinks"]), case["heads"], case["hd"]
    a.sliding_window, a.ratio, a.attention_class = case["window"], case["ratio"], case["cls"]
    a.phase_start_position, a.token_count, a.candidate_block_visible = case["start"], case["tokens"], block_visible
    if frequency is not None:
        a.rope_dims, a.rope_frequency = 2 * len(frequency), ptr(frequency)
    return a
