"""Host-side description of the Q8 KV record (see include/yvex_b200/cuda_shim.h).

`record_offsets()` gives, for every (token, dim) of a 64-token x 128-dim head
block, where its lane and its f16 scale live inside the 17408-byte record. A lane
is stored as one byte holding int8 + 128 (the GGUF byte with its top bit flipped),
which is the form the kernel's byte-to-f16 placement wants.
It is the layout's definition in executable form: tests check the device pack
kernel against it byte for byte, and callers can use it to append or inspect
tokens without the library.
"""
import numpy as np

RECORD_BYTES = 17408
K_LANES, V_LANES, K_SCALES, V_SCALES = 0, 8192, 16384, 16896
LANE_BIAS = np.uint8(0x80)   # stored byte = GGUF int8 byte ^ 0x80 = int8 + 128


def record_offsets():
    t = np.arange(64)[:, None]
    d = np.arange(128)[None, :]
    e = d % 16
    k_lane = ((t // 8 * 2 + d // 64) * 32 + (t % 8) * 4 + (e % 8) // 2) * 16 + (d % 64 // 16) * 4 + (d % 2) + 2 * (e // 8)
    et = t % 16
    v_lane = V_LANES + (((t // 16 * 4 + d // 32) * 32 + (d % 8) * 4 + (et % 8) // 2) * 4 + (d // 8) % 4) * 4 + (t % 2) + 2 * (et // 8)
    q = np.arange(4)[None, :]
    k_scale = K_SCALES + (t * 4 + q) * 2
    v_scale = V_SCALES + (((t // 16 * 4 + (et % 8) // 2) * 4 + q) * 4 + (t % 2) + 2 * (et // 8)) * 2
    return k_lane, v_lane, k_scale, v_scale


def pack_records(k_rows, v_rows, kv_heads, block_ids=None, pool_blocks=None):
    """GGUF Q8_0 rows uint8 [tokens, kv_heads*4*34] -> records uint8
    [pool_blocks, kv_heads, 17408]; unused slots are zero bytes."""
    tokens = k_rows.shape[0]
    blocks = (tokens + 63) // 64
    if block_ids is None:
        block_ids = np.arange(blocks)
    pool_blocks = pool_blocks or int(max(block_ids[:blocks])) + 1
    out = np.zeros((pool_blocks, kv_heads, RECORD_BYTES), np.uint8)
    k_lane, v_lane, k_scale, v_scale = record_offsets()
    kb = k_rows.reshape(tokens, kv_heads, 4, 34)
    vb = v_rows.reshape(tokens, kv_heads, 4, 34)
    for j in range(blocks):
        lo, hi = j * 64, min(tokens, j * 64 + 64)
        n = hi - lo
        for h in range(kv_heads):
            rec = out[block_ids[j], h]
            rec[k_lane[:n].reshape(-1)] = kb[lo:hi, h, :, 2:].reshape(n, 128).reshape(-1) ^ LANE_BIAS
            rec[v_lane[:n].reshape(-1)] = vb[lo:hi, h, :, 2:].reshape(n, 128).reshape(-1) ^ LANE_BIAS
            for byte in range(2):
                rec[(k_scale[:n] + byte).reshape(-1)] = kb[lo:hi, h, :, byte].reshape(-1)
                rec[(v_scale[:n] + byte).reshape(-1)] = vb[lo:hi, h, :, byte].reshape(-1)
    return out
