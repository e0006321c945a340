"""Seeded synthetic inputs with the shapes of the five benchmark configurations.

Generator: numpy's PCG64 seeded as stated per configuration, `standard_normal`
in float32 (and `integers` / `random` for lengths, permutations, int8 lanes and
scales). Nothing here computes attention. `scale_down` shrinks token counts so
the CPU oracle finishes in seconds; head counts and head_dim keep their values.
"""
import numpy as np

from .operator import f32_to_bf16_bits


def decode_f32(seed=0, kv_tokens=4096, query_heads=32, kv_heads=8, head_dim=128):
    """Config 1: one session, one query token, F32 Q/K/V ~ N(0,1)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    q = rng.standard_normal((1, query_heads * head_dim), dtype=np.float32)
    k = rng.standard_normal((kv_tokens, kv_heads * head_dim), dtype=np.float32)
    v = rng.standard_normal((kv_tokens, kv_heads * head_dim), dtype=np.float32)
    return q, k, v


def session_lengths(seed=1, sessions=64, low=512, high=32768):
    """Config 2 lengths: uniform integers in [low, high]."""
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.integers(low, high + 1, size=sessions).astype(np.int32)


def block_table(lengths, block_tokens=64, seed=1):
    """A random permutation of a shared pool, dealt to sessions in order.

    Returns (table int32 [sessions, max_blocks] padded with -1, pool_blocks)."""
    rng = np.random.Generator(np.random.PCG64(seed + 1000))
    blocks = (np.asarray(lengths, np.int64) + block_tokens - 1) // block_tokens
    pool_blocks = int(blocks.sum())
    order = rng.permutation(pool_blocks).astype(np.int32)
    table = np.full((len(lengths), int(blocks.max())), -1, np.int32)
    cursor = 0
    for s, n in enumerate(blocks):
        table[s, :n] = order[cursor:cursor + n]
        cursor += int(n)
    return table, pool_blocks


def batched_decode_bf16(seed=1, sessions=64, low=512, high=32768, query_heads=40, kv_heads=8,
                        head_dim=128, block_tokens=64, rows=1):
    """Config 2 on the host (use small sessions/high for tests): bf16 bits.

    Pools are [pool_blocks, block_tokens, kv_heads*head_dim] (token-major rows,
    the reference's row layout). Rows of a block beyond a session's length hold
    random data too, so a kernel that reads past the length is caught."""
    rng = np.random.Generator(np.random.PCG64(seed))
    lengths = rng.integers(low, high + 1, size=sessions).astype(np.int32)
    table, pool_blocks = block_table(lengths, block_tokens, seed)
    width = kv_heads * head_dim
    q = f32_to_bf16_bits(rng.standard_normal((sessions, rows, query_heads * head_dim), dtype=np.float32))
    kpool = f32_to_bf16_bits(rng.standard_normal((pool_blocks, block_tokens, width), dtype=np.float32))
    vpool = f32_to_bf16_bits(rng.standard_normal((pool_blocks, block_tokens, width), dtype=np.float32))
    return lengths, table, q, kpool, vpool


def rope_rotate_half(x, positions, theta=1.0e6):
    """Rotate-half RoPE over the full head width, the reference's convention
    (src/runtime/decoder.c:1080-1094: freq = theta^(-2*pair/width), cos/sin
    tables rounded to bf16, pairs (lane, lane + width/2)). x: [..., T, H, D]."""
    d = x.shape[-1]
    half = d // 2
    freq = np.power(np.float64(theta), -2.0 * np.arange(half, dtype=np.float64) / d)
    angle = positions.astype(np.float64)[:, None] * freq[None, :]
    from .operator import bf16_bits_to_f32
    cos = bf16_bits_to_f32(f32_to_bf16_bits(np.cos(angle).astype(np.float32)))[:, None, :]
    sin = bf16_bits_to_f32(f32_to_bf16_bits(np.sin(angle).astype(np.float32)))[:, None, :]
    lo, hi = x[..., :half], x[..., half:]
    return np.concatenate([lo * cos - hi * sin, hi * cos + lo * sin], axis=-1).astype(np.float32)


def prefill_bf16(seed=2, batch=2, tokens=8192, query_heads=40, kv_heads=8, head_dim=128,
                 sigma=0.5, theta=1.0e6):
    """Config 3: bf16 Q/K/V ~ N(0, sigma^2), RoPE applied to Q and K, bf16 bits.

    Returns q [batch, T, Hq*D], k, v [batch, T, Hkv*D] as uint16."""
    rng = np.random.Generator(np.random.PCG64(seed))
    positions = np.arange(tokens)
    out = []
    for heads, rotate in ((query_heads, True), (kv_heads, True), (kv_heads, False)):
        x = rng.standard_normal((batch, tokens, heads, head_dim), dtype=np.float32) * np.float32(sigma)
        if rotate:
            x = rope_rotate_half(x, positions, theta)
        out.append(f32_to_bf16_bits(x.reshape(batch, tokens, heads * head_dim)))
    return tuple(out)


def q8_0_kv(seed=3, kv_tokens=131072, kv_heads=8, head_dim=128):
    """Config 4 KV as GGUF Q8_0 rows: int8 lanes uniform in [-127,127], one f16
    scale ~ U(0.002, 0.02) per 32 lanes. Returns (k_rows, v_rows) uint8
    [kv_tokens, kv_heads*head_dim/32*34]."""
    rng = np.random.Generator(np.random.PCG64(seed))
    blocks = kv_tokens * kv_heads * head_dim // 32
    rows = []
    for _ in range(2):
        lanes = rng.integers(-127, 128, size=(blocks, 32)).astype(np.int8)
        scales = rng.uniform(0.002, 0.02, size=blocks).astype(np.float16)
        enc = np.empty((blocks, 34), np.uint8)
        enc[:, :2] = scales.view(np.uint8).reshape(blocks, 2)
        enc[:, 2:] = lanes.view(np.uint8)
        rows.append(enc.reshape(kv_tokens, kv_heads * head_dim // 32 * 34))
    return rows[0], rows[1]


def verify_queries_bf16(seed=3, rows=4, query_heads=32, head_dim=128):
    rng = np.random.Generator(np.random.PCG64(seed + 500))
    return f32_to_bf16_bits(rng.standard_normal((rows, query_heads * head_dim), dtype=np.float32))


def mla_decode_bf16(seed=4, batch=32, heads=128, nope_dim=128, latent_dim=512, rope_dim=64,
                    context=16384):
    """Config 5: returns bf16 bit arrays q_nope [B,H,dn], q_rope [B,H,dr],
    w_uk [H,dn,dc] ~ N(0, 1/dc), latent [B,L,dc], rope_key [B,L,dr]."""
    rng = np.random.Generator(np.random.PCG64(seed))
    q_nope = f32_to_bf16_bits(rng.standard_normal((batch, heads, nope_dim), dtype=np.float32))
    q_rope = f32_to_bf16_bits(rng.standard_normal((batch, heads, rope_dim), dtype=np.float32))
    w_uk = f32_to_bf16_bits(rng.standard_normal((heads, nope_dim, latent_dim), dtype=np.float32)
                            * np.float32(1.0 / np.sqrt(latent_dim)))
    latent = f32_to_bf16_bits(rng.standard_normal((batch, context, latent_dim), dtype=np.float32))
    rope_key = f32_to_bf16_bits(rng.standard_normal((batch, context, rope_dim), dtype=np.float32))
    return q_nope, q_rope, w_uk, latent, rope_key
