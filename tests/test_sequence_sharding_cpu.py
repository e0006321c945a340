"""KV-sequence sharding across ranks, exercised on CPU: the shard planner, the
(o, m, l) partial protocol and the log-sum-exp merge, with two gloo ranks
exchanging partials through an all-gather exactly as the GPU ranks do over
NCCL. The per-shard attention here is the CPU oracle (test infrastructure)."""
import ctypes as C
import os
import socket
import subprocess
import sys

import numpy as np

from clori_b200 import abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def shard(lib, tokens, shards, index, block=64):
    begin, end = abi.u64(), abi.u64()
    assert lib.yvex_b200_kv_sequence_shard(tokens, shards, index, block, C.byref(begin), C.byref(end))
    return begin.value, end.value


def test_shard_ranges_partition_the_sequence(library):
    for tokens, shards in [(131072, 8), (131072, 1), (1000, 4), (65, 2), (10, 4), (64 * 5, 3), (1, 8)]:
        cursor = 0
        sizes = []
        for g in range(shards):
            lo, hi = shard(library, tokens, shards, g)
            assert lo == cursor and hi >= lo
            assert lo % 64 == 0 or lo == tokens
            cursor = hi
            sizes.append(hi - lo)
        assert cursor == tokens
        full = [s for s in sizes if s % 64 == 0 and s]
        assert not full or max(full) - min(full) <= 64
    lo, hi = abi.u64(), abi.u64()
    assert not library.yvex_b200_kv_sequence_shard(100, 0, 0, 64, C.byref(lo), C.byref(hi))
    assert not library.yvex_b200_kv_sequence_shard(100, 2, 2, 64, C.byref(lo), C.byref(hi))


WORKER = r'''
import os, sys, ctypes as C
import numpy as np
import torch, torch.distributed as dist
sys.path.insert(0, os.environ["YVX_ROOT"])
from clori_b200 import abi
from oracle.binding import Oracle

def partial(oracle, q, k, v, lo, hi, qstart, hq, hkv, hd):
    """(o, m, l) of rows of q over tokens [lo, hi) with absolute causal positions."""
    rows = q.shape[0]
    out = np.zeros((rows, hq, hd + 2), np.float32)
    scale = 1.0 / np.sqrt(hd)
    for r in range(rows):
        visible = min(hi, qstart + r + 1) - lo
        for h in range(hq):
            if visible <= 0:
                out[r, h, hd] = -np.inf
                continue
            kk = k[lo:lo + visible, (h // (hq // hkv)) * hd:(h // (hq // hkv) + 1) * hd]
            vv = v[lo:lo + visible, (h // (hq // hkv)) * hd:(h // (hq // hkv) + 1) * hd]
            rc, o, scores, probs = oracle.op_attention(q[r, h * hd:(h + 1) * hd], kk, vv, visible - 1, scale, 1)
            m = float(scores[:visible].max())
            out[r, h, :hd] = o
            out[r, h, hd] = m
            out[r, h, hd + 1] = float(np.exp(scores[:visible].astype(np.float64) - m).sum())
    return out

def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    lib = abi.load()
    oracle = Oracle()
    hq, hkv, hd, rows, tokens = 4, 2, 32, 3, 300
    rng = np.random.default_rng(77)   # same inputs on every rank
    q = rng.standard_normal((rows, hq * hd)).astype(np.float32)
    k = rng.standard_normal((tokens, hkv * hd)).astype(np.float32)
    v = rng.standard_normal((tokens, hkv * hd)).astype(np.float32)
    lo, hi = abi.u64(), abi.u64()
    assert lib.yvex_b200_kv_sequence_shard(tokens, world, rank, 64, C.byref(lo), C.byref(hi))
    mine = torch.from_numpy(partial(oracle, q, k, v, lo.value, hi.value, tokens - rows, hq, hkv, hd))
    pieces = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(pieces, mine)
    parts = torch.stack(pieces).numpy()                     # [rank][row][head][hd+2]
    m = parts[..., hd]
    mm = m.max(axis=0)
    w = np.where(np.isinf(m), 0.0, parts[..., hd + 1] * np.exp(m - mm))
    merged = (parts[..., :hd] * w[..., None]).sum(axis=0) / w.sum(axis=0)[..., None]
    whole = oracle.gqa_attention(q, k, v, tokens - rows, hq, hkv, hd).reshape(rows, hq, hd)
    err = float(np.abs(merged - whole).max())
    ok = torch.tensor([1 if err < 2e-6 else 0])
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("sharded-merge max-abs", err, "all ranks ok", int(ok.item()))
    dist.destroy_process_group()
    sys.exit(0 if int(ok.item()) == 1 else 3)

main()
'''


def test_two_gloo_ranks_merge_sharded_partials(tmp_path, oracle, library):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, YVX_ROOT=ROOT, OMP_NUM_THREADS="1")
    result = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
         "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
        env=env, capture_output=True, text=True, timeout=240)
    assert result.returncode == 0, result.stdout + result.stderr
    assert "all ranks ok 1" in result.stdout
