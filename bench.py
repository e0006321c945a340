"""Benchmark of the attention hot path on B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One "step" is one batched decode-attention call over the headline workload:
64 sessions with context lengths uniform in [512, 32768] (seed 1), 40 query /
8 KV heads, head_dim 128, bf16 Q/K/V ~ N(0,1), KV in 64-token blocks addressed
through a block table that is a random permutation of a shared pool, one query
token per session. Rank 0 prints ONE JSON line.

  value      tokens/s with every input resident in HBM (operator call, async)
  e2e        tokens/s through the same operator with host buffers: the step's
             query, lengths and block table go host->device and the output
             comes device->host inside the timed region (the KV pool is the
             session state and stays on the device, as in the reference)
  roofline   the attention kernel alone, CUDA events around its launch
  cpu_baseline  the reference's own CPU attention on a bounded sample

With N > 1 (torchrun) every rank runs its own 64 sessions (weak scaling, no
communication on the data path); the time is the max over ranks.
`--impl reference` times the reference's CPU attention (oracle/_ref when it
was built from the reference tree, else the C restatement) on the same
workload, sampled, on rank 0 only.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SESSIONS, QUERY_HEADS, KV_HEADS, HEAD_DIM, BLOCK_TOKENS = 64, 40, 8, 128, 64
LOW, HIGH, SEED = 512, 32768, 1
# dram__bytes_read.sum + dram__bytes_write.sum over algorithmic bytes, from the ncu capture
# summarised under profiles/ (decode kernel, batched block-table workload).
TRAFFIC_PER_ALGORITHMIC_BYTE = 1.011
METRIC = "decode_attention_tokens_per_s"
UNIT = "tokens/s"
WORKLOAD = ("batched_decode_block_table: 64 sessions, ctx~U[512,32768] seed 1, 40q/8kv heads, "
            "hd128, bf16, 64-token blocks, 1 query token/session")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            peaks = json.load(f)
        return float(peaks["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device, self.proc, self.path = device, None, None

    def start(self):
        try:
            handle, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(handle)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, maxima, reasons = [], [], set()
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    clocks.append(float(parts[1]))
                    maxima.append(float(parts[2]))
                except ValueError:
                    continue
                for name, flag in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                       "sw_power_cap"), parts[5:9]):
                    if flag.lower().startswith("active"):
                        reasons.add(name)
        os.unlink(self.path)
        return {"sm_mhz": float(np.median(clocks)) if clocks else None,
                "sm_max_mhz": max(maxima) if maxima else None,
                "samples": len(clocks), "reasons": sorted(reasons)}


def algorithmic_bytes(lengths, out_bytes):
    """K and V rows once per KV head + block-table entries + query + output."""
    lengths = np.asarray(lengths, np.int64)
    kv = int(lengths.sum()) * 2 * KV_HEADS * HEAD_DIM * 2
    table = int(((lengths + BLOCK_TOKENS - 1) // BLOCK_TOKENS).sum()) * 4
    qo = len(lengths) * QUERY_HEADS * HEAD_DIM * (2 + out_bytes)
    return kv + table + qo


class Workload:
    """The headline workload resident on one GPU, driven through the C-ABI."""

    def __init__(self, device, seed):
        import clori_b200
        from clori_b200 import abi, workloads
        self.abi, self.cl = abi, clori_b200
        self.lib = abi.load()
        self.backend = clori_b200.Backend(device)
        b = self.backend
        self.lengths = workloads.session_lengths(seed, SESSIONS, LOW, HIGH)
        self.table, self.pool_blocks = workloads.block_table(self.lengths, BLOCK_TOKENS, seed)
        width = KV_HEADS * HEAD_DIM
        pool_elems = self.pool_blocks * BLOCK_TOKENS * width
        self.kpool = b.alloc("kpool", abi.DTYPE_BF16, (self.pool_blocks, BLOCK_TOKENS, width))
        self.vpool = b.alloc("vpool", abi.DTYPE_BF16, (self.pool_blocks, BLOCK_TOKENS, width))
        for tensor, salt in ((self.kpool, 11), (self.vpool, 12)):
            rc = self.lib.yvx_cuda_fill_normal(tensor.data_ptr, abi.DTYPE_BF16, pool_elems,
                                               seed * 100 + salt, 1.0, b.stream)
            assert rc == 0, self.lib.yvx_cuda_last_error_text()
            tensor.struct.is_written = 1
        rng = np.random.Generator(np.random.PCG64(seed + 77))
        self.q_host = clori_b200.f32_to_bf16_bits(
            rng.standard_normal((SESSIONS, 1, QUERY_HEADS * HEAD_DIM), dtype=np.float32))
        self.q = b.tensor("q", self.q_host)
        self.kv_tokens = b.tensor("kv_tokens", self.lengths)
        self.block_table = b.tensor("block_table", self.table)
        self.out = b.alloc("out", abi.DTYPE_BF16, (SESSIONS, 1, QUERY_HEADS * HEAD_DIM))
        self.requirement = clori_b200.attention_requirement(
            1, int(self.lengths.max()), 0, QUERY_HEADS, KV_HEADS, HEAD_DIM, dtype=abi.DTYPE_BF16,
            output_dtype=abi.DTYPE_BF16, numeric_contract=abi.NUMERIC_BF16_F32_ACCUMULATE)
        b.sync()
        self.bytes = algorithmic_bytes(self.lengths, 2)
        self._pinned = None

    def step(self):
        rc, facts = self.backend.attention_batch_execute(
            self.requirement, self.q, self.kpool, self.vpool, self.kv_tokens, self.out,
            block_table=self.block_table, block_tokens=BLOCK_TOKENS,
            max_blocks_per_session=self.table.shape[1])
        return facts

    # -- events on the backend's stream -------------------------------------
    def event(self):
        e = C.c_void_p()
        assert self.lib.yvx_cuda_event_create(C.byref(e)) == 0
        return e

    def record(self, event):
        assert self.lib.yvx_cuda_event_record(event, self.backend.stream) == 0

    def elapsed_ms(self, start, stop):
        ms = C.c_float()
        assert self.lib.yvx_cuda_event_elapsed_ms(start, stop, C.byref(ms)) == 0
        return float(ms.value)

    # -- end to end: host buffers in, host buffer out -----------------------
    def pinned(self):
        if self._pinned is None:
            sizes = {"q": self.q_host.nbytes, "lens": self.lengths.nbytes, "table": self.table.nbytes,
                     "out": SESSIONS * QUERY_HEADS * HEAD_DIM * 2}
            self._pinned = {}
            for name, size in sizes.items():
                p = C.c_void_p()
                assert self.lib.yvx_cuda_host_alloc(C.byref(p), size) == 0
                self._pinned[name] = (p, size)
            C.memmove(self._pinned["q"][0], self.q_host.ctypes.data, self.q_host.nbytes)
            C.memmove(self._pinned["lens"][0], self.lengths.ctypes.data, self.lengths.nbytes)
            C.memmove(self._pinned["table"][0], self.table.ctypes.data, self.table.nbytes)
        return self._pinned

    def step_e2e(self):
        pin, s, lib = self.pinned(), self.backend.stream, self.lib
        lib.yvx_cuda_upload_async(self.q.data_ptr, pin["q"][0], pin["q"][1], s)
        lib.yvx_cuda_upload_async(self.kv_tokens.data_ptr, pin["lens"][0], pin["lens"][1], s)
        lib.yvx_cuda_upload_async(self.block_table.data_ptr, pin["table"][0], pin["table"][1], s)
        facts = self.step()
        lib.yvx_cuda_download_async(pin["out"][0], self.out.data_ptr, pin["out"][1], s)
        lib.yvx_cuda_stream_synchronize(s)
        return facts

    def e2e_bytes(self):
        pin = self.pinned()
        return pin["q"][1] + pin["lens"][1] + pin["table"][1], pin["out"][1]

    # -- the dominant kernel alone -------------------------------------------
    def kernel_ms(self, repeats):
        """Average duration of the attention kernel (without the combine)."""
        abi, lib, b = self.abi, self.lib, self.backend
        p = abi.GqaProblem()
        width = KV_HEADS * HEAD_DIM
        p.sessions, p.query_rows, p.query_heads, p.kv_heads, p.head_dim = SESSIONS, 1, QUERY_HEADS, KV_HEADS, HEAD_DIM
        p.causal, p.scale = 1, 1.0 / np.sqrt(HEAD_DIM)
        p.query_dtype = p.kv_dtype = p.output_dtype = abi.DTYPE_BF16
        p.query, p.query_row_stride, p.query_session_stride = self.q.data_ptr, QUERY_HEADS * HEAD_DIM, QUERY_HEADS * HEAD_DIM
        p.output = self.out.data_ptr
        p.key, p.value = self.kpool.data_ptr, self.vpool.data_ptr
        p.key_token_stride = p.value_token_stride = width
        p.key_head_stride = p.value_head_stride = HEAD_DIM
        p.block_table, p.block_tokens, p.block_table_stride = self.block_table.data_ptr, BLOCK_TOKENS, self.table.shape[1]
        p.pool_blocks = self.pool_blocks
        p.key_block_stride = p.value_block_stride = BLOCK_TOKENS * width
        p.kv_tokens, p.kv_tokens_max = self.kv_tokens.data_ptr, int(self.lengths.max())
        p.query_start_from_end = 1
        lib.yvx_cuda_gqa_plan_splits(C.byref(p), b.sm_count)
        scratch, status = C.c_void_p(), C.c_void_p()
        assert lib.yvx_cuda_malloc(C.byref(scratch), max(lib.yvx_cuda_gqa_partials_bytes(C.byref(p)), 16)) == 0
        assert lib.yvx_cuda_malloc(C.byref(status), 4) == 0
        lib.yvx_cuda_memset_async(status, 0, 4, b.stream)
        p.partials, p.status = scratch, status
        triples = [(self.event(), self.event(), self.event()) for _ in range(repeats)]
        launches = C.c_uint()
        for triple in triples:
            events = (C.c_void_p * 3)(*triple)
            rc = lib.yvx_cuda_gqa_attention_profiled(C.byref(p), b.stream, events, C.byref(launches))
            assert rc == 0, lib.yvx_cuda_last_error_text()
        lib.yvx_cuda_stream_synchronize(b.stream)
        main = [self.elapsed_ms(t[0], t[1]) for t in triples]
        combine = [self.elapsed_ms(t[1], t[2]) for t in triples]
        for triple in triples:
            for e in triple:
                lib.yvx_cuda_event_destroy(e)
        lib.yvx_cuda_free(scratch)
        lib.yvx_cuda_free(status)
        return float(np.mean(main)), float(np.mean(combine)), (p.chunk_tokens, p.max_splits)

    # -- CPU sample: the same sessions' KV copied back to the host ----------
    def host_session(self, s):
        """(q f32 [1,Hq*D], k f32 [L,Hkv*D], v f32 [L,Hkv*D]) of session s."""
        width = KV_HEADS * HEAD_DIM
        length = int(self.lengths[s])
        blocks = (length + BLOCK_TOKENS - 1) // BLOCK_TOKENS
        block_bytes = BLOCK_TOKENS * width * 2
        out = []
        for pool in (self.kpool, self.vpool):
            rows = np.empty((blocks * BLOCK_TOKENS, width), np.uint16)
            for j in range(blocks):
                src = pool.data_ptr + int(self.table[s, j]) * block_bytes
                dst = rows.ctypes.data + j * block_bytes
                assert self.lib.yvx_cuda_download_async(dst, src, block_bytes, self.backend.stream) == 0
            self.lib.yvx_cuda_stream_synchronize(self.backend.stream)
            out.append(self.cl.bf16_bits_to_f32(rows[:length]))
        return self.cl.bf16_bits_to_f32(self.q_host[s]), out[0], out[1]


def cpu_engine():
    from oracle.binding import Oracle, Reference, build_oracle, reference_available
    if reference_available():
        return Reference(), "reference"
    build_oracle()
    return Oracle(), "port"


def cpu_sample_run(engine, sample, threads):
    """One pass of the CPU attention over the sampled sessions; returns seconds."""
    start = time.perf_counter()
    outs = []
    for q, k, v in sample:
        outs.append(engine.gqa_attention(q, k, v, k.shape[0] - 1, QUERY_HEADS, KV_HEADS, HEAD_DIM,
                                         threads=threads))
    return time.perf_counter() - start, outs


def synth_host_sample(sample_ids, lengths, seed):
    """Host-generated inputs of the sampled sessions (reference arm: no GPU)."""
    rng = np.random.Generator(np.random.PCG64(seed + 5))
    sample = []
    width = KV_HEADS * HEAD_DIM
    import clori_b200
    rnd = lambda shape: clori_b200.bf16_bits_to_f32(clori_b200.f32_to_bf16_bits(
        rng.standard_normal(shape, dtype=np.float32)))
    for s in sample_ids:
        length = int(lengths[s])
        sample.append((rnd((1, QUERY_HEADS * HEAD_DIM)), rnd((length, width)), rnd((length, width))))
    return sample


def run_reference(args, rank):
    from clori_b200 import workloads
    if rank != 0:
        return
    engine, kind = cpu_engine()
    threads = os.cpu_count() or 1
    lengths = workloads.session_lengths(SEED, SESSIONS, LOW, HIGH)
    sample_ids = list(range(0, SESSIONS, 8))
    sample = synth_host_sample(sample_ids, lengths, SEED)
    times = []
    for i in range(args.warmup + args.steps):
        seconds, _ = cpu_sample_run(engine, sample, threads)
        if i >= args.warmup:
            times.append(seconds)
    per_step = float(np.mean(times))
    value = len(sample_ids) / per_step
    sample_text = (f"sessions {sample_ids} of {SESSIONS} ({int(lengths[sample_ids].sum())} of "
                   f"{int(lengths.sum())} KV tokens) per step, F32 host arrays widened from bf16")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic", "config": {"workload": WORKLOAD},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind,
                         "sample": sample_text},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    parser.add_argument("--sessions", type=int, default=SESSIONS,
                        help="shrink the batch (profiling captures only; not a bench value)")
    args = parser.parse_args()
    globals()["SESSIONS"] = args.sessions
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if dist is not None:
            dist.barrier()

    def max_over_ranks(x):
        if dist is None:
            return x
        import torch
        t = torch.tensor([x], dtype=torch.float64, device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    w = Workload(local_rank, SEED + 1000 * rank if world > 1 else SEED)
    lib, b = w.lib, w.backend

    # ---- device-resident throughput: operator call, asynchronous ----------
    b.bind_stream(None, synchronous=False)
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(args.warmup):
        facts = w.step()
    b.sync()
    barrier()
    start, stop = w.event(), w.event()
    lib.yvx_cuda_stream_synchronize(b.stream)
    w.record(start)
    launches = 0
    for _ in range(args.steps):
        facts = w.step()
        launches += int(facts.kernel_launches)
    w.record(stop)
    b.sync()
    barrier()
    device_ms = max_over_ranks(w.elapsed_ms(start, stop))

    # ---- end to end: host buffers, synchronous operator --------------------
    b.bind_stream(None, synchronous=True)
    for _ in range(3):
        w.step_e2e()
    barrier()
    lib.yvx_cuda_stream_synchronize(b.stream)
    e2e_start = time.perf_counter()
    w.record(start)
    for _ in range(args.steps):
        w.step_e2e()
    w.record(stop)
    lib.yvx_cuda_stream_synchronize(b.stream)
    e2e_wall_ms = (time.perf_counter() - e2e_start) * 1e3
    e2e_ms = max_over_ranks(max(w.elapsed_ms(start, stop), e2e_wall_ms))
    barrier()

    # ---- the attention kernel alone ----------------------------------------
    kernel_ms, combine_ms, (chunk, splits) = w.kernel_ms(min(max(args.steps, 10), 100))
    clocks = sampler.stop()

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    peak, peak_kind = measured_peaks()
    ms_per_step = device_ms / args.steps
    tokens = SESSIONS * world
    achieved = w.bytes / (kernel_ms * 1e-3) / 1e9
    h2d, d2h = w.e2e_bytes()
    line = {
        "metric": METRIC, "value": tokens / (ms_per_step * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": WORKLOAD if SESSIONS == 64 else f"REDUCED to {SESSIONS} sessions (profiling only): " + WORKLOAD, "l2": "inputs_exceed_l2 (KV pool %.2f GB per GPU)" % (
                       2 * w.pool_blocks * BLOCK_TOKENS * KV_HEADS * HEAD_DIM * 2 / 1e9),
                   "kv_tokens_total": int(w.lengths.sum()), "chunk_tokens": chunk,
                   "max_splits": splits, "sharding": "sessions per rank, no collective"},
        "hbm_gbs_whole_step": w.bytes / (ms_per_step * 1e-3) / 1e9,
        "e2e": {"value": tokens / (e2e_ms / args.steps * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms / args.steps},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": TRAFFIC_PER_ALGORITHMIC_BYTE * w.bytes,
                     "traffic_source": "ncu dram read+write of a reduced launch (8 sessions), "
                                       "scaled by KV tokens: 1.011 x algorithmic bytes",
                     "peak_kind": peak_kind,
                     "kernel": "gqa split attention (combine excluded)",
                     "kernel_ms": kernel_ms, "combine_ms": combine_ms,
                     "algorithmic_bytes": w.bytes, "frac_of_8000_spec": achieved / 8000.0},
    }
    if world == 1 and not args.no_cpu:
        engine, kind = cpu_engine()
        threads = os.cpu_count() or 1
        sample_ids = list(range(0, SESSIONS, 8))
        sample = [w.host_session(s) for s in sample_ids]
        best, outs = None, None
        for _ in range(3):
            seconds, outs = cpu_sample_run(engine, sample, threads)
            best = seconds if best is None else min(best, seconds)
        gpu = w.cl.bf16_bits_to_f32(w.out.read())
        worst = max(float(np.abs(gpu[s, 0] - o[0]).max()) for s, o in zip(sample_ids, outs))
        line["cpu_baseline"] = {
            "value": len(sample_ids) / best, "unit": UNIT, "cores": threads, "kind": kind,
            "sample": f"sessions {sample_ids} of {SESSIONS} "
                      f"({int(w.lengths[sample_ids].sum())} of {int(w.lengths.sum())} KV tokens), "
                      "best of 3 passes, KV copied back from the device and widened to F32",
            "seconds": best, "gpu_vs_cpu_max_abs_on_sample": worst}
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
