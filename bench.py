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
SUSTAIN_SECONDS = 2.0          # length of the back-to-back run reported as "sustained"
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
    """Samples nvidia-smi clocks and throttle reasons (with timestamps) from before the first
    timed region until after the last leg; `window` summarises the samples of one leg."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, device):
        self.device, self.proc, self.path, self.samples = device, None, None, None

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
        """Ends the sampling and parses the samples: (epoch seconds, MHz, max MHz, watts, reasons)."""
        self.samples = []
        if not self.proc:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        import datetime
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    stamp = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    clock, maximum = float(parts[1]), float(parts[2])
                except ValueError:
                    continue
                try:
                    watts = float(parts[3])
                except ValueError:
                    watts = None
                active = [name for name, flag in zip(self.REASONS, parts[5:9]) if flag.lower().startswith("active")]
                self.samples.append((stamp, clock, maximum, watts, active))
        os.unlink(self.path)

    def window(self, begin=None, end=None):
        """Median SM clock and the throttle reasons seen between two time.time() stamps (the
        whole record without them). A leg shorter than the sampling period takes the samples
        within 0.1 s of it."""
        if self.samples is None:
            self.stop()
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
        chosen = self.samples
        if begin is not None:
            chosen = [x for x in self.samples if begin - 0.1 <= x[0] <= end + 0.1]
            if not chosen:
                middle = 0.5 * (begin + end)
                chosen = [min(self.samples, key=lambda x: abs(x[0] - middle))]
        reasons = sorted({r for x in chosen for r in x[4]})
        watts = [x[3] for x in chosen if x[3] is not None]
        return {"sm_mhz": float(np.median([x[1] for x in chosen])), "sm_max_mhz": max(x[2] for x in chosen),
                "samples": len(chosen), "reasons": reasons,
                "power_w_max": max(watts) if watts else None}


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
        # Every rank draws the SAME session lengths (seed 1), so per-GPU work is identical
        # (weak scaling); the block-table permutation and the data differ per rank.
        self.lengths = workloads.session_lengths(SEED, SESSIONS, LOW, HIGH)
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
        # The per-step inputs (queries, lengths, block table) live in ONE device allocation, so the
        # end-to-end leg moves them with one host->device copy; the operator sees three tensors.
        parts = (("q", self.q_host, abi.DTYPE_BF16), ("kv_tokens", self.lengths, abi.DTYPE_I32),
                 ("block_table", self.table, abi.DTYPE_I32))
        self.input_offsets, total = {}, 0
        for name, array, _ in parts:
            self.input_offsets[name] = total
            total += (np.ascontiguousarray(array).nbytes + 255) // 256 * 256
        self.inputs = b.alloc("step_inputs", abi.DTYPE_I8, (total,))
        self.inputs_host = np.zeros(total, np.uint8)
        for name, array, dtype in parts:
            array = np.ascontiguousarray(array)
            offset = self.input_offsets[name]
            self.inputs_host[offset:offset + array.nbytes] = array.view(np.uint8).reshape(-1)
            view = b.wrap(name, dtype, array.shape, self.inputs.data_ptr + offset, array.nbytes)
            view.struct.is_written = 1
            setattr(self, name if name != "q" else "q", view)
        assert self.lib.yvx_cuda_upload_async(self.inputs.data_ptr, self.inputs_host.ctypes.data, total, b.stream) == 0
        self.inputs.struct.is_written = 1
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
            sizes = {"inputs": self.inputs_host.nbytes, "out": SESSIONS * QUERY_HEADS * HEAD_DIM * 2}
            self._pinned = {}
            for name, size in sizes.items():
                p = C.c_void_p()
                assert self.lib.yvx_cuda_host_alloc(C.byref(p), size) == 0
                self._pinned[name] = (p, size)
            C.memmove(self._pinned["inputs"][0], self.inputs_host.ctypes.data, self.inputs_host.nbytes)
        return self._pinned

    def step_e2e(self):
        pin, s, lib = self.pinned(), self.backend.stream, self.lib
        lib.yvx_cuda_upload_async(self.inputs.data_ptr, pin["inputs"][0], pin["inputs"][1], s)
        facts = self.step()
        lib.yvx_cuda_download_async(pin["out"][0], self.out.data_ptr, pin["out"][1], s)
        lib.yvx_cuda_stream_synchronize(s)
        return facts

    def e2e_bytes(self):
        pin = self.pinned()
        return pin["inputs"][1], pin["out"][1]

    # -- the dominant kernel alone -------------------------------------------
    def kernel_ms(self, repeats, chunk=0):
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
        if chunk:
            p.chunk_tokens, p.max_splits = chunk, (p.kv_tokens_max + chunk - 1) // chunk
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



# ---------------------------------------------------------------------------
# The other single-GPU configurations: measured in the same run and reported
# under "other_workloads" (the headline line stays the batched decode).
# ---------------------------------------------------------------------------

def _alloc(lib, nbytes):
    p = C.c_void_p()
    assert lib.yvx_cuda_malloc(C.byref(p), nbytes) == 0, lib.yvx_cuda_last_error_text()
    return p


def _timed_launches(lib, backend, problems, repeats):
    """Profiled launches cycling through `problems` (copies of the inputs larger
    than L2 in total); returns mean ms of the attention kernel and the combine."""
    def event():
        e = C.c_void_p()
        assert lib.yvx_cuda_event_create(C.byref(e)) == 0
        return e
    for i in range(3):
        n = C.c_uint()
        assert lib.yvx_cuda_gqa_attention(C.byref(problems[i % len(problems)]), backend.stream, C.byref(n)) == 0
    triples = [(event(), event(), event()) for _ in range(repeats)]
    for i, triple in enumerate(triples):
        n = C.c_uint()
        rc = lib.yvx_cuda_gqa_attention_profiled(C.byref(problems[i % len(problems)]), backend.stream,
                                                 (C.c_void_p * 3)(*triple), C.byref(n))
        assert rc == 0, lib.yvx_cuda_last_error_text()
    assert lib.yvx_cuda_stream_synchronize(backend.stream) == 0, lib.yvx_cuda_last_error_text()
    ms = C.c_float()
    main, combine = [], []
    for a, b, c in triples:
        lib.yvx_cuda_event_elapsed_ms(a, b, C.byref(ms)); main.append(ms.value)
        lib.yvx_cuda_event_elapsed_ms(b, c, C.byref(ms)); combine.append(ms.value)
        for e in (a, b, c):
            lib.yvx_cuda_event_destroy(e)
    # Whole calls back to back, as a decode loop issues them (no events between the
    # attention kernel and its combine, so the combine's launch can overlap the tail).
    first, last = event(), event()
    lib.yvx_cuda_event_record(first, backend.stream)
    for i in range(repeats):
        assert lib.yvx_cuda_gqa_attention(C.byref(problems[i % len(problems)]), backend.stream, C.byref(n)) == 0
    lib.yvx_cuda_event_record(last, backend.stream)
    assert lib.yvx_cuda_stream_synchronize(backend.stream) == 0, lib.yvx_cuda_last_error_text()
    lib.yvx_cuda_event_elapsed_ms(first, last, C.byref(ms))
    _timed_launches.step_ms = ms.value / repeats
    # The same calls captured once into a CUDA graph and replayed (launch gaps shrink).
    _timed_launches.graph_step_ms = None
    _timed_launches.last_problem = (repeats - 1) % len(problems)     # whose outputs the buffers hold now
    calls = max(len(problems), 8)
    if lib.yvx_cuda_graph_capture_begin(backend.stream) == 0:
        ok = all(lib.yvx_cuda_gqa_attention(C.byref(problems[i % len(problems)]), backend.stream, C.byref(n)) == 0
                 for i in range(calls))
        graph = C.c_void_p()
        if lib.yvx_cuda_graph_capture_end(backend.stream, C.byref(graph)) == 0 and ok:
            replays = max(repeats // calls, 3)
            lib.yvx_cuda_graph_launch(graph, backend.stream)
            lib.yvx_cuda_event_record(first, backend.stream)
            for _ in range(replays):
                lib.yvx_cuda_graph_launch(graph, backend.stream)
            _timed_launches.last_problem = (calls - 1) % len(problems)
            lib.yvx_cuda_event_record(last, backend.stream)
            if lib.yvx_cuda_stream_synchronize(backend.stream) == 0:
                lib.yvx_cuda_event_elapsed_ms(first, last, C.byref(ms))
                _timed_launches.graph_step_ms = ms.value / (replays * calls)
            lib.yvx_cuda_graph_destroy(graph)
    for e in (first, last):
        lib.yvx_cuda_event_destroy(e)
    return float(np.mean(main)), float(np.mean(combine)), n.value


def bench_decode_f32(lib, backend, abi, peak, repeats):
    """Config 1: 1 session, 1 query token, 32/8 heads, hd 128, KV 4096, F32."""
    hq, hkv, hd, tokens, copies = 32, 8, 128, 4096, 16
    width = hkv * hd
    kv_elems = tokens * width
    k = _alloc(lib, copies * kv_elems * 4)
    v = _alloc(lib, copies * kv_elems * 4)
    q = _alloc(lib, hq * hd * 4)
    out = _alloc(lib, hq * hd * 4)
    status = _alloc(lib, 4)
    tickets = _alloc(lib, 8 * hkv)
    lib.yvx_cuda_memset_async(tickets, 0, 8 * hkv, backend.stream)
    lib.yvx_cuda_fill_normal(k, abi.DTYPE_F32, copies * kv_elems, 101, 1.0, backend.stream)
    lib.yvx_cuda_fill_normal(v, abi.DTYPE_F32, copies * kv_elems, 102, 1.0, backend.stream)
    lib.yvx_cuda_fill_normal(q, abi.DTYPE_F32, hq * hd, 103, 1.0, backend.stream)
    lib.yvx_cuda_memset_async(status, 0, 4, backend.stream)
    problems, scratch = [], None
    for i in range(copies):
        p = abi.GqaProblem()
        p.sessions, p.query_rows, p.query_heads, p.kv_heads, p.head_dim = 1, 1, hq, hkv, hd
        p.causal, p.scale = 1, 1.0 / np.sqrt(hd)
        p.query_dtype = p.kv_dtype = p.output_dtype = abi.DTYPE_F32
        p.query, p.query_row_stride, p.output = q, hq * hd, out
        p.key, p.value = k.value + i * kv_elems * 4, v.value + i * kv_elems * 4
        p.key_token_stride = p.value_token_stride = width
        p.key_head_stride = p.value_head_stride = hd
        p.kv_tokens_uniform = p.kv_tokens_max = tokens
        p.query_start_uniform = tokens - 1
        lib.yvx_cuda_gqa_plan_splits(C.byref(p), backend.sm_count)
        if scratch is None:
            scratch = _alloc(lib, max(lib.yvx_cuda_gqa_partials_bytes(C.byref(p)), 16))
        p.partials, p.status, p.tickets = scratch, status, tickets
        problems.append(p)
    main, combine, launches = _timed_launches(lib, backend, problems, repeats)
    # full-size parity of the copy the last launch read, against the CPU oracle
    last = _timed_launches.last_problem
    host = {}
    for name, ptr, count in (("q", q.value, hq * hd), ("k", k.value + last * kv_elems * 4, kv_elems),
                             ("v", v.value + last * kv_elems * 4, kv_elems), ("o", out.value, hq * hd)):
        host[name] = np.empty(count, np.float32)
        lib.yvx_cuda_download_async(host[name].ctypes.data, ptr, count * 4, backend.stream)
    st = np.zeros(1, np.int32)
    lib.yvx_cuda_download_async(st.ctypes.data, status, 4, backend.stream)
    lib.yvx_cuda_stream_synchronize(backend.stream)
    nbytes = 2 * kv_elems * 4 + 2 * hq * hd * 4
    # One launch per step: the step replayed from a CUDA graph IS the kernel back to back; a pair
    # of events around every single launch adds the gap the host takes to enqueue it.
    best = min(x for x in (main, _timed_launches.step_ms, _timed_launches.graph_step_ms) if x)
    result = {"workload": "decode 1x1 token, 32q/8kv heads, hd128, KV 4096, F32 (exact-F32 contract)",
              "kernel": "gqa_decode_f32_kernel", "launches_per_step": launches,
              "kernel_ms": best, "event_bracketed_launch_ms": main, "combine_ms": combine, "algorithmic_bytes": nbytes,
              "achieved_gbs": nbytes / (best * 1e-3) / 1e9, "frac_of_measured_hbm": nbytes / (best * 1e-3) / 1e9 / peak,
              "step_ms": _timed_launches.step_ms, "graph_step_ms": _timed_launches.graph_step_ms,
              "tokens_per_s": 1.0 / (_timed_launches.step_ms * 1e-3),
              "l2": f"{copies} rotating KV copies ({copies * 2 * kv_elems * 4 / 1e6:.0f} MB) exceed L2",
              "chunk_tokens": problems[0].chunk_tokens, "status_word": int(st[0])}
    for ptr in (k, v, q, out, status, scratch, tickets):
        lib.yvx_cuda_free(ptr)
    return result, host


def bench_verify_q8(lib, backend, abi, peak, repeats, chunk=None):
    """Config 4 on one GPU: 1 session, KV 131072, 32/8 heads, hd 128, Q8_0 KV,
    4 speculative rows causal among themselves."""
    from clori_b200 import q8_records
    hq, hkv, hd, tokens, rows, copies = 32, 8, 128, 131072, 4, 2
    blocks = tokens // 64
    record = q8_records.RECORD_BYTES
    pool_bytes = blocks * hkv * record
    records = _alloc(lib, copies * pool_bytes)
    q = _alloc(lib, rows * hq * hd * 2)
    out = _alloc(lib, rows * hq * hd * 4)
    status = _alloc(lib, 4)
    lib.yvx_cuda_fill_q8_records(records, copies * blocks * hkv, 201, 0.002, 0.02, backend.stream)
    lib.yvx_cuda_fill_normal(q, abi.DTYPE_BF16, rows * hq * hd, 202, 1.0, backend.stream)
    lib.yvx_cuda_memset_async(status, 0, 4, backend.stream)
    problems, scratch = [], None
    for i in range(copies):
        p = abi.GqaProblem()
        p.sessions, p.query_rows, p.query_heads, p.kv_heads, p.head_dim = 1, rows, hq, hkv, hd
        p.causal, p.scale = 1, 1.0 / np.sqrt(hd)
        p.query_dtype, p.kv_dtype, p.output_dtype = abi.DTYPE_BF16, abi.DTYPE_Q8_0, abi.DTYPE_F32
        p.query, p.query_row_stride, p.query_session_stride, p.output = q, hq * hd, rows * hq * hd, out
        p.key = records.value + i * pool_bytes
        p.key_head_stride, p.key_block_stride, p.block_tokens = record, hkv * record, 64
        p.kv_tokens_uniform = p.kv_tokens_max = tokens
        p.query_start_from_end = 1
        lib.yvx_cuda_gqa_plan_splits(C.byref(p), backend.sm_count)
        if chunk:
            p.chunk_tokens, p.max_splits = chunk, (tokens + chunk - 1) // chunk
        if scratch is None:
            scratch = _alloc(lib, max(lib.yvx_cuda_gqa_partials_bytes(C.byref(p)), 16))
        p.partials, p.status = scratch, status
        problems.append(p)
    main, combine, launches = _timed_launches(lib, backend, problems, repeats)
    step_ms, graph_step_ms = _timed_launches.step_ms, _timed_launches.graph_step_ms
    # The same step as ONE cooperative launch: the splits are folded by the kernel's own CTAs
    # (the exchange tail with a single rank, whose area is this GPU's own memory).
    items = rows * hq
    area_bytes = lib.yvx_cuda_lse_exchange_bytes(1, items, hd)
    area, table, mine = _alloc(lib, area_bytes), _alloc(lib, 16), _alloc(lib, items * (hd + 2) * 4)
    lib.yvx_cuda_memset_async(area, 0, area_bytes, backend.stream)
    pointers = np.array([area.value, area.value + lib.yvx_cuda_lse_exchange_counter_offset(1, items, hd)], np.uint64)
    lib.yvx_cuda_upload_async(table, pointers.ctypes.data, 16, backend.stream)
    lib.yvx_cuda_stream_synchronize(backend.stream)
    exchange = abi.LseExchange()
    exchange.ranks, exchange.rank, exchange.gather, exchange.arrivals, exchange.one_launch = 1, 0, table.value, table.value + 8, 1
    for p in problems:
        p.partial_output = mine
    first, final, ms, n = C.c_void_p(), C.c_void_p(), C.c_float(), C.c_uint()
    lib.yvx_cuda_event_create(C.byref(first)); lib.yvx_cuda_event_create(C.byref(final))
    epoch = 0
    for timed in (False, True):
        if timed:
            lib.yvx_cuda_event_record(first, backend.stream)
        for i in range(repeats if timed else 3):
            epoch += 1
            exchange.epoch = epoch
            rc = lib.yvx_cuda_gqa_attention_exchange(C.byref(problems[i % copies]), C.byref(exchange), backend.stream, C.byref(n))
            assert rc == 0, lib.yvx_cuda_last_error_text()
    lib.yvx_cuda_event_record(final, backend.stream)
    assert lib.yvx_cuda_stream_synchronize(backend.stream) == 0, lib.yvx_cuda_last_error_text()
    lib.yvx_cuda_event_elapsed_ms(first, final, C.byref(ms))
    one_launch_ms, one_launch_launches = ms.value / repeats, int(n.value)
    lib.yvx_cuda_event_destroy(first); lib.yvx_cuda_event_destroy(final)
    for p in problems:
        p.partial_output = None
    last = (repeats - 1) % copies
    # sample for the CPU check: KV head 0 (query heads 0..3), every record of it
    head0 = np.empty((blocks, record), np.uint8)
    for j in range(blocks):
        lib.yvx_cuda_download_async(head0.ctypes.data + j * record,
                                    records.value + last * pool_bytes + j * hkv * record, record, backend.stream)
    q_host = np.empty(rows * hq * hd, np.uint16)
    o_host = np.empty(rows * hq * hd, np.float32)
    lib.yvx_cuda_download_async(q_host.ctypes.data, q, q_host.nbytes, backend.stream)
    lib.yvx_cuda_download_async(o_host.ctypes.data, out, o_host.nbytes, backend.stream)
    st = np.zeros(1, np.int32)
    lib.yvx_cuda_download_async(st.ctypes.data, status, 4, backend.stream)
    lib.yvx_cuda_stream_synchronize(backend.stream)
    nbytes = pool_bytes + rows * hq * hd * (2 + 4)
    result = {"workload": "speculative verify, 1 session, KV 131072, 32q/8kv heads, hd128, Q8_0 KV, 4 rows",
              "kernel": "gqa_decode_q8_kernel", "launches_per_step": launches, "kernel_ms": main,
              "combine_ms": combine, "algorithmic_bytes": nbytes, "status_word": int(st[0]),
              "achieved_gbs": nbytes / (main * 1e-3) / 1e9, "frac_of_measured_hbm": nbytes / (main * 1e-3) / 1e9 / peak,
              "step_ms": step_ms, "graph_step_ms": graph_step_ms,
              "one_launch_step_ms": one_launch_ms, "one_launch_launches": one_launch_launches,
              "tokens_per_s": rows / (min(step_ms, one_launch_ms) * 1e-3),
              "l2": f"{copies} rotating record pools ({copies * pool_bytes / 1e6:.0f} MB) exceed L2",
              "chunk_tokens": problems[0].chunk_tokens}
    for ptr in (records, q, out, status, scratch, area, table, mine):
        lib.yvx_cuda_free(ptr)
    return result, (head0, q_host.reshape(rows, hq * hd), o_host.reshape(rows, hq * hd))



def bench_prefill(lib, backend, abi, repeats, tokens=8192, batch=2):
    """Config 3: causal prefill, batch x tokens, 40/8 heads, hd 128, bf16 in and out.
    Device-generated N(0, 0.5^2), Q and K rotated (theta 1e6, positions 0..tokens-1,
    rotate-half over the full head width) before the bf16 rounding, V left as drawn."""
    hq, hkv, hd = 40, 8, 128
    qn, kn = batch * tokens * hq * hd, batch * tokens * hkv * hd
    q, k, v, out = _alloc(lib, qn * 2), _alloc(lib, kn * 2), _alloc(lib, kn * 2), _alloc(lib, qn * 2)
    status = _alloc(lib, 4)
    for ptr, heads, seed in ((q, hq, 301), (k, hkv, 302)):
        rc = lib.yvx_cuda_fill_normal_rope_bf16(ptr, batch * tokens, tokens, heads, hd, seed, 0.5, 1.0e6,
                                                backend.stream)
        assert rc == 0, lib.yvx_cuda_last_error_text()
    lib.yvx_cuda_fill_normal(v, abi.DTYPE_BF16, kn, 303, 0.5, backend.stream)
    lib.yvx_cuda_memset_async(status, 0, 4, backend.stream)
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
    p.query_start_uniform = 0
    lib.yvx_cuda_gqa_plan_splits(C.byref(p), backend.sm_count)
    scratch = _alloc(lib, max(lib.yvx_cuda_gqa_partials_bytes(C.byref(p)), 16))
    p.partials, p.status = scratch, status
    main, combine, launches = _timed_launches(lib, backend, [p], repeats)
    flops = 4.0 * batch * hq * hd * tokens * (tokens + 1) / 2.0
    # sustained: launches back to back for about two seconds (power-capped clocks)
    sustained_launches = max(int(2000.0 / max(main, 1e-3)), repeats) if tokens >= 8192 else repeats
    first, last, ms, n = C.c_void_p(), C.c_void_p(), C.c_float(), C.c_uint()
    lib.yvx_cuda_event_create(C.byref(first)); lib.yvx_cuda_event_create(C.byref(last))
    lib.yvx_cuda_event_record(first, backend.stream)
    for _ in range(sustained_launches):
        assert lib.yvx_cuda_gqa_attention(C.byref(p), backend.stream, C.byref(n)) == 0
    lib.yvx_cuda_event_record(last, backend.stream)
    assert lib.yvx_cuda_stream_synchronize(backend.stream) == 0, lib.yvx_cuda_last_error_text()
    lib.yvx_cuda_event_elapsed_ms(first, last, C.byref(ms))
    sustained_ms = ms.value / sustained_launches
    lib.yvx_cuda_event_destroy(first); lib.yvx_cuda_event_destroy(last)
    st = np.zeros(1, np.int32)
    lib.yvx_cuda_download_async(st.ctypes.data, status, 4, backend.stream)
    # sample for the CPU check: batch 0, KV head 0, query head 0, the last 128 rows
    rows = 128
    q_host = np.empty((rows, hq * hd), np.uint16)
    o_host = np.empty((rows, hq * hd), np.uint16)
    k_host = np.empty((tokens, hkv * hd), np.uint16)
    v_host = np.empty((tokens, hkv * hd), np.uint16)
    lib.yvx_cuda_download_async(q_host.ctypes.data, q.value + (tokens - rows) * hq * hd * 2, q_host.nbytes, backend.stream)
    lib.yvx_cuda_download_async(o_host.ctypes.data, out.value + (tokens - rows) * hq * hd * 2, o_host.nbytes, backend.stream)
    lib.yvx_cuda_download_async(k_host.ctypes.data, k, k_host.nbytes, backend.stream)
    lib.yvx_cuda_download_async(v_host.ctypes.data, v, v_host.nbytes, backend.stream)
    lib.yvx_cuda_stream_synchronize(backend.stream)
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    tf_peak, tf_sustained_peak, tf_kind = 1590.0, 1400.0, "fallback"
    if os.path.exists(peaks_path):
        with open(peaks_path) as f:
            peaks = json.load(f)
        tf_peak, tf_kind = float(peaks["bf16_tflops"]), "measured"
        tf_sustained_peak = float(peaks.get("bf16_tflops_sustained", tf_peak))
    achieved = flops / (main * 1e-3) / 1e12
    result = {"workload": f"causal prefill {batch} x {tokens} tokens, 40q/8kv heads, hd128, bf16",
              "kernel": "prefill_tcgen05_kernel", "launches_per_step": launches, "kernel_ms": main,
              "flops_causal": flops, "achieved_tflops": achieved, "peak_tflops": tf_peak,
              "peak_kind": tf_kind + " (burst, kernel timed alone)", "frac_of_bf16_peak": achieved / tf_peak,
              "sustained_ms": sustained_ms, "sustained_launches": sustained_launches,
              "sustained_tflops": flops / (sustained_ms * 1e-3) / 1e12,
              "sustained_frac_of_burst_peak": flops / (sustained_ms * 1e-3) / 1e12 / tf_peak,
              "sustained_frac_of_sustained_peak": flops / (sustained_ms * 1e-3) / 1e12 / tf_sustained_peak,
              "peak_tflops_sustained": tf_sustained_peak,
              "tokens_per_s": batch * tokens / (main * 1e-3), "status_word": int(st[0]),
              "l2": "Q+K+V+O = %.0f MB exceed L2" % ((2 * qn + 2 * kn) * 2 / 1e6)}
    for ptr in (q, k, v, out, status, scratch):
        lib.yvx_cuda_free(ptr)
    return result, (q_host, k_host, v_host, o_host, tokens, rows)


def bench_prefill_f32(lib, backend, abi, repeats, tokens=21741, heads=56):
    """The exact-F32 contract at the reference's largest tested prefill geometry (MHA, 21741 tokens x 56
    heads, hd 128, tests/unit/cuda/quant_qtype.c:2868-2970): F32 Q/K/V whose values bf16 holds exactly
    (what the reference's linears publish), F32 output. Staging to bf16, the tensor-core kernel and the
    (idle) exact kernel are all inside the timed step."""
    hd = 128
    n = tokens * heads * hd
    q, k, v, out = (_alloc(lib, n * 4) for _ in range(4))
    status = _alloc(lib, 4)
    for ptr, seed in ((q, 701), (k, 702), (v, 703)):
        assert lib.yvx_cuda_fill_normal(ptr, -abi.DTYPE_F32, n, seed, 0.5, backend.stream) == 0
    lib.yvx_cuda_memset_async(status, 0, 4, backend.stream)
    p = abi.GqaProblem()
    p.sessions, p.query_rows, p.query_heads, p.kv_heads, p.head_dim = 1, tokens, heads, heads, hd
    p.causal, p.scale = 1, 1.0 / np.sqrt(hd)
    p.query_dtype = p.kv_dtype = p.output_dtype = abi.DTYPE_F32
    p.query, p.query_row_stride, p.output = q, heads * hd, out
    p.key, p.value = k, v
    p.key_token_stride = p.value_token_stride = heads * hd
    p.key_head_stride = p.value_head_stride = hd
    p.kv_tokens_uniform = p.kv_tokens_max = tokens
    lib.yvx_cuda_gqa_plan_splits(C.byref(p), backend.sm_count)
    partial_bytes = (lib.yvx_cuda_gqa_partials_bytes(C.byref(p)) + 255) & ~255
    staging_bytes = lib.yvx_cuda_gqa_f32_staging_bytes(C.byref(p))
    scratch = _alloc(lib, max(partial_bytes + staging_bytes, 16))
    p.partials, p.status = scratch, status
    p.f32_staging = scratch.value + partial_bytes
    first, last, ms, launches = C.c_void_p(), C.c_void_p(), C.c_float(), C.c_uint()
    lib.yvx_cuda_event_create(C.byref(first)); lib.yvx_cuda_event_create(C.byref(last))
    assert lib.yvx_cuda_gqa_attention(C.byref(p), backend.stream, C.byref(launches)) == 0, lib.yvx_cuda_last_error_text()
    lib.yvx_cuda_event_record(first, backend.stream)
    for _ in range(repeats):
        assert lib.yvx_cuda_gqa_attention(C.byref(p), backend.stream, C.byref(launches)) == 0
    lib.yvx_cuda_event_record(last, backend.stream)
    assert lib.yvx_cuda_stream_synchronize(backend.stream) == 0, lib.yvx_cuda_last_error_text()
    lib.yvx_cuda_event_elapsed_ms(first, last, C.byref(ms))
    step_ms = ms.value / repeats
    st = np.zeros(1, np.int32)
    lib.yvx_cuda_download_async(st.ctypes.data, status, 4, backend.stream)
    # sample for the CPU check: head 0, the last 64 rows against every token
    rows = 64
    host = {}
    for name, ptr, first_row, count in (("q", q, tokens - rows, rows), ("o", out, tokens - rows, rows),
                                        ("k", k, 0, tokens), ("v", v, 0, tokens)):
        full = np.empty((count, heads * hd), np.float32)
        lib.yvx_cuda_download_async(full.ctypes.data, ptr.value + first_row * heads * hd * 4, full.nbytes, backend.stream)
        host[name] = full
    lib.yvx_cuda_stream_synchronize(backend.stream)
    sample = {name: np.ascontiguousarray(a[:, :hd]) for name, a in host.items()}
    flops = 4.0 * heads * hd * tokens * (tokens + 1) / 2.0
    tf_peak = 1699.0
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        with open(peaks_path) as f:
            tf_peak = float(json.load(f)["bf16_tflops"])
    result = {"workload": f"exact-F32 contract causal prefill, {tokens} tokens x {heads} heads (MHA), hd128, F32 in/out, bf16-valued",
              "kernel": "f32_stage_rows_kernel x3 + prefill_tcgen05_kernel (+ gated exact kernel)",
              "launches_per_step": int(launches.value), "step_ms": step_ms, "kernel_ms": step_ms, "flops_causal": flops,
              "achieved_tflops": flops / (step_ms * 1e-3) / 1e12, "frac_of_bf16_peak": flops / (step_ms * 1e-3) / 1e12 / tf_peak,
              "tokens_per_s": tokens / (step_ms * 1e-3), "status_word": int(st[0]),
              "l2": "Q+K+V+O = %.0f MB exceed L2" % (4 * n * 4 / 1e6)}
    for ptr in (q, k, v, out, status, scratch):
        lib.yvx_cuda_free(ptr)
    lib.yvx_cuda_event_destroy(first); lib.yvx_cuda_event_destroy(last)
    return result, (sample, tokens, rows)


def check_prefill_f32(engine, sample_tuple, threads):
    sample, tokens, rows = sample_tuple
    start = time.perf_counter()
    ref = engine.gqa_attention(sample["q"], sample["k"], sample["v"], tokens - rows, 1, 1, 128, threads=threads)
    seconds = time.perf_counter() - start
    return float((np.abs(ref - sample["o"]) / (1.0 + np.abs(ref))).max()), seconds


def check_prefill(engine, sample, threads):
    from clori_b200 import bf16_bits_to_f32
    q, k, v, o, tokens, rows = sample
    hd = 128
    qf = bf16_bits_to_f32(q)[:, :hd]
    kf, vf = bf16_bits_to_f32(k)[:, :hd], bf16_bits_to_f32(v)[:, :hd]
    start = time.perf_counter()
    ref = engine.gqa_attention(np.ascontiguousarray(qf), np.ascontiguousarray(kf), np.ascontiguousarray(vf),
                               tokens - rows, 1, 1, hd, threads=threads)
    seconds = time.perf_counter() - start
    got = bf16_bits_to_f32(o)[:, :hd]
    return float(np.abs(ref - got).max()), seconds



def bench_mla(lib, backend, abi, hbm_peak, repeats, sessions=32, context=16384):
    """Config 5: latent-compressed decode, 128 heads, latent 512 + rope 64, bf16."""
    heads, nope, dc, dr = 128, 128, 512, 64
    sizes = {"q_nope": sessions * heads * nope, "q_rope": sessions * heads * dr, "w_uk": heads * nope * dc,
             "latent": sessions * context * dc, "rope_key": sessions * context * dr}
    bufs = {k: _alloc(lib, n * 2) for k, n in sizes.items()}
    for i, (k, n) in enumerate(sizes.items()):
        sigma = 1.0 / np.sqrt(dc) if k == "w_uk" else 1.0
        lib.yvx_cuda_fill_normal(bufs[k], abi.DTYPE_BF16, n, 401 + i, sigma, backend.stream)
    p = abi.MlaProblem()
    p.sessions, p.heads, p.nope_dim, p.latent_dim, p.rope_dim = sessions, heads, nope, dc, dr
    p.scale = 1.0 / np.sqrt(192.0)
    p.q_nope, p.q_rope, p.w_uk = bufs["q_nope"], bufs["q_rope"], bufs["w_uk"]
    p.latent, p.rope_key = bufs["latent"], bufs["rope_key"]
    p.latent_session_stride, p.rope_session_stride = context * dc, context * dr
    p.kv_tokens_uniform = p.kv_tokens_max = context
    lib.yvx_cuda_mla_plan(C.byref(p), backend.sm_count)
    q_abs = _alloc(lib, lib.yvx_cuda_mla_absorbed_bytes(C.byref(p)))
    parts = _alloc(lib, lib.yvx_cuda_mla_partials_bytes(C.byref(p)))
    out = _alloc(lib, sessions * heads * dc * 4)
    status = _alloc(lib, 4)
    lib.yvx_cuda_memset_async(status, 0, 4, backend.stream)
    p.q_absorbed, p.partials, p.output, p.status = q_abs, parts, out, status

    def event():
        e = C.c_void_p()
        assert lib.yvx_cuda_event_create(C.byref(e)) == 0
        return e
    n = C.c_uint()
    for _ in range(3):
        assert lib.yvx_cuda_mla_decode(C.byref(p), backend.stream, None, C.byref(n)) == 0, lib.yvx_cuda_last_error_text()
    quads = [tuple(event() for _ in range(4)) for _ in range(repeats)]
    for quad in quads:
        rc = lib.yvx_cuda_mla_decode(C.byref(p), backend.stream, (C.c_void_p * 4)(*quad), C.byref(n))
        assert rc == 0, lib.yvx_cuda_last_error_text()
    assert lib.yvx_cuda_stream_synchronize(backend.stream) == 0, lib.yvx_cuda_last_error_text()
    ms = C.c_float()
    spans = [[], [], []]
    for quad in quads:
        for i in range(3):
            lib.yvx_cuda_event_elapsed_ms(quad[i], quad[i + 1], C.byref(ms))
            spans[i].append(ms.value)
        for e in quad:
            lib.yvx_cuda_event_destroy(e)
    absorb, attend, combine = (float(np.mean(x)) for x in spans)
    nbytes = sessions * context * (dc + dr) * 2 + sizes["w_uk"] * 2 + sessions * heads * ((nope + dr) * 2 + dc * 4)
    flops = 2.0 * sessions * heads * context * (dc + dr + dc) + 2.0 * sessions * heads * nope * dc
    # sample for the CPU check: session 0, heads 0..7
    h = 8
    host = {"q_nope": np.empty((h, nope), np.uint16), "q_rope": np.empty((h, dr), np.uint16),
            "w_uk": np.empty((h, nope, dc), np.uint16), "latent": np.empty((context, dc), np.uint16),
            "rope_key": np.empty((context, dr), np.uint16)}
    for k, a in host.items():
        lib.yvx_cuda_download_async(a.ctypes.data, bufs[k], a.nbytes, backend.stream)
    o_host = np.empty((h, dc), np.float32)
    st = np.zeros(1, np.int32)
    lib.yvx_cuda_download_async(o_host.ctypes.data, out, o_host.nbytes, backend.stream)
    lib.yvx_cuda_download_async(st.ctypes.data, status, 4, backend.stream)
    lib.yvx_cuda_stream_synchronize(backend.stream)
    total = absorb + attend + combine
    tf_peak = 1699.0
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        with open(peaks_path) as f:
            tf_peak = float(json.load(f)["bf16_tflops"])
    result = {"workload": f"latent decode, {sessions} sessions x {context} tokens, 128 heads, latent 512 + rope 64, bf16",
              "kernel": "mla_decode_tcgen05_kernel", "launches_per_step": int(n.value),
              "absorb_ms": absorb, "kernel_ms": attend, "combine_ms": combine,
              "algorithmic_bytes": nbytes, "flops": flops,
              "achieved_gbs": nbytes / (attend * 1e-3) / 1e9, "frac_of_measured_hbm": nbytes / (attend * 1e-3) / 1e9 / hbm_peak,
              "achieved_tflops": flops / (attend * 1e-3) / 1e12, "frac_of_bf16_peak": flops / (attend * 1e-3) / 1e12 / tf_peak,
              "tokens_per_s": sessions / (total * 1e-3), "status_word": int(st[0]),
              "chunk_tokens": p.chunk_tokens, "max_splits": p.max_splits,
              "l2": "latent + rope cache %.0f MB exceed L2" % (sessions * context * (dc + dr) * 2 / 1e6)}
    for ptr in list(bufs.values()) + [q_abs, parts, out, status]:
        lib.yvx_cuda_free(ptr)
    return result, (host, o_host)


def bench_kv_append(lib, backend, abi, hbm_peak, repeats, sessions=2, tokens=8192):
    """KV append + rotary for the new rows of a step (prefill-sized: sessions x tokens rows,
    40q/8kv heads, hd 128, full rotary width, bf16-staged arithmetic): Q rotated in place,
    K rotated and V copied into bf16 pools behind an identity block table."""
    hq, hkv, hd, block = 40, 8, 128, 64
    rows = sessions * tokens
    sizes = {"q": rows * hq * hd, "k": rows * hkv * hd, "v": rows * hkv * hd, "cos": rows * hd, "sin": rows * hd}
    bufs = {k: _alloc(lib, n * 4) for k, n in sizes.items()}
    for i, (k, n) in enumerate(sizes.items()):
        lib.yvx_cuda_fill_normal(bufs[k], abi.DTYPE_F32, n, 601 + i, 0.5, backend.stream)
    blocks = (tokens + block - 1) // block
    kpool, vpool = _alloc(lib, rows * hkv * hd * 2), _alloc(lib, rows * hkv * hd * 2)
    table_host = np.arange(sessions * blocks, dtype=np.int32).reshape(sessions, blocks)
    table, status = _alloc(lib, table_host.nbytes), _alloc(lib, 4)
    lib.yvx_cuda_upload_async(table, table_host.ctypes.data, table_host.nbytes, backend.stream)
    lib.yvx_cuda_memset_async(status, 0, 4, backend.stream)
    a = abi.KvAppendArgs()
    a.sessions, a.tokens, a.query_heads, a.kv_heads, a.head_dim, a.rotary_dim = sessions, tokens, hq, hkv, hd, hd
    a.staged_bf16 = 1
    a.query, a.key, a.value, a.cosines, a.sines = bufs["q"], bufs["k"], bufs["v"], bufs["cos"], bufs["sin"]
    a.kv_tokens_uniform = 0
    a.key_pool, a.value_pool, a.block_table = kpool, vpool, table
    a.block_tokens, a.block_table_stride, a.pool_blocks = block, blocks, sessions * blocks
    a.pool_token_stride, a.pool_head_stride, a.pool_block_stride = hkv * hd, hd, block * hkv * hd
    a.status = status

    def event():
        e = C.c_void_p()
        assert lib.yvx_cuda_event_create(C.byref(e)) == 0
        return e
    for _ in range(3):
        assert lib.yvx_cuda_kv_append_rotary(C.byref(a), backend.stream) == 0
    first, last = event(), event()
    lib.yvx_cuda_event_record(first, backend.stream)
    for _ in range(repeats):
        assert lib.yvx_cuda_kv_append_rotary(C.byref(a), backend.stream) == 0
    lib.yvx_cuda_event_record(last, backend.stream)
    assert lib.yvx_cuda_stream_synchronize(backend.stream) == 0, lib.yvx_cuda_last_error_text()
    ms = C.c_float()
    lib.yvx_cuda_event_elapsed_ms(first, last, C.byref(ms))
    step = ms.value / repeats
    # per row: Q read + written (F32), K and V read (F32), tables read, K and V written (bf16)
    nbytes = rows * (2 * hq * hd * 4 + 2 * hkv * hd * 4 + 2 * hd * 4 + 2 * hkv * hd * 2)
    st = np.zeros(1, np.int32)
    lib.yvx_cuda_download_async(st.ctypes.data, status, 4, backend.stream)
    lib.yvx_cuda_stream_synchronize(backend.stream)
    result = {"workload": f"KV append + rotary, {sessions} x {tokens} new rows, 40q/8kv heads, hd128, "
                          "F32 in, bf16 pools behind a block table",
              "kernel": "kv_append_rotary_kernel", "launches_per_step": 1, "kernel_ms": step,
              "algorithmic_bytes": nbytes, "achieved_gbs": nbytes / (step * 1e-3) / 1e9,
              "frac_of_measured_hbm": nbytes / (step * 1e-3) / 1e9 / hbm_peak,
              "rows_per_s": rows / (step * 1e-3), "status_word": int(st[0]),
              "l2": "%.0f MB per launch exceed L2" % (nbytes / 1e6),
              "replaces": "2 rotary launches + 2 device copies per new token + a position upload"}
    for ptr in list(bufs.values()) + [kpool, vpool, table, status]:
        lib.yvx_cuda_free(ptr)
    return result, None


def bench_compressor(lib, backend, abi, hbm_peak, repeats, tokens=32768):
    """Rolling compressor over a prefill-sized chunk of the sparse class's main rows (ratio 4,
    head dimension 512, two halves: 1024-lane token rows) with the publication chain (bf16, RMS
    norm, bf16, rotation of the last 64 lanes, bf16); a CPU-computed sample of rows is compared."""
    from oracle.binding import Oracle, PositionPolicy, compressor_initial_state
    ratio, hd, rope, width = 4, 512, 64, 1024
    oracle = Oracle()
    frequency = oracle.rope_frequencies(PositionPolicy(10000, 16, 65536, 32, 1), rope)
    sizes = {"kv": tokens * width, "score": tokens * width, "ape": ratio * width, "norm": hd}
    dev = {k: _alloc(lib, n * 4) for k, n in sizes.items()}
    for i, (k, n) in enumerate(sizes.items()):
        lib.yvx_cuda_fill_normal(dev[k], abi.DTYPE_F32, n, 701 + i, 1.0, backend.stream)
    kv0, score0 = compressor_initial_state(ratio, hd, 1)
    emitted = tokens // ratio
    for name, nbytes in (("skv", kv0.nbytes), ("ssc", kv0.nbytes), ("akv", kv0.nbytes), ("asc", kv0.nbytes),
                         ("rows", emitted * hd * 4), ("positions", emitted * 8), ("freq", frequency.nbytes),
                         ("status", 4)):
        dev[name] = _alloc(lib, nbytes)
    for name, array in (("skv", kv0), ("ssc", score0), ("freq", frequency)):
        lib.yvx_cuda_upload_async(dev[name], array.ctypes.data, array.nbytes, backend.stream)
    lib.yvx_cuda_memset_async(dev["status"], 0, 4, backend.stream)
    a = abi.CompressorArgs()
    a.ratio, a.head_dim, a.overlap, a.start_position, a.token_count = ratio, hd, 1, 0, tokens
    a.token_kv, a.token_score, a.token_stride, a.ape = dev["kv"], dev["score"], width, dev["ape"]
    a.state_kv, a.state_score, a.after_kv, a.after_score = dev["skv"], dev["ssc"], dev["akv"], dev["asc"]
    a.compressed, a.compressed_stride, a.positions = dev["rows"], hd, dev["positions"]
    a.norm_weights, a.epsilon, a.rope_dims, a.rope_frequency = dev["norm"], 1e-6, rope, dev["freq"]
    a.status = dev["status"]
    count = C.c_ulonglong()

    def event():
        e = C.c_void_p()
        assert lib.yvx_cuda_event_create(C.byref(e)) == 0
        return e
    for _ in range(3):
        assert lib.yvx_cuda_compressor_chunk(C.byref(a), backend.stream, C.byref(count)) == 0
    first, last = event(), event()
    lib.yvx_cuda_event_record(first, backend.stream)
    for _ in range(repeats):
        assert lib.yvx_cuda_compressor_chunk(C.byref(a), backend.stream, C.byref(count)) == 0
    lib.yvx_cuda_event_record(last, backend.stream)
    assert lib.yvx_cuda_stream_synchronize(backend.stream) == 0, lib.yvx_cuda_last_error_text()
    ms = C.c_float()
    lib.yvx_cuda_event_elapsed_ms(first, last, C.byref(ms))
    step = ms.value / repeats
    # per token: its kv and score rows read once; per emitted row: head_dim floats and a position written
    nbytes = tokens * 2 * width * 4 + emitted * (hd * 4 + 8)
    sample_tokens = 64
    host = {k: np.zeros((sample_tokens, width) if k in ("kv", "score") else ((ratio, width) if k == "ape" else (hd,)),
                        np.float32) for k in ("kv", "score", "ape", "norm")}
    rows, st = np.zeros((sample_tokens // ratio, hd), np.float32), np.zeros(1, np.int32)
    for k, array in host.items():
        lib.yvx_cuda_download_async(array.ctypes.data, dev[k], array.nbytes, backend.stream)
    lib.yvx_cuda_download_async(rows.ctypes.data, dev["rows"], rows.nbytes, backend.stream)
    lib.yvx_cuda_download_async(st.ctypes.data, dev["status"], 4, backend.stream)
    lib.yvx_cuda_stream_synchronize(backend.stream)
    begin = time.perf_counter()
    ref = oracle.compressor_chunk(ratio, hd, 1, 0, host["kv"], host["score"], host["ape"], kv0, score0, host["norm"],
                                  1e-6, rope, frequency)
    cpu_seconds = time.perf_counter() - begin
    result = {"workload": f"rolling compressor, {tokens} tokens in one chunk, ratio 4, head dimension 512, two halves "
                          "(1024-lane rows), publication chain with rotation fused",
              "kernel": "compressor_chunk_kernel", "launches_per_step": 1, "kernel_ms": step,
              "algorithmic_bytes": nbytes, "achieved_gbs": nbytes / (step * 1e-3) / 1e9,
              "frac_of_measured_hbm": nbytes / (step * 1e-3) / 1e9 / hbm_peak,
              "tokens_per_s": tokens / (step * 1e-3), "emitted_rows": int(count.value), "status_word": int(st[0]),
              "l2": "%.0f MB per launch exceed L2" % (nbytes / 1e6),
              "replaces": "one single-CTA launch per token that copies the whole state",
              "rows_differing_from_cpu_on_sample": int((ref[0] != rows).sum()) if ref is not None else -1,
              "gpu_vs_cpu_max_abs_on_sample": float(np.abs(ref[0] - rows).max()) if ref is not None else -1.0,
              "cpu_sample": f"first {sample_tokens} tokens (CPU restatement, 1 core)",
              "cpu_sample_ms": cpu_seconds * 1e3, "cpu_cores": 1}
    for ptr in dev.values():
        lib.yvx_cuda_free(ptr)
    return result, None


def bench_reference_gpu(lib, backend, abi, repeats=5):
    """The reference's OWN CUDA attention kernel (yvex_gqa_f32, src/backend/cuda/transformer_kernels.cu:137-238,
    compiled for sm_100 from its source into oracle/_ref by `make -C oracle ref_cuda`) launched with the
    reference's geometry (src/backend/cuda/transformer.c:790-803: 128 threads = 4 query rows per block, one block
    per (row tile, query head), 2 * head_dim floats of shared memory) on config 1 and on a small F32 causal
    prefill, timed between CUDA events, its output compared with this library's on the same device buffers."""
    from oracle.binding import REFERENCE_CUBIN
    if not os.path.exists(REFERENCE_CUBIN):
        return {"unavailable": "oracle/_ref/transformer_kernels.sm_100.cubin is not built (make -C oracle ref_cuda)"}
    try:
        from cuda.bindings import driver as cu
    except Exception as error:       # pragma: no cover
        return {"unavailable": f"cuda-python is not importable: {error}"}
    err, module = cu.cuModuleLoadData(open(REFERENCE_CUBIN, "rb").read())
    if int(err) != 0:
        return {"unavailable": f"cuModuleLoadData: {err}"}
    err, function = cu.cuModuleGetFunction(module, b"yvex_gqa_f32")
    assert int(err) == 0, err

    def event():
        e = C.c_void_p()
        assert lib.yvx_cuda_event_create(C.byref(e)) == 0
        return e
    first, last, ms = event(), event(), C.c_float()
    out = {}
    # the third case has bf16-valued F32 inputs (what the reference's runtime feeds its attention) and
    # takes this library's default dispatch: staged to bf16 for the tensor cores behind the device gate
    for name, rows, tokens, hq, hkv, hd, copies, valued in (("config1_decode_f32", 1, 4096, 32, 8, 128, 16, 0),
                                                            ("prefill_f32_2048x16q4kv_exact", 2048, 2048, 16, 4, 128, 1, 0),
                                                            ("prefill_f32_2048x16q4kv_bf16_valued", 2048, 2048, 16, 4, 128, 1, 1)):
        width = hkv * hd
        kv_elems = tokens * width
        k, v = _alloc(lib, copies * kv_elems * 4), _alloc(lib, copies * kv_elems * 4)
        q, mine, theirs = _alloc(lib, rows * hq * hd * 4), _alloc(lib, rows * hq * hd * 4), _alloc(lib, rows * hq * hd * 4)
        status, tickets = _alloc(lib, 4), _alloc(lib, 8 * hkv)
        lib.yvx_cuda_memset_async(tickets, 0, 8 * hkv, backend.stream)
        lib.yvx_cuda_memset_async(status, 0, 4, backend.stream)
        fill = -abi.DTYPE_F32 if valued else abi.DTYPE_F32
        lib.yvx_cuda_fill_normal(k, fill, copies * kv_elems, 601, 1.0, backend.stream)
        lib.yvx_cuda_fill_normal(v, fill, copies * kv_elems, 602, 1.0, backend.stream)
        lib.yvx_cuda_fill_normal(q, fill, rows * hq * hd, 603, 1.0, backend.stream)
        staging = None
        problems, scratch = [], None
        for i in range(copies):
            p = abi.GqaProblem()
            p.sessions, p.query_rows, p.query_heads, p.kv_heads, p.head_dim = 1, rows, hq, hkv, hd
            p.causal, p.scale = 1, 1.0 / np.sqrt(hd)
            p.query_dtype = p.kv_dtype = p.output_dtype = abi.DTYPE_F32
            p.query, p.query_row_stride, p.output = q, hq * hd, mine
            p.key, p.value = k.value + i * kv_elems * 4, v.value + i * kv_elems * 4
            p.key_token_stride = p.value_token_stride = width
            p.key_head_stride = p.value_head_stride = hd
            p.kv_tokens_uniform = p.kv_tokens_max = tokens
            p.query_start_uniform = tokens - rows
            p.force_general = 1 if rows > 1 and not valued else 0
            lib.yvx_cuda_gqa_plan_splits(C.byref(p), backend.sm_count)
            if scratch is None:
                scratch = _alloc(lib, max(lib.yvx_cuda_gqa_partials_bytes(C.byref(p)), 16))
                staging_bytes = lib.yvx_cuda_gqa_f32_staging_bytes(C.byref(p)) if valued else 0
                staging = _alloc(lib, staging_bytes) if staging_bytes else None
            p.partials, p.status, p.tickets = scratch, status, tickets
            if staging is not None:
                p.f32_staging = staging
            problems.append(p)
        n = C.c_uint()

        def ours(i):
            assert lib.yvx_cuda_gqa_attention(C.byref(problems[i % copies]), backend.stream, C.byref(n)) == 0

        def reference(i):
            values = [C.c_void_p(q.value), C.c_void_p(k.value + (i % copies) * kv_elems * 4),
                      C.c_void_p(v.value + (i % copies) * kv_elems * 4), C.c_void_p(theirs.value),
                      C.c_ulonglong(rows), C.c_ulonglong(tokens), C.c_ulonglong(tokens - rows), C.c_ulonglong(hq),
                      C.c_ulonglong(hkv), C.c_ulonglong(hd), C.c_ulonglong(hq * hd), C.c_ulonglong(width),
                      C.c_ulonglong(width), C.c_float(1.0 / np.sqrt(hd)), C.c_int(1)]
            params = (C.c_void_p * len(values))(*[C.addressof(x) for x in values])
            grid = ((rows + 3) // 4) * hq
            stream = cu.CUstream(backend.stream.value if hasattr(backend.stream, "value") else int(backend.stream))
            err, = cu.cuLaunchKernel(function, grid, 1, 1, 128, 1, 1, 2 * hd * 4, stream, C.addressof(params), 0)
            assert int(err) == 0, err
        timings = {}
        for label, run in (("ours", ours), ("reference", reference)):
            run(0)
            lib.yvx_cuda_event_record(first, backend.stream)
            for i in range(repeats):
                run(i)
            lib.yvx_cuda_event_record(last, backend.stream)
            assert lib.yvx_cuda_stream_synchronize(backend.stream) == 0, lib.yvx_cuda_last_error_text()
            lib.yvx_cuda_event_elapsed_ms(first, last, C.byref(ms))
            timings[label] = ms.value / repeats
        # both on the same copy, then compare
        ours(0)
        reference(0)
        a, b = np.empty(rows * hq * hd, np.float32), np.empty(rows * hq * hd, np.float32)
        lib.yvx_cuda_download_async(a.ctypes.data, mine, a.nbytes, backend.stream)
        lib.yvx_cuda_download_async(b.ctypes.data, theirs, b.nbytes, backend.stream)
        lib.yvx_cuda_stream_synchronize(backend.stream)
        out[name] = {"reference_gpu_ms": timings["reference"], "this_library_ms": timings["ours"],
                     "speedup": timings["reference"] / timings["ours"],
                     "max_scaled_difference": float(np.max(np.abs(a - b) / (1.0 + np.abs(b)))),
                     "grid": ((rows + 3) // 4) * hq}
        for ptr in (k, v, q, mine, theirs, status, tickets, scratch) + ((staging,) if staging is not None else ()):
            lib.yvx_cuda_free(ptr)
    for e in (first, last):
        lib.yvx_cuda_event_destroy(e)
    cu.cuModuleUnload(module)
    return {"kernel": "yvex_gqa_f32 (the reference's CUDA kernel, compiled for sm_100 from its source)", **out}


def bench_projections(lib, backend, abi, hbm_peak, repeats, tokens=1):
    """The five projections around the latent attention of one decode step at the reference
    configuration's widths (hidden 4096, query rank 1024, 64 heads x 512, 8 output groups,
    output rank 1024): q_a [1024 x 4096], q_b [32768 x 1024], kv [512 x 4096], grouped out_a
    [8 x 1024 x 4096], out_b [4096 x 8192]; 106.9 M weights, once as BF16 and once as Q8_0.
    Every weight byte is read once per step (two copies of the weights alternate so that no
    step finds them in L2); the roofline is encoded bytes / measured HBM peak. Sample rows of
    every projection are compared with the CPU restatement of the reference's dot bit for bit."""
    from oracle.binding import Oracle
    oracle = Oracle()
    shapes = (("q_a", 1024, 4096, 1), ("q_b", 32768, 1024, 1), ("kv", 512, 4096, 1), ("out_a", 1024, 4096, 8),
              ("out_b", 4096, 8192, 1))
    rng = np.random.default_rng(SEED + 91)
    copies, sample_rows = 2, 16
    out = {}

    def event():
        e = C.c_void_p()
        assert lib.yvx_cuda_event_create(C.byref(e)) == 0
        return e
    first, last, ms = event(), event(), C.c_float()
    status = _alloc(lib, 4)
    lib.yvx_cuda_memset_async(status, 0, 4, backend.stream)
    for label, qtype in (("bf16", abi.QTYPE_BF16), ("q8_0", abi.QTYPE_Q8_0)):
        owned, calls, checks, weight_bytes = [], [[] for _ in range(copies)], [], 0
        for name, rows, width, groups in shapes:
            row_bytes = lib.yvx_cuda_qtype_row_bytes(qtype, width)
            total_rows = rows * groups
            weight_bytes += total_rows * row_bytes
            if qtype == abi.QTYPE_Q8_0:
                blocks = np.zeros((total_rows * (width // 32), 34), np.uint8)
                blocks[:, :2] = rng.uniform(0.002, 0.02, blocks.shape[0]).astype(np.float16).view(np.uint8).reshape(-1, 2)
                blocks[:, 2:] = rng.integers(-127, 128, (blocks.shape[0], 32), dtype=np.int8).view(np.uint8)
                host = blocks.reshape(total_rows, row_bytes)
            else:
                host = None
            x_host = np.zeros((tokens, groups * width), np.float32)
            x = _alloc(lib, x_host.nbytes)
            lib.yvx_cuda_fill_normal(x, -abi.DTYPE_F32, x_host.size, 300 + len(owned), 1.0, backend.stream)
            lib.yvx_cuda_download_async(x_host.ctypes.data, x, x_host.nbytes, backend.stream)
            y = _alloc(lib, tokens * total_rows * 4)
            owned += [x, y]
            for c in range(copies):
                w = _alloc(lib, total_rows * row_bytes)
                owned.append(w)
                if host is not None:
                    lib.yvx_cuda_upload_async(w, host.ctypes.data, host.nbytes, backend.stream)
                else:
                    lib.yvx_cuda_fill_normal(w, abi.DTYPE_BF16, total_rows * width, 400 + len(owned), 0.02, backend.stream)
                a = abi.MatvecArgs()
                a.weights, a.qtype, a.rows, a.width, a.row_bytes = w, qtype, rows, width, row_bytes
                a.input, a.tokens, a.input_stride = x, tokens, groups * width
                a.output, a.output_stride, a.groups, a.round_bf16, a.status = y, total_rows, groups, 1, status
                calls[c].append(a)
            lib.yvx_cuda_stream_synchronize(backend.stream)     # the host block array may go
            checks.append((name, rows, width, groups, row_bytes, x_host, y, calls[(repeats - 1) % copies][-1]))

        def step(i):
            for a in calls[i % copies]:
                assert lib.yvx_cuda_qtype_matvec(C.byref(a), backend.stream) == 0, lib.yvx_cuda_last_error_text()
        for i in range(3):
            step(i)
        lib.yvx_cuda_event_record(first, backend.stream)
        for i in range(repeats):
            step(i)
        lib.yvx_cuda_event_record(last, backend.stream)
        assert lib.yvx_cuda_stream_synchronize(backend.stream) == 0, lib.yvx_cuda_last_error_text()
        lib.yvx_cuda_event_elapsed_ms(first, last, C.byref(ms))
        step_ms = ms.value / repeats
        # each projection alone (events around its launch)
        alone = {}
        for k, (name, rows, width, groups, row_bytes, _, _, _) in enumerate(checks):
            total = 0.0
            for i in range(repeats):
                a = calls[i % copies][k]
                lib.yvx_cuda_event_record(first, backend.stream)
                lib.yvx_cuda_qtype_matvec(C.byref(a), backend.stream)
                lib.yvx_cuda_event_record(last, backend.stream)
                lib.yvx_cuda_stream_synchronize(backend.stream)
                lib.yvx_cuda_event_elapsed_ms(first, last, C.byref(ms))
                total += ms.value
            nbytes = rows * groups * row_bytes
            alone[name] = {"kernel_us": total / repeats * 1e3, "gbs": nbytes / (total / repeats * 1e-3) / 1e9}
        graph_ms = None
        if lib.yvx_cuda_graph_capture_begin(backend.stream) == 0:
            for i in range(2 * copies):
                step(i)
            graph = C.c_void_p()
            if lib.yvx_cuda_graph_capture_end(backend.stream, C.byref(graph)) == 0:
                lib.yvx_cuda_graph_launch(graph, backend.stream)
                lib.yvx_cuda_event_record(first, backend.stream)
                replays = max(repeats // (2 * copies), 3)
                for _ in range(replays):
                    lib.yvx_cuda_graph_launch(graph, backend.stream)
                lib.yvx_cuda_event_record(last, backend.stream)
                if lib.yvx_cuda_stream_synchronize(backend.stream) == 0:
                    lib.yvx_cuda_event_elapsed_ms(first, last, C.byref(ms))
                    graph_ms = ms.value / (replays * 2 * copies)
                lib.yvx_cuda_graph_destroy(graph)
        # sample rows against the CPU dot
        equal = True
        for name, rows, width, groups, row_bytes, x_host, y, a in checks:
            got = np.zeros((tokens, rows * groups), np.float32)
            lib.yvx_cuda_qtype_matvec(C.byref(a), backend.stream)
            lib.yvx_cuda_download_async(got.ctypes.data, y, got.nbytes, backend.stream)
            sample = np.zeros((sample_rows, row_bytes), np.uint8)
            last_group_first = (groups - 1) * rows
            lib.yvx_cuda_download_async(sample.ctypes.data, a.weights + last_group_first * row_bytes, sample.nbytes,
                                        backend.stream)
            lib.yvx_cuda_stream_synchronize(backend.stream)
            want = oracle.qtype_matvec(sample, qtype, width,
                                       np.ascontiguousarray(x_host[:, (groups - 1) * width:groups * width]), 0,
                                       sample_rows, True)
            equal = equal and want is not None and bool(np.array_equal(
                got[:, last_group_first:last_group_first + sample_rows].view(np.uint32), want.view(np.uint32)))
        best = min(step_ms, graph_ms or step_ms)
        out[label] = {"step_ms": step_ms, "graph_step_ms": graph_ms, "encoded_bytes": weight_bytes,
                      "bytes_per_weight": weight_bytes / 106954752.0,
                      "achieved_gbs": weight_bytes / (best * 1e-3) / 1e9,
                      "frac_of_measured_hbm": weight_bytes / (best * 1e-3) / 1e9 / hbm_peak,
                      "per_projection": alone, "sample_rows_bit_equal_to_cpu_dot": equal}
        for ptr in owned:
            lib.yvx_cuda_free(ptr)
    st = np.zeros(1, np.int32)
    lib.yvx_cuda_download_async(st.ctypes.data, status, 4, backend.stream)
    lib.yvx_cuda_stream_synchronize(backend.stream)
    lib.yvx_cuda_free(status)
    for e in (first, last):
        lib.yvx_cuda_event_destroy(e)
    result = {"workload": "projections of one latent decode step (q_a, q_b, kv, grouped out_a, out_b; 106.9 M weights, "
                          "%d token%s), encoded weights read once per step" % (tokens, "" if tokens == 1 else "s"),
              "kernel": "qtype_matvec_kernel", "launches_per_step": 5, "status_word": int(st[0]),
              "roofline_unit": "encoded weight bytes / measured HBM peak", **out}
    return result, None


def bench_projections_prefill(lib, backend, abi, repeats, tokens=4096):
    """The same five projections for a prefill chunk of `tokens` tokens on the tensor cores
    (yvx_cuda_bf16_gemm: tcgen05, BF16 weights, bf16-valued activations, publication fused into the
    epilogue): 2 * tokens * 106.9 M flop per step. A sample of tokens is compared with the CPU twin."""
    from oracle.binding import Oracle
    oracle = Oracle()
    shapes = (("q_a", 1024, 4096, 1), ("q_b", 32768, 1024, 1), ("kv", 512, 4096, 1), ("out_a", 1024, 4096, 8),
              ("out_b", 4096, 8192, 1))
    status = _alloc(lib, 4)
    lib.yvx_cuda_memset_async(status, 0, 4, backend.stream)

    def event():
        e = C.c_void_p()
        assert lib.yvx_cuda_event_create(C.byref(e)) == 0
        return e
    first, last, ms = event(), event(), C.c_float()
    calls, owned, flops = [], [status], 0.0
    for k, (name, rows, width, groups) in enumerate(shapes):
        total_rows, lanes = rows * groups, groups * width
        w, x, y = _alloc(lib, total_rows * width * 2), _alloc(lib, tokens * lanes * 4), _alloc(lib, tokens * total_rows * 4)
        staging = _alloc(lib, lib.yvx_cuda_bf16_gemm_staging_bytes(tokens, groups, width))
        owned += [w, x, y, staging]
        lib.yvx_cuda_fill_normal(w, abi.DTYPE_BF16, total_rows * width, 500 + k, 0.02, backend.stream)
        lib.yvx_cuda_fill_normal(x, -abi.DTYPE_F32, tokens * lanes, 520 + k, 1.0, backend.stream)
        a = abi.GemmArgs()
        a.weights, a.rows, a.width, a.input, a.tokens, a.input_stride = w, rows, width, x, tokens, lanes
        a.output, a.output_stride, a.groups, a.round_bf16, a.staging, a.status = y, total_rows, groups, 1, staging, status
        calls.append(a)
        flops += 2.0 * tokens * total_rows * width

    def step():
        for a in calls:
            assert lib.yvx_cuda_bf16_gemm(C.byref(a), backend.stream) == 0, lib.yvx_cuda_last_error_text()
    for _ in range(2):
        step()
    lib.yvx_cuda_event_record(first, backend.stream)
    for _ in range(repeats):
        step()
    lib.yvx_cuda_event_record(last, backend.stream)
    assert lib.yvx_cuda_stream_synchronize(backend.stream) == 0, lib.yvx_cuda_last_error_text()
    lib.yvx_cuda_event_elapsed_ms(first, last, C.byref(ms))
    step_ms = ms.value / repeats
    alone = {}
    for (name, rows, width, groups), a in zip(shapes, calls):
        lib.yvx_cuda_event_record(first, backend.stream)
        for _ in range(repeats):
            lib.yvx_cuda_bf16_gemm(C.byref(a), backend.stream)
        lib.yvx_cuda_event_record(last, backend.stream)
        lib.yvx_cuda_stream_synchronize(backend.stream)
        lib.yvx_cuda_event_elapsed_ms(first, last, C.byref(ms))
        t = ms.value / repeats
        alone[name] = {"ms": t, "tflops": 2.0 * tokens * rows * groups * width / (t * 1e-3) / 1e12}
    # sample: 4 tokens x 16 rows of every projection against the CPU twin
    worst_steps, differing, compared = 0.0, 0, 0
    for (name, rows, width, groups), a in zip(shapes, calls):
        lanes, total_rows = groups * width, rows * groups
        xs = np.zeros((4, lanes), np.float32)
        ws = np.zeros((16, width * 2), np.uint8)
        ys = np.zeros((4, total_rows), np.float32)
        lib.yvx_cuda_download_async(xs.ctypes.data, a.input, xs.nbytes, backend.stream)
        lib.yvx_cuda_download_async(ws.ctypes.data, a.weights + (groups - 1) * rows * width * 2, ws.nbytes, backend.stream)
        lib.yvx_cuda_download_async(ys.ctypes.data, a.output, ys.nbytes, backend.stream)
        lib.yvx_cuda_stream_synchronize(backend.stream)
        want = oracle.qtype_matvec(ws, abi.QTYPE_BF16, width, np.ascontiguousarray(xs[:, (groups - 1) * width:]), 0, 16, True)
        got = ys[:, (groups - 1) * rows:(groups - 1) * rows + 16]
        step_size = np.exp2(np.floor(np.log2(np.maximum(np.maximum(np.abs(want), np.abs(got)), 1e-3))) - 7.0)
        worst_steps = max(worst_steps, float(np.max(np.abs(got - want) / step_size)))
        differing += int((got != want).sum())
        compared += got.size
    st = np.zeros(1, np.int32)
    lib.yvx_cuda_download_async(st.ctypes.data, status, 4, backend.stream)
    lib.yvx_cuda_stream_synchronize(backend.stream)
    for e in (first, last):
        lib.yvx_cuda_event_destroy(e)
    for ptr in owned:
        lib.yvx_cuda_free(ptr)
    tf_peak = 1590.0
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        with open(peaks_path) as f:
            tf_peak = float(json.load(f)["bf16_tflops"])
    result = {"workload": "projections of one latent layer for a prefill chunk of %d tokens (BF16 weights, 106.9 M; "
                          "activation staging inside the timed step)" % tokens,
              "kernel": "bf16_gemm_tcgen05_kernel", "launches_per_step": 10, "step_ms": step_ms, "kernel_ms": step_ms,
              "flops": flops, "achieved_tflops": flops / (step_ms * 1e-3) / 1e12,
              "frac_of_bf16_peak": flops / (step_ms * 1e-3) / 1e12 / tf_peak, "per_projection": alone,
              "status_word": int(st[0]), "sample_values": compared, "sample_values_differing_from_cpu": differing,
              "sample_worst_difference_in_bf16_steps": worst_steps}
    return result, None


def bench_activation(lib, backend, abi, hbm_peak, repeats, rows=131072):
    """Activation fake quantisation in place: FP8 E4M3 in blocks of 64 over the 448 leading lanes of
    512-lane rows (what the reference applies to new local rows and emitted compressed rows), and the
    transform + FP4 E2M1 variant over 128-lane rows (index queries). A sample of rows is compared with
    the CPU restatement bit for bit."""
    from oracle.binding import Oracle
    oracle = Oracle()
    out = {}
    for name, stride, count, quantization, block, hadamard in (("fp8_rows_512x448", 512, 448, 8, 64, 0),
                                                               ("fp4_hadamard_rows_128", 128, 128, 4, 32, 1)):
        n = rows if stride == 512 else rows * 4
        values, source, status = _alloc(lib, n * stride * 4), _alloc(lib, n * stride * 4), _alloc(lib, 4)
        lib.yvx_cuda_fill_normal(source, abi.DTYPE_F32, n * stride, 811, 1.0, backend.stream)
        lib.yvx_cuda_memset_async(status, 0, 4, backend.stream)
        a = abi.ActivationArgs()
        a.values, a.rows, a.row_stride, a.count = values, n, stride, count
        a.quantization, a.block_width, a.hadamard = quantization, block, hadamard
        a.hadamard_scale = float(np.float32(1.0) / np.sqrt(np.float32(count)))
        a.status = status
        sample = np.zeros((64, stride), np.float32)
        lib.yvx_cuda_download_async(sample.ctypes.data, source, sample.nbytes, backend.stream)

        def event():
            e = C.c_void_p()
            assert lib.yvx_cuda_event_create(C.byref(e)) == 0
            return e
        # the operation is in place and not idempotent behind a transform: time it on a fresh copy each
        # time and subtract nothing; the copy is timed separately and reported
        first, middle, last = event(), event(), event()
        for _ in range(2):
            lib.yvx_cuda_copy_async(values, source, n * stride * 4, backend.stream)
            assert lib.yvx_cuda_activation_quant(C.byref(a), backend.stream) == 0
        total = 0.0
        for _ in range(repeats):
            lib.yvx_cuda_copy_async(values, source, n * stride * 4, backend.stream)
            lib.yvx_cuda_event_record(first, backend.stream)
            assert lib.yvx_cuda_activation_quant(C.byref(a), backend.stream) == 0
            lib.yvx_cuda_event_record(last, backend.stream)
            assert lib.yvx_cuda_stream_synchronize(backend.stream) == 0, lib.yvx_cuda_last_error_text()
            ms = C.c_float()
            lib.yvx_cuda_event_elapsed_ms(first, last, C.byref(ms))
            total += ms.value
        step = total / repeats
        got, st = np.zeros((64, stride), np.float32), np.zeros(1, np.int32)
        lib.yvx_cuda_download_async(got.ctypes.data, values, got.nbytes, backend.stream)
        lib.yvx_cuda_download_async(st.ctypes.data, status, 4, backend.stream)
        lib.yvx_cuda_stream_synchronize(backend.stream)
        expected = sample.copy()
        expected[:, :count] = oracle.activation_quant(np.ascontiguousarray(sample[:, :count]), quantization, block,
                                                      hadamard)
        nbytes = n * count * 4 * 2     # every active lane read once and written once
        out[name] = {"rows": n, "kernel_ms": step, "algorithmic_bytes": nbytes,
                     "achieved_gbs": nbytes / (step * 1e-3) / 1e9,
                     "frac_of_measured_hbm": nbytes / (step * 1e-3) / 1e9 / hbm_peak,
                     "status_word": int(st[0]),
                     "sample_rows_bit_equal_to_cpu": bool(np.array_equal(got.view(np.uint32), expected.view(np.uint32)))}
        for ptr in (values, source, status):
            lib.yvx_cuda_free(ptr)
    result = {"workload": f"activation fake quantisation in place, {rows} rows of 512 lanes (448 quantised, FP8, blocks "
                          f"of 64) and {rows * 4} rows of 128 lanes (transform + FP4, blocks of 32)",
              "kernel": "activation_quant_kernel", "launches_per_step": 1,
              "l2": "each launch works on a fresh 268 MB copy of its rows", **out}
    return result, None


def bench_publish(lib, backend, abi, hbm_peak, repeats, tokens=4096):
    """Publication chain of projected rows in place: the query heads of `tokens` tokens (64 heads of 512
    lanes: unit RMS norm, bf16, rotation of the last 64 lanes, bf16) and the new local rows of 16 x as many
    tokens (512 lanes: weighted norm, bf16, rotation, bf16, FP8 activation of the 448 leading lanes)."""
    from oracle.binding import Oracle, PositionPolicy
    oracle = Oracle()
    frequency = oracle.rope_frequencies(PositionPolicy(10000, 16, 65536, 32, 1), 64)
    out = {}
    for name, rpt, n_tokens, chain in (("query_heads", 64, tokens, dict(norm_mode=1, rope_dims=64)),
                                       ("local_rows", 1, tokens * 16, dict(norm_mode=2, rope_dims=64, quantization=8,
                                                                           activation_count=448, block_width=64))):
        rows, width = rpt * n_tokens, 512
        nbytes = rows * width * 4
        dev = {k: _alloc(lib, n) for k, n in (("values", nbytes), ("source", nbytes), ("weights", width * 4),
                                              ("freq", frequency.nbytes), ("status", 4))}
        lib.yvx_cuda_fill_normal(dev["source"], abi.DTYPE_F32, rows * width, 821, 1.0, backend.stream)
        lib.yvx_cuda_fill_normal(dev["weights"], abi.DTYPE_F32, width, 822, 1.0, backend.stream)
        lib.yvx_cuda_upload_async(dev["freq"], frequency.ctypes.data, frequency.nbytes, backend.stream)
        lib.yvx_cuda_memset_async(dev["status"], 0, 4, backend.stream)
        a = abi.RowsPublishArgs()
        a.values, a.rows, a.rows_per_token, a.row_stride, a.width = dev["values"], rows, rpt, width, width
        a.norm_mode, a.norm_weights, a.epsilon = chain["norm_mode"], dev["weights"], 1e-6
        a.rope_dims, a.rope_frequency, a.start_position = 64, dev["freq"], 5000
        a.quantization, a.activation_count = chain.get("quantization", 0), chain.get("activation_count", 0)
        a.block_width, a.status = chain.get("block_width", 0), dev["status"]
        sample, weights = np.zeros((rpt * 2, width), np.float32), np.zeros(width, np.float32)
        lib.yvx_cuda_download_async(sample.ctypes.data, dev["source"], sample.nbytes, backend.stream)
        lib.yvx_cuda_download_async(weights.ctypes.data, dev["weights"], weights.nbytes, backend.stream)

        def event():
            e = C.c_void_p()
            assert lib.yvx_cuda_event_create(C.byref(e)) == 0
            return e
        first, last = event(), event()
        total = 0.0
        for i in range(repeats + 2):
            lib.yvx_cuda_copy_async(dev["values"], dev["source"], nbytes, backend.stream)
            lib.yvx_cuda_event_record(first, backend.stream)
            assert lib.yvx_cuda_rows_publish(C.byref(a), backend.stream) == 0
            lib.yvx_cuda_event_record(last, backend.stream)
            assert lib.yvx_cuda_stream_synchronize(backend.stream) == 0, lib.yvx_cuda_last_error_text()
            ms = C.c_float()
            lib.yvx_cuda_event_elapsed_ms(first, last, C.byref(ms))
            total += ms.value if i >= 2 else 0.0
        step = total / repeats
        got, st = np.zeros_like(sample), np.zeros(1, np.int32)
        lib.yvx_cuda_download_async(got.ctypes.data, dev["values"], got.nbytes, backend.stream)
        lib.yvx_cuda_download_async(st.ctypes.data, dev["status"], 4, backend.stream)
        lib.yvx_cuda_stream_synchronize(backend.stream)
        plain = {k: v for k, v in chain.items() if k in ("norm_mode", "rope_dims")}
        expected = oracle.rows_publish(sample, rpt, 5000, norm_weights=weights, rope_frequency=frequency, **plain)
        out[name] = {"rows": rows, "kernel_ms": step, "algorithmic_bytes": 2 * nbytes,
                     "achieved_gbs": 2 * nbytes / (step * 1e-3) / 1e9,
                     "frac_of_measured_hbm": 2 * nbytes / (step * 1e-3) / 1e9 / hbm_peak, "status_word": int(st[0])}
        if "quantization" not in chain:
            out[name]["lanes_differing_from_cpu_on_sample"] = int((got != expected).sum())
            out[name]["sample_lanes"] = int(got.size)
        for ptr in dev.values():
            lib.yvx_cuda_free(ptr)
    return {"workload": f"publication chain of projected rows in place: query heads of {tokens} tokens (64 x 512 lanes) "
                        f"and local rows of {tokens * 16} tokens (512 lanes, FP8 activation on 448)",
            "kernel": "rows_publish_kernel", "launches_per_step": 1,
            "l2": "each launch works on a fresh copy of its rows (537 MB)",
            "replaces": "a norm launch, a rotation launch and an activation launch per step of the chain", **out}, None


def bench_latent_sparse(lib, backend, abi, repeats, context=131072, tokens=1):
    """One decode step of a sparse shared-latent layer at the reference configuration's
    widths (64 heads x 512 with the last 64 lanes rotated, window 128, ratio 4, 64 index
    heads x 128, top-k 512) over a `context`-token history: index selection (scores in
    double precision in the reference's order + ranked top-k), then the reduce with the
    inverse rotation fused. Checked on the host against the CPU restatement: selected
    rows identical, published output within the reduce stage's tolerance."""
    import clori_b200
    from oracle.binding import Oracle, indexer_struct
    heads, hd, rope, window, ratio, ih, idim, topk = 64, 512, 64, 128, 4, 64, 128, 512
    start = context - tokens
    rows = context // ratio
    rng = np.random.default_rng(SEED + 77)
    rounded = lambda x: clori_b200.bf16_bits_to_f32(clori_b200.f32_to_bf16_bits(x.astype(np.float32)))
    host = dict(keys=rounded(rng.standard_normal((rows, idim))), iq=rounded(rng.standard_normal((tokens, ih * idim))),
                iw=rounded(rng.standard_normal((tokens, ih)) * 0.5),
                positions=np.arange(rows, dtype=np.uint64) * np.uint64(ratio),
                query=rounded(rng.standard_normal((tokens, heads * hd))),
                local=rounded(rng.standard_normal((window - 1 + tokens, hd))),
                local_positions=np.arange(start - (window - 1), start + tokens, dtype=np.uint64),
                compressed=rounded(rng.standard_normal((rows, hd))), sinks=rng.standard_normal(heads).astype(np.float32))
    policy = (10000, 16, 65536, 32, 1)
    frequency = np.zeros(rope // 2, np.float64)
    assert lib.yvex_b200_rope_frequencies(C.byref(abi.PositionPolicy(*policy)), rope, frequency.ctypes.data) == 0
    host["frequency"] = frequency
    dev = {}
    for name, array in host.items():
        dev[name] = _alloc(lib, array.nbytes)
        lib.yvx_cuda_upload_async(dev[name], array.ctypes.data, array.nbytes, backend.stream)
    out_bytes = {"scores": tokens * rows * 4, "selected": tokens * topk * 8, "count": tokens * 8, "status": 4,
                 "out": tokens * heads * hd * 4,
                 "work": int(lib.yvx_cuda_csa_select_workspace_bytes(rows, tokens, topk))}
    for name, nbytes in out_bytes.items():
        dev[name] = _alloc(lib, nbytes)
    lib.yvx_cuda_memset_async(dev["status"], 0, 4, backend.stream)
    s = abi.CsaSelectArgs()
    s.keys, s.positions, s.rows, s.key_stride = dev["keys"], dev["positions"], rows, idim
    s.query, s.weights, s.heads, s.head_dim, s.topk = dev["iq"], dev["iw"], ih, idim, topk
    s.ratio, s.phase_start_position, s.token_count = ratio, start, tokens
    s.scores, s.selected, s.selected_count = dev["scores"], dev["selected"], dev["count"]
    s.topk_capacity, s.workspace, s.status = topk, dev["work"], dev["status"]
    r = abi.LatentReduceArgs()
    r.query, r.local, r.local_positions = dev["query"], dev["local"], dev["local_positions"]
    r.initial_local_count, r.local_stride = window - 1, hd
    r.compressed, r.compressed_positions, r.compressed_stride = dev["compressed"], dev["positions"], hd
    r.selected, r.selected_count, r.topk_capacity = dev["selected"], dev["count"], topk
    r.sinks, r.query_heads, r.head_dim, r.sliding_window, r.ratio = dev["sinks"], heads, hd, window, ratio
    r.attention_class, r.phase_start_position, r.token_count = 1, start, tokens
    r.out, r.status, r.rope_dims, r.rope_frequency = dev["out"], dev["status"], rope, dev["frequency"]
    dev["reduce_work"] = _alloc(lib, max(int(lib.yvx_cuda_latent_reduce_workspace_bytes(C.byref(r))), 16))
    r.workspace = dev["reduce_work"]
    launches, reduce_launches = C.c_uint(), C.c_uint()

    def select():
        assert lib.yvx_cuda_csa_select(C.byref(s), backend.stream, C.byref(launches)) == 0, lib.yvx_cuda_last_error_text()

    def reduce():
        assert lib.yvx_cuda_latent_reduce_launches(C.byref(r), backend.stream, C.byref(reduce_launches)) == 0, \
            lib.yvx_cuda_last_error_text()

    def timed(*calls):
        first, last = C.c_void_p(), C.c_void_p()
        lib.yvx_cuda_event_create(C.byref(first)); lib.yvx_cuda_event_create(C.byref(last))
        for _ in range(3):
            for call in calls:
                call()
        lib.yvx_cuda_event_record(first, backend.stream)
        for _ in range(repeats):
            for call in calls:
                call()
        lib.yvx_cuda_event_record(last, backend.stream)
        assert lib.yvx_cuda_stream_synchronize(backend.stream) == 0, lib.yvx_cuda_last_error_text()
        ms = C.c_float()
        lib.yvx_cuda_event_elapsed_ms(first, last, C.byref(ms))
        return ms.value / repeats
    select_ms, reduce_ms, step_ms = timed(select), timed(reduce), timed(select, reduce)

    # ---- the whole device side of the step between the projections and the output projection: the
    # publication chains of the query heads, the new local row and the index queries, both rolling
    # compressors with their activation, then selection and reduce. The preparation stages work on
    # scratch rows of their own so that the CPU check of selection and reduce below stays valid.
    from oracle.binding import compressor_initial_state
    prep = {"q": tokens * heads * hd, "l": tokens * hd, "iq": tokens * ih * idim, "w": hd,
            "mkv": tokens * 2 * hd, "msc": tokens * 2 * hd, "mape": ratio * 2 * hd, "mrow": hd,
            "ikv": tokens * 2 * idim, "isc": tokens * 2 * idim, "iape": ratio * 2 * idim, "irow": idim}
    for i, (name, n) in enumerate(prep.items()):
        dev["p_" + name] = _alloc(lib, n * 4)
        lib.yvx_cuda_fill_normal(dev["p_" + name], abi.DTYPE_F32, n, 901 + i, 1.0, backend.stream)
    for name, width in (("m", hd), ("i", idim)):
        kv0, score0 = compressor_initial_state(ratio, width, 1)
        for part, array in (("skv", kv0), ("ssc", score0), ("akv", kv0), ("asc", score0)):
            dev[f"p_{name}{part}"] = _alloc(lib, array.nbytes)
            lib.yvx_cuda_upload_async(dev[f"p_{name}{part}"], array.ctypes.data, array.nbytes, backend.stream)
        lib.yvx_cuda_stream_synchronize(backend.stream)

    def publish_args(values, n_rows, rpt, width, **kw):
        a = abi.RowsPublishArgs()
        a.values, a.rows, a.rows_per_token, a.row_stride, a.width = values, n_rows, rpt, width, width
        a.epsilon, a.rope_dims, a.rope_frequency, a.start_position = 1e-6, rope, dev["frequency"], start
        a.status = dev["status"]
        for k, v in kw.items():
            setattr(a, k, v)
        return a

    def compressor_args(tag, width, row):
        a = abi.CompressorArgs()
        a.ratio, a.head_dim, a.overlap, a.start_position, a.token_count = ratio, width, 1, start, tokens
        a.token_kv, a.token_score, a.token_stride, a.ape = dev[f"p_{tag}kv"], dev[f"p_{tag}sc"], 2 * width, dev[f"p_{tag}ape"]
        a.state_kv, a.state_score = dev[f"p_{tag}skv"], dev[f"p_{tag}ssc"]
        a.after_kv, a.after_score = dev[f"p_{tag}akv"], dev[f"p_{tag}asc"]
        a.compressed, a.compressed_stride = dev[row], width
        a.norm_weights, a.epsilon, a.rope_dims, a.rope_frequency = dev["p_w"], 1e-6, rope, dev["frequency"]
        a.status = dev["status"]
        return a

    def activation_args(values, width, count, quantization, block, hadamard):
        a = abi.ActivationArgs()
        a.values, a.rows, a.row_stride, a.count = values, 1, width, count
        a.quantization, a.block_width, a.hadamard = quantization, block, hadamard
        a.hadamard_scale, a.status = float(np.float32(1.0) / np.sqrt(np.float32(count))), dev["status"]
        return a
    stages = [
        (lib.yvx_cuda_rows_publish, publish_args(dev["p_q"], tokens * heads, heads, hd, norm_mode=1)),
        (lib.yvx_cuda_rows_publish, publish_args(dev["p_l"], tokens, 1, hd, norm_mode=2, norm_weights=dev["p_w"],
                                                 quantization=8, activation_count=hd - rope, block_width=64)),
        (lib.yvx_cuda_rows_publish, publish_args(dev["p_iq"], tokens * ih, ih, idim, quantization=4,
                                                 activation_count=idim, block_width=32, hadamard=1)),
        (lib.yvx_cuda_activation_quant, activation_args(dev["p_mrow"], hd, hd - rope, 8, 64, 0)),
        (lib.yvx_cuda_activation_quant, activation_args(dev["p_irow"], idim, idim, 4, 32, 1)),
    ]
    compressors = [compressor_args("m", hd, "p_mrow"), compressor_args("i", idim, "p_irow")]
    emitted = C.c_ulonglong()

    # one launch for the three publication chains; the activation rides in each compressor's launch
    batch = (abi.RowsPublishArgs * 3)(*[a for _, a in stages[:3]])
    for a, (_, q) in zip(compressors, stages[3:]):
        a.activation_quantization, a.activation_count = q.quantization, q.count
        a.activation_block_width, a.activation_hadamard = q.block_width, q.hadamard

    def prepare():
        assert lib.yvx_cuda_rows_publish_batch(batch, 3, backend.stream) == 0, lib.yvx_cuda_last_error_text()
        for a in compressors:
            assert lib.yvx_cuda_compressor_chunk(C.byref(a), backend.stream, C.byref(emitted)) == 0, \
                lib.yvx_cuda_last_error_text()
    prepare_ms, full_ms = timed(prepare), timed(prepare, select, reduce)
    prepare_launches = 3
    graph_ms = forked_ms = None
    graph = C.c_void_p()
    if lib.yvx_cuda_graph_capture_begin(backend.stream) == 0:
        prepare(); select(); reduce()
        if lib.yvx_cuda_graph_capture_end(backend.stream, C.byref(graph)) == 0 and graph:
            graph_ms = timed(lambda: lib.yvx_cuda_graph_launch(graph, backend.stream))
            lib.yvx_cuda_graph_destroy(graph)
    # The same step captured with its data flow: the main compressor feeds only the reduce, so it runs
    # on a second stream beside publication -> index compressor -> selection and joins before the reduce.
    side, fork, join = C.c_void_p(), C.c_void_p(), C.c_void_p()
    if (lib.yvx_cuda_stream_create(C.byref(side)) == 0 and lib.yvx_cuda_event_create(C.byref(fork)) == 0 and
            lib.yvx_cuda_event_create(C.byref(join)) == 0 and lib.yvx_cuda_graph_capture_begin(backend.stream) == 0):
        main = backend.stream
        ok = lib.yvx_cuda_event_record(fork, main) == 0 and lib.yvx_cuda_stream_wait_event(side, fork) == 0
        ok = ok and lib.yvx_cuda_compressor_chunk(C.byref(compressors[0]), side, C.byref(emitted)) == 0
        ok = ok and lib.yvx_cuda_event_record(join, side) == 0
        ok = ok and lib.yvx_cuda_rows_publish_batch(batch, 3, main) == 0
        ok = ok and lib.yvx_cuda_compressor_chunk(C.byref(compressors[1]), main, C.byref(emitted)) == 0
        if ok:
            select()
        ok = ok and lib.yvx_cuda_stream_wait_event(main, join) == 0
        if ok:
            reduce()
        graph = C.c_void_p()
        if lib.yvx_cuda_graph_capture_end(main, C.byref(graph)) == 0 and graph and ok:
            forked_ms = timed(lambda: lib.yvx_cuda_graph_launch(graph, main))
            lib.yvx_cuda_graph_destroy(graph)
        lib.yvx_cuda_stream_synchronize(main)
        lib.yvx_cuda_stream_destroy(side)
    got = {name: np.zeros(shape, dtype) for name, shape, dtype in (
        ("selected", (tokens, topk), np.uint64), ("count", (tokens,), np.uint64), ("status", (1,), np.int32),
        ("out", (tokens, heads * hd), np.float32))}
    for name, array in got.items():
        lib.yvx_cuda_download_async(array.ctypes.data, dev[name], array.nbytes, backend.stream)
    lib.yvx_cuda_stream_synchronize(backend.stream)
    flops = 2.0 * tokens * rows * ih * idim
    result = {"workload": f"sparse shared-latent decode step, context {context}, {tokens} token(s): index selection over "
                          f"{rows} rows (64 index heads x 128, top-k 512) + reduce (64 heads x 512, window 128, "
                          "512 selected rows) with the inverse rotation fused",
              "kernels": "csa_score_kernel, csa_rank_rows_kernel, csa_rank_lists_kernel, latent_reduce_kernel, latent_fold_kernel",
              "launches_per_step": int(launches.value) + int(reduce_launches.value), "select_ms": select_ms, "reduce_ms": reduce_ms,
              "step_ms": step_ms, "score_fp64_tflops": flops / (select_ms * 1e-3) / 1e12,
              "prepare_ms": prepare_ms, "prepare_launches": prepare_launches,
              "prepare_stages": "publication chains of query heads, local row and index queries; main and index "
                                "rolling compressors with their activation",
              "full_step_ms": full_ms, "full_step_graph_replay_ms": graph_ms,
              "full_step_graph_replay_two_streams_ms": forked_ms,
              "score_note": "scores keep the reference's double-precision order: FP64 pipe bound, keys (%.0f MB) stay in L2"
                            % (rows * idim * 4 / 1e6),
              "status_word": int(got["status"][0])}
    oracle = Oracle()
    begin = time.perf_counter()
    ix = indexer_struct(host["keys"], host["positions"], host["iq"], host["iw"], ih, idim, topk, ratio)
    selected, counts = np.zeros((tokens, topk), np.uint64), np.zeros(tokens, np.uint64)
    for t in range(tokens):
        picked, _, _ = oracle.csa_select(ix, t, start + t)
        counts[t], selected[t, :len(picked)] = len(picked), picked
    a = abi.LatentReduceArgs()
    ptr = lambda x: x.ctypes.data
    a.query, a.local, a.local_positions = ptr(host["query"]), ptr(host["local"]), ptr(host["local_positions"])
    a.initial_local_count, a.local_stride = window - 1, hd
    a.compressed, a.compressed_positions, a.compressed_stride = ptr(host["compressed"]), ptr(host["positions"]), hd
    a.selected, a.selected_count, a.topk_capacity = ptr(selected), ptr(counts), topk
    a.sinks, a.query_heads, a.head_dim, a.sliding_window, a.ratio = ptr(host["sinks"]), heads, hd, window, ratio
    a.attention_class, a.phase_start_position, a.token_count = 1, start, tokens
    a.rope_dims, a.rope_frequency = rope, ptr(frequency)
    ref = oracle.latent_reduce_full(a, tokens, heads, hd)
    cpu_seconds = time.perf_counter() - begin
    result.update(selected_rows_equal_cpu=bool(np.array_equal(counts, got["count"]) and
                                               np.array_equal(selected, got["selected"])),
                  out_max_abs_vs_cpu=float(np.abs(ref - got["out"]).max()), cpu_port_step_ms=cpu_seconds * 1e3,
                  cpu_cores=1)
    for ptr_ in dev.values():
        lib.yvx_cuda_free(ptr_)
    return result, None


def check_mla(sample):
    from oracle.binding import Oracle
    host, o = sample
    start = time.perf_counter()
    ref = Oracle().mla_decode(host["q_nope"], host["q_rope"], host["w_uk"], host["latent"], host["rope_key"],
                              1.0 / np.sqrt(192.0))
    return float(np.abs(ref - o).max()), time.perf_counter() - start



def bench_verify_q8_sharded(lib, backend, abi, rank, world, dist, torch, repeats):
    """Config 4 across `world` GPUs: the KV sequence of ONE session is sharded in
    contiguous block-aligned ranges; every rank runs the same kernel over its shard
    (absolute positions through kv_position_base) and emits (o, m, l) per (row, head);
    one NCCL all-gather of 66 560 bytes per rank; the LSE combine folds the shards in
    rank order. Every rank fills the whole record pool identically (same seed) and
    reads only its slice, so rank 0 can also run the unsharded problem as a cross-check."""
    from clori_b200 import q8_records
    hq, hkv, hd, tokens, rows = 32, 8, 128, 131072, 4
    record = q8_records.RECORD_BYTES
    blocks = tokens // 64
    pool_bytes = blocks * hkv * record
    copies = 2
    records = _alloc(lib, copies * pool_bytes)
    q = _alloc(lib, rows * hq * hd * 2)
    status = _alloc(lib, 4)
    for i in range(copies):
        lib.yvx_cuda_fill_q8_records(records.value + i * pool_bytes, blocks * hkv, 201 + i, 0.002, 0.02, backend.stream)
    lib.yvx_cuda_fill_normal(q, abi.DTYPE_BF16, rows * hq * hd, 202, 1.0, backend.stream)
    lib.yvx_cuda_memset_async(status, 0, 4, backend.stream)
    begin, end = abi.u64(), abi.u64()
    assert lib.yvex_b200_kv_sequence_shard(tokens, world, rank, 64, C.byref(begin), C.byref(end))
    items = rows * hq
    device = torch.device("cuda", torch.cuda.current_device())
    mine = torch.zeros((items, hd + 2), dtype=torch.float32, device=device)
    gathered = torch.zeros((world, items, hd + 2), dtype=torch.float32, device=device)
    out = torch.zeros((rows, hq * hd), dtype=torch.float32, device=device)

    def problem(copy, lo, hi, partial):
        p = abi.GqaProblem()
        p.sessions, p.query_rows, p.query_heads, p.kv_heads, p.head_dim = 1, rows, hq, hkv, hd
        p.causal, p.scale = 1, 1.0 / np.sqrt(hd)
        p.query_dtype, p.kv_dtype, p.output_dtype = abi.DTYPE_BF16, abi.DTYPE_Q8_0, abi.DTYPE_F32
        p.query, p.query_row_stride, p.query_session_stride = q, hq * hd, rows * hq * hd
        p.key = records.value + copy * pool_bytes + (lo // 64) * hkv * record
        p.key_head_stride, p.key_block_stride, p.block_tokens = record, hkv * record, 64
        p.kv_tokens_uniform = p.kv_tokens_max = hi - lo
        p.query_start_uniform, p.kv_position_base = tokens - rows, lo
        if partial is not None:
            p.partial_output = partial.data_ptr()
        else:
            p.output = out.data_ptr()
        lib.yvx_cuda_gqa_plan_splits(C.byref(p), backend.sm_count)
        p.status = status
        return p
    local = [problem(i, begin.value, end.value, mine) for i in range(copies)]
    scratch = _alloc(lib, max(max(lib.yvx_cuda_gqa_partials_bytes(C.byref(p)) for p in local), 16))
    for p in local:
        p.partials = scratch

    def step(i):
        n = C.c_uint()
        rc = lib.yvx_cuda_gqa_attention(C.byref(local[i % copies]), backend.stream, C.byref(n))
        assert rc == 0, lib.yvx_cuda_last_error_text()
        dist.all_gather_into_tensor(gathered, mine)
        rc = lib.yvx_cuda_lse_combine_strided(gathered.data_ptr(), items, world, hd, hd + 2, items * (hd + 2),
                                              out.data_ptr(), abi.DTYPE_F32, status, backend.stream)
        assert rc == 0, lib.yvx_cuda_last_error_text()
        return n.value + 1
    for i in range(3):
        step(i)
    torch.cuda.synchronize()
    dist.barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(repeats):
        launches = step(i)
    stop.record()
    torch.cuda.synchronize()
    dist.barrier()
    t = torch.tensor([start.elapsed_time(stop) / repeats], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    sharded = out.clone()

    # ---- the same step without NCCL on the data path: each rank's (o, m, l) rows go to every
    # rank by peer stores over NVLink, with arrival counters and bounded waits. Twice: the
    # exchange as a second (dependent) launch, and folded into the attention kernel's own tail
    # (ONE cooperative launch per step). Each variant has its own exchange area.
    area_bytes = lib.yvx_cuda_lse_exchange_bytes(world, items, hd)
    counter_offset = lib.yvx_cuda_lse_exchange_counter_offset(world, items, hd)
    opened, owned = [], []

    def exchange_area():
        """Allocates, zeroes and maps one exchange area on every rank -> LseExchange or None."""
        area = _alloc(lib, area_bytes)
        owned.append(area)
        lib.yvx_cuda_memset_async(area, 0, area_bytes, backend.stream)
        torch.cuda.synchronize()
        handle = (C.c_ubyte * 64)()
        exported = lib.yvx_cuda_ipc_export(area, handle) == 0
        handles = [None] * world
        dist.all_gather_object(handles, bytes(handle) if exported else None)
        peers, mapped_ok = [], exported and all(h is not None for h in handles)
        for r in range(world):
            if r == rank or not mapped_ok:
                peers.append(area.value)
                continue
            mapped = C.c_void_p()
            raw = (C.c_ubyte * 64).from_buffer_copy(handles[r])
            if lib.yvx_cuda_ipc_open(raw, C.byref(mapped)) != 0:
                mapped_ok = False
                peers.append(area.value)
            else:
                peers.append(mapped.value)
                opened.append(mapped.value)
        agreed = torch.tensor([1 if mapped_ok else 0], dtype=torch.int32, device=device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed.item()) != 1:
            return None
        table = _alloc(lib, 2 * world * 8)
        owned.append(table)
        gather_host = np.array(peers, np.uint64)
        arrivals_host = gather_host + np.uint64(counter_offset)
        lib.yvx_cuda_upload_async(table, gather_host.ctypes.data, world * 8, backend.stream)
        lib.yvx_cuda_upload_async(table.value + world * 8, arrivals_host.ctypes.data, world * 8, backend.stream)
        lib.yvx_cuda_stream_synchronize(backend.stream)
        exchange = abi.LseExchange()
        exchange.ranks, exchange.rank = world, rank
        exchange.gather, exchange.arrivals = table.value, table.value + world * 8
        return exchange

    fused_out = torch.zeros((rows, hq * hd), dtype=torch.float32, device=device)
    fused = []
    for i in range(copies):
        fp = problem(i, begin.value, end.value, mine)
        fp.output = fused_out.data_ptr()
        fp.partials = scratch
        fused.append(fp)

    def exchange_run(one_launch, tagged=0):
        exchange = exchange_area()
        if exchange is None or os.environ.get("YVEX_BENCH_NO_FUSED_EXCHANGE"):
            return {"unavailable": "peer mapping of the exchange areas failed on some rank"}
        exchange.one_launch = one_launch
        exchange.tagged_words = tagged
        epoch = [0]

        def fused_step(i):
            epoch[0] += 1
            exchange.epoch = epoch[0]
            n = C.c_uint()
            rc = lib.yvx_cuda_gqa_attention_exchange(C.byref(fused[i % copies]), C.byref(exchange), backend.stream,
                                                     C.byref(n))
            assert rc == 0, lib.yvx_cuda_last_error_text()
            return n.value
        fused_out.zero_()
        torch.cuda.synchronize()
        dist.barrier()          # every area is zeroed and mapped before the first peer store
        for i in range(3):
            fused_step(i)
        torch.cuda.synchronize()
        dist.barrier()
        start.record()
        for i in range(repeats):
            fused_launches = fused_step(i)
        stop.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([start.elapsed_time(stop) / repeats], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        fused_ms = float(t.item())
        return {"ms_per_step": fused_ms, "tokens_per_s": rows / (fused_ms * 1e-3),
                "aggregate_gbs": (pool_bytes + rows * hq * hd * (2 + 4)) / (fused_ms * 1e-3) / 1e9,
                "launches_per_step": fused_launches,
                "collective": "none: peer stores of %d bytes to each rank inside the %s%s"
                              % (items * (hd + 2) * (8 if tagged else 4),
                                 "attention kernel's tail" if one_launch else "fold kernel",
                                 " as (value, epoch) words, no fence, no counter" if tagged else ""),
                "max_abs_vs_nccl_path": float((fused_out - sharded).abs().max().item())}
    fused_result = exchange_run(0)
    one_launch_result = exchange_run(1)
    fused_tagged_result = exchange_run(0, 1)
    one_launch_tagged_result = exchange_run(1, 1)
    # this rank's shard alone (no exchange, no collective): what the step adds on top of it
    shard_main_ms, shard_combine_ms, _ = _timed_launches(lib, backend, local, repeats)
    shard = torch.tensor([shard_main_ms + shard_combine_ms, _timed_launches.step_ms,
                          _timed_launches.graph_step_ms or 0.0], dtype=torch.float64, device=device)
    dist.all_reduce(shard, op=dist.ReduceOp.MAX)
    # cross-check on rank 0: the same pool copy, unsharded, on one GPU
    diff = None
    if rank == 0:
        whole = problem((repeats - 1) % copies, 0, tokens, None)
        whole_scratch = _alloc(lib, max(lib.yvx_cuda_gqa_partials_bytes(C.byref(whole)), 16))
        whole.partials = whole_scratch
        n = C.c_uint()
        assert lib.yvx_cuda_gqa_attention(C.byref(whole), backend.stream, C.byref(n)) == 0
        torch.cuda.synchronize()
        diff = float((out - sharded).abs().max().item())
        lib.yvx_cuda_free(whole_scratch)
    st = torch.zeros(1, dtype=torch.int32)
    lib.yvx_cuda_download_async(st.data_ptr(), status, 4, backend.stream)
    torch.cuda.synchronize()
    nbytes = pool_bytes + rows * hq * hd * (2 + 4)
    result = {"workload": "speculative verify, 1 session, KV 131072 sharded over %d GPUs, Q8_0 KV, 4 rows" % world,
              "n_gpus": world, "scaling": "strong", "ms_per_step": ms, "tokens_per_s": rows / (ms * 1e-3),
              "aggregate_gbs": nbytes / (ms * 1e-3) / 1e9, "launches_per_step": launches,
              "collective": "one NCCL all-gather of %d bytes per rank" % (items * (hd + 2) * 4),
              "shard_tokens": end.value - begin.value, "status_word": int(st[0]),
              "sharded_vs_single_gpu_max_abs": diff,
              "fused_exchange": fused_result, "one_launch_exchange": one_launch_result,
              "fused_tagged_exchange": fused_tagged_result, "one_launch_tagged_exchange": one_launch_tagged_result,
              "fused_tagged_step_us": fused_tagged_result.get("ms_per_step", float("nan")) * 1e3,
              "one_launch_tagged_step_us": one_launch_tagged_result.get("ms_per_step", float("nan")) * 1e3,
              "shard_alone": {"kernels_ms": float(shard[0]), "step_ms": float(shard[1]),
                              "graph_step_ms": float(shard[2]) or None},
              "ranks": world, "nccl_step_us": ms * 1e3,
              "fused_step_us": fused_result.get("ms_per_step", float("nan")) * 1e3,
              "one_launch_step_us": one_launch_result.get("ms_per_step", float("nan")) * 1e3,
              "shard_alone_us": float(shard[2] or shard[1]) * 1e3}
    dist.barrier()          # nobody unmaps while a peer may still store
    for mapped in opened:
        lib.yvx_cuda_ipc_close(C.c_void_p(mapped))
    for ptr in [records, q, status, scratch] + owned:
        lib.yvx_cuda_free(ptr)
    return result


def check_decode_f32(engine, host, threads):
    start = time.perf_counter()
    ref = engine.gqa_attention(host["q"].reshape(1, -1), host["k"].reshape(4096, -1), host["v"].reshape(4096, -1),
                               4095, 32, 8, 128, threads=threads)
    seconds = time.perf_counter() - start
    return float(np.abs(ref.reshape(-1) - host["o"]).max()), seconds


def check_verify_q8(engine, sample, threads):
    """CPU attention of KV head 0's group (4 query heads x 4 rows) over all 131072 tokens."""
    from clori_b200 import bf16_bits_to_f32, q8_records
    head0, q_bits, o = sample
    k_lane, v_lane, k_scale, v_scale = q8_records.record_offsets()
    blocks = head0.shape[0]
    def dequant(lane, scale):
        lanes = (head0[:, lane.reshape(-1)] ^ q8_records.LANE_BIAS).reshape(blocks * 64, 128).view(np.int8).astype(np.float32)
        lo = head0[:, scale.reshape(-1)].astype(np.uint16)
        hi = head0[:, (scale + 1).reshape(-1)].astype(np.uint16)
        d = (lo | (hi << 8)).view(np.float16).astype(np.float32).reshape(blocks * 64, 4)
        return lanes * np.repeat(d, 32, axis=1)
    k, v = dequant(k_lane, k_scale), dequant(v_lane, v_scale)
    q = bf16_bits_to_f32(q_bits).reshape(4, 32, 128)[:, :4].reshape(4, 4 * 128)
    start = time.perf_counter()
    ref = engine.gqa_attention(np.ascontiguousarray(q), k, v, k.shape[0] - 4, 4, 1, 128, threads=threads)
    seconds = time.perf_counter() - start
    got = o.reshape(4, 32, 128)[:, :4].reshape(4, 4 * 128)
    return float(np.abs(ref - got).max()), seconds


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


def cpu_sample_sessions(lengths):
    """Eight sessions spread over the length distribution (every eighth by rank of length,
    starting at the fourth shortest), so the sample's share of KV tokens is close to its
    share of sessions; the CPU time is scaled to the whole batch by KV tokens either way."""
    order = np.argsort(np.asarray(lengths), kind="stable")
    step = max(len(order) // 8, 1)
    return sorted(int(s) for s in order[step // 2::step][:8])


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


def pin_to_gpu_cores(device_index):
    """Runs this rank's host thread on the CPU cores NVML names as nearest to its GPU (the
    same NUMA node as the GPU's PCIe root), so that the per-step host copies of the
    end-to-end leg do not cross the socket interconnect. Reads NVML only; changes nothing
    on the GPU. A process that cannot ask (no NVML, no permission) keeps its affinity."""
    try:
        import pynvml
        pynvml.nvmlInit()
        visible = os.environ.get("CUDA_VISIBLE_DEVICES", "")
        entry = visible.split(",")[device_index].strip() if visible else ""
        if entry.startswith("GPU-"):
            handle = pynvml.nvmlDeviceGetHandleByUUID(entry)
        else:
            handle = pynvml.nvmlDeviceGetHandleByIndex(int(entry) if entry else device_index)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        cores = {64 * i + bit for i, word in enumerate(words) for bit in range(64) if word >> bit & 1}
        allowed = cores & os.sched_getaffinity(0)
        if allowed:
            os.sched_setaffinity(0, allowed)
        pynvml.nvmlShutdown()
        return sorted(allowed)
    except Exception:
        return None


def run_reference(args, rank):
    from clori_b200 import workloads
    if rank != 0:
        return
    engine, kind = cpu_engine()
    threads = os.cpu_count() or 1
    lengths = workloads.session_lengths(SEED, SESSIONS, LOW, HIGH)
    sample_ids = cpu_sample_sessions(lengths)
    sample = synth_host_sample(sample_ids, lengths, SEED)
    times = []
    for i in range(args.warmup + args.steps):
        seconds, _ = cpu_sample_run(engine, sample, threads)
        if i >= args.warmup:
            times.append(seconds)
    sample_tokens, total_tokens = int(lengths[sample_ids].sum()), int(lengths.sum())
    # one step of the whole batch = the sample's time scaled by KV tokens (the work is linear in them)
    per_step = float(np.mean(times)) * total_tokens / sample_tokens
    value = SESSIONS / per_step
    sample_text = (f"sessions {sample_ids} of {SESSIONS} ({sample_tokens} of {total_tokens} KV tokens) "
                   "per step, F32 host arrays widened from bf16; time scaled to the whole batch by KV tokens")
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
    parser.add_argument("--workload", default="headline",
                        choices=["headline", "decode_f32", "verify_q8", "prefill", "mla", "kv_append", "latent_sparse",
                                 "compressor", "activation", "publish", "prefill_f32", "verify_q8_sharded",
                                 "projections", "reference_gpu", "projections_prefill"],
                        help="run ONE of the other configurations alone and print its numbers "
                             "(for profiler captures; not the bench line)")
    parser.add_argument("--tokens", type=int, default=8192,
                        help="sequence length of --workload prefill (profiling captures)")
    parser.add_argument("--chunk", type=int, default=0,
                        help="override the split size of --workload verify_q8 (experiments)")
    parser.add_argument("--headline-only", action="store_true",
                        help="skip the other single-GPU configurations")
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

    pin_to_gpu_cores(local_rank)
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

    if args.workload != "headline":
        import clori_b200
        from clori_b200 import abi
        backend = clori_b200.Backend(local_rank)
        if args.workload == "verify_q8_sharded":
            if dist is None:
                print(json.dumps({"workload_only": args.workload, "unavailable": "needs two or more ranks"}))
                return
            import torch
            side = torch.cuda.Stream()      # kernels and the all-gather ordered on one stream
            with torch.cuda.stream(side):
                backend.bind_stream(side.cuda_stream, synchronous=False)
                result = bench_verify_q8_sharded(abi.load(), backend, abi, rank, world, dist, torch,
                                                 max(args.steps, 3))
            side.synchronize()
            if rank == 0:
                print(json.dumps({"workload_only": args.workload, **result}))
            dist.barrier()
            dist.destroy_process_group()
            return
        if args.workload == "mla":
            result, _ = bench_mla(abi.load(), backend, abi, measured_peaks()[0], max(args.steps, 3),
                                  sessions=min(args.sessions, 32))
        elif args.workload == "latent_sparse":
            result, _ = bench_latent_sparse(abi.load(), backend, abi, max(args.steps, 3))
        elif args.workload == "projections_prefill":
            result, _ = bench_projections_prefill(abi.load(), backend, abi, max(min(args.steps, 20), 3),
                                                  tokens=args.tokens if args.tokens != 8192 else 4096)
        elif args.workload == "reference_gpu":
            result = bench_reference_gpu(abi.load(), backend, abi, max(args.steps, 3) if args.steps != 200 else 5)
        elif args.workload == "projections":
            result, _ = bench_projections(abi.load(), backend, abi, measured_peaks()[0], max(args.steps, 3),
                                          tokens=max(1, min(args.tokens, 4)) if args.tokens != 8192 else 1)
        elif args.workload == "publish":
            result, _ = bench_publish(abi.load(), backend, abi, measured_peaks()[0], max(args.steps, 3),
                                      tokens=min(args.tokens // 2, 4096))
        elif args.workload == "activation":
            result, _ = bench_activation(abi.load(), backend, abi, measured_peaks()[0], max(args.steps, 3),
                                         rows=min(args.tokens * 16, 131072))
        elif args.workload == "compressor":
            result, _ = bench_compressor(abi.load(), backend, abi, measured_peaks()[0], max(args.steps, 3),
                                         tokens=min(args.tokens * 4, 32768))
        elif args.workload == "kv_append":
            result, _ = bench_kv_append(abi.load(), backend, abi, measured_peaks()[0], max(args.steps, 3),
                                        tokens=args.tokens)
        elif args.workload == "prefill":
            result, _ = bench_prefill(abi.load(), backend, abi, max(args.steps, 3), tokens=args.tokens)
        elif args.workload == "prefill_f32":
            result, _ = bench_prefill_f32(abi.load(), backend, abi, max(args.steps, 3),
                                          tokens=args.tokens if args.tokens != 8192 else 21741)
        else:
            run = {"decode_f32": bench_decode_f32, "verify_q8": bench_verify_q8}[args.workload]
            extra = {"chunk": args.chunk} if args.workload == "verify_q8" and args.chunk else {}
            result, _ = run(abi.load(), backend, abi, measured_peaks()[0], max(args.steps, 3), **extra)
        print(json.dumps({"workload_only": args.workload, **result}))
        return

    w = Workload(local_rank, SEED + 1000 * rank if world > 1 else SEED)
    lib, b = w.lib, w.backend
    legs = {}                      # leg name -> (time.time() at its start, at its end)

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
    leg_begin = time.time()
    w.record(start)
    launches = 0
    for _ in range(args.steps):
        facts = w.step()
        launches += int(facts.kernel_launches)
    w.record(stop)
    b.sync()
    legs["headline"] = (leg_begin, time.time())
    barrier()
    device_ms = max_over_ranks(w.elapsed_ms(start, stop))

    # ---- end to end: host buffers, synchronous operator --------------------
    b.bind_stream(None, synchronous=True)
    for _ in range(3):
        w.step_e2e()
    barrier()
    lib.yvx_cuda_stream_synchronize(b.stream)
    leg_begin = time.time()
    e2e_start = time.perf_counter()
    w.record(start)
    for _ in range(args.steps):
        w.step_e2e()
    w.record(stop)
    lib.yvx_cuda_stream_synchronize(b.stream)
    e2e_wall_ms = (time.perf_counter() - e2e_start) * 1e3
    legs["e2e"] = (leg_begin, time.time())
    e2e_ms = max_over_ranks(max(w.elapsed_ms(start, stop), e2e_wall_ms))
    barrier()

    # ---- the attention kernel alone ----------------------------------------
    leg_begin = time.time()
    kernel_ms, combine_ms, (chunk, splits) = w.kernel_ms(min(max(args.steps, 10), 100), args.chunk)
    legs["kernel"] = (leg_begin, time.time())
    sharded = None
    if world > 1 and not args.headline_only:
        import torch
        # The kernels and the NCCL all-gather must be ordered on ONE stream: a torch
        # side stream (the legacy default stream has no handle to bind).
        side = torch.cuda.Stream()
        leg_begin = time.time()
        with torch.cuda.stream(side):
            b.bind_stream(side.cuda_stream, synchronous=False)
            sharded = bench_verify_q8_sharded(lib, b, w.abi, rank, world, dist, torch, 20)
        side.synchronize()
        legs["cfg4_sharded"] = (leg_begin, time.time())
        b.bind_stream(None, synchronous=True)
    others, other_samples = {}, {}
    if world == 1 and not args.headline_only:
        hbm_peak = measured_peaks()[0]
        plan = (("decode_f32_config1", "f32", lambda: bench_decode_f32(lib, b, w.abi, hbm_peak, 200)),
                ("verify_q8_config4_1gpu", "q8", lambda: bench_verify_q8(lib, b, w.abi, hbm_peak, 100)),
                ("prefill_config3", "prefill", lambda: bench_prefill(lib, b, w.abi, 10)),
                ("prefill_f32_contract", "prefill_f32", lambda: bench_prefill_f32(lib, b, w.abi, 3)),
                ("latent_decode_config5", "mla", lambda: bench_mla(lib, b, w.abi, hbm_peak, 20)),
                ("projections_decode_step", "proj", lambda: bench_projections(lib, b, w.abi, hbm_peak, 20)),
                ("projections_prefill_4096", None, lambda: bench_projections_prefill(lib, b, w.abi, 5)),
                ("reference_gpu_kernels", None, lambda: (bench_reference_gpu(lib, b, w.abi), None)),
                ("kv_append_rotary", None, lambda: bench_kv_append(lib, b, w.abi, hbm_peak, 10)),
                ("latent_sparse_decode", None, lambda: bench_latent_sparse(lib, b, w.abi, 20)),
                ("rolling_compressor", None, lambda: bench_compressor(lib, b, w.abi, hbm_peak, 10)),
                ("activation_quant", None, lambda: bench_activation(lib, b, w.abi, hbm_peak, 5)),
                ("rows_publish", None, lambda: bench_publish(lib, b, w.abi, hbm_peak, 5)))
        for name, sample_key, run in plan:
            leg_begin = time.time()
            others[name], sample = run()
            legs[name] = (leg_begin, time.time())
            if sample_key:
                other_samples[sample_key] = sample
    # ---- the same step back to back for SUSTAIN_SECONDS (power-capped clocks); last, so that the
    # short legs above are not measured on a GPU this run has just heated ----
    b.bind_stream(None, synchronous=False)
    sustained_steps = max(int(SUSTAIN_SECONDS * 1e3 / (device_ms / args.steps)), args.steps)
    leg_begin = time.time()
    w.record(start)
    for _ in range(sustained_steps):
        w.step()
    w.record(stop)
    b.sync()
    legs["sustained"] = (leg_begin, time.time())
    barrier()
    sustained_ms = max_over_ranks(w.elapsed_ms(start, stop)) / sustained_steps

    sampler.stop()
    clocks = sampler.window(*legs["headline"])
    for name, result in others.items():
        result["clocks"] = {k: v for k, v in sampler.window(*legs[name]).items() if k != "sm_max_mhz"}
        # time x median SM clock (ms x MHz = thousands of cycles): comparable across runs whose clocks differ
        if result.get("kernel_ms") and result["clocks"].get("sm_mhz"):
            result["kernel_kcycles"] = result["kernel_ms"] * result["clocks"]["sm_mhz"]
    if sharded:
        sharded["clocks"] = sampler.window(*legs["cfg4_sharded"])

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
        "sustained": {"value": tokens / (sustained_ms * 1e-3), "unit": UNIT, "ms_per_step": sustained_ms,
                      "steps": sustained_steps, "seconds": sustained_ms * sustained_steps * 1e-3,
                      "hbm_gbs_whole_step": w.bytes / (sustained_ms * 1e-3) / 1e9,
                      "clocks": sampler.window(*legs["sustained"])},
        "e2e": {"value": tokens / (e2e_ms / args.steps * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms / args.steps, "clocks": sampler.window(*legs["e2e"])},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": TRAFFIC_PER_ALGORITHMIC_BYTE * w.bytes,
                     "traffic_source": "ncu dram read+write of a reduced launch (8 sessions), "
                                       "scaled by KV tokens: 1.011 x algorithmic bytes",
                     "peak_kind": peak_kind,
                     "peak_note": "the peak is a read+write copy (half reads, half writes); a kernel "
                                  "that almost only reads can exceed it",
                     "kernel": "gqa split attention (combine excluded)",
                     "kernel_ms": kernel_ms, "combine_ms": combine_ms,
                     "algorithmic_bytes": w.bytes, "frac_of_8000_spec": achieved / 8000.0,
                     "clocks": sampler.window(*legs["kernel"])},
    }
    if world == 1 and not args.no_cpu:
        engine, kind = cpu_engine()
        threads = os.cpu_count() or 1
        sample_ids = cpu_sample_sessions(w.lengths)
        sample = [w.host_session(s) for s in sample_ids]
        best, outs = None, None
        for _ in range(3):
            seconds, outs = cpu_sample_run(engine, sample, threads)
            best = seconds if best is None else min(best, seconds)
        gpu = w.cl.bf16_bits_to_f32(w.out.read())
        worst = max(float(np.abs(gpu[s, 0] - o[0]).max()) for s, o in zip(sample_ids, outs))
        sample_tokens, total_tokens = int(w.lengths[sample_ids].sum()), int(w.lengths.sum())
        whole_job_seconds = best * total_tokens / sample_tokens
        line["cpu_baseline"] = {
            "value": SESSIONS / whole_job_seconds, "unit": UNIT, "cores": threads, "kind": kind,
            "sample": f"sessions {sample_ids} of {SESSIONS} "
                      f"({sample_tokens} of {total_tokens} KV tokens), best of 3 passes, KV copied back "
                      "from the device and widened to F32; time scaled to the whole batch by KV tokens",
            "seconds": best, "whole_job_seconds_by_tokens": whole_job_seconds,
            "gpu_vs_cpu_max_abs_on_sample": worst}
        if "f32" in other_samples:
            err, seconds = check_decode_f32(engine, other_samples["f32"], threads)
            others["decode_f32_config1"].update(gpu_vs_cpu_max_abs=err, cpu_ms=seconds * 1e3, cpu_cores=threads)
        if "q8" in other_samples:
            err, seconds = check_verify_q8(engine, other_samples["q8"], threads)
            others["verify_q8_config4_1gpu"].update(
                gpu_vs_cpu_max_abs_on_sample=err, cpu_sample="KV head 0: 4 query heads x 4 rows x 131072 tokens",
                cpu_sample_ms=seconds * 1e3, cpu_cores=threads)
        if "prefill" in other_samples:
            err, seconds = check_prefill(engine, other_samples["prefill"], threads)
            others["prefill_config3"].update(
                gpu_vs_cpu_max_abs_on_sample=err, cpu_sample_ms=seconds * 1e3, cpu_cores=threads,
                cpu_sample="batch 0, query head 0: last 128 rows x 8192 tokens")
        if "prefill_f32" in other_samples:
            err, seconds = check_prefill_f32(engine, other_samples["prefill_f32"], threads)
            others["prefill_f32_contract"].update(
                gpu_vs_cpu_max_scaled_error_on_sample=err, tolerance="2e-3 * (1 + |ref|)", cpu_sample_ms=seconds * 1e3,
                cpu_sample="head 0: last 64 rows x 21741 tokens")
        if "mla" in other_samples:
            err, seconds = check_mla(other_samples["mla"])
            others["latent_decode_config5"].update(
                gpu_vs_cpu_max_abs_on_sample=err, cpu_sample_ms=seconds * 1e3, cpu_cores=1,
                cpu_sample="session 0, heads 0..7 (CPU restatement, pinned to the reference's reduce)")
    if sharded:
        others["verify_q8_config4_sharded"] = sharded
    if others:
        line["other_workloads"] = others
    # Last and compact, so a reader that keeps only the end of the line still has every
    # configuration: [kernel ms, fraction of the binding measured peak, median SM MHz, max-abs vs CPU].
    line["summary"] = summary_of(line, others)
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def _r(x, digits=4):
    return None if x is None else float(f"{x:.{digits}g}")


def summary_of(line, others):
    out = {"cfg2": {"ms": _r(line["roofline"]["kernel_ms"]), "hbm": _r(line["roofline"]["frac"], 3),
                    "burst_tok_s": _r(line["value"]), "sustained_tok_s": _r(line["sustained"]["value"]),
                    "e2e_tok_s": _r(line["e2e"]["value"]), "mhz": line["clocks"]["sm_mhz"],
                    "err": _r(line.get("cpu_baseline", {}).get("gpu_vs_cpu_max_abs_on_sample"), 2)}}
    short = (("cfg1", "decode_f32_config1", "frac_of_measured_hbm", "hbm", "gpu_vs_cpu_max_abs"),
             ("cfg4", "verify_q8_config4_1gpu", "frac_of_measured_hbm", "hbm", "gpu_vs_cpu_max_abs_on_sample"),
             ("cfg3", "prefill_config3", "frac_of_bf16_peak", "tc", "gpu_vs_cpu_max_abs_on_sample"),
             ("f32_prefill", "prefill_f32_contract", "frac_of_bf16_peak", "tc", "gpu_vs_cpu_max_scaled_error_on_sample"),
             ("cfg5", "latent_decode_config5", "frac_of_measured_hbm", "hbm", "gpu_vs_cpu_max_abs_on_sample"))
    for tag, name, frac_key, frac_tag, err_key in short:
        r = others.get(name)
        if not r:
            continue
        entry = {"ms": _r(r["kernel_ms"]), frac_tag: _r(r[frac_key], 3), "mhz": r.get("clocks", {}).get("sm_mhz"),
                 "kcyc": _r(r.get("kernel_kcycles"), 3), "err": _r(r.get(err_key), 2)}
        if "graph_step_ms" in r:
            entry["graph_ms"] = _r(r["graph_step_ms"])
        if tag == "cfg3":
            entry["tflops"] = _r(r["achieved_tflops"])
            if "sustained_tflops" in r:
                entry["sustained_tflops"] = _r(r["sustained_tflops"])
        if tag == "cfg5":
            entry["tc"] = _r(r["frac_of_bf16_peak"], 3)
            entry["step_ms"] = _r(r["absorb_ms"] + r["kernel_ms"] + r["combine_ms"])
        out[tag] = entry
    ref_gpu = others.get("reference_gpu_kernels")
    if ref_gpu and "config1_decode_f32" in ref_gpu:
        out["vs_reference_gpu"] = {k.replace("prefill_f32_2048x16q4kv_", "prefill_"): _r(v["speedup"], 3)
                                   for k, v in ref_gpu.items() if isinstance(v, dict) and "speedup" in v}
    gemm = others.get("projections_prefill_4096")
    if gemm:
        out["proj_prefill"] = {"ms": _r(gemm["step_ms"]), "tflops": _r(gemm["achieved_tflops"]),
                               "tc": _r(gemm["frac_of_bf16_peak"], 3),
                               "worst_bf16_steps": _r(gemm["sample_worst_difference_in_bf16_steps"], 2)}
    proj = others.get("projections_decode_step")
    if proj:
        out["proj"] = {k: {"us": _r((proj[k]["graph_step_ms"] or proj[k]["step_ms"]) * 1e3), "hbm": _r(proj[k]["frac_of_measured_hbm"], 3),
                           "bit_equal": proj[k]["sample_rows_bit_equal_to_cpu_dot"]} for k in ("bf16", "q8_0")}
    sharded = others.get("verify_q8_config4_sharded")
    if sharded:
        out["cfg4_sharded"] = {k: _r(v) if isinstance(v, float) else v for k, v in sharded.items()
                               if k in ("ranks", "nccl_step_us", "fused_step_us", "one_launch_step_us",
                                        "fused_tagged_step_us", "one_launch_tagged_step_us",
                                        "single_gpu_step_us", "max_abs_vs_nccl_path", "shard_alone_us")}
    return out


if __name__ == "__main__":
    main()
