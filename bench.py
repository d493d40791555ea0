#!/usr/bin/env python
"""Benchmark of the B200 provider's hot path.

Headline workload (the only one that shards): the Q8_0 sweep point R x 8192 bf16 -> Q8_0 blocks +
decoded bf16 + sum of squares, row-sharded over the ranks, per-rank sums combined by one NCCL
all-reduce.  A step is one pass over the whole tensor.  `value` is Gelem/s with the input resident
in HBM; `e2e` is the same pass from pinned HOST buffers through the C ABI (host->device and
device->host copies inside the timed region); `ops` lists the other operators' largest shapes.

    python bench.py [--gpus N] [--steps K] [--warmup W]            # this library
    python bench.py --impl reference [...]                          # the CPU provider restated, host cores
    torchrun --nproc-per-node N bench.py --gpus N ...               # one rank per GPU
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

SWEEP_COLS = 8192
DEFAULT_ROWS = 262144                       # 4 GiB of bf16: the largest sweep point
BYTES_PER_ELEMENT = 2 + 34 / 32 + 2         # read bf16, write Q8_0 block share, write decoded bf16
# dram__bytes_read.sum + dram__bytes_write.sum per element of the roundtrip kernel, from the ncu
# capture summarised in profiles/ (the rest of the 3.06 B/value of output is written back from L2 after the kernel).
NCU_TRAFFIC_BYTES_PER_ELEMENT = 4.66  # profiles/q8_0_roundtrip_R16384.md: 2.00 read + 2.66 written by kernel end
FALLBACK_HBM_GBS = 6650.0
METRIC = "Q8_0 quantise+dequantise+sum-of-squares sweep throughput"
UNIT = "Gelem/s"


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """SM clock and throttle reasons sampled every few milliseconds while the timed region runs.

    Reads only (NVML queries); nothing about the GPU is changed.  Falls back to one `nvidia-smi`
    query when the NVML binding is missing.
    """

    REASONS = {  # nvmlClocksEventReasons bits
        0x0000000000000004: "sw_power_cap",
        0x0000000000000008: "hw_slowdown",
        0x0000000000000020: "sw_thermal_slowdown",
        0x0000000000000040: "hw_thermal_slowdown",
    }

    def __init__(self, device_index: int, period_s: float = 0.005):
        self.device_index = device_index
        self.period_s = period_s
        self.samples, self.reason_bits, self.max_clock = [], 0, None
        self._stop = None
        self._thread = None
        self._nvml = None

    def _physical_index(self) -> int:
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        if visible:
            entries = [e.strip() for e in visible.split(",") if e.strip()]
            if self.device_index < len(entries) and entries[self.device_index].isdigit():
                return int(entries[self.device_index])
        return self.device_index

    def start(self):
        import threading
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.max_clock = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nvml = None
            return
        self._nvml = pynvml
        self._stop = threading.Event()

        def loop():
            while not self._stop.is_set():
                try:
                    self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)))
                    self.reason_bits |= int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle))
                except Exception:
                    pass
                self._stop.wait(self.period_s)

        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()

    def stop(self):
        if self._nvml is None:
            return self._smi_once()
        self._stop.set()
        self._thread.join(timeout=2)
        reasons = sorted(name for bit, name in self.REASONS.items() if self.reason_bits & bit)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_clock,
                "reasons": reasons, "samples": len(self.samples), "source": "nvml"}

    def _smi_once(self):
        try:
            out = subprocess.run(["nvidia-smi", "--query-gpu=clocks.sm,clocks.max.sm", "--format=csv,noheader,nounits",
                                  "-i", str(self.device_index)], capture_output=True, text=True, timeout=20).stdout
            clock, maximum = [float(v) for v in out.strip().splitlines()[0].split(",")]
            return {"sm_mhz": clock, "sm_max_mhz": maximum, "reasons": [], "samples": 1, "source": "nvidia-smi after the run"}
        except Exception:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock query unavailable"], "samples": 0}


# ---------------------------------------------------------------------------------------------------------
# reference arm: the CPU restatement of the provider's Q8_0 path on the host cores
# ---------------------------------------------------------------------------------------------------------
def cpu_sample_rows(oracle, target_seconds: float, max_rows: int) -> int:
    """Rows of the sweep tensor the CPU gets through in about `target_seconds` (power of two)."""
    from hyle_b200 import workloads as wl

    probe_rows = 256
    w = wl.q8_sweep_inputs(probe_rows)
    oracle.q8_0_roundtrip(w)
    t0 = time.perf_counter()
    oracle.q8_0_roundtrip(w)
    per_row = (time.perf_counter() - t0) / probe_rows
    rows = probe_rows
    while rows * 2 * per_row <= target_seconds and rows * 2 <= max_rows:
        rows *= 2
    return rows


def time_cpu(oracle, rows: int, steps: int, warmup: int):
    from hyle_b200 import workloads as wl

    w = np.tile(wl.q8_sweep_inputs(min(rows, 1024)), (max(1, rows // 1024), 1))[:rows]
    blocks = np.empty(w.size // 32 * 34, np.uint8)
    decoded = np.empty(w.size, np.uint16)
    for _ in range(warmup):
        oracle.q8_0_roundtrip(w, blocks, decoded)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.q8_0_roundtrip(w, blocks, decoded)
    seconds = (time.perf_counter() - t0) / steps
    return w.size / seconds / 1e9, seconds


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return  # the CPU arm is one process on the host cores
    from oracle.binding import Oracle

    oracle = Oracle()
    cores = os.cpu_count() or 1
    oracle.set_threads(cores)
    total_steps = max(1, args.steps + args.warmup)
    rows = cpu_sample_rows(oracle, target_seconds=max(0.5, 120.0 / total_steps), max_rows=args.rows)
    value, seconds = time_cpu(oracle, rows, args.steps, args.warmup)
    sample = f"{rows} of {args.rows} rows x {SWEEP_COLS} per step ({rows * SWEEP_COLS * 2 / 2**20:.0f} MiB of bf16)"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16->q8_0(int8+f16)", "data": "synthetic",
        "config": {"workload": f"Q8_0 sweep R={args.rows} x {SWEEP_COLS} bf16 (CPU sample: {sample})",
                   "l2": "working set larger than the host caches"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------
# this library
# ---------------------------------------------------------------------------------------------------------
def event_pairs_ms(pairs):
    return [a.elapsed_time(b) for a, b in pairs]


def time_op(torch, launch, sets: int, iterations: int = 40, warmup: int = 5):
    """Average device time of `launch(i)` over rotating buffer sets (footprint >> L2), CUDA events."""
    for i in range(warmup):
        code = launch(i % sets)
        if code not in (None, 0):
            raise RuntimeError(f"a timed entry point returned {code}")
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(iterations):
        launch(i % sets)
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / iterations


def other_ops(torch, peak_gbs, only=None, iterations=40):
    """Largest single-GPU shape of workloads 1-4: GB/s against algorithmic bytes, rotating inputs.

    `only` restricts the run to some operators (for profiling one kernel on a short command)."""
    from hyle_b200 import abi, ops

    results = []
    dev = "cuda"
    lib, stream = abi.load(), torch.cuda.current_stream().cuda_stream

    def wanted(name):
        return only is None or name in only

    def report(name, shape, elements, algorithmic_bytes, ms, sets):
        gbs = algorithmic_bytes / (ms * 1e-3) / 1e9
        results.append({"op": name, "shape": shape, "us": ms * 1e3, "GB/s": gbs, "Gelem/s": elements / (ms * 1e-3) / 1e9,
                        "roofline_frac": gbs / peak_gbs, "algorithmic_bytes": algorithmic_bytes,
                        "buffer_sets": sets})

    # 1: f32 broadcast add + row sum + row max, 4096 x 4096
    if wanted("add_bias_row_sum_max_f32"):
        sets = 8
        a = [torch.randn(4096, 4096, device=dev) for _ in range(sets)]
        bias = torch.rand(4096, device=dev) * 2 - 1
        c = [torch.empty_like(a[0]) for _ in range(sets)]
        rs, rm = torch.empty(4096, device=dev), torch.empty(4096, device=dev)
        ms = time_op(torch, lambda i: lib.hyle_b200_add_bias_row_sum_max_f32(
            stream, a[i].data_ptr(), bias.data_ptr(), c[i].data_ptr(), rs.data_ptr(), rm.data_ptr(), 4096, 4096),
            sets, iterations)
        report("add_bias_row_sum_max_f32", "4096x4096", 4096 * 4096, 2 * 4096 * 4096 * 4 + 3 * 4096 * 4, ms, sets)
        del a, c

    # 2: bf16 residual add + RMSNorm, T = 4096, hidden 2048
    if wanted("add_rms_norm_bf16"):
        sets = 16
        x = [torch.randn(4096, 2048, device=dev).bfloat16() for _ in range(sets)]
        r = [torch.randn(4096, 2048, device=dev).bfloat16() for _ in range(sets)]
        w = (torch.rand(2048, device=dev) + 0.5).bfloat16()
        y = [torch.empty_like(x[0]) for _ in range(sets)]
        h = [torch.empty_like(x[0]) for _ in range(sets)]
        ms = time_op(torch, lambda i: lib.hyle_b200_add_rms_norm_bf16(
            stream, x[i].data_ptr(), r[i].data_ptr(), w.data_ptr(), abi.BF16, y[i].data_ptr(), h[i].data_ptr(),
            4096, 2048, 1e-6), sets, iterations)
        report("add_rms_norm_bf16", "4096x2048", 4096 * 2048, 4 * 4096 * 2048 * 2 + 2048 * 2, ms, sets)
        del x, r, y, h

    # 3: bf16 SwiGLU, T = 4096, 6144 columns
    if wanted("swiglu_bf16"):
        sets = 8
        g = [(1.5 * torch.randn(4096, 6144, device=dev)).bfloat16() for _ in range(sets)]
        u = [(1.5 * torch.randn(4096, 6144, device=dev)).bfloat16() for _ in range(sets)]
        o = [torch.empty_like(g[0]) for _ in range(sets)]
        ms = time_op(torch, lambda i: lib.hyle_b200_swiglu_bf16(
            stream, g[i].data_ptr(), u[i].data_ptr(), o[i].data_ptr(), 4096, 6144, 6144, 6144), sets, iterations)
        report("swiglu_bf16", "4096x6144", 4096 * 6144, 3 * 4096 * 6144 * 2, ms, sets)
        del g, u, o

    # the widened elementwise catalogue on the same shapes: one Unary and one Binary kind per storage type
    if wanted("unary_binary"):
        sets = 8
        x32 = [torch.randn(4096, 4096, device=dev) for _ in range(sets)]
        y32 = [torch.empty_like(x32[0]) for _ in range(sets)]
        for name, kind in (("unary_tanh_f32", abi.UNARY_TANH), ("unary_gelu_f32", abi.UNARY_GELU)):
            ms = time_op(torch, lambda i: lib.hyle_b200_unary(
                stream, kind, abi.F32, x32[i].data_ptr(), y32[i].data_ptr(), 4096 * 4096), sets, iterations)
            report(name, "4096x4096", 4096 * 4096, 2 * 4096 * 4096 * 4, ms, sets)
        ms = time_op(torch, lambda i: lib.hyle_b200_binary(
            stream, abi.BINARY_DIVIDE, abi.F32, x32[i].data_ptr(), x32[(i + 1) % sets].data_ptr(), y32[i].data_ptr(),
            4096 * 4096, 4096 * 4096), sets, iterations)
        report("binary_divide_f32", "4096x4096", 4096 * 4096, 3 * 4096 * 4096 * 4, ms, sets)
        del x32, y32
        x16 = [(torch.randn(4096, 6144, device=dev) * 1.5).to(torch.bfloat16) for _ in range(sets)]
        y16 = [torch.empty_like(x16[0]) for _ in range(sets)]
        for name, kind in (("unary_silu_bf16", abi.UNARY_SILU), ("unary_gelu_tanh_bf16", abi.UNARY_GELU_TANH)):
            ms = time_op(torch, lambda i: lib.hyle_b200_unary(
                stream, kind, abi.BF16, x16[i].data_ptr(), y16[i].data_ptr(), 4096 * 6144), sets, iterations)
            report(name, "4096x6144", 4096 * 6144, 2 * 4096 * 6144 * 2, ms, sets)
        ms = time_op(torch, lambda i: lib.hyle_b200_binary(
            stream, abi.BINARY_MAXIMUM, abi.BF16, x16[i].data_ptr(), x16[(i + 1) % sets].data_ptr(), y16[i].data_ptr(),
            4096 * 6144, 4096 * 6144), sets, iterations)
        report("binary_maximum_bf16", "4096x6144", 4096 * 6144, 3 * 4096 * 6144 * 2, ms, sets)
        del x16, y16

    # LayerNorm, Cast, FP8 cache encode and the sampling operators
    if wanted("norm_cast_sampling"):
        sets = 8
        x16 = [torch.randn(4096, 2048, device=dev).to(torch.bfloat16) for _ in range(sets)]
        y16 = [torch.empty_like(x16[0]) for _ in range(sets)]
        scale = (torch.rand(2048, device=dev) + 0.5).to(torch.bfloat16)
        bias = torch.randn(2048, device=dev).to(torch.bfloat16)
        ms = time_op(torch, lambda i: lib.hyle_b200_layer_norm_bf16(
            stream, x16[i].data_ptr(), scale.data_ptr(), bias.data_ptr(), y16[i].data_ptr(), 4096, 2048, 1e-5), sets, iterations)
        report("layer_norm_bf16", "4096x2048", 4096 * 2048, 2 * 4096 * 2048 * 2, ms, sets)
        del x16, y16
        x32 = [torch.randn(4096, 4096, device=dev) for _ in range(sets)]
        codes = [torch.empty(4096, 4096, dtype=torch.uint8, device=dev) for _ in range(sets)]
        ms = time_op(torch, lambda i: lib.hyle_b200_cast(
            stream, abi.F32, abi.E4M3, x32[i].data_ptr(), codes[i].data_ptr(), 4096 * 4096), sets, iterations)
        report("cast_f32_to_e4m3", "4096x4096", 4096 * 4096, 4096 * 4096 * 5, ms, sets)
        ms = time_op(torch, lambda i: lib.hyle_b200_fp8_e4m3_encode(
            stream, abi.F32, x32[i].data_ptr(), 4096 * 4096, 0.37, codes[i].data_ptr(), None), sets, iterations)
        report("fp8_e4m3_encode_f32", "4096x4096", 4096 * 4096, 4096 * 4096 * 5, ms, sets)
        ms = time_op(torch, lambda i: lib.hyle_b200_cast(
            stream, abi.E4M3, abi.F32, codes[i].data_ptr(), x32[i].data_ptr(), 4096 * 4096), sets, iterations)
        report("cast_e4m3_to_f32", "4096x4096", 4096 * 4096, 4096 * 4096 * 5, ms, sets)
        del x32, codes
        identities = torch.randint(-2 ** 31, 2 ** 31 - 1, (4096, 4), dtype=torch.int32, device=dev)
        words = [torch.empty(4096, 4096, dtype=torch.int32, device=dev) for _ in range(sets)]
        ms = time_op(torch, lambda i: lib.hyle_b200_random_bits(
            stream, identities.data_ptr(), 4096, 4096, words[i].data_ptr()), sets, iterations)
        report("random_bits", "4096x4096 words", 4096 * 4096, 4096 * 4096 * 4, ms, sets)
        del words
        rows, cols = 256, 151936
        logits = [4.0 * torch.randn(rows, cols, device=dev) for _ in range(2)]
        ids = torch.randint(-2 ** 31, 2 ** 31 - 1, (rows, 4), dtype=torch.int32, device=dev)
        picked, logp = torch.empty(rows, dtype=torch.int32, device=dev), torch.empty(rows, device=dev)
        ms = time_op(torch, lambda i: lib.hyle_b200_categorical(
            stream, abi.F32, logits[i].data_ptr(), ids.data_ptr(), rows, cols, picked.data_ptr(), logp.data_ptr(), None),
            2, max(1, iterations // 2))
        report("categorical_f32", "256x151936", rows * cols, rows * cols * 4, ms, 2)
        del logits

    # Select, the masked f16 Softmax, and the gather-and-cast of strided views
    if wanted("select_softmax_strided"):
        import ctypes

        sets = 4
        n = 4096 * 4096
        cond = [(torch.rand(n, device=dev) < 0.5).to(torch.uint8) for _ in range(sets)]
        a = [torch.randn(n, device=dev) for _ in range(sets)]
        b = [torch.randn(n, device=dev) for _ in range(sets)]
        y = [torch.empty(n, device=dev) for _ in range(sets)]
        ms = time_op(torch, lambda i: lib.hyle_b200_select(
            stream, abi.F32, cond[i].data_ptr(), a[i].data_ptr(), b[i].data_ptr(), y[i].data_ptr(), n, n, n), sets, iterations)
        report("select_f32", "4096x4096, both branches full", n, n * 13, ms, sets)
        del cond, a, b, y
        rows, cols = 32768, 2048  # 16 heads x 2048 queries x 2048 keys, one causal mask for all heads
        scores = [torch.randn(rows, cols, device=dev).to(torch.float16) for _ in range(sets)]
        probs = [torch.empty_like(scores[0]) for _ in range(sets)]
        mask = torch.tril(torch.ones(cols, cols, dtype=torch.uint8, device=dev)).contiguous()
        ms = time_op(torch, lambda i: lib.hyle_b200_masked_softmax_f16(
            stream, scores[i].data_ptr(), mask.data_ptr(), mask.numel(), 0.125, probs[i].data_ptr(), rows, cols), sets, iterations)
        report("masked_softmax_f16", "32768x2048, causal mask 2048x2048", rows * cols, rows * cols * 4 + mask.numel(), ms, sets)
        del scores, probs, mask
        side = 4096
        x = [torch.randn(side, side, device=dev) for _ in range(sets)]
        y = [torch.empty(side, side, device=dev) for _ in range(sets)]
        dims = (ctypes.c_int64 * 2)(side, side)
        transposed = (ctypes.c_int64 * 2)(4, 4 * side)
        ms = time_op(torch, lambda i: lib.hyle_b200_strided_cast(
            stream, abi.F32, abi.F32, x[i].data_ptr(), y[i].data_ptr(), 2, dims, transposed), sets, iterations)
        report("strided_copy_f32_transpose", "4096x4096 read through a transposed view", side * side, side * side * 8, ms, sets)
        half = (ctypes.c_int64 * 2)(side, side // 2)
        sliced = (ctypes.c_int64 * 2)(4 * side, 4)
        y16 = [torch.empty(side, side // 2, dtype=torch.bfloat16, device=dev) for _ in range(sets)]
        ms = time_op(torch, lambda i: lib.hyle_b200_strided_cast(
            stream, abi.F32, abi.BF16, x[i].data_ptr(), y16[i].data_ptr(), 2, half, sliced), sets, iterations)
        report("strided_cast_f32_to_bf16_slice", "4096x2048 slice of 4096x4096 rows", side * side // 2, side * side // 2 * 6, ms, sets)
        del x, y, y16

    # Scan{axis=-1}: f32 over vocabulary rows and over 4096 x 4096; i32 (two passes: check, then write)
    if wanted("scan"):
        for rows, cols, sets in ((256, 151936, 2), (4096, 4096, 4)):
            x = [torch.randn(rows, cols, device=dev) for _ in range(sets)]
            y = [torch.empty_like(x[0]) for _ in range(sets)]
            ms = time_op(torch, lambda i: lib.hyle_b200_scan(
                stream, abi.F32, x[i].data_ptr(), y[i].data_ptr(), rows, cols, 0, None), sets, iterations)
            report("scan_f32", f"{rows}x{cols}", rows * cols, rows * cols * 8, ms, sets)
            del x, y
        sets = 4
        n = [torch.randint(-1000, 1000, (4096, 4096), dtype=torch.int32, device=dev) for _ in range(sets)]
        m = [torch.empty_like(n[0]) for _ in range(sets)]
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        ms = time_op(torch, lambda i: lib.hyle_b200_scan(
            stream, abi.I32, n[i].data_ptr(), m[i].data_ptr(), 4096, 4096, 0, status.data_ptr()), sets, iterations)
        report("scan_i32_checked", "4096x4096", 4096 * 4096, 4096 * 4096 * 8, ms, sets)
        del n, m

    # Paged append: 4096 new Q8_0 rows of 8192 values (8704 bytes) into 256 pages of 16 rows
    if wanted("paged_append"):
        sets, page_rows, pages, new_count, row_bytes = 4, 16, 1024, 4096, 8704
        arenas = [torch.zeros(pages * page_rows, row_bytes, dtype=torch.uint8, device=dev) for _ in range(sets)]
        fresh = [torch.randint(0, 256, (new_count, row_bytes), dtype=torch.uint8, device=dev) for _ in range(sets)]
        order = torch.randperm(pages)[: new_count // page_rows].tolist()
        episode = ops.paged_append_metadata([(0, 0, i * page_rows, page, 0, page_rows) for i, page in enumerate(order)],
                                            new_count // page_rows, dev)
        ms = time_op(torch, lambda i: lib.hyle_b200_paged_append(
            stream, arenas[i].data_ptr(), fresh[i].data_ptr(), episode.data_ptr(), page_rows, pages, new_count,
            new_count // page_rows, row_bytes), sets, iterations)
        report("paged_append", "4096 rows x 8704 B into 16-row pages", new_count, 2 * new_count * row_bytes, ms, sets)
        # the same rows through the device-lengths variant: 32 requests of 128 new rows after 24 old ones
        requests, per_request, history = 32, new_count // 32, 24
        words = np.zeros(4 + 8 * (1 + requests + 320), dtype=np.uint32)
        spare = torch.randperm(pages // 2).tolist()
        records = []
        for r in range(requests):
            words[12 + 8 * r: 16 + 8 * r] = (per_request, history, history, history + per_request)
            for logical in range(history // page_rows, (history + per_request - 1) // page_rows + 1):
                inherited = max(0, min(page_rows, history - logical * page_rows))
                records.append((r, logical, spare.pop(), page_rows, pages // 2 + r if inherited else 0xFFFFFFFF, inherited))
        words[0], words[4], words[5] = 1 + requests + len(records), requests, len(records)
        for i, record in enumerate(records):
            words[12 + 8 * (requests + i): 18 + 8 * (requests + i)] = record
        episode = torch.from_numpy(words.view(np.int32)).to(dev)
        q = torch.full((requests,), per_request, dtype=torch.int32, device=dev)
        kv = torch.full((requests,), history + per_request, dtype=torch.int32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        ms = time_op(torch, lambda i: lib.hyle_b200_paged_append_device_lengths(
            stream, arenas[i].data_ptr(), fresh[i].data_ptr(), episode.data_ptr(), q.data_ptr(), kv.data_ptr(), page_rows,
            pages, new_count, (words.size - 4) // 8, row_bytes, requests, status.data_ptr()), sets, iterations)
        assert int(status.item()) == 0
        moved = sum(record[3] for record in records) * row_bytes  # every initialised row is written once
        read = (new_count + sum(record[5] for record in records)) * row_bytes
        report("paged_append_device_lengths", "32 requests x 128 new rows x 8704 B, 16-row pages", new_count, moved + read, ms, sets)
        del arenas, fresh

    # 4: f32 logits -> lse, softmax bf16, argmax, B = 256, vocabulary 151936
    if wanted("logits_reduce_f32"):
        sets = 4
        rows, cols = 256, 151936
        logits = [4.0 * torch.randn(rows, cols, device=dev) for _ in range(sets)]
        probs = [torch.empty(rows, cols, dtype=torch.bfloat16, device=dev) for _ in range(sets)]
        lse = torch.empty(rows, device=dev)
        idx = torch.empty(rows, dtype=torch.int32, device=dev)
        val = torch.empty(rows, device=dev)
        scratch = ops.make_logits_workspace(dev, rows, cols)
        ms = time_op(torch, lambda i: lib.hyle_b200_logits_reduce_f32(
            stream, logits[i].data_ptr(), rows, cols, lse.data_ptr(), probs[i].data_ptr(), idx.data_ptr(),
            val.data_ptr(), scratch.data_ptr(), scratch.numel(), None), sets, max(1, iterations // 2))
        report("logits_reduce_f32", "256x151936", rows * cols, rows * cols * 6 + rows * 12, ms, sets)
        if os.environ.get("HYLE_B200_LOGITS_CLUSTER_KERNEL"):  # the other kernel, for comparison
            ms = time_op(torch, lambda i: lib.hyle_b200_logits_reduce_f32(
                stream, logits[i].data_ptr(), rows, cols, lse.data_ptr(), probs[i].data_ptr(), idx.data_ptr(),
                val.data_ptr(), None, 0, None), sets, max(1, iterations // 2))
            report("logits_reduce_f32_cluster_kernel", "256x151936", rows * cols, rows * cols * 6 + rows * 12, ms, sets)
        del logits, probs, scratch
    torch.cuda.empty_cache()
    return results


def sweep(torch, dist, ops, abi, wl, world: int, rank: int, peak_gbs: float, reducer, peers, iterations: int = 20):
    """The whole sweep R = 1024 ... 262144 (16 MiB ... 4 GiB of bf16), row-sharded over the ranks:
    per point the step time (kernel + all-reduce, max over ranks), Gelem/s and GB/s per GPU."""
    points = []
    lib = abi.load()
    stream = torch.cuda.current_stream().cuda_stream
    workspace = ops.make_workspace("cuda", (wl.SWEEP_ROWS[-1] + world - 1) // world * SWEEP_COLS)
    partial = torch.zeros(1, dtype=torch.float64, device="cuda")
    for total_rows in wl.SWEEP_ROWS:
        shard = wl.shard_rows(total_rows, world, rank)
        # small points rotate over several buffers so that no launch finds its input in L2
        sets = max(1, min(8, int(600e6 // max(1, shard.rows * SWEEP_COLS * 2))))
        w = [wl.q8_sweep_device_shard(shard) for _ in range(sets)]
        count = w[0].numel()
        blocks = [torch.empty(ops.q8_0_bytes(count), dtype=torch.uint8, device="cuda") for _ in range(sets)]
        decoded = [torch.empty_like(w[0]) for _ in range(sets)]

        def one(i):
            if peers is not None:
                abi.check("roundtrip_exchange", lib.hyle_b200_q8_0_roundtrip_bf16_exchange(
                    stream, w[i % sets].data_ptr(), count, blocks[i % sets].data_ptr(), decoded[i % sets].data_ptr(),
                    partial.data_ptr(), None, workspace.data_ptr(), workspace.numel(), peers.pointers, world, rank,
                    peers.next_epoch(), 0))
                return
            abi.check("roundtrip", lib.hyle_b200_q8_0_roundtrip_bf16(
                stream, w[i % sets].data_ptr(), count, blocks[i % sets].data_ptr(), decoded[i % sets].data_ptr(),
                partial.data_ptr(), None, workspace.data_ptr(), workspace.numel()))
            if reducer is not None:
                reducer.sum_f64(partial, stream)

        for i in range(3):
            one(i)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(iterations):
            one(i)
        stop.record()
        torch.cuda.synchronize()
        ms = torch.tensor([start.elapsed_time(stop) / iterations], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        seconds = float(ms.item()) * 1e-3
        elements = total_rows * SWEEP_COLS
        gbs_per_gpu = BYTES_PER_ELEMENT * count / seconds / 1e9
        points.append({"rows": total_rows, "MiB_in": elements * 2 // 2**20, "us_per_step": seconds * 1e6,
                       "Gelem/s": elements / seconds / 1e9, "GB/s_per_gpu": gbs_per_gpu,
                       "roofline_frac": gbs_per_gpu / peak_gbs, "buffer_sets": sets})
        del w, blocks, decoded
        torch.cuda.empty_cache()
    return points


def run_e2e(torch, ops, abi, shard_rows: int, steps: int, warmup: int):
    """One pass from pinned host buffers: chunks flow host -> device -> kernel -> host on rotating
    streams so both copy directions and the kernels overlap."""
    chunk_rows = min(shard_rows, 4096)                     # 64 MiB of bf16 per chunk
    chunks = (shard_rows + chunk_rows - 1) // chunk_rows
    lanes = min(3, chunks)
    host_in = torch.empty((shard_rows, SWEEP_COLS), dtype=torch.bfloat16, pin_memory=True)
    host_in.copy_(torch.randn(1024, SWEEP_COLS).mul_(0.02).bfloat16().repeat((shard_rows + 1023) // 1024, 1)[:shard_rows])
    host_blocks = torch.empty(shard_rows * SWEEP_COLS // 32 * 34, dtype=torch.uint8, pin_memory=True)
    host_decoded = torch.empty((shard_rows, SWEEP_COLS), dtype=torch.bfloat16, pin_memory=True)
    host_sums = torch.empty(chunks, dtype=torch.float64, pin_memory=True)
    streams = [torch.cuda.Stream() for _ in range(lanes)]
    dev_in = [torch.empty((chunk_rows, SWEEP_COLS), dtype=torch.bfloat16, device="cuda") for _ in range(lanes)]
    dev_blocks = [torch.empty(chunk_rows * SWEEP_COLS // 32 * 34, dtype=torch.uint8, device="cuda") for _ in range(lanes)]
    dev_decoded = [torch.empty((chunk_rows, SWEEP_COLS), dtype=torch.bfloat16, device="cuda") for _ in range(lanes)]
    dev_sums = torch.zeros(chunks, dtype=torch.float64, device="cuda")
    workspaces = [ops.make_workspace("cuda", chunk_rows * SWEEP_COLS) for _ in range(lanes)]
    lib = abi.load()
    block_bytes_per_row = SWEEP_COLS // 32 * 34

    def one_pass():
        for c in range(chunks):
            lane = c % lanes
            first = c * chunk_rows
            rows = min(chunk_rows, shard_rows - first)
            with torch.cuda.stream(streams[lane]):
                dev_in[lane][:rows].copy_(host_in[first:first + rows], non_blocking=True)
                abi.check("roundtrip", lib.hyle_b200_q8_0_roundtrip_bf16(
                    streams[lane].cuda_stream, dev_in[lane].data_ptr(), rows * SWEEP_COLS, dev_blocks[lane].data_ptr(),
                    dev_decoded[lane].data_ptr(), dev_sums[c:].data_ptr(), None, workspaces[lane].data_ptr(),
                    workspaces[lane].numel()))
                host_blocks[first * block_bytes_per_row:(first + rows) * block_bytes_per_row].copy_(
                    dev_blocks[lane][:rows * block_bytes_per_row], non_blocking=True)
                host_decoded[first:first + rows].copy_(dev_decoded[lane][:rows], non_blocking=True)
        for s in streams:
            s.synchronize()
        host_sums.copy_(dev_sums)
        return float(host_sums.sum())

    for _ in range(warmup):
        one_pass()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        total = one_pass()
    torch.cuda.synchronize()
    seconds = (time.perf_counter() - t0) / steps
    h2d = shard_rows * SWEEP_COLS * 2
    d2h = shard_rows * block_bytes_per_row + shard_rows * SWEEP_COLS * 2 + chunks * 8
    return seconds, h2d, d2h, total


def run_ops_only(args):
    """Time only the named operators of workloads 1-4 (short command for profiling one kernel)."""
    import torch

    from hyle_b200 import abi

    torch.cuda.set_device(0)
    abi.load()
    peak_gbs, peak_kind = hbm_peak()
    names = set(args.ops_only.split(","))
    print(json.dumps({"ops": other_ops(torch, peak_gbs, names, args.steps), "peak_gbs": peak_gbs,
                      "peak_kind": peak_kind}), flush=True)


def run_gpu(args):
    import torch
    import torch.distributed as dist

    from hyle_b200 import abi, ops
    from hyle_b200 import workloads as wl

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("for --gpus N > 1 launch with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N ...")
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    abi.load()  # fails loudly when libhyle_b200.so is missing

    peak_gbs, peak_kind = hbm_peak()
    shard = wl.shard_rows(args.rows, world, rank)
    w = wl.q8_sweep_device_shard(shard)
    count = w.numel()
    blocks = torch.empty(ops.q8_0_bytes(count), dtype=torch.uint8, device="cuda")
    decoded = torch.empty_like(w)
    partial = torch.zeros(1, dtype=torch.float64, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    workspace = ops.make_workspace("cuda", count)
    lib = abi.load()
    stream = torch.cuda.current_stream().cuda_stream

    # The one exchange of the path: 8 bytes per rank.  "fused": the kernel's finishing CTA writes
    # them into the peers' mailboxes over NVLink and adds what it receives (one kernel per step).
    # "nccl": kernel, then ncclAllReduce on the same stream.
    reducer, peers, exchange = None, None, "none"
    if world > 1:
        from hyle_b200.collective import PeerExchange, PeerMappingUnavailable, StreamAllReduce

        if args.exchange == "fused":
            try:
                peers = PeerExchange()
                exchange = "fused into the kernel: 8-byte stores to peer mailboxes over NVLink, summed in rank order"
            except PeerMappingUnavailable as problem:  # raised on every rank together
                exchange = f"ncclAllReduce of one f64 on the kernels' stream (peer mapping unavailable: {problem})"
        if peers is None:
            reducer = StreamAllReduce()
            if args.exchange != "fused":
                exchange = "ncclAllReduce of one f64 on the kernels' stream"

    def step():
        if peers is not None:
            abi.check("roundtrip_exchange", lib.hyle_b200_q8_0_roundtrip_bf16_exchange(
                stream, w.data_ptr(), count, blocks.data_ptr(), decoded.data_ptr(), partial.data_ptr(),
                status.data_ptr(), workspace.data_ptr(), workspace.numel(), peers.pointers, world, rank,
                peers.next_epoch(), 0))
        else:
            abi.check("roundtrip", lib.hyle_b200_q8_0_roundtrip_bf16(
                stream, w.data_ptr(), count, blocks.data_ptr(), decoded.data_ptr(), partial.data_ptr(),
                status.data_ptr(), workspace.data_ptr(), workspace.numel()))

    def combine():
        if reducer is not None:
            reducer.sum_f64(partial, stream)

    for _ in range(args.warmup):
        step()
        combine()
    torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    kernel_events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for k in range(args.steps):
        kernel_events[k][0].record()
        step()
        kernel_events[k][1].record()
        combine()
    stop.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    elapsed_ms = torch.tensor([start.elapsed_time(stop)], dtype=torch.float64, device="cuda")
    kernel_ms = torch.tensor([statistics.mean(event_pairs_ms(kernel_events))], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(elapsed_ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(kernel_ms, op=dist.ReduceOp.MAX)
    clocks = sampler.stop() if rank == 0 else None
    sum_squares = float(partial.item())
    if int(status.item()) != 0:
        raise SystemExit("the Q8_0 kernel flagged invalid input on synthetic data")

    # end-to-end from host buffers (every rank moves its own shard).  The pinned staging is
    # 6.06 bytes per element; if that is more than a quarter of the free host memory per rank,
    # time a leading part of the shard instead and say so.
    e2e_steps = max(1, min(args.steps, 3))
    e2e_rows = shard.rows
    try:
        import psutil
        budget = psutil.virtual_memory().available // (4 * world)
        while e2e_rows > 1024 and e2e_rows * SWEEP_COLS * 6.0625 > budget:
            e2e_rows //= 2
    except ImportError:
        pass
    if args.skip_e2e:
        e2e_seconds, h2d, d2h = float("nan"), 0, 0
    else:
        e2e_seconds, h2d, d2h, _ = run_e2e(torch, ops, abi, e2e_rows, e2e_steps, 1)
    e2e_seconds *= shard.rows / e2e_rows
    h2d, d2h = h2d * shard.rows // e2e_rows, d2h * shard.rows // e2e_rows
    e2e_t = torch.tensor([e2e_seconds], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)

    sweep_points = None
    if args.sweep:
        del w, blocks, decoded
        torch.cuda.empty_cache()
        sweep_points = sweep(torch, dist, ops, abi, wl, world, rank, peak_gbs, reducer, peers)

    if peers is not None:
        peers.close()  # collective (it ends with a barrier), so before rank 0 goes on alone

    def shut_down():
        if world > 1:
            if reducer is not None:
                reducer.close()
            dist.destroy_process_group()

    if rank != 0:
        shut_down()
        return

    total_elements = args.rows * SWEEP_COLS
    ms_per_step = float(elapsed_ms.item()) / args.steps
    value = total_elements / (ms_per_step * 1e-3) / 1e9
    kernel_s = float(kernel_ms.item()) * 1e-3
    algorithmic = BYTES_PER_ELEMENT * count
    achieved = algorithmic / kernel_s / 1e9
    roofline = {"bound": "hbm", "kernel": "q8_0_kernel<bf16, encode, decode, sum_squares>",
                "achieved": achieved, "peak": peak_gbs, "unit": "GB/s", "frac": achieved / peak_gbs,
                "peak_kind": peak_kind, "algorithmic_bytes_per_launch": algorithmic,
                "launch_us": kernel_s * 1e6,
                "traffic": None if NCU_TRAFFIC_BYTES_PER_ELEMENT is None else NCU_TRAFFIC_BYTES_PER_ELEMENT * count}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16->q8_0(int8+f16)", "data": "synthetic",
        "config": {"workload": f"Q8_0 sweep R={args.rows} x {SWEEP_COLS} bf16 -> Q8_0 + decoded bf16 + sum of squares",
                   "rows_per_gpu": shard.rows, "parallelism": f"row-sharded x{world}, one exchange of 8 bytes per rank", "exchange": exchange,
                   "l2": "inputs larger than L2 (no flush needed)" if count * 2 > 4 * 126e6 else "input fits L2: cold-cache not guaranteed"},
        "roofline": roofline,
        "e2e": {"value": total_elements / float(e2e_t.item()) / 1e9, "unit": UNIT,
                "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world, "steps": e2e_steps,
                "rows_timed_per_gpu": e2e_rows, "rows_per_gpu": shard.rows},
        "gpu_launches": args.steps,
        "clocks": clocks,
        "sum_squares": sum_squares,
    }

    if args.sweep:
        line["sweep"] = sweep_points
    if world == 1:
        if not args.skip_ops:
            line["ops"] = other_ops(torch, peak_gbs)
        if not args.skip_cpu:
            from oracle.binding import Oracle

            oracle = Oracle()
            cores = os.cpu_count() or 1
            oracle.set_threads(cores)
            rows = cpu_sample_rows(oracle, target_seconds=4.0, max_rows=args.rows)
            cpu_value, _ = time_cpu(oracle, rows, steps=3, warmup=1)
            line["cpu_baseline"] = {"value": cpu_value, "unit": UNIT, "cores": cores, "kind": "port",
                                    "sample": f"{rows} of {args.rows} rows x {SWEEP_COLS} per step, 3 timed steps"}
    print(json.dumps(line), flush=True)
    shut_down()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=50)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--rows", type=int, default=DEFAULT_ROWS, help="total rows of the sweep point")
    parser.add_argument("--skip-ops", action="store_true", help="do not time workloads 1-4")
    parser.add_argument("--skip-cpu", action="store_true", help="do not time the CPU baseline")
    parser.add_argument("--sweep", action="store_true", help="also time every sweep point R = 1024 ... 262144")
    parser.add_argument("--skip-e2e", action="store_true", help="do not time the host-buffer pass (profiling runs)")
    parser.add_argument("--exchange", default="fused", choices=["fused", "nccl"],
                        help="how the per-GPU sums of squares are combined when --gpus > 1")
    parser.add_argument("--ops-only", default=None,
                        help="comma list of add_bias_row_sum_max_f32,add_rms_norm_bf16,swiglu_bf16,logits_reduce_f32: "
                             "time only these, --steps iterations each")
    args = parser.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.ops_only:
        run_ops_only(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
