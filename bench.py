#!/usr/bin/env python
"""Benchmark of the B200 provider's hot path.

Headline workload (the only one that shards): the Q8_0 sweep point R x 8192 bf16 -> Q8_0 blocks +
decoded bf16 + sum of squares, row-sharded over the ranks, per-rank sums combined by one exchange of
8 bytes per rank.  A step is one pass over the whole tensor.  `value` is Gelem/s with the input
resident in HBM; `e2e` is the same pass from pinned HOST buffers through the C ABI (host->device and
device->host copies inside the timed region) beside the pinned-copy bandwidth measured in the same
run; `sweep` holds every point R = 1024 ... 262144; `ops` lists the other operators; `workloads`
(printed last) is the compact record of the five benchmark workloads: largest shape against the HBM
roofline, the small shapes in microseconds, and the reference CPU code timed on the host cores.
Before anything is timed the round trip's output is compared with the CPU checker on three 1024-row
chunks of the very tensor that is timed (`parity`).

    python bench.py [--gpus N] [--steps K] [--warmup W]            # this library
    python bench.py --impl reference [...]                          # the CPU provider restated, host cores
    torchrun --nproc-per-node N bench.py --gpus N ...               # one rank per GPU
"""
from __future__ import annotations

import argparse
import ctypes
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
# dram__bytes_read.sum + dram__bytes_write.sum per element of the round-trip kernel in an ncu capture of a
# 16384-row launch: 2.00 read + 2.73 written by the end of the kernel (the rest of the 3.06 B/value of
# output is still in L2 then and is written back afterwards).  Traffic grows in proportion to the tensor.
NCU_TRAFFIC_BYTES_PER_ELEMENT = 4.73
FALLBACK_HBM_GBS = 6650.0
METRIC = "Q8_0 quantise+dequantise+sum-of-squares sweep throughput"
UNIT = "Gelem/s"
DTYPE = "bf16->q8_0(int8+f16)"
PARITY_CHUNK_ROWS = 1024


def job_config(rows: int, world: int) -> dict:
    """What is measured, in the same words for this library and for the reference arm."""
    return {"workload": f"Q8_0 sweep R={rows} x {SWEEP_COLS} bf16 -> Q8_0 + decoded bf16 + sum of squares",
            "rows": rows, "cols": SWEEP_COLS, "parallelism": f"row-sharded x{world}, one exchange of 8 bytes per rank",
            "l2": "inputs larger than L2 (no flush needed)" if rows * SWEEP_COLS * 2 // world > 4 * 126e6
            else "input fits L2: launches rotate over distinct buffers"}


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
        "scaling": "strong", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
        "config": job_config(args.rows, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                         "what": "the CPU provider's Q8_0 path restated in C (the reference delegates it to ggml, "
                                 "which is not part of its tree), OpenMP over blocks on all host cores"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------
# this library
# ---------------------------------------------------------------------------------------------------------
def event_pairs_ms(pairs):
    return [a.elapsed_time(b) for a, b in pairs]


class StreamArgument:
    """The stream argument of the timed ctypes calls: a handle that `time_op` can redirect, so the same
    `launch` closure runs on the default stream and, for the graph measurement, on the capturing one.  (A
    plain attribute: resolving torch's current stream on every launch costs more than a small kernel.)"""

    def __init__(self, torch):
        self.use(torch.cuda.current_stream())

    def use(self, stream):
        self._as_parameter_ = ctypes.c_void_p(stream.cuda_stream)


STREAM = None  # set by the functions that time operators


class Timed(float):
    """Milliseconds per launch in a stream of eager launches; `.graph` = the same launches replayed from a
    CUDA graph (no host launch cost between them), or None where that was not measured."""
    graph = None


def time_op(torch, launch, sets: int, iterations: int = 40, warmup: int = 5, graph: bool = True):
    """Average device time of `launch(i)` over rotating buffer sets (footprint >> L2), CUDA events: issued
    eagerly back to back, and (`.graph`) the same sequence captured once into a CUDA graph and replayed."""
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
    result = Timed(start.elapsed_time(stop) / iterations)
    if graph and STREAM is not None:
        side = torch.cuda.Stream()
        captured = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            STREAM.use(side)
            launch(0)
            side.synchronize()
            with torch.cuda.graph(captured, stream=side):
                for i in range(iterations):
                    launch(i % sets)
            captured.replay()
            side.synchronize()
            start.record(side)
            captured.replay()
            stop.record(side)
            side.synchronize()
        STREAM.use(torch.cuda.current_stream())  # outside the `with`: the stream the eager launches use
        result.graph = start.elapsed_time(stop) / iterations
        del captured
    return result


def other_ops(torch, peak_gbs, only=None, iterations=40):
    """Largest single-GPU shape of workloads 1-4: GB/s against algorithmic bytes, rotating inputs.

    `only` restricts the run to some operators (for profiling one kernel on a short command)."""
    from hyle_b200 import abi, ops

    results = []
    dev = "cuda"
    global STREAM
    lib, stream = abi.load(), StreamArgument(torch)
    STREAM = stream

    def wanted(name):
        return only is None or name in only

    def report(name, shape, elements, algorithmic_bytes, ms, sets):
        gbs = algorithmic_bytes / (ms * 1e-3) / 1e9
        entry = {"op": name, "shape": shape, "us": ms * 1e3, "GB/s": gbs, "Gelem/s": elements / (ms * 1e-3) / 1e9,
                 "roofline_frac": gbs / peak_gbs, "algorithmic_bytes": algorithmic_bytes, "buffer_sets": sets}
        replayed = getattr(ms, "graph", None)
        if replayed:  # the same launches replayed from a CUDA graph
            entry["us_graph"] = replayed * 1e3
            entry["roofline_frac_graph"] = algorithmic_bytes / (replayed * 1e-3) / 1e9 / peak_gbs
        results.append(entry)

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
        # the same kernel on eight times the rows: an 8 us launch is dominated by the launch-to-launch boundary
        sets = 3
        x16 = [torch.randn(32768, 2048, device=dev).to(torch.bfloat16) for _ in range(sets)]
        y16 = [torch.empty_like(x16[0]) for _ in range(sets)]
        ms = time_op(torch, lambda i: lib.hyle_b200_layer_norm_bf16(
            stream, x16[i].data_ptr(), scale.data_ptr(), bias.data_ptr(), y16[i].data_ptr(), 32768, 2048, 1e-5), sets, iterations)
        report("layer_norm_bf16", "32768x2048", 32768 * 2048, 2 * 32768 * 2048 * 2, ms, sets)
        del x16, y16
        sets = 8
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
        addend = torch.where(mask != 0, 0.0, float("-inf")).to(torch.float16).contiguous()
        ms = time_op(torch, lambda i: lib.hyle_b200_additive_masked_softmax_f16(
            stream, scores[i].data_ptr(), addend.data_ptr(), addend.numel(), 0.125, probs[i].data_ptr(), rows, cols), sets, iterations)
        report("additive_masked_softmax_f16", "32768x2048, causal f16 addends 2048x2048", rows * cols,
               rows * cols * 4 + addend.numel() * 2, ms, sets)
        ms = time_op(torch, lambda i: lib.hyle_b200_reduce_rows_extremum(
            stream, abi.REDUCE_MAXIMUM, abi.F16, scores[i].data_ptr(), probs[i].data_ptr(), rows, cols), sets, iterations)
        report("reduce_max_f16", "32768x2048", rows * cols, rows * cols * 2 + rows * 2, ms, sets)
        ms = time_op(torch, lambda i: lib.hyle_b200_rms_norm(
            stream, abi.F16, scores[i].data_ptr(), None, abi.F16, probs[i].data_ptr(), rows, cols, 1e-6), sets, iterations)
        report("rms_norm_f16", "32768x2048", rows * cols, rows * cols * 4, ms, sets)
        del scores, probs, mask, addend
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
        # the mirror: dense rows placed into the left half of wider rows (16-byte groups), and into a transposed layout
        narrow = [torch.randn(side, side // 2, device=dev) for _ in range(sets)]
        ms = time_op(torch, lambda i: lib.hyle_b200_strided_scatter(
            stream, abi.F32, narrow[i].data_ptr(), y[i].data_ptr(), 2, half, sliced), sets, iterations)
        report("strided_scatter_f32_slice", "4096x2048 placed into a slice of 4096x4096 rows", side * side // 2, side * side // 2 * 8, ms, sets)
        ms = time_op(torch, lambda i: lib.hyle_b200_strided_scatter(
            stream, abi.F32, x[i].data_ptr(), y[i].data_ptr(), 2, dims, transposed), sets, iterations)
        report("strided_scatter_f32_transpose", "4096x4096 written through a transposed view (the tiled transposition, from the destination's side)", side * side,
               side * side * 8, ms, sets)
        del x, y, y16, narrow

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
        # "an overflow writes nothing" forces the whole input to be checked before the first store: a tensor that
        # does not stay in L2 between the two passes is read twice, 12 bytes per value moved
        report("scan_i32_checked (12 B per value: input read twice)", "4096x4096", 4096 * 4096, 4096 * 4096 * 12, ms, sets)
        del n, m
        sets = 8
        n = [torch.randint(-1000, 1000, (2048, 4096), dtype=torch.int32, device=dev) for _ in range(sets)]
        m = [torch.empty_like(n[0]) for _ in range(sets)]
        ms = time_op(torch, lambda i: lib.hyle_b200_scan(
            stream, abi.I32, n[i].data_ptr(), m[i].data_ptr(), 2048, 4096, 0, status.data_ptr()), sets, iterations)
        report("scan_i32_checked", "2048x4096 (32 MiB: the writing pass reads it from L2)", 2048 * 4096, 2048 * 4096 * 8, ms, sets)
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
        # The same episode through the REFERENCE's own CUDA kernel (compiled in place into oracle/_ref, used
        # by the tests as the checker): reported beside the product's number, never part of a product timing.
        from oracle.binding import RefPaged

        if RefPaged.available():
            reference = RefPaged()
            ms = time_op(torch, lambda i: reference.paged_append(
                stream, arenas[i].data_ptr(), fresh[i].data_ptr(), episode.data_ptr(), page_rows, pages, new_count,
                new_count // page_rows, row_bytes), sets, iterations, graph=False)
            report("paged_append_REFERENCE_KERNEL", "the reference's cuda_paged_append.cu on the same episode (not this library)",
                   new_count, 2 * new_count * row_bytes, ms, sets)
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
        # Softmax and LogSoftmax alone (f32 in, f32 out: 8 B per value), the same streaming kernel
        del probs
        out32 = [torch.empty(rows, cols, device=dev) for _ in range(2)]
        for name, kind in (("softmax_f32", abi.SOFTMAX), ("log_softmax_f32", abi.LOG_SOFTMAX)):
            ms = time_op(torch, lambda i: lib.hyle_b200_softmax_f32(
                stream, kind, logits[i].data_ptr(), out32[i % 2].data_ptr(), rows, cols, scratch.data_ptr(), scratch.numel(),
                None), sets, max(1, iterations // 2))
            report(name, "256x151936", rows * cols, rows * cols * 8, ms, sets)
        del logits, out32, scratch
    torch.cuda.empty_cache()
    return results


def sweep(torch, dist, abi, wl, world: int, rank: int, peak_gbs: float, reducer, peers, resident, iterations: int = 20):
    """The whole sweep R = 1024 ... 262144 (16 MiB ... 4 GiB of bf16), row-sharded over the ranks:
    per point the step time (kernel + exchange, max over ranks), Gelem/s and GB/s per GPU.

    The points run on row ranges of the tensors that are already resident (`resident` = input,
    blocks, decoded, workspace, partial of the headline point); a small point rotates over distinct
    ranges, so that no launch finds its input in L2."""
    w, blocks, decoded, workspace, partial = resident
    points = []
    lib = abi.load()
    stream = torch.cuda.current_stream().cuda_stream
    block_row_bytes = SWEEP_COLS // 32 * 34
    for total_rows in wl.SWEEP_ROWS:
        rows = wl.shard_rows(total_rows, world, rank).rows
        if rows == 0 or rows > w.shape[0]:
            continue
        sets = max(1, min(8, w.shape[0] // rows, int(600e6 // max(1, rows * SWEEP_COLS * 2))))
        count = rows * SWEEP_COLS

        def one(i):
            first = (i % sets) * rows
            arguments = (stream, w[first:].data_ptr(), count, blocks[first * block_row_bytes:].data_ptr(),
                         decoded[first:].data_ptr(), partial.data_ptr(), None, workspace.data_ptr(), workspace.numel())
            if peers is not None:
                abi.check("roundtrip_exchange", lib.hyle_b200_q8_0_roundtrip_bf16_exchange(
                    *arguments, peers.pointers, world, rank, peers.next_epoch(), 0))
                return
            abi.check("roundtrip", lib.hyle_b200_q8_0_roundtrip_bf16(*arguments))
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
        points.append({"rows": total_rows, "MiB_in": elements * 2 // 2**20, "us_per_step": round(seconds * 1e6, 2),
                       "Gelem/s": round(elements / seconds / 1e9, 2), "GB/s_per_gpu": round(gbs_per_gpu, 1),
                       "roofline_frac": round(gbs_per_gpu / peak_gbs, 4), "buffer_sets": sets})
    return points


def parity_check(torch, ops, w, blocks, decoded, first_row: int):
    """The round trip's output on the tensor that is about to be timed against the CPU checker: the
    first 1024 rows, the 1024 rows around the middle (at the full size they straddle the 2 GiB byte
    offset of both bf16 tensors) and the last 1024 rows; bytes of blocks and decoded values must be equal."""
    from oracle.binding import Oracle

    oracle = Oracle()
    rows = w.shape[0]
    chunk = min(PARITY_CHUNK_ROWS, rows)
    starts = sorted({0, max(0, rows // 2 - chunk // 2), rows - chunk})
    block_row_bytes = SWEEP_COLS // 32 * 34
    for first in starts:
        words = w[first:first + chunk].view(torch.int16).cpu().numpy().view(np.uint16).copy()
        want_blocks, want_decoded, _, invalid = oracle.q8_0_roundtrip(words)
        got_blocks = blocks[first * block_row_bytes:(first + chunk) * block_row_bytes].cpu().numpy()
        got_decoded = decoded[first:first + chunk].view(torch.int16).cpu().numpy().view(np.uint16).ravel()
        if invalid or not np.array_equal(got_blocks, want_blocks) or not np.array_equal(got_decoded, want_decoded):
            return f"MISMATCH in rows {first_row + first}..{first_row + first + chunk}"
    return "checked"


def numa_affinity(local_rank: int):
    """Pin the calling thread to the CPUs next to this rank's GPU (NVML's ideal affinity), so that the pinned
    staging buffers allocated afterwards are on that NUMA node.  A host-side setting of this process only.
    Returns (previous affinity, description) or (None, reason)."""
    try:
        import pynvml

        pynvml.nvmlInit()
        index = local_rank
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        if visible:
            entries = [e.strip() for e in visible.split(",") if e.strip()]
            if local_rank < len(entries) and entries[local_rank].isdigit():
                index = int(entries[local_rank])
        handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        previous = os.sched_getaffinity(0)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        cpus = {64 * w + b for w, word in enumerate(words) for b in range(64) if word >> b & 1} & previous
        if not cpus:
            return None, "NVML reports no CPU near the GPU inside this process's CPU set"
        os.sched_setaffinity(0, cpus)
        return previous, f"{len(cpus)} CPUs near the GPU"
    except Exception as problem:  # no NVML, no permission: run unpinned and say so
        return None, f"not pinned ({type(problem).__name__})"


def pinned_copy_bandwidth(torch, chunk_bytes: int = 64 << 20, chunks: int = 24, together=None):
    """GB/s of pinned-memory copies, one cudaMemcpyAsync per chunk: host->device alone, device->host alone,
    both directions at once on two streams, and both at once in the proportion of the end-to-end pass (per
    64 MiB copied in, 98 MiB copied out: the Q8_0 blocks and the decoded tensor), which is the copy-only
    version of that pass and the denominator of its roofline.  `together` (a barrier among the ranks) is
    called before each measurement so that all ranks measure the same thing at the same time."""
    out_chunk = chunk_bytes // 32 * 17 + chunk_bytes                  # 34 bytes of blocks per 64 bytes of bf16, plus the decoded bf16
    host_a = torch.empty(chunk_bytes * chunks, dtype=torch.uint8, pin_memory=True)
    host_b = torch.empty(out_chunk * chunks, dtype=torch.uint8, pin_memory=True)
    host_a.zero_(), host_b.zero_()
    dev_a = torch.empty(chunk_bytes * chunks, dtype=torch.uint8, device="cuda")
    dev_b = torch.empty(out_chunk * chunks, dtype=torch.uint8, device="cuda")
    up, down = torch.cuda.Stream(), torch.cuda.Stream()

    def run(h2d: bool, d2h: bool, out_bytes: int = chunk_bytes):
        if together is not None:
            together()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for c in range(chunks):
            if h2d:
                piece = slice(c * chunk_bytes, (c + 1) * chunk_bytes)
                with torch.cuda.stream(up):
                    dev_a[piece].copy_(host_a[piece], non_blocking=True)
            if d2h:
                piece = slice(c * out_bytes, (c + 1) * out_bytes)
                with torch.cuda.stream(down):
                    host_b[piece].copy_(dev_b[piece], non_blocking=True)
        torch.cuda.synchronize()
        return (int(h2d) * chunk_bytes + int(d2h) * out_bytes) * chunks / (time.perf_counter() - t0) / 1e9

    run(True, True)
    return {"h2d_GB/s": round(run(True, False), 2), "d2h_GB/s": round(run(False, True), 2),
            "both_GB/s": round(run(True, True), 2), "pass_mix_GB/s": round(run(True, True, out_chunk), 2),
            "how": f"pinned host memory, one cudaMemcpyAsync per chunk of 64 MiB (98 MiB out in the mix), {chunks} chunks per direction"}


def time_host(call, repeats: int = 2) -> float:
    """Seconds of one host-side call: one warm-up, then the mean of `repeats`."""
    call()
    t0 = time.perf_counter()
    for _ in range(repeats):
        call()
    return (time.perf_counter() - t0) / repeats


def cpu_baselines():
    """The reference's CPU code for workloads 1-4, timed on the host cores: all cores and one thread.

    Workloads 2-4 run the reference's own Highway-free scalar floor compiled in place from its tree
    (oracle/_ref/libhyle_ref_floor.so: rms_norm_bf16, swiglu_bf16, softmax_f32, top_k_f32), with the
    residual add and the f32 -> bf16 cast of the fused forms from the C restatement; workload 1 and
    the floor's absence fall back to the restatement alone (kind "port").  Rows are split over
    threads like the reference's parallel_for_ranges.  Returns {workload: record}."""
    from hyle_b200 import workloads as wl
    from oracle import binding as ob

    oracle = ob.Oracle()
    floor = ob.RefFloor() if ob.RefFloor.available() else None
    cores = os.cpu_count() or 1
    ptr = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    records = {}

    def measure(name, kind, full_rows, single_rows, elements_per_row, run):
        record = {"kind": kind, "unit": "Gelem/s", "cores": cores}
        for label, threads, rows in (("all_cores", cores, full_rows), ("one_thread", 1, single_rows)):
            oracle.set_threads(threads)
            if floor is not None:
                floor.set_threads(threads)
            seconds = time_host(lambda: run(rows))
            record[label] = {"value": round(rows * elements_per_row / seconds / 1e9, 4), "threads": threads,
                             "sample": f"{rows} of {full_rows} rows", "ms": round(seconds * 1e3, 2)}
        oracle.set_threads(cores)
        if floor is not None:
            floor.set_threads(cores)
        records[name] = record

    # 1: C = A + bias, row sums and row maxima of C (three operators on the CPU route)
    a, bias = wl.broadcast_add_inputs(4096, 4096)
    c, row_sum, row_max = np.empty_like(a), np.empty(4096, np.float32), np.empty(4096, np.float32)

    def add_reduce(rows):
        oracle.lib.hyle_oracle_binary(ob.ADD, ob.F32, ptr(a), ptr(bias), ptr(c), rows * 4096, 4096)
        oracle.lib.hyle_oracle_reduce_rows_f32(ob.SUM, ptr(c), ptr(row_sum), rows, 4096)
        oracle.lib.hyle_oracle_reduce_rows_f32(ob.MAXIMUM, ptr(c), ptr(row_max), rows, 4096)
    measure("add_bias_row_sum_max_f32", "port", 4096, 512, 4096, add_reduce)

    # 2: h = x + residual, y = RmsNorm(h) * w
    x, residual, weight, _ = wl.rms_norm_inputs(4096)
    h, y, y32 = np.empty_like(x), np.empty_like(x), np.empty(x.shape, np.float32)

    def add_norm(rows):
        oracle.lib.hyle_oracle_binary(ob.ADD, ob.BF16, ptr(x), ptr(residual), ptr(h), rows * 2048, rows * 2048)
        if floor is not None:
            floor.lib.hyle_ref_rms_norm_bf16(ptr(h), ptr(weight), ptr(y), rows, 2048, 1e-6)
        else:
            oracle.lib.hyle_oracle_rms_norm_bf16(ptr(h), ptr(weight), ob.BF16, ptr(y), ptr(y32), rows, 2048, 1e-6)
    measure("add_rms_norm_bf16", "reference-floor" if floor else "port", 4096, 512, 2048, add_norm)
    del y32

    # 3: out = silu(gate) * up
    gate, up = wl.swiglu_inputs(4096)
    out, out32 = np.empty_like(gate), None

    def gated(rows):
        if floor is not None:
            floor.lib.hyle_ref_swiglu_bf16(ptr(gate), ptr(up), ptr(out), rows, 6144, 6144, 6144)
        else:
            nonlocal out32
            out32 = np.empty(gate.shape, np.float32) if out32 is None else out32
            oracle.lib.hyle_oracle_swiglu_bf16(ptr(gate), ptr(up), ptr(out), ptr(out32), rows, 6144, 6144, 6144)
    measure("swiglu_bf16", "reference-floor" if floor else "port", 4096, 256, 6144, gated)

    # 4: softmax (f32) -> bf16, log-sum-exp (the log-softmax shift) and argmax of 151936-wide rows
    logits, _ = wl.logits_inputs(256)
    probs32, probs16 = np.empty_like(logits), np.empty(logits.shape, np.uint16)
    index, value = np.empty(256, np.int32), np.empty(256, np.float32)

    def reduce_logits(rows):
        if floor is not None:
            floor.lib.hyle_ref_softmax_f32(0, ptr(logits), ptr(probs32), rows, wl.VOCAB)
            floor.lib.hyle_ref_argmax_f32(ptr(logits), ptr(index), ptr(value), rows, wl.VOCAB)
        else:
            oracle.lib.hyle_oracle_softmax_f32(0, ptr(logits), ptr(probs32), rows, wl.VOCAB)
            oracle.lib.hyle_oracle_argmax_f32(ptr(logits), ptr(index), ptr(value), rows, wl.VOCAB)
        oracle.lib.hyle_oracle_cast_f32_to_bf16(ptr(probs32), ptr(probs16), rows * wl.VOCAB)
    measure("logits_reduce_f32", "reference-floor" if floor else "port", 256, 16, wl.VOCAB, reduce_logits)
    return records


def small_shapes(torch, iterations: int = 200):
    """The decode-sized shapes of workloads 2-4 in microseconds per launch (launch-bound: no roofline
    fraction is meaningful at 4 KiB ... 10 MB), back to back on one stream with their inputs in L2."""
    from hyle_b200 import abi

    global STREAM
    lib, stream, dev = abi.load(), StreamArgument(torch), "cuda"
    STREAM = stream
    shapes = {}

    def record(name, ms):
        shapes[name] = round(ms * 1e3, 2)
        if ms.graph:
            shapes[name + " (graph replay)"] = round(ms.graph * 1e3, 2)
    weight = (torch.rand(2048, device=dev) + 0.5).bfloat16()
    for tokens in (1, 64):
        x, r = torch.randn(tokens, 2048, device=dev).bfloat16(), torch.randn(tokens, 2048, device=dev).bfloat16()
        y, h = torch.empty_like(x), torch.empty_like(x)
        ms = time_op(torch, lambda i: lib.hyle_b200_add_rms_norm_bf16(
            stream, x.data_ptr(), r.data_ptr(), weight.data_ptr(), abi.BF16, y.data_ptr(), h.data_ptr(), tokens, 2048, 1e-6),
            1, iterations)
        record(f"add_rms_norm_bf16 T={tokens}", ms)
    for tokens in (1, 8, 32):
        g, u = torch.randn(tokens, 6144, device=dev).bfloat16(), torch.randn(tokens, 6144, device=dev).bfloat16()
        o = torch.empty_like(g)
        ms = time_op(torch, lambda i: lib.hyle_b200_swiglu_bf16(
            stream, g.data_ptr(), u.data_ptr(), o.data_ptr(), tokens, 6144, 6144, 6144), 1, iterations)
        record(f"swiglu_bf16 T={tokens}", ms)
    for batch in (1, 16):
        logits = 4.0 * torch.randn(batch, 151936, device=dev)
        probs = torch.empty(batch, 151936, dtype=torch.bfloat16, device=dev)
        lse, val = torch.empty(batch, device=dev), torch.empty(batch, device=dev)
        idx = torch.empty(batch, dtype=torch.int32, device=dev)
        ms = time_op(torch, lambda i: lib.hyle_b200_logits_reduce_f32(
            stream, logits.data_ptr(), batch, 151936, lse.data_ptr(), probs.data_ptr(), idx.data_ptr(), val.data_ptr(),
            None, 0, None), 1, iterations)
        record(f"logits_reduce_f32 B={batch}", ms)
    return shapes


def run_e2e(torch, ops, abi, shard_rows: int, steps: int, warmup: int, copies_only: bool = False, together=None):
    """One pass from pinned host buffers through the C ABI and back, as a three-stage pipeline: a stream that
    only copies host -> device, one that only runs the kernel, one that only copies device -> host, chained
    per chunk by events over four rotating sets of device buffers.  Both copy directions therefore run all
    the time (chunks on one stream each would fall into step: all copying in, then all copying out).  Timed
    with CUDA events from the first copy in to the last copy out.  `copies_only` records the same pipeline
    without the kernel launches: the same copies in the same order behind the same events, which is the
    ceiling the host link sets for this pass.  `together` (a barrier among the ranks) is called before every
    timed pass: the ranks share the host's memory and links, so their passes must run at the same time for
    the max over ranks to be the time of the job (buffer set-up takes each rank a different time)."""
    chunk_rows = min(shard_rows, 4096, max(1024, shard_rows // 16))   # 64 MiB of bf16 per chunk, at least 16 chunks
    chunks = (shard_rows + chunk_rows - 1) // chunk_rows
    lanes = min(4, chunks)
    host_in = torch.empty((shard_rows, SWEEP_COLS), dtype=torch.bfloat16, pin_memory=True)
    host_in.copy_(torch.randn(1024, SWEEP_COLS).mul_(0.02).bfloat16().repeat((shard_rows + 1023) // 1024, 1)[:shard_rows])
    host_blocks = torch.empty(shard_rows * SWEEP_COLS // 32 * 34, dtype=torch.uint8, pin_memory=True)
    host_decoded = torch.empty((shard_rows, SWEEP_COLS), dtype=torch.bfloat16, pin_memory=True)
    host_sums = torch.empty(chunks, dtype=torch.float64, pin_memory=True)
    copy_in, compute, copy_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    dev_in = [torch.empty((chunk_rows, SWEEP_COLS), dtype=torch.bfloat16, device="cuda") for _ in range(lanes)]
    dev_blocks = [torch.empty(chunk_rows * SWEEP_COLS // 32 * 34, dtype=torch.uint8, device="cuda") for _ in range(lanes)]
    dev_decoded = [torch.empty((chunk_rows, SWEEP_COLS), dtype=torch.bfloat16, device="cuda") for _ in range(lanes)]
    dev_sums = torch.zeros(chunks, dtype=torch.float64, device="cuda")
    workspaces = [ops.make_workspace("cuda", chunk_rows * SWEEP_COLS) for _ in range(lanes)]
    arrived = [torch.cuda.Event() for _ in range(lanes)]     # the chunk is on the device
    consumed = [torch.cuda.Event() for _ in range(lanes)]    # the kernel has read it: the input set is free
    produced = [torch.cuda.Event() for _ in range(lanes)]    # the kernel's outputs are complete
    drained = [torch.cuda.Event() for _ in range(lanes)]     # the outputs are on the host: the output set is free
    first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    lib = abi.load()
    block_bytes_per_row = SWEEP_COLS // 32 * 34

    def one_pass():
        first.record(copy_in)
        for c in range(chunks):
            lane = c % lanes
            begin = c * chunk_rows
            rows = min(chunk_rows, shard_rows - begin)
            with torch.cuda.stream(copy_in):
                if c >= lanes:
                    copy_in.wait_event(consumed[lane])
                dev_in[lane][:rows].copy_(host_in[begin:begin + rows], non_blocking=True)
                arrived[lane].record(copy_in)
            with torch.cuda.stream(compute):
                compute.wait_event(arrived[lane])
                if c >= lanes:
                    compute.wait_event(drained[lane])
                if not copies_only:
                    abi.check("roundtrip", lib.hyle_b200_q8_0_roundtrip_bf16(
                        compute.cuda_stream, dev_in[lane].data_ptr(), rows * SWEEP_COLS, dev_blocks[lane].data_ptr(),
                        dev_decoded[lane].data_ptr(), dev_sums[c:].data_ptr(), None, workspaces[lane].data_ptr(),
                        workspaces[lane].numel()))
                consumed[lane].record(compute)
                produced[lane].record(compute)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(produced[lane])
                host_blocks[begin * block_bytes_per_row:(begin + rows) * block_bytes_per_row].copy_(
                    dev_blocks[lane][:rows * block_bytes_per_row], non_blocking=True)
                host_decoded[begin:begin + rows].copy_(dev_decoded[lane][:rows], non_blocking=True)
                drained[lane].record(copy_out)
        with torch.cuda.stream(copy_out):
            host_sums.copy_(dev_sums, non_blocking=True)   # ordered behind the last kernel through produced[]
            last.record(copy_out)
        last.synchronize()
        return float(host_sums.sum()), first.elapsed_time(last) * 1e-3

    for _ in range(warmup):
        one_pass()
    torch.cuda.synchronize()
    seconds = 0.0
    for _ in range(steps):
        if together is not None:
            together()
        total, elapsed = one_pass()
        seconds += elapsed / steps
    torch.cuda.synchronize()
    h2d = shard_rows * SWEEP_COLS * 2
    d2h = shard_rows * block_bytes_per_row + shard_rows * SWEEP_COLS * 2 + chunks * 8
    return seconds, h2d, d2h, total


def file_stream_bench(torch, ops, abi, blocks, values: int = 512 * 1024 * 1024 // 34 * 32, passes: int = 3):
    """The on-disk form of the path: a Q8_0 bank (the blocks the headline launch just produced) is written to a
    temporary file and streamed back through `hyle_b200_file_stream_*` into the decode kernel (file -> pinned
    slots -> device -> `hyle_b200_q8_0_decode_bf16` per chunk).  Reads come from the page cache, so this times
    the pipeline, not a disk.  Wall clock, best of `passes` after a warm-up: the streaming phase (first next()
    to the last decode's completion) in GB/s of file bytes, and open() / close(), which allocate and free the
    pinned and device slots, on their own."""
    import tempfile

    values -= values % 256
    size = values // 32 * 34
    if blocks.numel() < size:
        return None
    lib = abi.load()
    out = torch.empty(values, dtype=torch.bfloat16, device="cuda")
    consumer = torch.cuda.current_stream().cuda_stream
    best = None
    with tempfile.NamedTemporaryFile(prefix="hyle_b200_bank_", suffix=".q8_0") as bank:
        bank.write(memoryview(blocks[:size].cpu().numpy()))
        bank.flush()
        for _ in range(passes + 1):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            stream = ops.FileStream(bank.name, size, granule=34 * 8)
            t1 = time.perf_counter()
            for pointer, nbytes, offset in stream:
                abi.check("decode", lib.hyle_b200_q8_0_decode_bf16(consumer, pointer, nbytes // 34 * 32,
                                                                   out.data_ptr() + offset // 34 * 64))
            torch.cuda.synchronize()
            t2 = time.perf_counter()
            report = stream.report()
            stream.close()
            t3 = time.perf_counter()
            if best is None or t2 - t1 < best[1]:
                best = (t1 - t0, t2 - t1, t3 - t2, report)
    opened, streamed, closed, report = best
    return {"bank_MiB": round(size / 2 ** 20, 1), "GB/s_of_file_bytes": round(size / streamed / 1e9, 2),
            "stream_ms": round(streamed * 1e3, 2), "open_ms": round(opened * 1e3, 2), "close_ms": round(closed * 1e3, 2),
            "chunk_MiB": round(report.chunk_bytes / 2 ** 20, 2), "chunks": int(report.chunks), "copies": int(report.copies),
            "pread_calls": int(report.io_calls), "pinned_MiB": round(report.staging_bytes / 2 ** 20, 1),
            "what": "Q8_0 bank from the page cache -> pinned slots (several threads read a chunk together) -> one "
                    "cudaMemcpyAsync per chunk -> decode kernel -> bf16 tensor"}


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

    # Parity first: one launch, three 1024-row chunks of its output against the CPU checker.
    parity = "skipped"
    if not args.skip_parity:
        step()
        combine()
        torch.cuda.synchronize()
        parity = parity_check(torch, ops, w, blocks, decoded, shard.first_row)
        if world > 1:
            verdicts = [None] * world
            dist.all_gather_object(verdicts, parity)
            bad = [v for v in verdicts if v != "checked"]
            parity = bad[0] if bad else "checked"
        if parity != "checked":
            raise SystemExit(f"parity check failed before timing: {parity}")

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
    # A step is ONE launch unless the sums are combined by a library call behind it; only then is the kernel
    # bracketed by events of its own (an event between two launches keeps the second from starting under the
    # first's tail, so the one-launch steps are timed as a whole and divided).
    bracket = reducer is not None
    kernel_events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)] if bracket else []
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for k in range(args.steps):
        if bracket:
            kernel_events[k][0].record()
        step()
        if bracket:
            kernel_events[k][1].record()
        combine()
    stop.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    elapsed_ms = torch.tensor([start.elapsed_time(stop)], dtype=torch.float64, device="cuda")
    launch_ms = statistics.mean(event_pairs_ms(kernel_events)) if bracket else start.elapsed_time(stop) / args.steps
    kernel_ms = torch.tensor([launch_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(elapsed_ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(kernel_ms, op=dist.ReduceOp.MAX)
    clocks = sampler.stop() if rank == 0 else None
    sum_squares = float(partial.item())
    if int(status.item()) != 0:
        raise SystemExit("the Q8_0 kernel flagged invalid input on synthetic data")

    # Where a multi-GPU step goes: every rank times the bare kernel on its shard (no exchange), and the
    # step as it ran above.  step - slowest bare kernel = waiting for the slowest rank + the exchange.
    rank_split = None
    if world > 1:
        # Blocks of ten bare launches and ten whole steps take turns, so both see the same clocks (a block measured
        # after the other would run under the power cap the first one provoked); each block is one pair of events
        # around its run of launches (an event between two launches costs more than the exchange looked for).
        def bare():
            lib.hyle_b200_q8_0_roundtrip_bf16(stream, w.data_ptr(), count, blocks.data_ptr(), decoded.data_ptr(),
                                              partial.data_ptr(), None, workspace.data_ptr(), workspace.numel())

        def whole():
            step()
            combine()

        def block_ms(launch, launches=10):
            first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            first.record()
            for _ in range(launches):
                launch()
            last.record()
            last.synchronize()
            return first.elapsed_time(last) / launches

        alone_ms, whole_ms = [], []
        for _ in range(4):
            dist.barrier()
            torch.cuda.synchronize()
            alone_ms.append(block_ms(bare))
            dist.barrier()
            torch.cuda.synchronize()
            whole_ms.append(block_ms(whole))
        mine = {"rank": rank, "kernel_alone_us": round(statistics.mean(alone_ms) * 1e3, 2),
                "step_us": round(statistics.mean(whole_ms) * 1e3, 2)}
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        slowest = max(g["kernel_alone_us"] for g in gathered)
        rank_split = {"per_rank": gathered, "slowest_kernel_alone_us": slowest,
                      "step_us_max": max(g["step_us"] for g in gathered),
                      "wait_and_exchange_us": round(max(g["step_us"] for g in gathered) - slowest, 2),
                      "note": "kernel_alone = the round trip without the exchange, step = the launch including the wait for the "
                              "slowest rank's sum (and the library all-reduce where that is the exchange); blocks of ten launches "
                              "of each kind taking turns, each block between one pair of CUDA events, mean of four blocks"}

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
    copy_peak, pinned_to = None, None
    if args.skip_e2e:
        e2e_seconds, h2d, d2h = float("nan"), 0, 0
    else:
        previous_affinity, pinned_to = numa_affinity(local_rank)  # pinned staging next to the GPU
        try:
            if world > 1:
                dist.barrier()  # all ranks copy at once: the bandwidth a rank sees is its share of the host's
            copy_peak = pinned_copy_bandwidth(torch, together=dist.barrier if world > 1 else None)
            if world > 1:
                dist.barrier()
            in_step = dist.barrier if world > 1 else None
            e2e_seconds, h2d, d2h, _ = run_e2e(torch, ops, abi, e2e_rows, e2e_steps, 1, together=in_step)
            # the ceiling of that pass: the same pipeline without its kernels, all ranks at once
            copies_seconds, _, _, _ = run_e2e(torch, ops, abi, e2e_rows, e2e_steps, 1, copies_only=True, together=in_step)
        finally:
            if previous_affinity is not None:
                os.sched_setaffinity(0, previous_affinity)
    e2e_seconds *= shard.rows / e2e_rows
    h2d, d2h = h2d * shard.rows // e2e_rows, d2h * shard.rows // e2e_rows
    e2e_t = torch.tensor([e2e_seconds, float("nan") if args.skip_e2e else copies_seconds * shard.rows / e2e_rows],
                         dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)

    copy_peaks = None
    if copy_peak is not None and world > 1:
        copy_peaks = [None] * world
        dist.all_gather_object(copy_peaks, copy_peak)

    sweep_points = None
    if not args.skip_sweep:
        sweep_points = sweep(torch, dist, abi, wl, world, rank, peak_gbs, reducer, peers,
                             (w, blocks, decoded, workspace, partial))

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

    e2e_seconds_max, copies_seconds_max = float(e2e_t[0].item()), float(e2e_t[1].item())
    e2e = {"value": total_elements / e2e_seconds_max / 1e9, "unit": UNIT,
           "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world, "steps": e2e_steps,
           "rows_timed_per_gpu": e2e_rows, "rows_per_gpu": shard.rows, "host_threads_pinned": pinned_to}
    if copy_peak is not None:
        # the end-to-end pass moves h2d + d2h bytes per GPU over its PCIe link while the kernels run beside
        # the copies: its roofline is the same bytes in the same proportion as bare pinned copies, both
        # directions busy, all ranks at once, measured just before; the slowest rank's link bounds the step
        per_gpu = (h2d + d2h) / e2e_seconds_max / 1e9
        ceiling = (h2d + d2h) / copies_seconds_max / 1e9
        e2e["roofline"] = {"bound": "pcie (pinned host memory <-> device): the same pipeline recorded without its kernels -- "
                                    "the same copies behind the same events, all ranks at once, max over ranks",
                           "achieved": round(per_gpu, 2), "peak": round(ceiling, 2), "unit": "GB/s per GPU",
                           "frac": round(per_gpu / ceiling, 3), "copy_bandwidth": copy_peak,
                           "copy_bandwidth_all_ranks_at_once": None if copy_peaks is None else
                           {"pass_mix_GB/s_per_rank": [p["pass_mix_GB/s"] for p in copy_peaks],
                            "both_GB/s_per_rank": [p["both_GB/s"] for p in copy_peaks],
                            "d2h_GB/s_per_rank": [p["d2h_GB/s"] for p in copy_peaks],
                            "h2d_GB/s_per_rank": [p["h2d_GB/s"] for p in copy_peaks],
                            "sum_pass_mix_GB/s": round(sum(p["pass_mix_GB/s"] for p in copy_peaks), 1)}}

    streamed = None
    if world == 1 and not args.skip_e2e:
        streamed = file_stream_bench(torch, ops, abi, blocks)
        if streamed is not None and copy_peak is not None:
            streamed["h2d_pinned_copy_GB/s"] = copy_peak["h2d_GB/s"]
            streamed["frac_of_pinned_copy"] = round(streamed["GB/s_of_file_bytes"] / copy_peak["h2d_GB/s"], 3)

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
        "config": job_config(args.rows, world),
        "details": {"rows_per_gpu": shard.rows, "exchange": exchange},
        "parity": parity,
        "roofline": roofline,
        "e2e": e2e,
        "file_stream": streamed,
        "gpu_launches": args.steps,
        "clocks": clocks,
        "sum_squares": sum_squares,
    }
    if rank_split is not None:
        line["multi_gpu_step"] = rank_split

    if world == 1:
        if not args.skip_cpu:
            from oracle.binding import Oracle

            oracle = Oracle()
            cores = os.cpu_count() or 1
            oracle.set_threads(cores)
            rows = cpu_sample_rows(oracle, target_seconds=4.0, max_rows=args.rows)
            cpu_value, _ = time_cpu(oracle, rows, steps=3, warmup=1)
            oracle.set_threads(1)
            single_rows = max(256, rows // 16)
            single_value, _ = time_cpu(oracle, single_rows, steps=2, warmup=1)
            oracle.set_threads(cores)
            line["cpu_baseline"] = {"value": cpu_value, "unit": UNIT, "cores": cores, "kind": "port",
                                    "sample": f"{rows} of {args.rows} rows x {SWEEP_COLS} per step, 3 timed steps",
                                    "one_thread": {"value": single_value, "sample": f"{single_rows} rows x {SWEEP_COLS}"}}
        if not args.skip_ops:
            line["ops"] = other_ops(torch, peak_gbs)
    if sweep_points is not None:
        line["sweep"] = sweep_points
    if world == 1 and not args.skip_ops:
        # Printed last, so that a reader of the line's tail still has it: the five benchmark workloads.
        by_name = {entry["op"]: entry for entry in line["ops"]}
        baselines = {} if args.skip_cpu else cpu_baselines()
        workloads = {}
        for number, name in ((1, "add_bias_row_sum_max_f32"), (2, "add_rms_norm_bf16"), (3, "swiglu_bf16"),
                             (4, "logits_reduce_f32")):
            entry = by_name.get(name)
            if entry is None:
                continue
            workloads[f"{number}:{name}"] = {
                "shape": entry["shape"], "us": round(entry["us"], 2), "GB/s": round(entry["GB/s"], 1),
                "Gelem/s": round(entry["Gelem/s"], 2), "frac_of_measured_hbm": round(entry["roofline_frac"], 4),
                "frac_of_nominal_8TB/s": round(entry["GB/s"] / 8000.0, 4),
                "us_graph": None if "us_graph" not in entry else round(entry["us_graph"], 2),
                "frac_of_measured_hbm_graph": None if "us_graph" not in entry else round(entry["roofline_frac_graph"], 4),
                "cpu_baseline": baselines.get(name)}
        workloads["5:q8_0_roundtrip_bf16"] = {
            "shape": f"{args.rows}x{SWEEP_COLS}", "us": round(kernel_s * 1e6, 1), "GB/s": round(achieved, 1),
            "Gelem/s": round(value, 2), "frac_of_measured_hbm": round(achieved / peak_gbs, 4),
            "frac_of_nominal_8TB/s": round(achieved / 8000.0, 4), "cpu_baseline": line.get("cpu_baseline")}
        workloads["small_shapes_us_per_launch"] = small_shapes(torch)
        workloads["host"] = {"nproc": os.cpu_count(), "peak_GB/s": peak_gbs, "peak_kind": peak_kind}
        line["workloads"] = workloads
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
    parser.add_argument("--skip-sweep", action="store_true", help="do not time the other sweep points R = 1024 ... 131072")
    parser.add_argument("--skip-parity", action="store_true", help="do not compare with the CPU checker before timing")
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
