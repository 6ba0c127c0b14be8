#!/usr/bin/env python
"""Benchmark of the B200 matmul path.  Prints ONE JSON line on rank 0.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME] [--no-extra]

Headline workload at EVERY N (1, 2, 4, 8): the large BF16 GEMM M=16384 N=53248 K=8192, B column-sharded over the ranks
(one process per GPU, launched by torch.distributed.run), A replicated, the output gathered on every rank - by the GEMM's
own epilogue, or by copies that run behind the next step's GEMM, whichever a ten-step trial on the machine finds faster
(`--gather`; the trial times are in the line) - strong scaling, so the per-N values form one curve.  It fits one GPU (2.9 GB), where the slab is the
whole result.  At N = 1 the other single-GPU configurations (BF16 4096^3, FP32 1024^3, INT8 4096x14336x4096, the three
weight-only decode shapes) are measured too and reported under "configs", each with its own `roofline`,
`cpu_baseline` and `e2e` record.

A step is one pass of the operator over one batch of synthetic input.  `value` is measured with the operands
resident in HBM (CUDA events on the launching stream, max over ranks); `e2e` runs the same step through the
operator bridge with pinned HOST buffers, host->device copies of the inputs and a device->host read of the
result inside the timed region.  `--impl reference` times the reference's own CPU matmul on the host cores.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys
import threading
import time
from ctypes import byref
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "GEMM TFLOP/s (BF16/INT8) & GB/s (decode) at 1/2/4/8 B200, % of roofline"
NOMINAL = {"bf16_tflops": 2250.0, "i8_tops": 4500.0, "hbm_gbs": 8000.0, "fp32_tflops": 74.4, "tf32_tflops": 1125.0}  # fp32: 148 SMs x 128 FMA lanes x 2 x 1.965 GHz
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, read from one ncu capture of that
# workload, with the committed summary the figure was taken from.  A workload without a capture reports null.
NCU_TRAFFIC = {
    "c1_f32_1024": (25.2e6, "profiles/f32_tf32x3__c1_f32_1024.md (the GEMM launch; the split pre-pass adds 8.4 MB)"),
    "c2_bf16_4096": (99.3e6, "profiles/gemm_tcgen05_bf16__c2_bf16_4096.md"),
    "c3_i8_4096x14336x4096": (282.6e6, "profiles/gemm_tcgen05_i8__c3_i8_4096x14336x4096.md"),
    "c4_w8_m1": (58.9e6, "profiles/w8_stream__c4_w8_m1.md"),
    "c4_w8_m16": (59.1e6, "profiles/w8_stream__c4_w8_m16.md"),
    "c4_w8_m128": (60.7e6, "profiles/gemm_tcgen05_w8__c4_w8_m128.md"),
}
# What a GPU can receive when all eight send to all eight at once: a store-only all-to-all probe on this pool
# (148 CTAs per GPU issuing the epilogue's own 32-row x 128-byte TMA stores to the seven peers) measured 668 GB/s per
# direction per GPU; a copy-engine copy between two GPUs 770.  Not measured in this run; they bound "result gathered on
# every rank" from below (the pipelined gather has run ten steps at 685 GB/s into every GPU, between the two).
NVLINK_RECEIVE_GBS = 668.0
NVLINK_PEER_COPY_GBS = 770.0
BURST_BELOW_MS = 5.0  # kernels shorter than this are held to the burst cuBLAS figure, longer ones to the sustained one


def measured_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return json.loads(path.read_text()), "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# ---------------------------------------------------------------------------------------------- clocks

class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a timed region runs (read-only)."""

    REASONS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
               0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
               0x100: "display_clock_setting"}

    def __init__(self, index: int) -> None:
        self.samples: list[int] = []
        self.reason_bits = 0
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
        except Exception:  # NVML missing: report nothing rather than guess
            self._nvml = None

    def _loop(self) -> None:
        nv = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM))
                self.reason_bits |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
            except Exception:
                try:
                    self.reason_bits |= int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle))
                except Exception:
                    pass
            time.sleep(0.002)

    def __enter__(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)

    def summary(self) -> dict:
        reasons = [name for bit, name in self.REASONS.items() if self.reason_bits & bit and name != "gpu_idle"]
        return {"sm_mhz": int(np.median(self.samples)) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(self.samples)}


# ---------------------------------------------------------------------------------------------- our arm

def device_sets(w, sets: int, dev, row0=0, row1=None):
    """`sets` operand sets for workload `w` on `dev`: set 0 is the seeded workload, the rest same-distribution fills."""
    import torch
    from vecops_b200 import workloads
    a0 = workloads.make_a(w)
    b0 = workloads.make_b_nk(w, row0, row1)
    s0 = workloads.make_scale(w, row0, row1)
    bf16_a = w.kind in ("bf16", "w8")
    bf16_b = w.kind == "bf16"

    def up(x, as_bf16):
        t = torch.from_numpy(x).to(dev)
        return t.view(torch.bfloat16) if as_bf16 else t

    out_dtype = {"f32": torch.float32, "i8": torch.int32}.get(w.kind, torch.bfloat16)
    result = []
    for i in range(sets):
        if i == 0:
            a, b = up(a0, bf16_a), up(b0, bf16_b)
        else:
            a, b = result[0]["a"].clone(), result[0]["b"][torch.randperm(b0.shape[0], device=dev)].contiguous()
        if w.b_layout == "kn":
            b = b.t().contiguous().t()  # stored as a row-major [K,N] matrix, addressed as its [N,K] view
        result.append({"a": a, "b": b, "c": torch.empty((w.m, b0.shape[0]), dtype=out_dtype, device=dev),
                       "scale": up(s0, False) if s0 is not None else None})
    return result, (a0, b0, s0)


def time_steps(step, steps: int, warmup: int, stream) -> float:
    """Average milliseconds per step over exactly `steps` steps, CUDA events on `stream`."""
    import torch
    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for i in range(steps):
        step(warmup + i)
    stop.record(stream)
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / steps


def time_graph(prepared, steps: int, warmup: int, dev) -> float:
    """Average milliseconds per step: `steps` launches (cycling through `prepared`) captured in ONE CUDA graph, replayed
    once inside the timed region; a second graph of `warmup` launches runs first.  Kernels of ~10 us are otherwise bound
    by the host's launch rate rather than by the GPU."""
    import torch
    from vecops_b200 import harness
    stream = torch.cuda.Stream(dev)
    order = [prepared[i % len(prepared)] for i in range(max(steps, warmup))]
    warm = harness.capture_graph(order[:warmup], stream)
    timed = harness.capture_graph(order[:steps], stream)
    with torch.cuda.stream(stream):
        warm.replay()
        stream.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        timed.replay()
        stop.record(stream)
        stream.synchronize()
    return start.elapsed_time(stop) / steps


def size_matched_read(byte_count: float, sets: int, steps: int, warmup: int, dev) -> dict:
    """Context for an HBM-bound roofline fraction: a library reduction (torch fp32 sum) over buffers of the same byte count,
    rotated and timed exactly as the kernel is.  The measured HBM peak comes from a copy of gigabytes; a launch that moves
    tens of megabytes spends a large part of its few microseconds filling and draining the memory system, and this figure
    says how much of the peak a plain read of that size reaches.  A yardstick only: nothing on the product path calls it."""
    import torch
    count = int(byte_count) // 4
    buffers = [torch.ones(count, dtype=torch.float32, device=dev) for _ in range(sets)]
    outs = [torch.empty(1, dtype=torch.float32, device=dev) for _ in range(sets)]
    stream = torch.cuda.Stream(dev)

    def capture(launches: int):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(launches):
                torch.sum(buffers[i % sets], dim=(0,), keepdim=True, out=outs[i % sets])
        return graph

    with torch.cuda.stream(stream):
        torch.sum(buffers[0], dim=(0,), keepdim=True, out=outs[0])
        stream.synchronize()
    warm, timed = capture(max(warmup, 3)), capture(steps)
    with torch.cuda.stream(stream):
        warm.replay()
        stream.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        timed.replay()
        stop.record(stream)
        stream.synchronize()
    ms = start.elapsed_time(stop) / steps
    del buffers, outs
    return {"kernel": "torch.sum over fp32, one launch per buffer", "bytes_per_launch": count * 4, "ms_per_launch": ms,
            "gb_per_s": count * 4 / (ms * 1e-3) / 1e9, "sets": sets}


def take_status(device: int = 0) -> int:
    from vecops_b200 import capi
    status = ctypes.c_uint32(0)
    error = capi.ErrorBuffer()
    capi.library().vecops_b200_take_device_status(device, byref(status), byref(error.record))
    return status.value


def parity_sample(w, host_inputs, c, port, rows: int = 16) -> dict:
    """Checker on a few output rows of the seeded operand set."""
    import torch
    from oracle.checker import bf16_bits_to_f32, rel_frobenius
    a0, b0, s0 = host_inputs
    pick = np.unique(np.linspace(0, a0.shape[0] - 1, rows).astype(np.int64))
    got = c[torch.from_numpy(pick).to(c.device)]
    if w.kind == "i8":
        want = port.matmul_i8(a0[pick], b0)
        return {"rows": len(pick), "bit_exact": bool(np.array_equal(got.cpu().numpy(), want))}
    if w.kind == "f32":
        return {"rows": len(pick), "rel_fro": rel_frobenius(got.cpu().numpy(), port.matmul_f32(a0[pick], b0))}
    got = bf16_bits_to_f32(got.contiguous().view(torch.int16).cpu().numpy().view(np.uint16))
    want = port.matmul_bf16(a0[pick], b0) if w.kind == "bf16" else port.matmul_w8(a0[pick], b0, s0)
    return {"rows": len(pick), "rel_fro": rel_frobenius(got, bf16_bits_to_f32(want))}


def bound_of(w, peaks, peak_source: str, kernel_ms: float, kernel: str = "") -> tuple[str, float, float, str, str]:
    """(bound, peak, nominal peak, unit, where the peak comes from) of the roofline that limits workload `w`."""
    if w.kind == "f32" and kernel == "f32_tf32x3":
        # three tf32 products per fp32 product: the ceiling for ALGORITHMIC fp32 flops is a third of the tf32 tensor rate
        third = NOMINAL["tf32_tflops"] / 3.0
        return "tensor", third, third, "TFLOP/s", ("NOMINAL dense tf32 rate / 3 (three tf32 products per fp32 product; no tf32 peak is measured on this pool); "
                                                   f"the FP32 FMA pipe's nominal rate is {NOMINAL['fp32_tflops']} TFLOP/s")
    burst = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    sustained = float(peaks.get("bf16_tflops_sustained", burst))
    tensor, which = (burst, "burst") if kernel_ms < BURST_BELOW_MS else (sustained, "sustained")
    if w.kind == "bf16":
        return "tensor", tensor, NOMINAL["bf16_tflops"], "TFLOP/s", f"{peak_source}: cuBLAS bf16 {which} ({'<' if which == 'burst' else '>='} {BURST_BELOW_MS:g} ms per launch)"
    if w.kind == "i8":
        return "tensor", 2.0 * tensor, NOMINAL["i8_tops"], "TOP/s", f"ASSUMED 2 x the {peak_source} cuBLAS bf16 {which} figure: no int8 peak is measured on this pool"
    if w.kind == "w8":
        return "hbm", float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"])), NOMINAL["hbm_gbs"], "GB/s", f"{peak_source}: device-to-device copy"
    return "fp32_fma", NOMINAL["fp32_tflops"], NOMINAL["fp32_tflops"], "TFLOP/s", "nominal FP32 FMA rate (128 lanes x 148 SMs x 2 x 1.965 GHz); no measured figure exists"


def roofline_record(w, name: str, kernel: str, kernel_ms: float, flops: float, algorithmic_bytes: float, peaks, peak_source: str) -> dict:
    """The roofline object of one kernel launch: achieved = algorithmic work per launch / measured launch time."""
    bound, peak, nominal, unit, source = bound_of(w, peaks, peak_source, kernel_ms, kernel)
    seconds = kernel_ms * 1e-3
    achieved = algorithmic_bytes / seconds / 1e9 if bound == "hbm" else flops / seconds / 1e12
    traffic, traffic_from = NCU_TRAFFIC.get(name, (None, None))
    return {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak, "traffic": traffic,
            "traffic_source": traffic_from, "peak_source": source, "frac_of_nominal": achieved / nominal, "nominal_peak": nominal,
            "kernel": kernel, "kernel_ms": kernel_ms, "algorithmic_flops_per_launch": flops,
            "algorithmic_bytes_per_launch": algorithmic_bytes}


def operand_sets_for(w) -> int:
    """Operand sets to rotate so that no launch finds its operands in the 126 MB L2."""
    l2 = 126e6
    return 1 if w.algorithmic_bytes > 1.5 * l2 else int(np.ceil(1.6 * l2 / w.algorithmic_bytes)) + 1


def measure_single(name: str, steps: int, warmup: int, dev, port, peaks, peak_source: str = "measured", fused: bool = False,
                   full_record: bool = True) -> dict:
    """One single-GPU configuration: the kernel with operands resident in HBM (value, roofline), the same step end to end
    through the operator bridge with host buffers (e2e), and the reference's CPU matmul on the host cores (cpu_baseline).
    `fused`: the same launches with a bias row as the accumulator input and SiLU as the output transform (what the fused
    epilogue costs on top of the plain GEMM); kernel figures only."""
    import torch

    import vecops_b200
    from vecops_b200 import capi, harness, workloads
    w = workloads.WORKLOADS[name]
    per_set = w.algorithmic_bytes
    sets = operand_sets_for(w)
    operands, host_inputs = device_sets(w, sets, dev)
    stream = torch.cuda.current_stream(dev)
    kernel = vecops_b200.select_kernel(vecops_b200.matmul_problem(operands[0]["a"], operands[0]["b"], operands[0]["c"], operands[0]["scale"]))
    kernel_name = capi.library().vecops_b200_kernel_name(kernel).decode()

    if fused:
        from oracle.checker import ACT_SILU, bf16_bits_to_f32, rel_frobenius
        bias_host = np.random.default_rng(5).uniform(-1, 1, w.n).astype(np.float32)
        bias = torch.from_numpy(bias_host).to(dev)
        record = harness.epilogue_record(bias, 1.0, capi.ACTIVATION_SILU, 0.0, 0.0, w.m, w.n)
        prepared = [harness.PreparedMatmul(o["a"], o["b"], o["c"], o["scale"], stream=stream, epilogue=record, keep=(bias,)) for o in operands]
        prepared[0].launch()
        torch.cuda.synchronize()
        a0, b0, _ = host_inputs
        pick = np.unique(np.linspace(0, w.m - 1, 8).astype(np.int64))
        got = operands[0]["c"][torch.from_numpy(pick).to(dev)].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
        want = port.matmul_bf16_fused(a0[pick], b0, bias_host, 1.0, None, ACT_SILU)
        parity = {"rows": len(pick), "rel_fro": rel_frobenius(bf16_bits_to_f32(got), bf16_bits_to_f32(want))}
    else:
        prepared = [harness.PreparedMatmul(o["a"], o["b"], o["c"], o["scale"], stream=stream) for o in operands]
        prepared[0].launch()
        torch.cuda.synchronize()
        parity = parity_sample(w, host_inputs, operands[0]["c"], port)
    before = capi.library().vecops_b200_launch_count()
    ms = time_graph(prepared, steps, warmup, dev)
    launches = capi.library().vecops_b200_launch_count() - before  # counted while the graphs were captured: steps + warm-up + set-up
    status = take_status(dev.index or 0)
    roofline = roofline_record(w, name, kernel_name, ms, w.flops, per_set, peaks, peak_source)
    record = {"workload": name + (" + bias row + SiLU, fused" if fused else ""), "description": w.description, "kernel": kernel_name,
              "ms_per_step": ms, "steps": steps, "warmup": warmup, "value": roofline["achieved"], "unit": roofline["unit"],
              "tflops": w.flops / (ms * 1e-3) / 1e12, "algorithmic_gb_per_s": per_set / (ms * 1e-3) / 1e9,
              "roofline": roofline, "gpu_launches_captured": int(launches),
              "l2": f"rotating {sets} operand sets ({sets * per_set / 1e6:.0f} MB) vs L2 126 MB",
              "launch": "one CUDA graph of all timed launches, CUDA events around its replay", "parity": parity, "device_status": status}
    if fused or not full_record:
        return record
    if roofline["bound"] == "hbm":
        try:
            read = size_matched_read(per_set, sets, steps, warmup, dev)
            read["frac_of_peak"] = read["gb_per_s"] / roofline["peak"]
            read["kernel_vs_read"] = roofline["achieved"] / read["gb_per_s"]
            roofline["size_matched_read"] = read
        except Exception as error:  # noqa: BLE001 - context only
            roofline["size_matched_read"] = {"error": repr(error)}
    try:
        e2e_steps = 20 if w.kind != "w8" else 200
        e2e = measure_e2e(w, operands, host_inputs, e2e_steps, 3, dev, resident_weights=w.kind == "w8")
        work = per_set / 1e9 if roofline["bound"] == "hbm" else w.flops / 1e12
        # steps of a few tens of microseconds gain nothing from three streams and their event traffic: the faster of the two ways counts
        best_ms = min(e2e["ms_per_step"], e2e["serial_ms_per_step"])
        record["e2e"] = {"value": work / (best_ms * 1e-3), "unit": roofline["unit"], "ms_per_step": best_ms,
                         "pipelined_ms_per_step": e2e["ms_per_step"],
                         "serial_ms_per_step": e2e["serial_ms_per_step"], "serial_value": work / (e2e["serial_ms_per_step"] * 1e-3),
                         "h2d_bytes_per_step": e2e["h2d_bytes_per_step"], "d2h_bytes_per_step": e2e["d2h_bytes_per_step"], "steps": e2e_steps,
                         "resident": e2e["resident"], "host_overhead_us_per_call": e2e["host_us_per_call"],
                         "bridge_calls": e2e["bridge_calls"],
                         "path": "vecops_operator_bridge_invoke_v1, pinned host buffers, copies inside the timed region"}
    except Exception as error:  # noqa: BLE001 - a failed side measurement must not lose the kernel number
        record["e2e"] = {"error": repr(error)}
    del operands, prepared
    torch.cuda.empty_cache()
    try:
        record["cpu_baseline"] = cpu_baseline(w)
    except Exception as error:  # noqa: BLE001
        record["cpu_baseline"] = {"error": repr(error)}
    return record


def measure_f16(steps: int, warmup: int, dev, port, peaks) -> dict:
    """The fp16 row at C2's shape (fp16 x fp16, fp32 accumulate, fp16 out) on the 16-bit tensor-core kernel."""
    import torch
    from oracle.checker import rel_frobenius
    from vecops_b200 import capi, harness
    m = n = k = 4096
    rng = np.random.default_rng(7)
    a_host = rng.standard_normal((m, k), dtype=np.float32).astype(np.float16)
    b_host = rng.standard_normal((n, k), dtype=np.float32).astype(np.float16)
    stream = torch.cuda.current_stream(dev)
    sets = []
    for i in range(4):  # 4 x 100 MB of operands and results: more than L2
        a = torch.from_numpy(a_host).to(dev)
        b = torch.from_numpy(b_host).to(dev) if i == 0 else sets[0][1][torch.randperm(n, device=dev)].contiguous()
        sets.append((a, b, torch.empty((m, n), dtype=torch.float16, device=dev)))
    prepared = [harness.PreparedMatmul(a, b, c, None, stream=stream) for a, b, c in sets]
    prepared[0].launch()
    torch.cuda.synchronize()
    pick = np.unique(np.linspace(0, m - 1, 8).astype(np.int64))
    want = port.matmul_f16(a_host[pick].view(np.uint16), b_host.view(np.uint16), out_f16=True).view(np.float16).astype(np.float32)
    got = sets[0][2][torch.from_numpy(pick).to(dev)].float().cpu().numpy()
    ms = time_graph(prepared, steps, warmup, dev)
    tflops = 2.0 * m * n * k / (ms * 1e-3) / 1e12
    return {"workload": "fp16 x fp16 -> fp16, M=N=K=4096, fp32 accumulate", "kernel": "bf16_tcgen05 (fp16 operand formats)", "ms_per_step": ms,
            "value": tflops, "unit": "TFLOP/s", "bound": "tensor", "frac_of_measured_peak": tflops / float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"])),
            "l2": "rotating 4 operand sets (403 MB) vs L2 126 MB", "parity": {"rows": len(pick), "rel_fro": rel_frobenius(got, want)},
            "device_status": take_status(dev.index or 0)}


def measure_pack(dev, peaks) -> dict:
    """Operand preparation at C4's weight shape: a [K, N]-stored matrix (N = 14336, K = 4096) transposed into the packed
    [N, K] form, and the row copy of an already K-contiguous one.  HBM-bound: every element read once, written once."""
    import torch
    from vecops_b200 import capi, harness
    n, k = 14336, 4096
    hbm = float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
    side = torch.cuda.Stream(dev)
    out = {}
    for name, dtype, narrow in [("bf16", torch.bfloat16, None), ("i8", torch.int8, None), ("f32_to_bf16", torch.float32, torch.bfloat16)]:
        sources = []
        for i in range(3):  # three sources and destinations in rotation: more than L2 between reuses
            if dtype == torch.int8:
                sources.append(torch.randint(-128, 128, (k, n), dtype=torch.int8, device=dev))
            else:
                sources.append(torch.randn((k, n), dtype=torch.float32, device=dev).to(dtype))
        pitch, size = harness.packed_layout(narrow or dtype, n, k)
        packed = [torch.empty((n, pitch), dtype=narrow or dtype, device=dev) for _ in sources]
        for form in ("transpose", "row_copy"):
            views = [x.t() if form == "transpose" else x.t().contiguous() for x in sources]
            records = [capi.VecopsB200Pack(ctypes.sizeof(capi.VecopsB200Pack), 1, n, k, v.data_ptr(), v.stride(0), v.stride(1),
                                           harness.torch_dtype_code(v.dtype), harness.torch_dtype_code(d.dtype), d.data_ptr(), size, dev.index or 0, 0,
                                           side.cuda_stream) for v, d in zip(views, packed)]
            error = capi.ErrorBuffer()
            count = 12
            torch.cuda.synchronize()
            with torch.cuda.stream(side):
                error.raise_for(capi.library().vecops_b200_matmul_pack(byref(records[0]), byref(error.record)))  # warm-up, outside the graph
                side.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for i in range(count):
                        error.raise_for(capi.library().vecops_b200_matmul_pack(byref(records[i % 3]), byref(error.record)))
                for _ in range(20):  # warm-up: clocks up, caches in their steady state
                    graph.replay()
                side.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(side)
                for _ in range(5):
                    graph.replay()
                e1.record(side)
                side.synchronize()
            ms = e0.elapsed_time(e1) / (5 * count)
            moved = n * k * (views[0].element_size() + packed[0].element_size())
            got = packed[2][:64, :64].float().cpu()
            want = views[2][:64, :64].to(narrow or dtype).float().cpu()
            out[f"{name}_{form}"] = {"ms": ms, "algorithmic_gb_per_s": moved / (ms * 1e-3) / 1e9, "frac_of_measured_hbm_peak": moved / (ms * 1e-3) / 1e9 / hbm,
                                     "equal_sample": bool(torch.equal(got, want))}
            del views, graph
        del sources, packed
        torch.cuda.empty_cache()
    return {"workload": "pack of a [14336, 4096] operand from a [K, N]-stored (transpose) or [N, K]-stored (row copy) source", "bound": "hbm",
            "timing": "a CUDA graph of 12 launches (three source/destination sets in rotation), 20 warm-up replays, 5 timed", "cases": out}


def measure_sdpa_case(dev, port, heads: int, length: int, d: int, strategy: int, sets: int, own_scratch: bool) -> dict:
    """Attention over `heads` heads of Lq = Lkv = `length`, head dim `d`, bottom-right causal, bf16 in and out, through
    vecops_b200_sdpa_run with the given strategy.  All launches of all timed steps are ONE CUDA graph (the host's launch rate
    is not what gets measured); `sets` operand sets are taken in turn so that no step finds its operands in the 126 MB L2."""
    import torch
    from oracle.checker import bf16_bits_to_f32, rel_frobenius
    from vecops_b200 import capi, harness
    rng = np.random.default_rng(9)
    scale = 1.0 / np.sqrt(d)
    host = [workloads_bf16(rng.standard_normal((heads, length, d)).astype(np.float32)) for _ in range(3)]
    stream = torch.cuda.current_stream(dev)
    error = capi.ErrorBuffer()
    records, keep_alive = [], []
    need = ctypes.c_uint64(0)
    shared = None
    for index in range(sets):
        q, k, v = (torch.from_numpy(x).to(dev).view(torch.bfloat16) for x in host)
        out = torch.empty((heads, length, d), dtype=torch.bfloat16, device=dev)
        record = harness.sdpa_record(q, k, v, out, scale, causal=capi.CAUSAL_BOTTOM_RIGHT, stream=stream, asynchronous=True, strategy=strategy)
        error.raise_for(capi.library().vecops_b200_sdpa_workspace(byref(record), byref(need), byref(error.record)))
        if own_scratch or shared is None:
            shared = torch.empty(need.value + 256, dtype=torch.uint8, device=dev)
        record.workspace, record.workspace_size = shared.data_ptr() + (-shared.data_ptr()) % 256, need.value
        records.append(record)
        keep_alive.append((q, k, v, out, shared))
    run = lambda r: error.raise_for(capi.library().vecops_b200_sdpa_run(byref(r), byref(error.record)))  # noqa: E731
    before = capi.library().vecops_b200_launch_count()
    run(records[0])
    launches = capi.library().vecops_b200_launch_count() - before
    torch.cuda.synchronize()
    chosen, tiles = harness.sdpa_plan(records[0])
    pick = np.unique(np.linspace(0, length - 1, 8).astype(np.int64))
    keep = (np.arange(length)[None, :] <= pick[:, None]).astype(np.uint8)
    last = heads - 1
    if chosen == capi.SDPA_STREAMING:  # held to the restatement of ITS strategy, keys cut into chunks as the launch cuts them
        want = port.sdpa_bf16_streaming(host[0][last][pick], host[1][last], host[2][last], scale, keep_mask=keep, out_bf16=True, chunk_blocks=tiles)
    else:
        want = port.sdpa_bf16(host[0][last][pick], host[1][last], host[2][last], scale, keep_mask=keep, out_bf16=True)
    got = keep_alive[0][3][last][torch.from_numpy(pick).to(dev)].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    count = max(sets, 24 // max(1, heads // 8) if heads > 1 else 48)
    side = torch.cuda.Stream(dev)
    for record in records:
        record.stream = side.cuda_stream
    side.wait_stream(stream)
    with torch.cuda.stream(side):
        for record in records:  # one-time set-up outside the capture
            run(record)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(count):
                run(records[i % sets])
        graph.replay()  # warm-up
        side.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(side)
        graph.replay()
        e1.record(side)
        side.synchronize()
    stream.wait_stream(side)
    ms = e0.elapsed_time(e1) / count
    dense = 4.0 * heads * length * length * d  # both products over the whole square
    needed = dense * (length + 1) / (2.0 * length)  # what the causal cut leaves
    names = {capi.SDPA_MATERIALIZED: "materialized", capi.SDPA_STREAMING: "streaming"}
    operand_mb = 4 * heads * length * d * 2 / 1e6
    return {"strategy": names[chosen], "heads": heads, "ms_per_step": ms, "launches_per_step": int(launches),
            "tiles_per_work_item": int(tiles), "dense_tflops": dense / (ms * 1e-3) / 1e12, "causal_tflops": needed / (ms * 1e-3) / 1e12,
            "scratch_mb": need.value / 1e6,
            "l2": f"{sets} operand sets of {operand_mb:.1f} MB" + (f" with {need.value / 1e6:.0f} MB of scratch each" if own_scratch else "") + " in turn vs L2 126 MB",
            "launch": f"one CUDA graph of {count} steps, CUDA events around its replay",
            "parity": {"rows": len(pick), "rel_fro": rel_frobenius(bf16_bits_to_f32(got), bf16_bits_to_f32(want))}, "device_status": take_status(dev.index or 0)}


def measure_sdpa(dev, port) -> dict:
    """The caller one step up: attention at Lq = Lkv = 4096, D = 128, bottom-right causal, bf16 - one head by both of the
    reference's strategies (streaming: one kernel, nothing of size Lq x Lkv in memory; materialized: two products
    through the matmul path around a row softmax, scores making a round trip), and 32 heads by the streaming one."""
    from vecops_b200 import capi
    one = measure_sdpa_case(dev, port, 1, 4096, 128, capi.SDPA_AUTOMATIC, sets=48, own_scratch=False)
    old = measure_sdpa_case(dev, port, 1, 4096, 128, capi.SDPA_MATERIALIZED, sets=2, own_scratch=True)
    many = measure_sdpa_case(dev, port, 32, 4096, 128, capi.SDPA_AUTOMATIC, sets=2, own_scratch=False)
    return {"workload": "attention, one head, Lq=Lkv=4096, D=128, bottom-right causal, bf16", **one,
            "materialized": old, "heads_32": many,
            "note": "automatic takes the streaming kernel; `materialized` is the same call forced onto the composition through "
                    "the matmul path (scores 67 MB f32 and probabilities 34 MB bf16 pass through device memory)"}


def workloads_bf16(values):
    from vecops_b200 import workloads
    return workloads.f32_to_bf16_bits(values)


def measure_quantized(steps: int, warmup: int, dev, port, peaks) -> dict:
    """The quantised form at C3's size: fp32 activations quantised to u8 (pre-pass), s8 weights, int32 correction row, dequantising
    transform with a per-column scale, bf16 out.  The timed launches are the product kernel alone; the pre-passes are timed beside it."""
    import torch
    from oracle.checker import bf16_bits_to_f32, rel_frobenius
    from vecops_b200 import capi, harness
    m, n, k = 4096, 14336, 4096
    rng = np.random.default_rng(6)
    a_host = rng.uniform(-20, 40, (m, k)).astype(np.float32)
    b_host = [rng.integers(-128, 128, (n, k), dtype=np.int8) for _ in range(2)]
    scale_host = rng.uniform(0.5, 2.0, n).astype(np.float32)
    a32 = torch.from_numpy(a_host).to(dev)
    qa = torch.empty((m, k), dtype=torch.uint8, device=dev)
    bs = [torch.from_numpy(x).to(dev) for x in b_host]
    scale = torch.from_numpy(scale_host).to(dev)
    corrections = [torch.empty(n, dtype=torch.int32, device=dev) for _ in bs]
    stream = torch.cuda.current_stream(dev)

    def timed(fn, count=20):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(count):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / count

    quantize_ms = timed(lambda: harness.quantize_rows(a32, qa, 2.0, 5.0))
    correction_ms = timed(lambda: harness.column_correction(bs[0], 5, corrections[0]))
    harness.column_correction(bs[1], 5, corrections[1])
    outs = [torch.empty((m, n), dtype=torch.bfloat16, device=dev) for _ in bs]
    prepared = [harness.PreparedMatmul(qa, bs[j], outs[j], scale, stream=stream,
                                       epilogue=harness.epilogue_record(corrections[j], 0.01, capi.ACTIVATION_NONE, 0.0, 0.0, m, n),
                                       keep=(corrections[j],)) for j in range(2)]
    prepared[0].launch()
    torch.cuda.synchronize()
    pick = np.unique(np.linspace(0, m - 1, 8).astype(np.int64))
    quantized_rows = port.quantize_rows(a_host[pick], 2.0, 5.0)
    correction_host = (-5 * b_host[0].astype(np.int64).sum(axis=1)).astype(np.int32)
    want = port.matmul_i8_dequant(quantized_rows, b_host[0], correction_host, 0.01, scale_host, out_bf16=True)
    got = outs[0][torch.from_numpy(pick).to(dev)].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    parity = {"rows": len(pick), "rel_fro": rel_frobenius(bf16_bits_to_f32(got), bf16_bits_to_f32(want)),
              "quantized_rows_equal": bool(np.array_equal(qa[torch.from_numpy(pick).to(dev)].cpu().numpy(), quantized_rows)),
              "correction_equal": bool(np.array_equal(corrections[0].cpu().numpy(), correction_host))}
    ms = time_graph(prepared, steps, warmup, dev)
    tops = 2.0 * m * n * k / (ms * 1e-3) / 1e12
    peak = 2.0 * float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))  # assumed: twice the measured bf16 burst figure
    return {"workload": "c3 shape, quantised form: u8 (quantised fp32) x s8 + int32 correction row, dequantised and column-scaled to bf16",
            "kernel": "i8_tcgen05", "ms_per_step": ms, "value": tops, "unit": "TOP/s", "bound": "tensor", "frac_of_measured_peak": tops / peak,
            "quantize_rows_ms": quantize_ms, "column_correction_ms": correction_ms,
            "ms_per_step_with_quantize_rows": ms + quantize_ms, "value_with_quantize_rows": 2.0 * m * n * k / ((ms + quantize_ms) * 1e-3) / 1e12,
            "note": "the activations are quantised by a pre-pass kernel, once per product; the correction row is computed once per weight matrix",
            "parity": parity, "device_status": take_status(dev.index or 0),
            "launch": "one CUDA graph of all timed launches; two weight sets (235 MB) > L2"}


def bridge_invoker():
    """Returns prepare(a, b, c, scale, stream) -> call(): the call frame is built once, as a C caller keeps it on its stack,
    and call() is ONE asynchronous vecops_operator_bridge_invoke_v1 (the reference-facing entry) over it."""
    from vecops_b200 import capi
    lib = capi.library()
    lib.vecops_b200_matmul_operator.restype = ctypes.c_uint64
    lib.vecops_operator_bridge_invoke_v1.argtypes = [ctypes.c_uint64, ctypes.POINTER(capi.VecopsCall), ctypes.c_uint32, ctypes.c_void_p,
                                                     ctypes.POINTER(capi.VecopsError)]
    lib.vecops_b200_operator_workspace.argtypes = [ctypes.c_uint64, ctypes.POINTER(capi.VecopsCall), ctypes.POINTER(ctypes.c_uint64),
                                                   ctypes.POINTER(capi.VecopsError)]
    handle = lib.vecops_b200_matmul_operator()
    invoke = lib.vecops_operator_bridge_invoke_v1

    import torch

    import vecops_b200

    def value_of(t, writable, keep):
        sizes = (ctypes.c_int64 * t.dim())(*t.shape)
        strides = (ctypes.c_int64 * t.dim())(*t.stride())
        keep += [sizes, strides]
        v = capi.VecopsValue()
        v.struct_size = ctypes.sizeof(capi.VecopsValue)
        v.kind = capi.VALUE_TENSOR
        tv = v.value.tensor
        tv.struct_size = ctypes.sizeof(capi.VecopsTensorView)
        tv.data, tv.byte_offset = t.data_ptr(), 0
        tv.device_type, tv.device_index = capi.DEVICE_CUDA, t.device.index
        tv.dtype, tv.rank, tv.sizes, tv.strides = vecops_b200.torch_dtype_code(t.dtype), t.dim(), sizes, strides
        tv.flags = capi.TENSOR_READ | (capi.TENSOR_WRITE if writable else 0)
        return v

    def prepare(a, b, c, scale, stream):
        keep: list = [a, b, c, scale]
        values = [value_of(a, False, keep), value_of(b, False, keep), value_of(c, True, keep)]
        if scale is not None:
            values.append(value_of(scale, False, keep))
        array = (capi.VecopsValue * len(values))(*values)
        context = capi.VecopsExecutionContext()
        context.struct_size = ctypes.sizeof(context)
        context.stream = stream.cuda_stream
        context.flags = capi.CONTEXT_FLAG_ASYNC
        frame = capi.VecopsCall(ctypes.sizeof(capi.VecopsCall), len(values), array, None, 0, ctypes.pointer(context))
        error = capi.ErrorBuffer()
        need = ctypes.c_uint64(0)
        error.raise_for(lib.vecops_b200_operator_workspace(handle, byref(frame), byref(need), byref(error.record)))
        if need.value:  # device workspace sized by the operator's own query, one per prepared call
            scratch = torch.empty(need.value, dtype=torch.uint8, device=c.device)
            frame.workspace, frame.workspace_size = scratch.data_ptr(), scratch.numel()
            keep.append(scratch)
        keep += [array, context]
        frame_ref, error_ref = byref(frame), byref(error.record)

        def call(_keep=keep):
            rc = invoke(handle, frame_ref, 0, None, error_ref)
            if rc != capi.OK:
                error.raise_for(rc)

        return call

    return prepare


def async_copier():
    """copy(dst_ptr, src_ptr, bytes, stream): cudaMemcpyAsync through the CUDA runtime the process already has loaded - what
    a C caller of the bridge issues around its call.  (torch's Tensor.copy_ costs ~10 us of Python per copy, which would
    be the measurement for the decode shapes.)"""
    try:
        runtime = ctypes.CDLL("libcudart.so.12")
        fn = runtime.cudaMemcpyAsync
        fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
        fn.restype = ctypes.c_int
    except (OSError, AttributeError):
        return None

    def copy(dst: int, src: int, count: int, stream) -> None:
        rc = fn(dst, src, count, 4, stream.cuda_stream)  # 4 = cudaMemcpyDefault
        if rc != 0:
            raise RuntimeError(f"cudaMemcpyAsync failed with code {rc}")

    return copy


def measure_e2e(w, operands, host_inputs, steps: int, warmup: int, dev, resident_weights: bool = False) -> dict:
    """The same step through the operator bridge with pinned host buffers; every step's copies are inside the timed region.

    Two measurements.  `serial`: copy in, run, copy out on one stream, one step after the other (the latency of a step).
    `pipelined` (the reported value): two operand sets in flight on three streams, so that the host-to-device copy of
    step i+1 and the device-to-host read of step i-1 overlap step i; still one copy-in and one read-back per step.
    `resident_weights` (the decode shapes): the weight matrix and its scales stay on the device, as a decode loop keeps
    them; a step copies the activations in and the result out.
    """
    import torch
    a0, b0, s0 = host_inputs
    prepare = bridge_invoker()
    copy = async_copier()
    host_a = torch.from_numpy(a0).pin_memory()
    host_b_src = b0 if w.b_layout == "nk" else np.ascontiguousarray(b0.T)
    host_b = None if resident_weights else torch.from_numpy(host_b_src).pin_memory()

    def nbytes(t):
        return t.numel() * t.element_size()

    lanes = []
    # resident weights must still come from HBM, not from L2: rotate over every operand set the caller made
    n_lanes = max(2, len(operands)) if resident_weights else 2
    for i in range(n_lanes):
        if i < len(operands):
            o = operands[i]
        else:  # a configuration that keeps one operand set: give the second lane its own buffers
            first = operands[0]
            o = {"a": torch.empty_like(first["a"]), "b": first["b"] if resident_weights else torch.empty_like(first["b"]),
                 "c": torch.empty_like(first["c"]), "scale": first["scale"]}
        b_storage = o["b"] if w.b_layout == "nk" else o["b"].t()  # the contiguous storage behind the [N,K] view
        assert o["a"].is_contiguous() and b_storage.is_contiguous() and o["c"].is_contiguous()
        lanes.append({"o": o, "a_ptr": o["a"].data_ptr(), "b_ptr": b_storage.data_ptr(), "c_ptr": o["c"].data_ptr(),
                      "host_c": torch.empty(o["c"].shape, dtype=o["c"].dtype).pin_memory(),
                      "loaded": torch.cuda.Event(), "computed": torch.cuda.Event(), "read": torch.cuda.Event(), "used": False})
    a_bytes, c_bytes = nbytes(host_a), nbytes(lanes[0]["host_c"])
    b_bytes = 0 if resident_weights else nbytes(host_b)
    main = torch.cuda.current_stream(dev)

    def copy_in(lane, stream):
        if copy is not None:
            copy(lane["a_ptr"], host_a.data_ptr(), a_bytes, stream)
            if not resident_weights:
                copy(lane["b_ptr"], host_b.data_ptr(), b_bytes, stream)
        else:
            with torch.cuda.stream(stream):
                lane["o"]["a"].view(torch.uint8).view(-1).copy_(host_a.view(torch.uint8).view(-1), non_blocking=True)
                if not resident_weights:
                    storage = lane["o"]["b"] if w.b_layout == "nk" else lane["o"]["b"].t()
                    storage.view(torch.uint8).view(-1).copy_(host_b.view(torch.uint8).view(-1), non_blocking=True)

    def copy_out(lane, stream):
        if copy is not None:
            copy(lane["host_c"].data_ptr(), lane["c_ptr"], c_bytes, stream)
        else:
            with torch.cuda.stream(stream):
                lane["host_c"].copy_(lane["o"]["c"], non_blocking=True)

    serial_calls = [prepare(lane["o"]["a"], lane["o"]["b"], lane["o"]["c"], lane["o"]["scale"], main) for lane in lanes]
    host_seconds = [0.0]

    def serial_step(i):
        lane = lanes[i % n_lanes]
        copy_in(lane, main)
        t0 = time.perf_counter()
        serial_calls[i % n_lanes]()
        host_seconds[0] += time.perf_counter() - t0
        copy_out(lane, main)

    for i in range(warmup):
        serial_step(i)
    torch.cuda.synchronize()
    host_seconds[0] = 0.0
    serial_ms = time_steps(serial_step, steps, 0, main)
    host_us = host_seconds[0] / steps * 1e6

    s_in, s_run, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    calls = [prepare(lane["o"]["a"], lane["o"]["b"], lane["o"]["c"], lane["o"]["scale"], s_run) for lane in lanes]

    def pipelined_step(i):
        lane = lanes[i % n_lanes]
        if lane["used"]:
            s_in.wait_event(lane["computed"])  # the lane's previous run has read its A and B
        copy_in(lane, s_in)
        lane["loaded"].record(s_in)
        s_run.wait_event(lane["loaded"])
        if lane["used"]:
            s_run.wait_event(lane["read"])  # the lane's previous C has reached the host
        calls[i % n_lanes]()
        lane["computed"].record(s_run)
        s_out.wait_event(lane["computed"])
        copy_out(lane, s_out)
        lane["read"].record(s_out)
        lane["used"] = True

    def drain():
        for side in (s_in, s_run, s_out):
            main.wait_stream(side)

    for i in range(warmup):
        pipelined_step(i)
    drain()
    torch.cuda.synchronize(dev)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(main)
    for side in (s_in, s_run, s_out):
        side.wait_event(start)
    for i in range(steps):
        pipelined_step(warmup + i)
    drain()
    stop.record(main)
    torch.cuda.synchronize(dev)
    pipelined_ms = start.elapsed_time(stop) / steps
    # the read-back is the product's result: compare what reached the host with the device copy
    last = lanes[(warmup + steps - 1) % n_lanes]
    if not torch.equal(last["host_c"], last["o"]["c"].cpu()):
        raise RuntimeError("end-to-end read-back differs from the device result")
    slow, prepared = ctypes.c_uint64(0), ctypes.c_uint64(0)
    from vecops_b200 import capi
    capi.library().vecops_b200_bridge_counters(byref(slow), byref(prepared))
    return {"ms_per_step": pipelined_ms, "serial_ms_per_step": serial_ms, "h2d_bytes_per_step": int(a_bytes + b_bytes),
            "bridge_calls": {"full_path": slow.value, "prepared_path": prepared.value, "note": "process totals: the full path (bind, validate, dispatch, resolve) runs once per call signature, the prepared path re-enters the resolved executable"},
            "d2h_bytes_per_step": int(c_bytes), "host_us_per_call": host_us,
            "resident": "weights and scales stay on the device; a step copies the activations in and the result out" if resident_weights else "nothing: every operand is copied in every step",
            "copies": "cudaMemcpyAsync from / to pinned host memory" + ("" if copy is not None else " (through torch)")}


def cpu_sample(w, ref, cores: int):
    """(run, rows, cols, kind, isa, note): the bounded sample of workload `w` the CPU baseline times, and how.

    The reference's own code wherever it has any for the row: ops::matmul on AMX for bf16, int8 and the weight-only
    expression, its AVX-512 fmadd leaf for fp32 (its matmul has no fp32 atom on x86).  Large problems are sampled and the
    throughput of the sample is reported: a row block of the big bf16 GEMM, a column block of the weight-only shapes
    (the reference's int8->bf16 conversion path is untuned and takes ~45 ms per 1024 columns)."""
    from oracle.checker import Port
    from vecops_b200 import workloads
    if ref is not None:
        rows = w.m if w.flops <= 6e11 else 256
        cols = w.n if w.kind != "w8" else min(w.n, 1024 * cores)
        a, b = workloads.make_a(w, 0, rows), workloads.make_b_nk(w, 0, cols)
        s = workloads.make_scale(w, 0, cols)
        run = {"bf16": lambda: ref.matmul_bf16(a, b, True, cores), "i8": lambda: ref.matmul_i8(a, b, cores),
               "w8": lambda: ref.matmul_w8(a, b, s, cores), "f32": lambda: ref.matmul_f32_leaf(a, b, cores)}[w.kind]
        isa = {"bf16": "AMX-BF16 (tdpbf16ps) through the reference's ops::matmul<AMX_BF16F32>",
               "i8": "AMX-INT8 (tdpbssd) through the reference's ops::matmul<AMX_I8I32>",
               "w8": "AMX-BF16 through the reference's ops::matmul<AMX_BF16F32> with input<bfloat16_t>(int8 W) and a per-column scale transform",
               "f32": "AVX-512 fmadd: the reference's small_vector_dense_matmul leaf (its matmul has no fp32 atom on x86), B transposed to [N,K] beforehand"}[w.kind]
        note = "" if (rows, cols) == (w.m, w.n) else " (throughput of the sample: the work is linear in the sampled extent)"
        return run, rows, cols, "reference", isa, note
    port = Port()
    rows, cols = min(w.m, 64), w.n
    a, b = workloads.make_a(w, 0, rows), workloads.make_b_nk(w, 0, cols)
    s = workloads.make_scale(w, 0, cols)
    run = {"bf16": lambda: port.matmul_bf16(a, b), "i8": lambda: port.matmul_i8(a, b), "w8": lambda: port.matmul_w8(a, b, s),
           "f32": lambda: port.matmul_f32(a, b)}[w.kind]
    return run, rows, cols, "port", "C restatement, OpenMP, compiler-vectorised", " (throughput of the sample)"


def cpu_baseline(w, repeats: int = 3) -> dict:
    """The reference's CPU matmul (or, where it cannot run, the C restatement) on a bounded sample of `w`, all host threads."""
    from oracle.checker import Port, Ref
    ref, why = Ref.load()
    cores = Ref.default_threads() if ref is not None else Port().threads
    run, rows, cols, kind, isa, note = cpu_sample(w, ref, cores)
    run()
    best = min(_timed(run) for _ in range(repeats))
    unit = "GB/s" if w.kind == "w8" else ("TOP/s" if w.kind == "i8" else "TFLOP/s")
    flops = 2.0 * rows * cols * w.k
    value = ((cols * w.k + 4 * cols + 2 * rows * w.k + 2 * rows * cols) / best / 1e9) if w.kind == "w8" else flops / best / 1e12
    record = {"value": value, "unit": unit, "cores": cores, "kind": kind, "isa": isa,
              "sample": f"{rows}x{cols}x{w.k} of {w.m}x{w.n}x{w.k}, best of {repeats}{note}", "seconds": best,
              "tflops": flops / best / 1e12}
    if why:
        record["reference_unavailable"] = why
    return record


def _timed(fn) -> float:
    t0 = time.perf_counter()
    fn()
    return time.perf_counter() - t0


HEADLINE = "c5_bf16_16384x53248x8192"
# the other single-GPU configurations, in the order they are reported: (workload, timed steps)
CONFIGS = [("c2_bf16_4096", 200), ("c1_f32_1024", 100), ("c3_i8_4096x14336x4096", 50), ("c4_w8_m1", 200), ("c4_w8_m16", 200),
           ("c4_w8_m128", 100)]


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    import vecops_b200
    from oracle.checker import Port
    from vecops_b200 import capi, harness, sharding, workloads

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        # NCCL may print a version banner on stdout when its communicator comes up; this program owes stdout ONE line,
        # so stdout is pointed at stderr until the first collective has run.
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=dev)
            warm = torch.zeros(1, device=dev)
            dist.all_reduce(warm)
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)
    lib = capi.library()
    peaks, peak_source = measured_peaks()
    port = Port()

    name = args.workload or HEADLINE
    w = workloads.WORKLOADS[name]
    if world > 1 and w.kind != "bf16":
        raise SystemExit("only the bf16 GEMM shards over GPUs; the other configurations are single-GPU")
    sharded = name == HEADLINE or world > 1   # the column-sharded operator (at one GPU its slab is the whole result)
    if not sharded:
        # any other workload alone on one GPU: the per-configuration record is the line
        steps = args.steps if args.steps is not None else dict(CONFIGS).get(name, 100)
        warmup = args.warmup if args.warmup is not None else 10
        with ClockSampler(local) as clocks:
            record = measure_single(name, steps, warmup, dev, port, peaks, peak_source)
        e2e = record.get("e2e", {})
        line = {"metric": METRIC, "value": record["value"], "unit": record["unit"], "n_gpus": 1, "steps": steps, "warmup": warmup,
                "ms_per_step": record["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": {"bf16": "bf16", "i8": "int8", "w8": "bf16 x int8 weights", "f32": "f32"}[w.kind],
                "data": "synthetic (seeded; shapes, layouts and value distributions of the named configuration)",
                "config": {"workload": name, "description": w.description, "m": w.m, "n": w.n, "k": w.k, "parallelism": "single GPU",
                           "l2": record["l2"], "timing": record["launch"]},
                "roofline": record["roofline"], "cpu_baseline": record.get("cpu_baseline"), "e2e": e2e,
                "gpu_launches": record["gpu_launches_captured"], "clocks": clocks.summary(), "parity": record["parity"],
                "device_status": record["device_status"]}
        print(json.dumps(line), flush=True)
        return

    steps = args.steps if args.steps is not None else 20
    warmup = args.warmup if args.warmup is not None else 3
    stream = torch.cuda.current_stream(dev)

    gather_mode = "none: one GPU owns every column, its slab is the result"
    n0, n1 = sharding.column_partition(w.n, world, rank)
    operands, host_inputs = device_sets(w, 1, dev, n0, n1)
    o = operands[0]
    a_peers = None
    if world > 1:
        # A lives in symmetric memory, so that the end-to-end step can copy in ONE row slice of A per rank and replicate
        # it over NVLink instead of pulling the whole of A over every rank's PCIe link
        try:
            import torch.distributed._symmetric_memory as symm_mem
            a_sym = symm_mem.empty(tuple(o["a"].shape), dtype=o["a"].dtype, device=dev)
            a_handle = symm_mem.rendezvous(a_sym, dist.group.WORLD)
            a_sym.copy_(o["a"])
            o["a"] = a_sym
            a_peers = {"handle": a_handle, "bases": [int(p) for p in a_handle.buffer_ptrs], "rank": rank, "world": world}
            built = 1
        except Exception as error:
            print(f"[bench] symmetric A unavailable on rank {rank}: {error!r}", file=sys.stderr)
            built = 0
        same = torch.tensor([built], device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        if int(same.item()) == 0:
            a_peers = None
    prepared = [harness.PreparedMatmul(o["a"], o["b"], o["c"], None, stream=stream)]  # the slab GEMM alone (roofline)
    full = pipe = full_of = None
    trials = {}
    step_join = lambda: None  # noqa: E731 - only the pipelined gather has work in flight on a second stream
    if world == 1:
        step_launch = prepared[0].launch
        launches_per_step = 1
    else:
        def fused_route(allow_multicast: bool):
            """The gather inside the GEMM's epilogue: each finished piece goes into every rank's result over NVLink."""
            result, hdl = sharding.symmetric_result(w.m, w.n, torch.bfloat16, dev)
            multicast = int(getattr(hdl, "multicast_ptr", 0) or 0) if allow_multicast else 0
            same = torch.tensor([1 if multicast else 0], device=dev)  # every rank must take the same route
            dist.all_reduce(same, op=dist.ReduceOp.MIN)
            if int(same.item()) == 1:
                # one store to the multicast address: the switch writes it into every rank's copy, own included
                targets = [multicast]
                mode = "fused: epilogue multimem.st to the NVSwitch multicast address of the result (one store, every rank's copy) + one device barrier"
            else:
                targets = [int(p) for p in hdl.buffer_ptrs]
                mode = "fused: epilogue TMA stores to every rank's result over NVLink peer pointers + one device barrier"
            gemm = sharding.FusedGatherGemm(o["a"], o["b"], targets, w.n, w.n, n0, torch.bfloat16, stream, multicast=len(targets) == 1)

            def launch():
                gemm.launch()
                hdl.barrier(channel=0)
            return {"launch": launch, "join": lambda: None, "full": lambda: result, "mode": mode, "launches_per_step": 1,
                    "buffers": result, "pipe": None, "keep": (gemm, hdl)}

        def pipelined_route(by_kernel: bool, lanes: int = 1):
            """The slab stored locally, pushed to the peers on a second stream behind the next step's GEMM (`lanes`:
            how many of the copy-engine copies to different peers are in flight at once, each on a stream of its own)."""
            results, hdl = sharding.symmetric_result(w.m, w.n, torch.bfloat16, dev, copies=2)
            lanes = 1 if by_kernel else int(os.environ.get("VECOPS_B200_PUSH_LANES", str(lanes)))
            gemm = sharding.PipelinedGatherGemm(o["a"], o["b"], results, [int(p) for p in hdl.buffer_ptrs], rank, n0,
                                                barrier=lambda: hdl.barrier(channel=0), compute_stream=stream,
                                                route=capi.PUSH_KERNEL if by_kernel else capi.PUSH_COPY_ENGINE, lanes=lanes)
            mode = ("pipelined: the slab GEMM stores into this rank's copy of the result; on a second stream "
                    + ("push_columns_kernel stores the slab" if by_kernel else f"the copy engines copy the slab (one strided copy per peer, {lanes} at a time)")
                    + " into every peer's copy over NVLink + one device barrier, while the next step's GEMM runs (two copies of the result, alternating)")
            return {"launch": gemm.launch, "join": gemm.join, "full": lambda: results[(gemm.steps - 1) & 1], "mode": mode,
                    "launches_per_step": 2 if by_kernel else 1, "buffers": results, "pipe": gemm, "keep": (hdl,)}

        makers = {"fused": lambda: fused_route(True), "fused-peer": lambda: fused_route(False),
                  "pipelined": lambda: pipelined_route(True), "pipelined-ce": lambda: pipelined_route(False)}
        # auto: both ways of hiding the gather are tried for a few steps on this machine and the faster one is measured.
        # (Copies to several peers in flight at once, VECOPS_B200_PUSH_LANES > 1, are not a candidate: 3 % faster than one
        # at a time in one 8-GPU run, 15-25 % slower in every 4-GPU run and twice as slow in another 8-GPU run.)
        wanted = ["fused", "pipelined-ce"] if args.gather == "auto" else [args.gather] if args.gather in makers else []
        routes, trials = {}, {}
        for key in wanted:
            try:
                route = makers[key]()
                route["launch"]()
                route["join"]()
                torch.cuda.synchronize()
                built = 1
            except Exception as error:  # symmetric memory unavailable: fall back to the library collective
                print(f"[bench] gather route {key} unavailable on rank {rank}: {error!r}", file=sys.stderr)
                built = 0
            ok = torch.tensor([built], device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) == 1:
                routes[key] = route
        if len(routes) > 1:
            for key, route in routes.items():
                def trial_step(_i, route=route):
                    route["launch"]()
                torch.cuda.synchronize()
                dist.barrier()
                for i in range(2):
                    trial_step(i)
                route["join"]()
                torch.cuda.synchronize()
                dist.barrier()
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record(stream)
                for i in range(10):
                    trial_step(i)
                route["join"]()
                t1.record(stream)
                torch.cuda.synchronize()
                took = torch.tensor([t0.elapsed_time(t1) / 10], dtype=torch.float64, device=dev)
                dist.all_reduce(took, op=dist.ReduceOp.MAX)
                trials[key] = float(took.item())
        if routes:
            chosen_key = min(routes, key=lambda k: trials.get(k, 0.0))
            chosen = routes[chosen_key]
            step_launch, step_join, pipe = chosen["launch"], chosen["join"], chosen["pipe"]
            gather_mode, launches_per_step = chosen["mode"], chosen["launches_per_step"]
            # nothing a trial step left behind may pass for the checked step's result
            torch.cuda.synchronize()
            dist.barrier()
            chosen["buffers"].zero_()
            torch.cuda.synchronize()
            dist.barrier()
            full_of = chosen["full"]
        else:
            gather_mode = "nccl: all_gather_into_tensor of the slabs + placement kernel per slab"
            full = torch.empty((w.m, w.n), dtype=torch.bfloat16, device=dev)
            staging = torch.empty((world, w.m, n1 - n0), dtype=torch.bfloat16, device=dev)
            place = sharding.cuda_place(stream)

            def step_launch():
                prepared[0].launch()
                sharding.gather_columns(o["c"], full, staging, world, place=place)
            launches_per_step = 1 + world
            full_of = lambda: full  # noqa: E731

    def step(_):
        step_launch()

    sets_note = f"operands and result {w.algorithmic_bytes / 1e9:.2f} GB > L2 126 MB"

    step(0)
    step_join()
    torch.cuda.synchronize()
    if full_of is not None:
        full = full_of()
    result_view = full[:, n0:n1] if full is not None else o["c"]
    parity = parity_sample(w, host_inputs, result_view, port, rows=8)
    if full is not None:
        # what a PEER computed must have arrived here too: the next rank's first 256 columns, four rows
        from oracle.checker import bf16_bits_to_f32, rel_frobenius
        p0, _ = sharding.column_partition(w.n, world, (rank + 1) % world)
        rows = np.array([0, w.m // 3, w.m // 2 + 1, w.m - 1])
        peer_b = workloads.make_b_nk(w, p0, p0 + 256)
        got = full[torch.from_numpy(rows).to(dev)][:, p0:p0 + 256].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
        parity["gathered_from_peer_rel_fro"] = rel_frobenius(bf16_bits_to_f32(got), bf16_bits_to_f32(port.matmul_bf16(host_inputs[0][rows], peer_b)))

    for i in range(warmup):
        step(i)
    step_join()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches_before = lib.vecops_b200_launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        start.record(stream)
        for i in range(steps):
            step(warmup + i)
        step_join()  # the last step's gather has landed on every rank before the clock stops
        stop.record(stream)
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches = lib.vecops_b200_launch_count() - launches_before
    elapsed = torch.tensor([start.elapsed_time(stop)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    ms = float(elapsed.item()) / steps
    status = take_status(local)

    # the GEMM kernel alone (what the roofline describes), timed live on the same stream
    def gemm_only(i):
        prepared[0].launch()

    kernel_ms = time_steps(gemm_only, steps, 3, stream) if world > 1 else ms
    gather_alone = None
    if pipe is not None:
        # the transfer by itself: this rank's slab to every peer + the barrier, nothing else running, max over ranks
        torch.cuda.synchronize()
        dist.barrier()
        gather_ms = torch.tensor([time_steps(lambda i: pipe.gather_alone(i & 1), steps, 3, pipe.send)], dtype=torch.float64, device=dev)
        dist.all_reduce(gather_ms, op=dist.ReduceOp.MAX)
        slab_bytes = 2.0 * w.m * (n1 - n0)
        gather_alone = {"note": "with the SMs idle; inside the pipelined step the same transfers have measured faster",
                        "ms": float(gather_ms.item()), "sent_bytes_per_gpu": slab_bytes * (world - 1),
                        "gb_per_s_per_direction": slab_bytes * (world - 1) / (float(gather_ms.item()) * 1e-3) / 1e9}
    slab_n = o["b"].shape[0]
    local_flops = 2.0 * w.m * slab_n * w.k
    local_bytes = 2.0 * (w.m * w.k + slab_n * w.k + w.m * slab_n)
    roofline = roofline_record(w, name, "gemm_tcgen05_kernel<bf16> (CTA pairs)", kernel_ms, local_flops, local_bytes, peaks, peak_source)
    value = w.flops / (ms * 1e-3) / 1e12

    # end to end through the operator bridge with host buffers
    e2e_steps = max(1, min(steps, 12 if world == 1 else 8))  # enough steps that filling the three-stream pipeline is not a third of the figure
    if world == 1:
        e2e = measure_e2e(w, operands, host_inputs, e2e_steps, 3, dev)
        e2e_note = {"serial_ms_per_step": e2e["serial_ms_per_step"], "serial_value": w.flops / (e2e["serial_ms_per_step"] * 1e-3) / 1e12,
                    "pipelining": "two operand sets in flight on copy-in / compute / read-back streams; serial_* is one step at a time on one stream",
                    "path": "vecops_operator_bridge_invoke_v1 (Operator -> MatmulRuntimeDispatch -> CudaExecutableProvider -> descriptor.run), pinned host buffers",
                    "resident": e2e["resident"], "copies": e2e["copies"]}
    else:
        def whole_step():  # end to end is one step at a time: the gather is waited for before the read-back
            step_launch()
            step_join()
        e2e = measure_e2e_sharded(w, o, host_inputs, whole_step, full_of, n0, n1, e2e_steps, 3, dev, a_peers)
        e2e_note = {"path": "per rank: " + e2e["a_route"] + " and this rank's B slab copied in from pinned host memory, the sharded operator "
                            "(slab GEMM + gather onto every rank + barrier), this rank's columns of the gathered result read back to the "
                            "host - the whole result reaches the host once per step, 1/N of it per rank",
                    "gather": "inside the timed region", "copies": e2e["copies"]}
    e2e_ms = torch.tensor([e2e["ms_per_step"]], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_value = w.flops / (float(e2e_ms.item()) * 1e-3) / 1e12

    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (seeded; shapes, layouts and value distributions of the named configuration)",
        "config": {"workload": name, "description": w.description, "m": w.m, "n": w.n, "k": w.k,
                   "parallelism": f"B column-sharded over {world} GPU" + ("s" if world > 1 else ""), "gather": gather_mode,
                   "l2": sets_note, "timing": "CUDA events on the launch stream, max over ranks"},
        "roofline": roofline,
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": e2e["h2d_bytes_per_step"],
                "d2h_bytes_per_step": e2e["d2h_bytes_per_step"], "ms_per_step": float(e2e_ms.item()), "steps": e2e_steps, **e2e_note},
        "gpu_launches": int(launches), "launches_per_step": launches_per_step, "clocks": clocks.summary(),
        "parity": parity, "device_status": status,
    }
    if gather_alone is not None:
        line["gather_alone"] = gather_alone
    if trials:
        line["config"]["gather_trials_ms_per_step"] = trials  # ten steps of each route before the measured run; the faster one was taken
    if world > 1:
        received = (world - 1) / world * w.m * w.n * 2.0
        line["scaling_ceiling"] = {"recv_bytes_per_gpu": received, "link_gbs_measured": NVLINK_RECEIVE_GBS,
                                   "floor_ms": received / (NVLINK_RECEIVE_GBS * 1e9) * 1e3,
                                   "peer_copy_gbs_measured": NVLINK_PEER_COPY_GBS,
                                   "floor_ms_at_peer_copy_rate": received / (NVLINK_PEER_COPY_GBS * 1e9) * 1e3,
                                   "achieved_gbs_into_every_gpu": received / (ms * 1e-3) / 1e9,
                                   "note": "gathering the result on every rank makes each GPU receive (N-1)/N of it per step; the link figures "
                                           "are a store-only all-to-all probe and a copy between two GPUs on this pool, not taken in this run"}

    if rank == 0 and world == 1:
        try:
            line["cpu_baseline"] = cpu_baseline(w)
        except Exception as error:  # the baseline is reported, never the reason a GPU number is lost
            line["cpu_baseline"] = {"error": repr(error)}
        if not args.no_extra and not args.workload:
            del operands, o, prepared, host_inputs
            torch.cuda.empty_cache()
            configs = {}
            for extra, k_steps in CONFIGS:
                try:
                    configs[extra] = measure_single(extra, k_steps, 10, dev, port, peaks, peak_source)
                except Exception as error:  # noqa: BLE001
                    configs[extra] = {"error": repr(error)}
                torch.cuda.empty_cache()
            line["configs"] = configs
            extras = {}
            for key, measure in [
                    ("c2_bf16_4096_fused_bias_silu", lambda: measure_single("c2_bf16_4096", 50, 5, dev, port, peaks, peak_source, fused=True)),
                    ("c3_quantized_u8s8", lambda: measure_quantized(50, 5, dev, port, peaks)),
                    ("attention_4096x4096x128", lambda: measure_sdpa(dev, port)),
                    ("pack_14336x4096", lambda: measure_pack(dev, peaks)),
                    ("c2_shape_f16", lambda: measure_f16(50, 5, dev, port, peaks))]:
                try:  # the rows beyond the five configurations
                    extras[key] = measure()
                except Exception as error:  # noqa: BLE001
                    extras[key] = {"error": repr(error)}
                torch.cuda.empty_cache()
            line["next_rows"] = extras
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def measure_e2e_sharded(w, o, host_inputs, step_launch, full, n0: int, n1: int, steps: int, warmup: int, dev, a_peers=None) -> dict:
    """One rank's share of the sharded operator end to end; every rank runs this at once.  Copy in from pinned host memory,
    run the slab GEMM with its gather (and the barrier that orders the ranks), read this rank's columns of the GATHERED
    result back - on a second stream, so that a step's read-back overlaps the next step's copy-in; the clock stops when the
    last result is on the host.  `full` is a callable returning the gathered result of the step
    just run.

    The inputs of a step are A, once, and B, once.  With `a_peers` (A in symmetric memory) each rank copies in its 1/N
    row slice of A and its slab of B, pushes the slice into every peer's A over NVLink (copy engines) and a device barrier
    orders the ranks before the GEMM: A crosses PCIe once per step in total, not once per rank.  Without it every rank
    pulls the whole of A over its own link."""
    import torch
    from vecops_b200 import capi
    a0, b0, _ = host_inputs
    copy = async_copier()
    main = torch.cuda.current_stream(dev)
    k_bytes = o["a"].shape[1] * o["a"].element_size()
    if a_peers is not None and copy is not None:
        rank, world = a_peers["rank"], a_peers["world"]
        r0, r1 = w.m * rank // world, w.m * (rank + 1) // world
        order = [(rank + 1 + j) % world for j in range(world - 1)]
        peers = (ctypes.c_void_p * len(order))(*[a_peers["bases"][r] + r0 * k_bytes for r in order])
        error = capi.ErrorBuffer()
        push = capi.library().vecops_b200_push_columns
        a_route = f"rows [{r0}, {r1}) of A (1/{world} of it; the slice is then pushed into every peer's A over NVLink by the copy engines, one device barrier)"
    else:
        a_peers, r0, r1 = None, 0, w.m
        a_route = "the whole of A"
    host_a = torch.from_numpy(np.ascontiguousarray(a0[r0:r1])).pin_memory()
    host_b = torch.from_numpy(b0).pin_memory()
    stage = torch.empty((w.m, n1 - n0), dtype=torch.bfloat16, device=dev)  # the rank's columns, made contiguous for the read-back
    host_c = torch.empty((w.m, n1 - n0), dtype=torch.bfloat16).pin_memory()
    a_bytes, b_bytes, c_bytes = (t.numel() * t.element_size() for t in (host_a, host_b, host_c))
    a_slice_ptr = o["a"].data_ptr() + r0 * k_bytes
    # the read-back of a step runs on a second stream, so that it shares the PCIe link (full duplex) with the next step's copy-in
    side = torch.cuda.Stream(dev)
    staged, read = torch.cuda.Event(), torch.cuda.Event()
    state = {"used": False}

    def step(_):
        if copy is not None:
            copy(a_slice_ptr, host_a.data_ptr(), a_bytes, main)
            copy(o["b"].data_ptr(), host_b.data_ptr(), b_bytes, main)
        else:
            o["a"].view(torch.int16).copy_(host_a.view(torch.int16), non_blocking=True)
            o["b"].view(torch.int16).copy_(host_b.view(torch.int16), non_blocking=True)
        if a_peers is not None:
            rc = push(a_slice_ptr, peers, len(order), o["a"].shape[1], 0, r1 - r0, o["a"].shape[1], o["a"].element_size(),
                      capi.PUSH_COPY_ENGINE, main.cuda_stream, byref(error.record))
            if rc != 0:
                error.raise_for(rc)
            a_peers["handle"].barrier(channel=0)  # every rank's slice has landed in this rank's A
        step_launch()
        if state["used"]:
            main.wait_event(read)  # the previous step's read-back has left `stage`
        stage.copy_(full()[:, n0:n1])
        staged.record(main)
        side.wait_event(staged)
        if copy is not None:
            copy(host_c.data_ptr(), stage.data_ptr(), c_bytes, side)
        else:
            with torch.cuda.stream(side):
                host_c.copy_(stage, non_blocking=True)
        read.record(side)
        state["used"] = True

    def timed(count: int) -> float:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(main)
        for i in range(count):
            step(i)
        main.wait_event(read)  # the last result has reached the host before the clock stops
        stop.record(main)
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / count

    if a_peers is not None:
        # the replication itself is checked: A is cleared on the device, one step rebuilds it from the ranks' slices
        torch.cuda.synchronize()
        a_peers["handle"].barrier(channel=0)
        o["a"].zero_()
        torch.cuda.synchronize()
        a_peers["handle"].barrier(channel=0)
        torch.cuda.synchronize()
    timed(warmup)
    ms = timed(steps)
    if not torch.equal(host_c, full()[:, n0:n1].cpu()):
        raise RuntimeError("end-to-end read-back differs from the gathered device result")
    if a_peers is not None and not torch.equal(o["a"].view(torch.int16).cpu(), torch.from_numpy(a0.view(np.int16) if a0.dtype != np.int16 else a0)):
        raise RuntimeError("A rebuilt from the ranks' row slices differs from the host's A")
    return {"ms_per_step": ms, "h2d_bytes_per_step": int(a_bytes + b_bytes), "d2h_bytes_per_step": int(c_bytes), "a_route": a_route,
            "copies": "cudaMemcpyAsync from / to pinned host memory" + ("" if copy is not None else " (through torch)")}


# ---------------------------------------------------------------------------------------------- reference arm

def run_reference(args) -> None:
    """The reference's own CPU matmul on the host cores, same metric and configuration as our arm."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    from oracle.checker import Port, Ref
    from vecops_b200 import workloads
    name = args.workload or HEADLINE
    w = workloads.WORKLOADS[name]
    steps = args.steps if args.steps is not None else 5
    warmup = args.warmup if args.warmup is not None else 1
    ref, why = Ref.load()
    cores = Ref.default_threads() if ref is not None else Port().threads
    run, rows, cols, kind, isa, note = cpu_sample(w, ref, cores)
    for _ in range(warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    seconds = (time.perf_counter() - t0) / steps
    unit = "GB/s" if w.kind == "w8" else ("TOP/s" if w.kind == "i8" else "TFLOP/s")
    value = ((cols * w.k + 4 * cols + 2 * rows * w.k + 2 * rows * cols) / seconds / 1e9) if w.kind == "w8" else 2.0 * rows * cols * w.k / seconds / 1e12
    sample = f"{rows}x{cols}x{w.k} of {w.m}x{w.n}x{w.k} per step{note}"
    how = f"{isa}; {cores} host threads each owning a slice of N" + (f" ({why})" if why else "")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": unit, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": seconds * 1e3, "higher_is_better": True, "scaling": "strong" if name == HEADLINE or world > 1 else "weak",
            "vs_baseline": None, "dtype": {"bf16": "bf16", "i8": "int8", "w8": "bf16 x int8 weights", "f32": "f32"}[w.kind],
            "data": "synthetic (same seeded inputs as the GPU arm)",
            "config": {"workload": name, "description": w.description, "m": w.m, "n": w.n, "k": w.k, "parallelism": f"{cores} host threads", "how": how},
            "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": kind, "isa": isa, "sample": sample},
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def measure_w8_size_curve(dev, peaks, steps: int = 60, warmup: int = 6) -> dict:
    """The weight-only streaming kernel at K=4096 over growing N (C4's N and 2, 4, 8, 16 times it), M=1 and M=16, each beside a
    library read of the same bytes: how much of the HBM-bound gap at C4 is the size of one launch and how much the kernel."""
    import torch
    from vecops_b200 import harness
    k, rows = 4096, []
    stream = torch.cuda.current_stream(dev)
    # VECOPS_B200_SIZE_CURVE_MULTIPLES="16" (or "1,4"): only these multiples of C4's N, e.g. to profile one size
    multiples = [int(x) for x in os.environ.get("VECOPS_B200_SIZE_CURVE_MULTIPLES", "1,2,4,8,16").split(",") if x.strip()]
    for n in [14336 * f for f in multiples]:
        sets = max(2, int(np.ceil(260e6 / (n * k))) + 1)
        weights = [torch.randint(-127, 128, (n, k), dtype=torch.int8, device=dev) for _ in range(sets)]
        scale = torch.rand(n, device=dev) * 0.02 + 0.001
        row = {"n": n, "k": k, "weight_bytes": n * k, "sets": sets}
        for m in (1, 16):
            a = torch.randn(m, k, device=dev).to(torch.bfloat16)
            outs = [torch.empty(m, n, dtype=torch.bfloat16, device=dev) for _ in range(sets)]
            prepared = [harness.PreparedMatmul(a, weights[i], outs[i], scale, stream=stream) for i in range(sets)]
            prepared[0].launch()
            torch.cuda.synchronize()
            ms = time_graph(prepared, steps, warmup, dev)
            want = (a.float() @ weights[0].float().t()) * scale
            algorithmic = n * k + 4 * n + 2 * m * k + 2 * m * n
            gbs = algorithmic / (ms * 1e-3) / 1e9
            row[f"m{m}"] = {"us": ms * 1e3, "gb_per_s": gbs, "frac_of_peak": gbs / peaks["hbm_gbs"],
                            "rel_fro_vs_torch_f32": ((outs[0].float() - want).norm() / want.norm()).item(), "device_status": take_status(dev.index or 0)}
            del prepared, outs
        read = size_matched_read(n * k, sets, steps, warmup, dev)
        row["read_of_the_same_bytes"] = {"us": read["ms_per_launch"] * 1e3, "gb_per_s": read["gb_per_s"], "frac_of_peak": read["gb_per_s"] / peaks["hbm_gbs"]}
        rows.append(row)
        del weights
        torch.cuda.empty_cache()
    return {"kernel": "w8_stream_kernel", "peak_gb_per_s": peaks["hbm_gbs"], "rows": rows}


def run_extra(which: str) -> None:
    """One of the extra measurements alone, on cuda:0."""
    import torch
    from oracle.checker import Port
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks, _ = measured_peaks()
    port = Port()
    record = {"attention": lambda: measure_sdpa(dev, port), "pack": lambda: measure_pack(dev, peaks),
              "f16": lambda: measure_f16(50, 5, dev, port, peaks), "quantized": lambda: measure_quantized(50, 5, dev, port, peaks),
              "w8-size-curve": lambda: measure_w8_size_curve(dev, peaks)}[which]()
    print(json.dumps({"extra": which, **record}), flush=True)


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=None)
    parser.add_argument("--warmup", type=int, default=None)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--workload", default=None, help="override the workload (a name from vecops_b200.workloads.WORKLOADS)")
    parser.add_argument("--gather", choices=["auto", "fused", "fused-peer", "pipelined", "pipelined-ce", "nccl"], default="auto",
                        help="how the sharded GEMM's output is gathered: auto = fused and pipelined-ce are both tried for ten steps and the "
                             "faster one is measured; fused = epilogue stores through the NVSwitch multicast address when "
                             "there is one, else to every rank's peer pointer; fused-peer = peer pointers only; pipelined = the slab is stored "
                             "locally and pushed to the peers by this library's kernel on a second stream, behind the next step's GEMM "
                             "(pipelined-ce: by the copy engines); nccl = library collective")
    parser.add_argument("--extra", choices=["attention", "pack", "f16", "quantized", "w8-size-curve"], default=None,
                        help="run ONLY this one of the extra single-GPU measurements and print its record (for profiling that kernel)")
    parser.add_argument("--no-extra", action="store_true", help="skip the brief measurements of the other single-GPU configurations")
    args = parser.parse_args()
    if args.warmup is not None and args.warmup < 3 and args.impl == "ours":
        args.warmup = 3  # timing rule: at least three warm-up steps
    if args.impl == "reference":
        run_reference(args)
    elif args.extra:
        run_extra(args.extra)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
