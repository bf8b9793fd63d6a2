#!/usr/bin/env python
"""Benchmark of the GEMM hot path.  `python bench.py --gpus N --steps K --warmup W` prints ONE
JSON line on rank 0.

Workload (default): the row-sharded BF16 GEMM  C[M,N] = A[M,K] @ B[K,N],  M = 131072,
K = N = 8192, FP32 accumulation, bf16 output.  A is made of 8 fixed row blocks (seed 1000 + b)
so it is identical for any rank count; rank r of N owns 8/N consecutive blocks, B (seed 0) is
broadcast once from rank 0 before the timed region and C stays sharded, so the timed loop holds
no collective.  A "step" is one pass of the GEMM over every rank's shard.

Every rank first runs PRELOAD_S seconds of untimed back-to-back launches, so that the timed steps
of every rank count are measured in the same regime: a board that has settled at its power cap.

* value       whole-job TFLOP/s = 2 M N K / (max over ranks of the device time per step), with
              operands resident in HBM (CUDA events on the launching stream).
* e2e         the same metric through the host-buffer C-ABI call (gemm_b200_gemm_bf16_host):
              operands start in pinned host memory and C ends there, copies inside the timing.
* roofline    achieved 2MNK/t of the GEMM kernel against the measured sustained cuBLAS bf16 peak.
* clocks      SM clock and throttle reasons of every rank's GPU, sampled while it is under load.
* cpu_baseline  the reference's oracle (torch.matmul on the host cores) on a bounded slice.
* per_dtype   (N = 1 only) the other benchmark configurations, each timed alone: median with the
              L2 flushed before every launch, best launch, and for the tensor-core shapes a 4 s
              back-to-back loop; the FP32 sweep beside the reference's three kernels and cuBLAS.

`--impl reference` times the reference's CPU-side computation instead (torch.matmul on all host
cores; the reference has no CPU kernels of its own, naive/test.py:23 is its check)."""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (M, K, N) of the whole job
    "bf16_rowsharded_131072x8192x8192": (131072, 8192, 8192),
    "bf16_8192": (8192, 8192, 8192),
    # the same row-sharded job on MXFP8 operands (quantising A and B is untimed preprocessing;
    # rank 0 quantises B and broadcasts its e4m3 data and packed scales)
    "mxfp8_rowsharded_131072x8192x8192": (131072, 8192, 8192),
}
DEFAULT_WORKLOAD = "bf16_rowsharded_131072x8192x8192"
L2_BYTES = 126 * 1024 * 1024
PRELOAD_S = 2.0                # untimed back-to-back launches before the warm-up steps, at every N
# DRAM traffic of a launch is not measured by this program (that takes a profiler); the last
# recorded capture of the default workload's kernel is quoted beside the line, labelled as such.
TRAFFIC_RECORD = {"file": "profiles/bench_launch_list.md", "workload": DEFAULT_WORKLOAD}


def measured_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return json.loads(p.read_text())
        except Exception:
            pass
    return {}


def recorded_traffic() -> dict | None:
    """The `dram bytes per launch` figure of the last committed capture (a line
    `recorded_dram_bytes_per_launch: <bytes> (<what, when>)` in the profile summary)."""
    p = ROOT / TRAFFIC_RECORD["file"]
    if not p.exists():
        return None
    for ln in p.read_text().splitlines():
        if ln.startswith("recorded_dram_bytes_per_launch:"):
            rest = ln.split(":", 1)[1].strip()
            num, _, note = rest.partition(" ")
            try:
                return {"bytes_per_launch_n1": float(num), "capture": TRAFFIC_RECORD["file"], "note": note.strip("() ")}
            except ValueError:
                return None
    return None


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi (read-only queries)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_id: str):
        self.gpu = gpu_id            # an nvidia-smi index or a "GPU-<uuid>" string
        self.proc = None
        self.lines: list = []
        self.t_mark = 0.0
        self.t_end = float("inf")

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def wait_first_sample(self, timeout: float = 3.0):
        t0 = time.perf_counter()
        while self.proc is not None and not self.lines and time.perf_counter() - t0 < timeout:
            time.sleep(0.02)

    def mark(self):
        """Samples taken before this call (idle GPU) are left out of the summary."""
        self.t_mark = time.perf_counter()

    def mark_end(self):
        """Samples taken after this call are left out of the summary."""
        self.t_end = time.perf_counter()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, smax, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, ln in self.lines:
            if ts < self.t_mark or ts > self.t_end:
                continue
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); smax.append(float(parts[2])); power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_min_mhz": sm[0] if sm else None,
                "sm_max_mhz": max(smax) if smax else None, "power_w_max": max(power) if power else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def gpu_smi_id(local: int) -> str:
    """nvidia-smi id of CUDA device `local` of this process (its UUID: CUDA_VISIBLE_DEVICES may renumber)."""
    import torch
    try:
        return "GPU-" + str(torch.cuda.get_device_properties(local).uuid)
    except Exception:
        return str(local)


def dist_setup(n_gpus: int):
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
    if world != n_gpus:
        raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {n_gpus}")
    return rank, world, local


def barrier(world):
    import torch
    import torch.distributed as dist
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def preload(fn, seconds: float) -> int:
    """Back-to-back launches of `fn` for about `seconds` (untimed).  Returns the launch count."""
    import torch
    if seconds <= 0:
        return 0
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize()
    per = max(e0.elapsed_time(e1) / 1e3, 1e-5)
    n = 1
    t0 = time.perf_counter()
    chunk = max(1, min(200, int(0.25 / per)))
    while time.perf_counter() - t0 < seconds:
        for _ in range(chunk):
            fn()
        torch.cuda.synchronize()
        n += chunk
    return n


def time_steps(fn, steps: int, warmup: int, world: int):
    """(device time in s of exactly `steps` calls, max over ranks; kernels this rank launched in that region)."""
    import torch
    from gemm_b200 import sharded
    import gemm_b200.ops as ops
    for _ in range(warmup):
        fn()
    barrier(world)
    n0 = ops.launch_count()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    launches = ops.launch_count() - n0
    secs = e0.elapsed_time(e1) / 1e3
    total = sharded.max_over_ranks(secs, device=torch.device("cuda", torch.cuda.current_device()))
    barrier(world)
    return total, launches


_FLUSH = None


def _flush_buffer():
    import torch
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device="cuda")
    return _FLUSH


def time_alone(fn, reps: int = 10, warmup: int = 3, both: bool = False, flush: str = "write"):
    """Device time (s) of single launches, L2 flushed before each (by writing 252 MB, or with
    flush="read" by reading them, which leaves no dirty lines behind): the median, or (median,
    best) with `both`."""
    import torch
    buf = _flush_buffer()
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(reps):
        if flush == "read":
            buf.sum()
        else:
            buf.zero_()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) / 1e3)
    ts.sort()
    return (ts[len(ts) // 2], ts[0]) if both else ts[len(ts) // 2]


def time_sustained(fn, seconds: float = 4.0) -> float:
    """Average device time (s) per launch over a back-to-back loop of about `seconds` (operands
    larger than L2): the power-capped regime."""
    import torch
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record(); fn(); e1.record()
    torch.cuda.synchronize()
    n = max(3, int(seconds / max(e0.elapsed_time(e1) / 1e3, 1e-5)))
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / 1e3 / n


def time_rotating(fns, reps: int = 30, warmup: int = 3) -> float:
    """Average device time (s) per launch of a back-to-back loop that walks `fns` in turn.  Each
    callable works on its own copy of the operands and the copies together exceed the L2 several
    times, so no launch finds its operands cached; no flush kernel runs between launches."""
    import torch
    for _ in range(warmup):
        for fn in fns:
            fn()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        for fn in fns:
            fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / 1e3 / (reps * len(fns))


def time_interleaved(fns, reps: int = 7, warmup: int = 2) -> list:
    """Median device time (s) of each callable, launched in turn (a, b, c, a, b, c, ...), L2 flushed
    before every launch."""
    import torch
    flush = _flush_buffer()
    for _ in range(warmup):
        for fn in fns:
            fn()
    ts = [[] for _ in fns]
    for _ in range(reps):
        for i, fn in enumerate(fns):
            flush.zero_()
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts[i].append(e0.elapsed_time(e1) / 1e3)
    return [sorted(t)[len(t) // 2] for t in ts]


def fp32_sweep(peaks: dict) -> dict:
    """FP32 square sweep: this library, the reference's three kernels (compiled unchanged, test
    infrastructure) and cuBLAS (torch.matmul) on the same seeded inputs, each launch timed alone
    with the L2 flushed; medians.  The reference kernels get fewer repetitions at the large sizes
    (a cap on repetitions, not on shapes)."""
    import torch
    import gemm_b200.ops as ops
    out = {}
    sm_max = float(peaks.get("sm_max_mhz", 1965.0))
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    f32_peak = sms * 128 * 2 * sm_max * 1e6 / 1e12
    ref = {}
    try:
        from oracle import oracle as O     # baseline reporting only: never on the library's path
        if O.reference_available():
            ref = {v: O.reference_launcher(v) for v in ("naive", "shared", "blocktile_1d")}
    except Exception:
        ref = {}
    allow_tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    g = torch.Generator(device="cuda").manual_seed(0)
    for n in (512, 1024, 2048, 4096, 8192):
        A = torch.rand(n, n, device="cuda", generator=g) * 2 - 1
        B = torch.rand(n, n, device="cuda", generator=g) * 2 - 1
        C = torch.empty(n, n, device="cuda")
        flops = 2.0 * n ** 3
        t, t_best = time_alone(lambda: ops.sgemm_f32(A, B, C), both=True)
        row = {"ours": round(flops / t / 1e12, 2), "ours_best": round(flops / t_best / 1e12, 2),
               "frac_of_simt_peak": round(flops / t / 1e12 / f32_peak, 4), "simt_peak_tflops": round(f32_peak, 1)}
        t = time_alone(lambda: torch.matmul(A, B, out=C))
        row["cublas"] = round(flops / t / 1e12, 2)
        for name, launch in ref.items():
            reps = 10 if n <= 2048 else (5 if n == 4096 else 2)
            t = time_alone(lambda: launch(A, B, C), reps=reps, warmup=1)
            row["ref_" + name] = round(flops / t / 1e12, 2)
        if not ref:
            row["ref"] = "oracle/_ref is not built"
        out[f"fp32_{n}"] = row
        del A, B, C
    torch.backends.cuda.matmul.allow_tf32 = allow_tf32
    return out


def per_dtype_table(peaks: dict) -> dict:
    """The other benchmark configurations at N = 1, each kernel timed alone."""
    import torch
    import gemm_b200.ops as ops
    out = fp32_sweep(peaks)
    g = torch.Generator(device="cuda").manual_seed(0)
    time.sleep(1.0)     # idle gap: these are kernels timed alone, not in the power-capped regime of a loop
    burst = float(peaks.get("bf16_tflops", 1590.0))
    sustained = float(peaks.get("bf16_tflops_sustained", 1400.0))
    for (M, K, N) in ((8192, 8192, 8192), (8192, 16384, 4096)):
        A = torch.randn(M, K, device="cuda", generator=g).bfloat16()
        B = torch.randn(K, N, device="cuda", generator=g).bfloat16()
        C = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        flops = 2.0 * M * N * K
        t, t_best = time_alone(lambda: ops.gemm_bf16(A, B, C), both=True)
        tf = flops / t / 1e12
        out[f"bf16_{M}x{K}x{N}"] = {
            "tflops": round(tf, 1), "tflops_best": round(flops / t_best / 1e12, 1),
            "frac_of_nominal_2250": round(tf / 2250.0, 4), "frac_of_measured_burst": round(tf / burst, 4)}
        # the vendor library on the same operands, same protocol (context, not the product path)
        torch.matmul(A, B, out=C)
        out[f"bf16_{M}x{K}x{N}"]["cublas"] = round(flops / time_alone(lambda: torch.matmul(A, B, out=C)) / 1e12, 1)
        del A, B, C
    if hasattr(ops, "gemm_mxfp8") and ops.gemm_mxfp8_configs():
        hbm = float(peaks.get("hbm_gbs", 6650.0))
        for (M, K, N) in ((8192, 8192, 8192), (16384, 8192, 28672), (16, 8192, 28672)):
            A = torch.randn(M, K, device="cuda", generator=g).bfloat16()
            B = torch.randn(K, N, device="cuda", generator=g).bfloat16()
            Aq = ops.quantize_mxfp8(A)
            Bq = ops.quantize_mxfp8(B, transposed_in=True)
            del A
            C = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            flops = 2.0 * M * N * K
            t, t_best = time_alone(lambda: ops.gemm_mxfp8(Aq, Bq, C), both=True)
            tf = flops / t / 1e12
            bytes_ = M * K + N * K + (M + N) * K // 32 + 2 * M * N
            row = {"tflops": round(tf, 1), "tflops_best": round(flops / t_best / 1e12, 1),
                   "frac_of_nominal_4500": round(tf / 4500.0, 4), "gbps": round(bytes_ / t / 1e9, 1),
                   "frac_of_measured_hbm": round(bytes_ / t / 1e9 / hbm, 4)}
            out[f"mxfp8_{M}x{K}x{N}"] = row
            try:
                # the vendor library's block-scaled GEMM on the same packed bytes (context only)
                a8, b8 = Aq.data.view(torch.float8_e4m3fn), Bq.data.view(torch.float8_e4m3fn).t()
                sa, sb = Aq.scales.view(torch.float8_e8m0fnu), Bq.scales.view(torch.float8_e8m0fnu)
                lib_mm = lambda: torch._scaled_mm(a8, b8, scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)
                lib_mm()
                t_l = time_alone(lib_mm)
                row["cublaslt_scaled_mm"] = round(flops / t_l / 1e12, 1)
                if M < 1024:
                    row["cublaslt_scaled_mm_gbps"] = round(bytes_ / t_l / 1e9, 1)
            except (RuntimeError, NotImplementedError, AttributeError):
                row["cublaslt_scaled_mm"] = None
            if M < 1024:
                # The HBM-bound decode shape.  `gbps` above is one call after the usual 252 MB WRITE
                # flush; that flush leaves the L2 full of dirty lines whose write-back competes with
                # this kernel's reads (a pure TMA stream of the same matrix: 55 us after the write
                # flush, 43 us after a read flush).  Per call with the L2 evicted by READING:
                t_c = time_alone(lambda: ops.gemm_mxfp8(Aq, Bq, C), flush="read")
                row["gbps_clean_l2"] = round(bytes_ / t_c / 1e9, 1)
                row["frac_of_measured_hbm_clean_l2"] = round(bytes_ / t_c / 1e9 / hbm, 4)
                row["protocol"] = ("gbps: per call after a 252 MB write flush; gbps_clean_l2: per call after a 252 MB read "
                                   "flush (no dirty lines); gbps_cuda_graph: write flush, call replayed from a CUDA graph; "
                                   "gbps_back_to_back: no flush kernel, four copies of B in turn")
                # A ~45 us HBM-bound kernel.  Two more views of the same call:
                #  * replayed from a CUDA graph (no Python / ctypes between the events);
                #  * back to back over four separate copies of B (4 x 235 MB, L2 = 126 MB) with no
                #    flush kernel in between: the flush writes 252 MB and leaves the L2 full of
                #    dirty lines, whose write-back then competes with this kernel's reads.
                st = torch.cuda.Stream()
                st.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(st):
                    ops.gemm_mxfp8(Aq, Bq, C)
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=st):
                        ops.gemm_mxfp8(Aq, Bq, C)
                torch.cuda.current_stream().wait_stream(st)
                t_g = time_alone(graph.replay)
                row["gbps_cuda_graph"] = round(bytes_ / t_g / 1e9, 1)
                row["frac_of_measured_hbm_cuda_graph"] = round(bytes_ / t_g / 1e9 / hbm, 4)
                del graph
                copies = [Bq] + [ops.quantize_mxfp8(B, transposed_in=True) for _ in range(3)]
                t_r = time_rotating([(lambda q=q: ops.gemm_mxfp8(Aq, q, C)) for q in copies])
                row["gbps_back_to_back"] = round(bytes_ / t_r / 1e9, 1)
                row["frac_of_measured_hbm_back_to_back"] = round(bytes_ / t_r / 1e9 / hbm, 4)
                row["back_to_back"] = "4 copies of B in turn (940 MB > L2), 30 rounds, no flush kernel"
                del copies
            elif N > 8192:
                # the same GEMM with the quantising epilogue vs GEMM (bf16 out) + separate quantise pass,
                # timed alternately: on a power-capped board the clock drifts with what ran just before
                t_f, t_p, t_q = time_interleaved([lambda: ops.gemm_mxfp8_quant_out(Aq, Bq),
                                                  lambda: ops.gemm_mxfp8(Aq, Bq, C),
                                                  lambda: ops.quantize_mxfp8(C)], reps=7)
                out[f"mxfp8_{M}x{K}x{N}_quant_out"] = {"fused_ms": round(t_f * 1e3, 3), "gemm_ms": round(t_p * 1e3, 3),
                                                       "gemm_plus_quantise_ms": round((t_p + t_q) * 1e3, 3),
                                                       "tflops_fused": round(flops / t_f / 1e12, 1)}
            del B, Aq, Bq, C
    # The 4 s back-to-back loops come last: they leave the board hot and at its power cap, and a
    # kernel timed alone right after one runs 15-20 % slower than after an idle gap.
    for (M, K, N) in ((8192, 8192, 8192), (8192, 16384, 4096)):
        A = torch.randn(M, K, device="cuda", generator=g).bfloat16()
        B = torch.randn(K, N, device="cuda", generator=g).bfloat16()
        C = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        t_sus = time_sustained(lambda: ops.gemm_bf16(A, B, C))
        row = out[f"bf16_{M}x{K}x{N}"]
        row["tflops_sustained_4s"] = round(2.0 * M * N * K / t_sus / 1e12, 1)
        row["sustained_frac_of_measured_sustained"] = round(2.0 * M * N * K / t_sus / 1e12 / sustained, 4)
        del A, B, C
    if "mxfp8_16384x8192x28672" in out:
        M, K, N = 16384, 8192, 28672
        Aq = ops.quantize_mxfp8(torch.randn(M, K, device="cuda", generator=g).bfloat16())
        Bq = ops.quantize_mxfp8(torch.randn(K, N, device="cuda", generator=g).bfloat16(), transposed_in=True)
        C = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        t_sus = time_sustained(lambda: ops.gemm_mxfp8(Aq, Bq, C))
        row = out["mxfp8_16384x8192x28672"]
        row["tflops_sustained_4s"] = round(2.0 * M * N * K / t_sus / 1e12, 1)
        row["sustained_frac_of_2x_measured_bf16_sustained"] = round(2.0 * M * N * K / t_sus / 1e12 / (2 * sustained), 4)
        del Aq, Bq, C
    return out


def host_threads() -> int:
    """Every core this process may run on; set explicitly because launchers such as
    torch.distributed.run export OMP_NUM_THREADS=1 to their children."""
    import torch
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def cpu_matmul_variants() -> dict:
    """The reference's host-side computation for BF16 operands, two ways: torch.matmul on the bf16
    tensors themselves (FP32 accumulation inside; the fast path on CPUs with bf16 matrix
    instructions) and the FP32 matmul of the same operands (the form the tolerance is stated on,
    oracle.bf16_matmul_oracle, with B converted once)."""
    import torch
    return {"bf16_matmul": lambda A, B, Bf: torch.matmul(A, B),
            "fp32_matmul_of_bf16": lambda A, B, Bf: torch.matmul(A.float(), Bf)}


def cpu_rate(K: int, N: int, pass_budget_s: float, M: int, steps: int = 3, warmup: int = 0):
    """Times both variants on a row slice sized for ~pass_budget_s of work per pass of the faster
    one.  Returns ({variant: {best, mean} TFLOP/s}, rows, seconds per pass of the faster variant,
    its name)."""
    import torch
    from oracle import oracle as O   # the CPU baseline leg: the oracle is what is timed here
    fns = cpu_matmul_variants()
    g = torch.Generator().manual_seed(0)
    B = torch.randn(K, N, generator=g).bfloat16()
    Bf = B.float()
    A = torch.randn(256, K, generator=g).bfloat16()
    assert torch.equal(fns["fp32_matmul_of_bf16"](A[:8], B, Bf), O.bf16_matmul_oracle(A[:8], B))
    probe = {}
    for name, f in fns.items():
        f(A, B, Bf)
        t0 = time.perf_counter(); f(A, B, Bf); probe[name] = time.perf_counter() - t0
    fast = min(probe, key=probe.get)
    rows = int(max(256, min(M, 65536, (pass_budget_s / max(probe[fast], 1e-4)) * 256 // 256 * 256)))
    A = torch.randn(rows, K, generator=g).bfloat16()
    out = {}
    per_pass = None
    for name, f in fns.items():
        # the slower variant gets a slice a quarter the size and one pass: it is reported, not the headline
        Av = A if name == fast else A[:max(256, rows // 4)]
        for _ in range(warmup if name == fast else 0):
            f(Av, B, Bf)
        best, total = None, 0.0
        n = steps if name == fast else 1
        for _ in range(n):
            t0 = time.perf_counter(); f(Av, B, Bf); dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
            total += dt
        out[name] = {"best": 2.0 * Av.shape[0] * N * K / best / 1e12, "mean": 2.0 * Av.shape[0] * N * K * n / total / 1e12}
        if name == fast:
            per_pass = total / n
    return out, rows, per_pass, fast


def cpu_baseline(M: int, K: int, N: int, budget_s: float = 12.0) -> dict:
    """torch.matmul on the host cores over a bounded row slice of the same workload."""
    cores = host_threads()
    rates, rows, per_pass, fast = cpu_rate(K, N, budget_s / 3, M, steps=3)
    return {"value": round(rates[fast]["best"], 4), "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "variant": fast, "variants": {k: round(v["best"], 4) for k, v in rates.items()},
            "sample": f"torch.matmul ({fast}) on the first {rows} of {M} rows, best of 3 passes of ~{per_pass:.2f} s, "
                      f"{cores} threads, os.cpu_count()={os.cpu_count()}"}


def run_reference_arm(args) -> int:
    """The reference's computation on the host cores (rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    cores = host_threads()
    M, K, N = WORKLOADS[args.workload]
    is_mx = args.workload.startswith("mxfp8")      # same host computation: a matmul of the bf16 operands
    # each step ~ 60 s / (steps + warmup) of CPU work (GEMM_B200_REF_BUDGET_S overrides the 60 s)
    per_step = float(os.environ.get("GEMM_B200_REF_BUDGET_S", "60")) / max(1, args.steps + args.warmup)
    rates, rows, per_pass, fast = cpu_rate(K, N, per_step, M, steps=max(1, args.steps), warmup=args.warmup)
    tf = rates[fast]["mean"]
    sample = f"torch.matmul ({fast}) on host cores, {rows} of {M} rows per step, {cores} threads"
    line = {
        "impl": "reference", "metric": "tflops", "value": round(tf, 4), "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(per_pass * 1e3, 3), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "mxfp8" if is_mx else "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "M": M, "K": K, "N": N, "rows_per_step": rows},
        "cpu_baseline": {"value": round(tf, 4), "unit": "TFLOP/s", "cores": cores, "kind": "port", "variant": fast,
                         "variants": {k: round(v["mean"], 4) for k, v in rates.items()}, "sample": sample},
        "e2e": {"value": round(tf, 4), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


def gather_objects(obj, world: int) -> list:
    if world == 1:
        return [obj]
    import torch.distributed as dist
    out = [None] * world
    dist.all_gather_object(out, obj)
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="gemm_b200", choices=["gemm_b200", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--no-extras", action="store_true", help="skip per_dtype, cpu_baseline and e2e (profiling runs)")
    ap.add_argument("--preload-s", type=float, default=PRELOAD_S, help="seconds of untimed launches before the warm-up")
    ap.add_argument("--e2e-steps", type=int, default=3)
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)

    import torch
    import gemm_b200.ops as ops        # raises if the CUDA library is missing: there is no fallback
    from gemm_b200 import sharded

    rank, world, local = dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    peaks = measured_peaks()
    M, K, N = WORKLOADS[args.workload]
    shard = sharded.shard_rows(M, world, rank)
    rows_per_block = M // sharded.BLOCKS

    # operands: A shard generated block by block on the device, B on rank 0 then broadcast
    A = torch.empty(shard.rows, K, device=dev, dtype=torch.bfloat16)
    for i, b in enumerate(shard.blocks):
        A[i * rows_per_block:(i + 1) * rows_per_block] = sharded.gen_a_block_cuda(b, rows_per_block, K, dev)
    B = sharded.gen_b_cuda(K, N, dev) if rank == 0 else torch.empty(K, N, device=dev, dtype=torch.bfloat16)
    sharded.broadcast_b(B, src=0)
    C = torch.empty(shard.rows, N, device=dev, dtype=torch.bfloat16)
    is_mx = args.workload.startswith("mxfp8")
    probe = torch.tensor([0, shard.rows // 2 + 1, shard.rows - 1], device=dev)
    want = torch.matmul(A[probe].float(), B.float())
    if is_mx:
        Aq = ops.quantize_mxfp8(A)
        Bq = ops.quantize_mxfp8(B, transposed_in=True)     # every rank runs it for the buffer shapes ...
        sharded.broadcast_mxfp8(Bq, src=0)                  # ... rank 0's bytes are the ones used

        def step():
            ops.gemm_mxfp8(Aq, Bq, C)
    else:
        def step():
            ops.gemm_bf16(A, B, C)

    # correctness guard before timing: a few rows against the FP32 product of the bf16 operands
    step()
    ops.check_status()
    if is_mx:
        # MXFP8 keeps ~3 significant bits per element: hold the rows to a few per cent overall
        err = float((C[probe].float() - want).norm() / want.norm())
        if not err < 0.06:
            raise SystemExit(f"mxfp8 probe rows differ from the bf16 product by {err:.3f}")
    else:
        torch.testing.assert_close(C[probe].float(), want, rtol=2e-2, atol=2e-2)

    # every rank samples its own GPU from the start of the pre-load to the end of the timed steps
    sampler = ClockSampler(gpu_smi_id(local))
    sampler.start()
    sampler.wait_first_sample()
    barrier(world)
    sampler.mark()
    preload_launches = preload(step, args.preload_s)
    secs, launches = time_steps(step, args.steps, max(args.warmup, 3), world)
    sampler.mark_end()
    launches = int(sharded.sum_over_ranks(float(launches), device=dev))
    my_clocks = sampler.stop()
    ops.check_status()
    all_clocks = gather_objects(my_clocks, world)
    per_step = secs / args.steps
    flops = 2.0 * M * N * K
    value = flops / per_step / 1e12

    clocks = {}
    if rank == 0:
        meds = [c.get("sm_mhz") for c in all_clocks]
        known = sorted(m for m in meds if m)
        reasons = sorted({r for c in all_clocks for r in (c.get("reasons") or [])})
        clocks = {"sm_mhz": known[len(known) // 2] if known else None,
                  "sm_max_mhz": max((c.get("sm_max_mhz") or 0) for c in all_clocks) or None,
                  "reasons": reasons, "per_rank_sm_mhz": meds,
                  "per_rank_sm_min_mhz": [c.get("sm_min_mhz") for c in all_clocks],
                  "per_rank_power_w_max": [c.get("power_w_max") for c in all_clocks],
                  "samples": [c.get("samples") for c in all_clocks],
                  "window": f"{args.preload_s:g} s pre-load + warm-up + timed steps, 20 ms period, every rank's own GPU"}

    # roofline of the GEMM kernel: one launch per rank per step, algorithmic flops of the rank's shard.
    # One denominator at every rank count: the pre-load puts every board in the power-capped regime
    # of the measured SUSTAINED cuBLAS figure; the burst and nominal fractions are quoted beside it.
    kernel_tflops = 2.0 * shard.rows * N * K / per_step / 1e12
    peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
    burst = float(peaks.get("bf16_tflops", 1590.0))
    nominal = 2250.0
    if is_mx:
        # no FP8 figure was measured on this pool: the FP8 pipe runs at twice the bf16 rate, so the
        # denominator is twice the measured bf16 figure
        peak, burst, nominal = 2 * peak, 2 * burst, 4500.0
    roofline = {"bound": "tensor", "achieved": round(kernel_tflops, 1), "peak": peak, "unit": "TFLOP/s",
                "frac": round(kernel_tflops / peak, 4), "traffic": None,
                "algorithmic_bytes": int((shard.rows * K + K * N) * (33 / 32 if is_mx else 2) + 2 * shard.rows * N),
                "peak_kind": ("2 x " if is_mx else "") + ("measured sustained" if peaks else "fallback sustained"),
                "frac_of_measured_burst": round(kernel_tflops / burst, 4),
                "frac_of_nominal_%d" % nominal: round(kernel_tflops / nominal, 4)}
    if rank == 0 and clocks.get("sm_mhz"):
        roofline["tflops_per_ghz"] = round(kernel_tflops / (clocks["sm_mhz"] / 1e3), 1)
    if args.workload == DEFAULT_WORKLOAD:
        rec = recorded_traffic()
        if rec is not None:
            rec["bytes_per_launch_this_rank"] = rec["bytes_per_launch_n1"] * shard.rows / M
            roofline["traffic_recorded"] = rec      # an earlier capture; `traffic` itself is not measured here

    e2e = None
    cpu = None
    extra = None
    mx_leg = None
    if not args.no_extras and not is_mx and ops.gemm_mxfp8_configs():
        # The MXFP8 half of the row-sharded configuration, same operands quantised along K, same
        # protocol (pre-load, barrier, device-timed steps, max over ranks) at this rank count.
        Aq = ops.quantize_mxfp8(A)
        Bq = ops.quantize_mxfp8(B, transposed_in=True)
        sharded.broadcast_mxfp8(Bq, src=0)

        def mx_step():
            ops.gemm_mxfp8(Aq, Bq, C)
        mx_step()
        ops.check_status()
        err = float((C[probe].float() - want).norm() / want.norm())
        if not err < 0.06:
            raise SystemExit(f"mxfp8 probe rows differ from the bf16 product by {err:.3f}")
        barrier(world)
        preload(mx_step, min(args.preload_s, 1.0))
        mx_secs, _ = time_steps(mx_step, args.steps, max(args.warmup, 3), world)
        ops.check_status()
        mx_tf = flops / (mx_secs / args.steps) / 1e12
        mx_leg = {"workload": "mxfp8_rowsharded_%dx%dx%d" % (M, K, N), "value": round(mx_tf, 1), "unit": "TFLOP/s",
                  "ms_per_step": round(mx_secs / args.steps * 1e3, 4), "steps": args.steps, "n_gpus": world,
                  "frac_of_2x_measured_bf16_sustained": round(mx_tf / world / (2 * float(peaks.get("bf16_tflops_sustained", 1400.0))), 4),
                  "operands": "e4m3 data + one ue8m0 scale per 32 k, quantised before the timed region; B's bytes broadcast from rank 0"}
        del Aq, Bq
    if not args.no_extras and not is_mx:
        # end to end: pinned host operands -> C in pinned host memory, through the host-buffer C-ABI call
        hA = torch.empty(shard.rows, K, dtype=torch.bfloat16, pin_memory=True); hA.copy_(A)
        hB = torch.empty(K, N, dtype=torch.bfloat16, pin_memory=True); hB.copy_(B)
        hC = torch.empty(shard.rows, N, dtype=torch.bfloat16, pin_memory=True)
        ops.gemm_bf16_host(hA, hB, hC)
        barrier(world)
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            ops.gemm_bf16_host(hA, hB, hC)
        dt = (time.perf_counter() - t0) / args.e2e_steps
        dt = sharded.max_over_ranks(dt, device=dev)
        torch.testing.assert_close(hC[:2].float(), torch.matmul(hA[:2].float(), hB.float()), rtol=2e-2, atol=2e-2)
        e2e = {"value": round(flops / dt / 1e12, 2), "unit": "TFLOP/s",
               "h2d_bytes_per_step": int(world * (hB.numel() * 2) + M * K * 2), "d2h_bytes_per_step": int(M * N * 2),
               "ms_per_step": round(dt * 1e3, 2)}
        del hA, hB, hC
        if rank == 0 and world == 1:
            cpu = cpu_baseline(M, K, N)
            del A, C
            torch.cuda.empty_cache()
            extra = per_dtype_table(peaks)

    if rank == 0:
        line = {
            "metric": "tflops", "value": round(value, 1), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(per_step * 1e3, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "mxfp8" if is_mx else "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "M": M, "K": K, "N": N, "rows_per_rank": shard.rows,
                       "parallelism": f"rows{world}", "l2": "inputs larger than L2 (A shard %.0f MiB)" % (shard.rows * K * 2 / 2 ** 20),
                       "out": "bf16", "accumulate": "fp32", "preload_s": args.preload_s, "preload_launches": preload_launches,
                       **({"operands": "e4m3 data + one ue8m0 scale per 32 k (quantised before the timed region)"} if is_mx else {})},
            "roofline": roofline, "clocks": clocks, "gpu_launches": int(launches),
        }
        if e2e is not None:
            line["e2e"] = e2e
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if mx_leg is not None:
            line["mxfp8_rowsharded"] = mx_leg
        if extra is not None:
            line["per_dtype"] = extra
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
