"""Runs one operator of the library a few times on seeded synthetic inputs:

    python -m gemm_b200.profiling.run_one {f32|bf16|mxfp8} [--m M --k K --n N] [--config C] [--reps R]

Meant as the target of a profiler (`ncu ... python -m gemm_b200.profiling.run_one bf16 --m 8192 ...`) or
for a quick timing; prints the median device time and TFLOP/s of the launches."""
from __future__ import annotations

import argparse
import json
import sys

import torch

from .. import ops


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("op", choices=["f32", "bf16", "mxfp8"])
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--config", type=int, default=-1)
    ap.add_argument("--reps", type=int, default=4)
    ap.add_argument("--out-f32", action="store_true", help="FP32 output for the tensor-core operators")
    ap.add_argument("--k-splits", type=int, default=0, help="bf16: K ranges of the two-launch split (0: library decides, 1: never)")
    ap.add_argument("--cluster-splits", type=int, default=0, help="bf16: split K over clusters of 2, 4 or 8 CTAs")
    ap.add_argument("--cublas", action="store_true", help="bf16 / f32: run torch.matmul instead (for comparison)")
    a = ap.parse_args(argv)
    M, K, N = a.m, a.k, a.n
    g = torch.Generator(device="cuda").manual_seed(0)
    od = torch.float32 if a.out_f32 else torch.bfloat16
    if a.op == "f32":
        A = torch.rand(M, K, device="cuda", generator=g) * 2 - 1
        B = torch.rand(K, N, device="cuda", generator=g) * 2 - 1
        C = torch.empty(M, N, device="cuda")
        fn = lambda: ops.sgemm_f32(A, B, C, config=a.config)
        if a.cublas:
            fn = lambda: torch.matmul(A, B, out=C)
    elif a.op == "bf16":
        A = torch.randn(M, K, device="cuda", generator=g).bfloat16()
        B = torch.randn(K, N, device="cuda", generator=g).bfloat16()
        C = torch.empty(M, N, device="cuda", dtype=od)
        fn = lambda: ops.gemm_bf16(A, B, C, out_dtype=od, config=a.config, k_splits=a.k_splits, cluster_splits=a.cluster_splits)
        if a.cublas:
            fn = lambda: torch.matmul(A, B, out=C)
    else:
        A = torch.randn(M, K, device="cuda", generator=g).bfloat16()
        B = torch.randn(K, N, device="cuda", generator=g).bfloat16()
        Aq = ops.quantize_mxfp8(A)
        Bq = ops.quantize_mxfp8(B, transposed_in=True)
        del A, B
        C = torch.empty(M, N, device="cuda", dtype=od)
        fn = lambda: ops.gemm_mxfp8(Aq, Bq, C, out_dtype=od, config=a.config)
    times = []
    for _ in range(a.reps):
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    ops.check_status()
    times.sort()
    med = times[len(times) // 2]
    print(json.dumps({"op": a.op, "M": M, "K": K, "N": N, "config": a.config, "median_ms": round(med, 4),
                      "tflops": round(2.0 * M * N * K / med / 1e9, 1)}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
