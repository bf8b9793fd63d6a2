"""Runs the MXFP8 quantiser a few times on a seeded synthetic matrix (profiler target / quick timing):

    python -m gemm_b200.profiling.run_quant [--rows R --k K] [--transposed] [--reps N]
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from .. import ops


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--transposed", action="store_true", help="input is [K, rows] (the layout of B[K, N])")
    ap.add_argument("--reps", type=int, default=4)
    a = ap.parse_args(argv)
    g = torch.Generator(device="cuda").manual_seed(0)
    X = torch.randn((a.k, a.rows) if a.transposed else (a.rows, a.k), device="cuda", generator=g).bfloat16()
    times = []
    for _ in range(a.reps):
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        ops.quantize_mxfp8(X, transposed_in=a.transposed)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    med = times[len(times) // 2]
    nbytes = a.rows * a.k * 3 + a.rows * a.k // 32
    print(json.dumps({"rows": a.rows, "K": a.k, "transposed": a.transposed, "median_ms": round(med, 4),
                      "gbps": round(nbytes / med / 1e6, 1)}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
