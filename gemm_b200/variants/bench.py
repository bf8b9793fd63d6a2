"""Benchmark of the three reference-named modules with the reference's own protocol
(naive/benchmark.py:14-60): square FP32 problems 128 / 512 / 1024, randn inputs, five warm-up
calls, then `triton.testing.do_bench(..., return_mode="median")` (L2 flushed before every timed
call, CUDA events), TFLOP/s = 2 M N K / t, next to `torch.matmul(A, B, out=C)`.

    python -m gemm_b200.variants.bench [--sizes 128 512 1024 ...]

The reference's scripts label microseconds as "ms"; this one prints microseconds as such."""
from __future__ import annotations

import argparse
import sys

import torch

from . import entry_point


def _median_us(fn) -> float:
    from triton.testing import do_bench
    return do_bench(fn, return_mode="median") * 1e3


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--sizes", type=int, nargs="*", default=[128, 512, 1024])
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("ERROR: CUDA is not available!")
        return 1
    print(f"CUDA Device: {torch.cuda.get_device_name(0)}")
    print(f"PyTorch version: {torch.__version__}")
    for variant in ("naive", "shared", "blocktile_1d"):
        f = entry_point(variant)
        print(f"\n== {variant} ==")
        for n in a.sizes:
            A = torch.randn(n, n, device="cuda", dtype=torch.float32)
            B = torch.randn(n, n, device="cuda", dtype=torch.float32)
            C = torch.zeros(n, n, device="cuda", dtype=torch.float32)
            for _ in range(5):
                f(A, B, C)
            torch.cuda.synchronize()
            custom_us = _median_us(lambda: f(A, B, C))
            for _ in range(5):
                torch.matmul(A, B, out=C)
            torch.cuda.synchronize()
            torch_us = _median_us(lambda: torch.matmul(A, B, out=C))
            flops = 2.0 * n * n * n
            print(f"  M=K=N={n}: custom {custom_us:8.2f} us ({flops / custom_us / 1e6:6.2f} TFLOP/s)   "
                  f"torch.matmul {torch_us:8.2f} us ({flops / torch_us / 1e6:6.2f} TFLOP/s)   speedup {torch_us / custom_us:.2f}x")
    return 0


if __name__ == "__main__":
    sys.exit(main())
