"""Stage timeline of one tensor-core launch (needs the trace build of the library):

    python -m gemm_b200.build --trace
    GEMM_B200_LIB=gemm_b200/profiling/libgemm_b200_trace.so \\
        python -m gemm_b200.profiling.run_trace {bf16|mxfp8} --m M --k K --n N [--config C] [--cluster-splits S]

Every CTA of the launch stamps the global nanosecond timer at fixed points (slots listed beside
trace_stamp in gemm_b200/csrc/tc_common.cuh); this prints, per slot, the earliest, median and
latest time over the CTAs, relative to the first CTA's entry."""
from __future__ import annotations

import argparse
import ctypes

import numpy as np
import torch

from .. import _lib, ops

SLOTS = ["kernel entry", "set-up done", "first TMA issued", "last load issued", "first stage arrived", "last MMA issued",
         "epilogue sees accumulator", "stores issued / partials sent", "stores complete / pieces landed",
         "before teardown barrier", "TMEM freed"]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("op", choices=["bf16", "mxfp8"])
    ap.add_argument("--m", type=int, default=128)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--config", type=int, default=-1)
    ap.add_argument("--k-splits", type=int, default=0, help="bf16: K ranges of the two-launch split (0: library decides, 1: never)")
    ap.add_argument("--cluster-splits", type=int, default=0)
    a = ap.parse_args(argv)
    lib = _lib.lib
    if not hasattr(lib, "gemm_b200_trace_read"):
        raise SystemExit("this build of the library has no stage timeline: build with `python -m gemm_b200.build --trace` "
                         "and point GEMM_B200_LIB at gemm_b200/profiling/libgemm_b200_trace.so")
    lib.gemm_b200_trace_read.argtypes = [ctypes.c_void_p, ctypes.c_int]
    lib.gemm_b200_trace_read.restype = ctypes.c_int
    g = torch.Generator(device="cuda").manual_seed(0)
    A = torch.randn(a.m, a.k, device="cuda", generator=g).bfloat16()
    B = torch.randn(a.k, a.n, device="cuda", generator=g).bfloat16()
    C = torch.empty(a.m, a.n, device="cuda", dtype=torch.bfloat16)
    if a.op == "bf16":
        fn = lambda: ops.gemm_bf16(A, B, C, config=a.config, k_splits=a.k_splits, cluster_splits=a.cluster_splits)
    else:
        Aq, Bq = ops.quantize_mxfp8(A), ops.quantize_mxfp8(B, transposed_in=True)
        fn = lambda: ops.gemm_mxfp8(Aq, Bq, C, config=a.config, cluster_splits=a.cluster_splits)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    flush.sum()                       # cold L2 without dirty lines
    torch.cuda.synchronize()
    fn()
    ops.check_status()
    buf = np.zeros((160, 16), dtype=np.uint64)
    _lib.check(lib.gemm_b200_trace_read(buf.ctypes.data, 160))
    entry = buf[:, 0]
    cur = (entry > 0) & (entry.max() - entry < 1_000_000)      # CTAs of the last launch
    t0 = int(entry[cur].min())
    print(f"{a.op} {a.m} x {a.k} x {a.n}: {int(cur.sum())} CTAs traced (of the first 160)")
    for i, name in enumerate(SLOTS):
        col = buf[cur][:, i]
        ok = col > 0
        if ok.any():
            rel = (col[ok].astype(np.int64) - t0) / 1e3
            print(f"  {name:34s} min {rel.min():7.2f}  median {np.median(rel):7.2f}  max {rel.max():7.2f} us")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
