"""Times the library's TMA streaming probe on a byte matrix of the given shape:

    python -m gemm_b200.run_stream [--rows 28672 --cols 8192 --rows-per-cta 256] [--reps 15]

Each launch only pulls the matrix through TMA into shared memory, tiled like the B operand of the
skinny GEMMs, so its time (CUDA events, L2 flushed before each launch) is the floor a
bandwidth-bound GEMM call of the same footprint can be compared with."""
from __future__ import annotations

import argparse
import json

import torch

from . import _lib
from ._lib import check, lib

# pattern -> (description, rows per box)
PATTERNS = {0: ("256 rows x 128 B, 4 stages", 256), 1: ("256 rows x 128 B, 6 stages", 256),
            2: ("64 rows x 512 B, 6 stages", 64), 3: ("32 rows x 1024 B, 6 stages", 32)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--rows", type=int, default=28672)
    ap.add_argument("--cols", type=int, default=8192)
    ap.add_argument("--rows-per-cta", type=int, default=256)
    ap.add_argument("--reps", type=int, default=15)
    a = ap.parse_args(argv)
    X = torch.ones(a.rows, a.cols, device="cuda", dtype=torch.uint8)
    flush = torch.empty(256 << 20, device="cuda", dtype=torch.uint8)
    stream = torch.cuda.current_stream().cuda_stream
    for pattern, (name, box_rows) in PATTERNS.items():
        if a.rows_per_cta % box_rows:
            continue
        times = []
        for i in range(a.reps + 2):
            flush.zero_()
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
            check(lib.gemm_b200_selftest_tma_stream(X.data_ptr(), a.rows, a.cols, a.rows_per_cta, pattern, stream))
            e1.record()
            torch.cuda.synchronize()
            if i >= 2:
                times.append(e0.elapsed_time(e1))
        times.sort()
        med = times[len(times) // 2]
        print(json.dumps({"pattern": name, "ctas": a.rows // a.rows_per_cta, "median_us": round(med * 1e3, 1),
                          "gbps": round(a.rows * a.cols / med / 1e6)}))
    check(lib.gemm_b200_check_status(stream, None))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
