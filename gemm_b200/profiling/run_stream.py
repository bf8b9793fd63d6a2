"""Times the TMA streaming probe (libgemm_b200_probe.so) on a byte matrix of the given shape:

    python -m gemm_b200.profiling.run_stream [--rows 28672 --cols 8192 --rows-per-cta 256] [--reps 15]

Each launch only pulls the matrix through TMA into shared memory, tiled like the B operand of the
skinny GEMMs, so its time (CUDA events, L2 flushed before each launch) is the floor a
bandwidth-bound GEMM call of the same footprint can be compared with."""
from __future__ import annotations

import argparse
import json

import torch

import ctypes as C
from pathlib import Path

PROBE_PATH = Path(__file__).resolve().parent / "libgemm_b200_probe.so"


def load_probe() -> C.CDLL:
    if not PROBE_PATH.exists():
        raise ImportError(f"{PROBE_PATH} is missing: build it with `python -m gemm_b200.build`")
    lib = C.CDLL(str(PROBE_PATH))
    lib.gemm_b200_probe_tma_stream.restype = C.c_int
    lib.gemm_b200_probe_tma_stream.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_void_p]
    lib.gemm_b200_probe_check_status.restype = C.c_int
    lib.gemm_b200_probe_check_status.argtypes = [C.c_void_p]
    lib.gemm_b200_probe_last_error.restype = C.c_char_p
    return lib


def check(lib: C.CDLL, rc: int) -> None:
    if rc != 0:
        raise RuntimeError(f"probe error {rc}: {(lib.gemm_b200_probe_last_error() or b'').decode()}")

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
    lib = load_probe()
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
            check(lib, lib.gemm_b200_probe_tma_stream(X.data_ptr(), a.rows, a.cols, a.rows_per_cta, pattern, stream))
            e1.record()
            torch.cuda.synchronize()
            if i >= 2:
                times.append(e0.elapsed_time(e1))
        times.sort()
        med = times[len(times) // 2]
        print(json.dumps({"pattern": name, "ctas": a.rows // a.rows_per_cta, "median_us": round(med * 1e3, 1),
                          "gbps": round(a.rows * a.cols / med / 1e6)}))
    check(lib, lib.gemm_b200_probe_check_status(stream))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
