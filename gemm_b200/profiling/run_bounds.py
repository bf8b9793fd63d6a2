"""Run the library's operators on ragged shapes under the bounds-checking build and report what
its checks saw (needs the debug build of the library):

    python -m gemm_b200.build --debug
    GEMM_B200_LIB=gemm_b200/profiling/libgemm_b200_debug.so python -m gemm_b200.profiling.run_bounds [--shrink BYTES]

Every global access the kernels address themselves is checked against the extent of its matrix
before it is made; an access outside is skipped and recorded, never made.  With --shrink the
checker is told that every matrix is BYTES shorter than it is, so it must refuse (and skip) the
accesses near the end of each matrix: this shows that the checks fire without any access ever
leaving a matrix.  Prints one line per case and exits 0 when every case met the expectation
(clean without --shrink, refused with it)."""
from __future__ import annotations

import argparse
import ctypes

import torch

from .. import _lib, ops


def _read(fn, shrink: int):
    out = (ctypes.c_int32 * 4)()
    code = fn(out, ctypes.c_longlong(shrink))
    if code not in (0, _lib.ERR_BOUNDS):
        raise SystemExit(f"reading the bounds status failed: {code}")
    return list(out)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--shrink", type=int, default=0)
    a = ap.parse_args(argv)
    lib = _lib.lib
    if not hasattr(lib, "gemm_b200_debug_bounds_f32"):
        raise SystemExit("this build of the library has no bounds checks: build with `python -m gemm_b200.build --debug` "
                         "and point GEMM_B200_LIB at gemm_b200/profiling/libgemm_b200_debug.so")
    for name in ("gemm_b200_debug_bounds_f32", "gemm_b200_debug_bounds_tc"):
        f = getattr(lib, name)
        f.argtypes = [ctypes.POINTER(ctypes.c_int32), ctypes.c_longlong]
        f.restype = ctypes.c_int
    f32, tc = lib.gemm_b200_debug_bounds_f32, lib.gemm_b200_debug_bounds_tc
    g = torch.Generator(device="cuda").manual_seed(0)
    rnd = lambda *s: torch.randn(*s, device="cuda", generator=g)

    def case_f32(M, K, N):
        A, B, C = rnd(M, K), rnd(K, N), torch.zeros(M, N, device="cuda")
        ops.sgemm_f32(A, B, C)
        return f32

    def case_bf16(M, K, N, **kw):
        A, B = rnd(M, K).bfloat16(), rnd(K, N).bfloat16()
        dtype = kw.pop("dtype", torch.bfloat16)
        C = torch.zeros(M, N, device="cuda", dtype=dtype)
        ops.gemm_bf16(A, B, C, out_dtype=dtype, **kw)
        return tc

    def case_mx(M, K, N, **kw):
        A, B = rnd(M, K).bfloat16(), rnd(K, N).bfloat16()
        Aq, Bq = ops.quantize_mxfp8(A), ops.quantize_mxfp8(B, transposed_in=True)
        C = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
        ops.gemm_mxfp8(Aq, Bq, C, **kw)
        return tc

    cases = [
        ("f32 257 x 100 x 131", lambda: case_f32(257, 100, 131)),
        ("f32 1000 x 333 x 1004", lambda: case_f32(1000, 333, 1004)),
        ("bf16 direct stores 200 x 512 x 136", lambda: case_bf16(200, 512, 136, config=0)),
        ("bf16 direct stores f32 out 130 x 256 x 72", lambda: case_bf16(130, 256, 72, config=0, dtype=torch.float32)),
        ("bf16 split-K with scratch 128 x 16384 x 256", lambda: case_bf16(128, 16384, 256, k_splits=4)),
        ("mxfp8 skinny 16 x 4096 x 520", lambda: case_mx(16, 4096, 520)),
        ("mxfp8 row quantiser 300 x 1024 (+ 300 x 1024 x 264 GEMM)", lambda: case_mx(300, 1024, 264)),
    ]
    for fn in (f32, tc):
        _read(fn, a.shrink)                                  # clear, set the knob
    bad = 0
    for name, run in cases:
        reader = run()
        st = _read(reader, a.shrink)
        refused = st[0] == _lib.ERR_BOUNDS
        ok = refused == (a.shrink > 0)
        bad += not ok
        print(f"{'ok ' if ok else 'BAD'} {name}: " + (f"refused at site {st[2]}, block {st[1]}, byte offset {st[3]}" if refused else "clean"))
    for fn in (f32, tc):
        _read(fn, 0)
    ops.check_status()
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main())
