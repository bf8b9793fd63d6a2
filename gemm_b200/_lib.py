"""ctypes binding of ``libgemm_b200.so`` (the C-ABI declared in ``include/gemm_b200.h``).

The library is the product: there is no Python or CPU fallback.  If the shared object is
missing or does not load, importing this module raises."""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

# GEMM_B200_LIB points at another build of the same library (e.g. a tuning build)
LIB_PATH = Path(os.environ.get("GEMM_B200_LIB") or (Path(__file__).resolve().parent / "libgemm_b200.so"))

OK = 0
ERR_INVALID_ARG, ERR_ALIGNMENT, ERR_UNSUPPORTED, ERR_CUDA, ERR_TIMEOUT, ERR_TOO_LARGE, ERR_BOUNDS = -1, -2, -3, -4, -5, -6, -7
OUT_BF16, OUT_F32 = 0, 1
B_ROW_MAJOR_KN, B_ROW_MAJOR_NK = 0, 1

i64, i32, vp, sz = C.c_int64, C.c_int, C.c_void_p, C.c_size_t

# name -> (restype, argtypes); every symbol include/gemm_b200.h declares
SIGNATURES = {
    "gemm_b200_sgemm_f32": (i32, [vp, vp, vp, i64, i64, i64, i64, i64, i64, vp]),
    "gemm_b200_sgemm_f32_cfg": (i32, [vp, vp, vp, i64, i64, i64, i64, i64, i64, i32, vp]),
    "gemm_b200_sgemm_f32_batched": (i32, [vp, vp, vp, i64, i64, i64, i64, i64, i64, i64, i64, i64, i64, vp]),
    "gemm_b200_sgemm_f32_num_configs": (i32, []),
    "gemm_b200_sgemm_f32_config_name": (C.c_char_p, [i32]),
    "gemm_b200_gemm_bf16": (i32, [vp, vp, vp, i64, i64, i64, i64, i64, i64, i32, i32, vp]),
    "gemm_b200_gemm_bf16_cfg": (i32, [vp, vp, vp, i64, i64, i64, i64, i64, i64, i32, i32, i32, vp]),
    "gemm_b200_gemm_bf16_batched": (i32, [vp, vp, vp, i64, i64, i64, i64, i64, i64, i64, i64, i64, i64, i32, i32, vp]),
    "gemm_b200_gemm_bf16_at": (i32, [vp, vp, vp, i64, i64, i64, i64, i64, i64, i32, i32, vp]),
    "gemm_b200_gemm_bf16_grouped": (i32, [vp, vp, vp, i64, C.POINTER(C.c_int64), i64, i64, i64, i64, i64, i64, i32, i32, vp]),
    "gemm_b200_gemm_bf16_splitk": (i32, [vp, vp, vp, i64, i64, i64, i64, i64, i64, i32, i32, i32, vp, sz, vp]),
    "gemm_b200_gemm_bf16_cluster_splitk": (i32, [vp, vp, vp, i64, i64, i64, i64, i64, i64, i32, i32, i32, vp]),
    "gemm_b200_gemm_bf16_splitk_scratch_bytes": (sz, [i64, i64, i32]),
    "gemm_b200_gemm_bf16_auto_splits": (i32, [i64, i64, i64]),
    "gemm_b200_gemm_bf16_num_configs": (i32, []),
    "gemm_b200_gemm_bf16_config_name": (C.c_char_p, [i32]),
    "gemm_b200_quantize_mxfp8": (i32, [vp, i64, i64, i64, i32, vp, vp, vp]),
    "gemm_b200_mxfp8_scale_bytes": (sz, [i64, i64]),
    "gemm_b200_mxfp8_scale_offset": (sz, [i64, i64, i64, i64]),
    "gemm_b200_gemm_mxfp8": (i32, [vp, vp, vp, vp, vp, i64, i64, i64, i64, i32, vp]),
    "gemm_b200_gemm_mxfp8_cfg": (i32, [vp, vp, vp, vp, vp, i64, i64, i64, i64, i32, i32, vp]),
    "gemm_b200_gemm_mxfp8_quant_out": (i32, [vp, vp, vp, vp, vp, vp, i64, i64, i64, vp]),
    "gemm_b200_gemm_mxfp8_splitk": (i32, [vp, vp, vp, vp, vp, i64, i64, i64, i64, i32, i32, vp, sz, vp]),
    "gemm_b200_gemm_mxfp8_grouped": (i32, [vp, vp, vp, vp, vp, i64, C.POINTER(C.c_int64), i64, i64, i64, i32, vp]),
    "gemm_b200_gemm_mxfp8_cluster_splitk": (i32, [vp, vp, vp, vp, vp, i64, i64, i64, i64, i32, i32, vp]),
    "gemm_b200_gemm_mxfp8_splitk_scratch_bytes": (sz, [i64, i64, i32]),
    "gemm_b200_gemm_mxfp8_splitk_static": (i32, [vp, vp, vp, vp, vp, i64, i64, i64, i64, i32, i32, vp]),
    "gemm_b200_gemm_mxfp8_auto_splits": (i32, [i64, i64, i64]),
    "gemm_b200_gemm_mxfp8_num_configs": (i32, []),
    "gemm_b200_gemm_mxfp8_config_name": (C.c_char_p, [i32]),
    "gemm_b200_sgemm_f32_host": (i32, [vp, vp, vp, i64, i64, i64]),
    "gemm_b200_gemm_bf16_host": (i32, [vp, vp, vp, i64, i64, i64, i32, i32]),
    "gemm_b200_release_workspace": (i32, []),
    "gemm_b200_check_status": (i32, [vp, C.POINTER(C.c_int32)]),
    "gemm_b200_selftest_wait_timeout": (i32, [i64, vp, vp]),
    "gemm_b200_last_error": (C.c_char_p, []),
    "gemm_b200_version": (i32, []),
    "gemm_b200_device_supported": (i32, [i32]),
    "gemm_b200_launch_count": (i64, []),
}


class GemmB200Error(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"gemm_b200 error {code}: {message}")
        self.code = code


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m gemm_b200.build` (needs nvcc); "
            "gemm_b200 has no fallback path")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)   # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def last_error() -> str:
    return (lib.gemm_b200_last_error() or b"").decode()


def check(rc: int) -> None:
    if rc != OK:
        raise GemmB200Error(rc, last_error())
