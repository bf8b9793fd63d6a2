"""The C-ABI library without a GPU: it loads, exports every symbol the header declares, and the
argument checks that precede any CUDA call behave."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "gemm_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gemm_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for must in ("gemm_b200_sgemm_f32", "gemm_b200_gemm_bf16", "gemm_b200_quantize_mxfp8", "gemm_b200_gemm_mxfp8",
                 "gemm_b200_sgemm_f32_host", "gemm_b200_check_status", "gemm_b200_last_error"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from gemm_b200 import _lib
    raw = C.CDLL(str(_lib.LIB_PATH))
    for name in declared_symbols():
        assert hasattr(raw, name), name
    assert set(_lib.SIGNATURES) == set(declared_symbols())


def test_diagnostic_builds_export_the_same_entry_points_plus_their_own():
    prof = ROOT / "gemm_b200" / "profiling"
    for lib, extra in (("libgemm_b200_debug.so", ["gemm_b200_debug_bounds_f32", "gemm_b200_debug_bounds_tc"]),
                       ("libgemm_b200_trace.so", ["gemm_b200_trace_read"])):
        raw = C.CDLL(str(prof / lib))
        for name in declared_symbols() + extra:
            assert hasattr(raw, name), (lib, name)
    release = C.CDLL(str(ROOT / "gemm_b200" / "libgemm_b200.so"))
    assert not hasattr(release, "gemm_b200_debug_bounds_tc") and not hasattr(release, "gemm_b200_trace_read")


def test_version_and_config_tables():
    from gemm_b200 import _lib
    assert _lib.lib.gemm_b200_version() == 100
    import gemm_b200.ops as ops
    assert len(ops.sgemm_f32_configs()) >= 3 and all(ops.sgemm_f32_configs())
    assert len(ops.gemm_bf16_configs()) >= 2
    assert len(ops.gemm_mxfp8_configs()) >= 2
    assert _lib.lib.gemm_b200_sgemm_f32_config_name(999) == b""


def test_argument_checks_need_no_gpu():
    from gemm_b200 import _lib
    L = _lib.lib
    assert L.gemm_b200_sgemm_f32(None, None, None, -1, 1, 1, 1, 1, 1, None) == _lib.ERR_INVALID_ARG
    assert "negative" in _lib.last_error()
    assert L.gemm_b200_sgemm_f32(None, None, None, 0, 5, 5, 5, 5, 5, None) == _lib.OK       # empty: no-op
    assert L.gemm_b200_sgemm_f32(None, None, None, 4, 4, 4, 4, 4, 4, None) == _lib.ERR_INVALID_ARG
    assert L.gemm_b200_gemm_bf16(None, None, None, 4, 4, 4, 4, 4, 4, 7, 0, None) == _lib.ERR_INVALID_ARG
    assert L.gemm_b200_gemm_bf16(None, None, None, 4, 4, 4, 4, 4, 4, 0, 9, None) == _lib.ERR_INVALID_ARG
    assert L.gemm_b200_gemm_mxfp8(None, None, None, None, None, 4, 4, 32, 4, 0, None) == _lib.ERR_INVALID_ARG
    assert L.gemm_b200_quantize_mxfp8(None, 4, 48, 48, 0, None, None, None) == _lib.ERR_INVALID_ARG


def test_scale_layout_helpers_match_the_oracle(oracle):
    from gemm_b200 import _lib
    L = _lib.lib
    for rows, K in [(1, 32), (128, 128), (130, 96), (300, 320), (16384, 8192)]:
        assert L.gemm_b200_mxfp8_scale_bytes(rows, K) == oracle.mxfp8_scale_bytes(rows, K)
        for r, kb in [(0, 0), (rows - 1, K // 32 - 1), (rows // 2, (K // 32) // 2)]:
            assert L.gemm_b200_mxfp8_scale_offset(rows, K, r, kb) == oracle.mxfp8_scale_offset(rows, K, r, kb)


def test_variant_modules_import_and_export_the_reference_names():
    from gemm_b200.variants import load_variant
    assert hasattr(load_variant("naive"), "naive_gemm")              # naive/naive.cpp:25
    assert hasattr(load_variant("shared"), "gemm_cuda")              # shared/shared.cpp:25
    assert hasattr(load_variant("blocktile_1d"), "gemm_cuda")        # blocktile_1d/blocktile_1d.cpp:25
    for v in ("naive", "shared", "blocktile_1d"):
        assert hasattr(load_variant(v), "matmul")


def test_ops_fail_loudly_without_cuda_tensors():
    import torch
    import gemm_b200.ops as ops
    with pytest.raises(ValueError):
        ops.sgemm_f32(torch.zeros(4, 4), torch.zeros(4, 4))
    with pytest.raises(ValueError):
        ops.gemm_bf16(torch.zeros(8, 8, dtype=torch.bfloat16), torch.zeros(8, 8, dtype=torch.bfloat16))


def test_environment_knobs_are_documented_in_the_sources():
    text = (ROOT / "gemm_b200" / "csrc" / "common.cuh").read_text()
    for knob in ("GEMM_B200_LOG", "GEMM_B200_F32_CONFIG", "GEMM_B200_BF16_CONFIG", "GEMM_B200_MXFP8_CONFIG"):
        assert knob in text
