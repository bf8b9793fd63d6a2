import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    return O


@pytest.fixture(scope="session")
def ops():
    """The product path: raises if the native library is missing (there is no fallback)."""
    import gemm_b200.ops as ops
    return ops


def pytest_sessionfinish(session, exitstatus):
    """Under the bounds-checking build (GEMM_B200_LIB pointing at libgemm_b200_debug.so) the whole GPU
    suite doubles as a bounds test: every access the kernels address themselves was checked against
    its matrix, and a refused access fails the session here."""
    mod = sys.modules.get("gemm_b200._lib")
    if mod is None or not hasattr(mod.lib, "gemm_b200_debug_bounds_f32"):
        return
    try:
        import torch
        if not torch.cuda.is_available():
            return
    except Exception:
        return
    import ctypes
    bad = []
    for name in ("gemm_b200_debug_bounds_f32", "gemm_b200_debug_bounds_tc"):
        fn = getattr(mod.lib, name)
        fn.argtypes = [ctypes.POINTER(ctypes.c_int32), ctypes.c_longlong]
        fn.restype = ctypes.c_int
        out = (ctypes.c_int32 * 4)()
        fn(out, ctypes.c_longlong(0))
        if out[0] != 0:
            bad.append(f"{name}: code {out[0]} block {out[1]} site {out[2]} byte offset {out[3]}")
    reporter = session.config.pluginmanager.get_plugin("terminalreporter")
    if bad:
        if reporter:
            reporter.write_line("bounds-checking build: an access outside its matrix was refused: " + "; ".join(bad), red=True)
        session.exitstatus = 1
    elif reporter:
        reporter.write_line("bounds-checking build: no access outside its matrix in this session")
