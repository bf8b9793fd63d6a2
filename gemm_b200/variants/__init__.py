"""The three reference-named PyTorch extension modules, prebuilt in-tree.

``load_variant("naive")`` returns the module the reference's scripts obtain from
``load(name='naive_gemm_cuda', sources=['naive.cpp', 'naive_1.cu'])`` (naive/test.py:5-11);
likewise ``"shared"`` -> ``shared_gemm`` (shared/test.py:5-11) and ``"blocktile_1d"`` ->
``blocktile_1d`` (blocktile_1d/test.py:5-11).  The sources in these directories carry the
reference's file names, so the reference's own two-file JIT build also works from here."""
from __future__ import annotations

import importlib.util
from pathlib import Path

HERE = Path(__file__).resolve().parent

MODULES = {"naive": "naive_gemm_cuda", "shared": "shared_gemm", "blocktile_1d": "blocktile_1d"}
ENTRY = {"naive": "naive_gemm", "shared": "gemm_cuda", "blocktile_1d": "gemm_cuda"}


def load_variant(variant: str):
    import torch  # noqa: F401  (the extension links against libtorch)

    name = MODULES[variant]
    path = HERE / variant / (name + ".so")
    if not path.exists():
        raise ImportError(f"{path} is missing: build it with `python -m gemm_b200.build`")
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def entry_point(variant: str):
    """The reference's exported function of that variant: f(A, B, C) -> C."""
    return getattr(load_variant(variant), ENTRY[variant])
