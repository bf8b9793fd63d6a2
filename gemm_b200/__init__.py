"""gemm_b200 — B200 (sm_100a) GEMM kernels behind the operator interface of danielvegamyhre/gemm.

``gemm_b200.ops`` binds the C-ABI shared library (``include/gemm_b200.h``);
``gemm_b200.variants`` loads the three reference-named PyTorch extension modules;
``gemm_b200.sharded`` holds the row-sharded multi-GPU driver;
``gemm_b200.build`` compiles the native parts in-tree.

The operators are re-exported here and resolved on first use, so ``python -m gemm_b200.build``
works before the library exists.  There is no fallback: touching an operator without the built
library raises ImportError."""
import importlib

_OPS = (
    "sgemm_f32", "sgemm_f32_batched", "gemm_bf16", "gemm_bf16_batched", "gemm_bf16_grouped", "gemm_bf16_at", "check_status", "sgemm_f32_host", "gemm_bf16_host",
    "sgemm_f32_configs", "gemm_bf16_configs", "launch_count",
    "quantize_mxfp8", "gemm_mxfp8", "gemm_mxfp8_configs", "MxFp8Tensor", "gemm_mxfp8_splitk", "gemm_mxfp8_auto_splits", "gemm_mxfp8_quant_out", "gemm_mxfp8_grouped", "quantize_mxfp8_stack",
)


def __getattr__(name):
    if name in _OPS:
        return getattr(importlib.import_module(".ops", __name__), name)
    if name == "GemmB200Error":
        return importlib.import_module("._lib", __name__).GemmB200Error
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__():
    return sorted(list(globals()) + list(_OPS) + ["GemmB200Error"])
