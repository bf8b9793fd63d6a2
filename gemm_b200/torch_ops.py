"""`torch.library` registration of the operators, so graph capture (`torch.compile`, export) can
call them as opaque ops:

    import gemm_b200.torch_ops
    C = torch.ops.gemm_b200.sgemm_f32(A, B)
    C = torch.ops.gemm_b200.gemm_bf16(A, B, b_is_nk=False, out_f32=False)
    C = torch.ops.gemm_b200.gemm_bf16_batched(A3, B3)         # [batch, M, K] x [batch, K, N] (or a shared 2-D B)

The allocating forms are registered (out-parameter forms alias their argument, which the
reference's wrappers do by design, naive/naive.cpp:17-21, and which functional graphs cannot
express); each has a fake implementation for shape inference."""
from __future__ import annotations

import torch

from . import ops


@torch.library.custom_op("gemm_b200::sgemm_f32", mutates_args=())
def sgemm_f32(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    return ops.sgemm_f32(A, B)


@sgemm_f32.register_fake
def _(A, B):
    torch._check(A.dim() == 2 and B.dim() == 2 and A.shape[1] == B.shape[0])
    return A.new_empty((A.shape[0], B.shape[1]))


@torch.library.custom_op("gemm_b200::gemm_bf16", mutates_args=())
def gemm_bf16(A: torch.Tensor, B: torch.Tensor, b_is_nk: bool = False, out_f32: bool = False) -> torch.Tensor:
    return ops.gemm_bf16(A, B, b_is_nk=b_is_nk, out_dtype=torch.float32 if out_f32 else torch.bfloat16)


@gemm_bf16.register_fake
def _(A, B, b_is_nk=False, out_f32=False):
    n = B.shape[0] if b_is_nk else B.shape[1]
    return A.new_empty((A.shape[0], n), dtype=torch.float32 if out_f32 else torch.bfloat16)


@torch.library.custom_op("gemm_b200::gemm_bf16_batched", mutates_args=())
def gemm_bf16_batched(A: torch.Tensor, B: torch.Tensor, b_is_nk: bool = False, out_f32: bool = False) -> torch.Tensor:
    return ops.gemm_bf16_batched(A, B, b_is_nk=b_is_nk, out_dtype=torch.float32 if out_f32 else torch.bfloat16)


@gemm_bf16_batched.register_fake
def _(A, B, b_is_nk=False, out_f32=False):
    torch._check(A.dim() == 3 and B.dim() in (2, 3))
    n = B.shape[-2] if b_is_nk else B.shape[-1]
    return A.new_empty((A.shape[0], A.shape[1], n), dtype=torch.float32 if out_f32 else torch.bfloat16)
