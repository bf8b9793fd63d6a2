"""`torch.library` registration of the operators, so graph capture (`torch.compile`, export) can
call them as opaque ops:

    import gemm_b200.torch_ops
    C = torch.ops.gemm_b200.sgemm_f32(A, B)
    C = torch.ops.gemm_b200.gemm_bf16(A, B, b_is_nk=False, out_f32=False)
    C = torch.ops.gemm_b200.gemm_bf16_batched(A3, B3)         # [batch, M, K] x [batch, K, N] (or a shared 2-D B)
    C = torch.ops.gemm_b200.gemm_bf16_at(At, B)               # At is A stored transposed, [K, M]
    C = torch.ops.gemm_b200.gemm_bf16_grouped(A, B3, [m0, m1, ...])   # ragged groups sharing N and K
    aq, asf = torch.ops.gemm_b200.quantize_mxfp8(A)           # e4m3 bytes [M, K] + packed UE8M0 scales
    bq, bsf = torch.ops.gemm_b200.quantize_mxfp8(B, True)     # B given as [K, N]
    C = torch.ops.gemm_b200.gemm_mxfp8(aq, asf, bq, bsf)

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


@torch.library.custom_op("gemm_b200::gemm_bf16_at", mutates_args=())
def gemm_bf16_at(At: torch.Tensor, B: torch.Tensor, b_is_nk: bool = False, out_f32: bool = False) -> torch.Tensor:
    return ops.gemm_bf16_at(At, B, b_is_nk=b_is_nk, out_dtype=torch.float32 if out_f32 else torch.bfloat16)


@gemm_bf16_at.register_fake
def _(At, B, b_is_nk=False, out_f32=False):
    torch._check(At.dim() == 2 and B.dim() == 2)
    n = B.shape[0] if b_is_nk else B.shape[1]
    return At.new_empty((At.shape[1], n), dtype=torch.float32 if out_f32 else torch.bfloat16)


@torch.library.custom_op("gemm_b200::gemm_bf16_grouped", mutates_args=())
def gemm_bf16_grouped(A: torch.Tensor, B: torch.Tensor, m_sizes: list[int], b_is_nk: bool = False,
                      out_f32: bool = False) -> torch.Tensor:
    return ops.gemm_bf16_grouped(A, B, m_sizes, b_is_nk=b_is_nk, out_dtype=torch.float32 if out_f32 else torch.bfloat16)


@gemm_bf16_grouped.register_fake
def _(A, B, m_sizes, b_is_nk=False, out_f32=False):
    torch._check(A.dim() == 2 and B.dim() == 3)
    n = B.shape[1] if b_is_nk else B.shape[2]
    return A.new_empty((A.shape[0], n), dtype=torch.float32 if out_f32 else torch.bfloat16)


# MXFP8: a quantised operand travels as two plain tensors, the e4m3 bytes [rows, K] and the packed
# UE8M0 scale buffer (layout of gemm_b200_mxfp8_scale_offset()).
@torch.library.custom_op("gemm_b200::quantize_mxfp8", mutates_args=())
def quantize_mxfp8(X: torch.Tensor, transposed_in: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    q = ops.quantize_mxfp8(X, transposed_in=transposed_in)
    return q.data, q.scales


def _scale_bytes(rows: int, K: int) -> int:
    return max(-(-rows // 128) * (-(-(K // 32) // 4)) * 512, 1)


@quantize_mxfp8.register_fake
def _(X, transposed_in=False):
    K, rows = (X.shape[0], X.shape[1]) if transposed_in else (X.shape[1], X.shape[0])
    return X.new_empty((rows, K), dtype=torch.uint8), X.new_empty((_scale_bytes(rows, K),), dtype=torch.uint8)


@torch.library.custom_op("gemm_b200::gemm_mxfp8", mutates_args=())
def gemm_mxfp8(a_data: torch.Tensor, a_scales: torch.Tensor, b_data: torch.Tensor, b_scales: torch.Tensor,
               out_f32: bool = False) -> torch.Tensor:
    A = ops.MxFp8Tensor(a_data, a_scales, a_data.shape[0], a_data.shape[1])
    B = ops.MxFp8Tensor(b_data, b_scales, b_data.shape[0], b_data.shape[1])
    return ops.gemm_mxfp8(A, B, out_dtype=torch.float32 if out_f32 else torch.bfloat16)


@gemm_mxfp8.register_fake
def _(a_data, a_scales, b_data, b_scales, out_f32=False):
    torch._check(a_data.dim() == 2 and b_data.dim() == 2 and a_data.shape[1] == b_data.shape[1])
    return a_data.new_empty((a_data.shape[0], b_data.shape[0]), dtype=torch.float32 if out_f32 else torch.bfloat16)
