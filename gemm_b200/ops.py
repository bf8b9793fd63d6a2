"""Operators of the library on torch CUDA tensors.

torch is used for device memory and streams only; every function here hands raw pointers to
the C-ABI (``include/gemm_b200.h``).  The calling convention mirrors the reference wrappers
(naive/naive.cpp:6-22): ``f(A, B, C) -> C`` writes the caller's C in place and returns it;
``out=None`` allocates."""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import lib, check

__all__ = [
    "sgemm_f32", "sgemm_f32_batched", "gemm_bf16", "gemm_bf16_batched", "gemm_bf16_grouped", "gemm_bf16_at", "check_status", "sgemm_f32_host", "gemm_bf16_host",
    "sgemm_f32_configs", "gemm_bf16_configs", "launch_count",
    "quantize_mxfp8", "gemm_mxfp8", "gemm_mxfp8_configs", "MxFp8Tensor", "gemm_mxfp8_splitk", "gemm_mxfp8_auto_splits", "gemm_mxfp8_quant_out", "gemm_mxfp8_grouped", "quantize_mxfp8_stack",
]


# torch's raw accessors (an integer handle instead of a Stream object, the device index without the
# lazy-initialisation check) when this build of torch has them: they take a few microseconds off
# every call, which is what a small GEMM costs on the device
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _current_device() -> int:
    return _raw_device() if _raw_device is not None else torch.cuda.current_device()


def _stream(t: torch.Tensor) -> int:
    if _raw_stream is not None:
        idx = t.device.index
        return _raw_stream(idx if idx is not None else _current_device())
    return torch.cuda.current_stream(t.device).cuda_stream


class _OnDevice:
    """Makes the tensor's device current for the duration of a C-ABI call; free when it already is
    (the usual case), which keeps the Python overhead of a small GEMM to a few microseconds."""

    __slots__ = ("idx", "prev")

    def __init__(self, device: torch.device):
        self.idx = device.index if device.index is not None else _current_device()
        self.prev = -1

    def __enter__(self):
        cur = _current_device()
        if cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)
        return self

    def __exit__(self, *exc):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
        return False


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)


def _row_major_ld(t: torch.Tensor) -> int:
    _require(t.dim() == 2, "expected a 2-D tensor")
    (rows, cols), (s0, s1) = t.shape, t.stride()
    _require(cols <= 1 or s1 == 1, "tensor must be row-major (unit column stride)")
    return s0 if rows > 1 else max(cols, 1)


def sgemm_f32(A: torch.Tensor, B: torch.Tensor, out: torch.Tensor | None = None, config: int = -1) -> torch.Tensor:
    """FP32 ``C = A @ B`` on CUDA cores, bit-identical to the reference kernels."""
    _require(A.is_cuda and B.is_cuda, "A and B must be CUDA tensors")
    _require(A.dtype == torch.float32 and B.dtype == torch.float32, "expected float32")
    M, K = A.shape
    _require(B.shape[0] == K, f"A is {tuple(A.shape)} but B is {tuple(B.shape)}")
    N = B.shape[1]
    if out is None:
        out = torch.empty((M, N), device=A.device, dtype=torch.float32)
    _require(out.is_cuda and out.dtype == torch.float32 and tuple(out.shape) == (M, N), "bad out tensor")
    with _OnDevice(A.device):
        check(lib.gemm_b200_sgemm_f32_cfg(A.data_ptr(), B.data_ptr(), out.data_ptr(), M, N, K, _row_major_ld(A),
                                          _row_major_ld(B), _row_major_ld(out), config, _stream(A)))
    return out


def gemm_bf16(A: torch.Tensor, B: torch.Tensor, out: torch.Tensor | None = None, *, b_is_nk: bool = False,
              out_dtype: torch.dtype = torch.bfloat16, config: int = -1, k_splits: int = 0,
              cluster_splits: int = 0) -> torch.Tensor:
    """BF16 ``C = A @ B`` on the tensor cores with FP32 accumulation.

    ``B`` is ``[K, N]`` row-major (the reference's layout) or, with ``b_is_nk``, its transpose
    ``[N, K]`` row-major.  ``k_splits``: 0 lets the library cut K when the output has few tiles,
    1 never splits, n > 1 splits into n ranges of K (FP32 partial sums, summed in split order).
    ``cluster_splits`` = 2, 4 or 8 splits K over the CTAs of a cluster instead (one launch, partial
    sums combined through distributed shared memory)."""
    _require(A.is_cuda and B.is_cuda, "A and B must be CUDA tensors")
    _require(A.dtype == torch.bfloat16 and B.dtype == torch.bfloat16, "expected bfloat16")
    _require(out_dtype in (torch.bfloat16, torch.float32), "out_dtype must be bfloat16 or float32")
    M, K = A.shape
    if b_is_nk:
        N = B.shape[0]
        _require(B.shape[1] == K, f"A is {tuple(A.shape)} but Bt is {tuple(B.shape)}")
    else:
        N = B.shape[1]
        _require(B.shape[0] == K, f"A is {tuple(A.shape)} but B is {tuple(B.shape)}")
    if out is None:
        out = torch.empty((M, N), device=A.device, dtype=out_dtype)
    _require(out.is_cuda and out.dtype == out_dtype and tuple(out.shape) == (M, N), "bad out tensor")
    layout = _lib.B_ROW_MAJOR_NK if b_is_nk else _lib.B_ROW_MAJOR_KN
    od = _lib.OUT_F32 if out_dtype == torch.float32 else _lib.OUT_BF16
    with _OnDevice(A.device):
        if cluster_splits:
            _require(config < 0 and k_splits == 0, "cluster_splits excludes k_splits and config")
            check(lib.gemm_b200_gemm_bf16_cluster_splitk(
                A.data_ptr(), B.data_ptr(), out.data_ptr(), M, N, K, _row_major_ld(A), _row_major_ld(B), _row_major_ld(out),
                layout, od, cluster_splits, _stream(A)))
        elif k_splits >= 1:
            _require(config < 0, "k_splits and config cannot both be given")
            nbytes = int(lib.gemm_b200_gemm_bf16_splitk_scratch_bytes(M, N, k_splits)) if k_splits > 1 else 0
            scratch = torch.empty((max(nbytes, 16),), device=A.device, dtype=torch.uint8)
            check(lib.gemm_b200_gemm_bf16_splitk(
                A.data_ptr(), B.data_ptr(), out.data_ptr(), M, N, K, _row_major_ld(A), _row_major_ld(B), _row_major_ld(out),
                layout, od, k_splits, scratch.data_ptr(), nbytes, _stream(A)))
        else:
            check(lib.gemm_b200_gemm_bf16_cfg(
                A.data_ptr(), B.data_ptr(), out.data_ptr(), M, N, K, _row_major_ld(A), _row_major_ld(B), _row_major_ld(out),
                layout, od, config, _stream(A)))
    return out


def gemm_bf16_at(At: torch.Tensor, B: torch.Tensor, out: torch.Tensor | None = None, *, b_is_nk: bool = False,
                 out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """BF16 ``C = At.T @ B`` with A given as its transpose ``At`` ``[K, M]`` row-major — the layout in which an
    activation matrix enters a weight-gradient product — without a transposing copy."""
    _require(At.is_cuda and B.is_cuda, "At and B must be CUDA tensors")
    _require(At.dtype == torch.bfloat16 and B.dtype == torch.bfloat16, "expected bfloat16")
    _require(out_dtype in (torch.bfloat16, torch.float32), "out_dtype must be bfloat16 or float32")
    K, M = At.shape
    if b_is_nk:
        N = B.shape[0]
        _require(B.shape[1] == K, f"At is {tuple(At.shape)} but Bt is {tuple(B.shape)}")
    else:
        N = B.shape[1]
        _require(B.shape[0] == K, f"At is {tuple(At.shape)} but B is {tuple(B.shape)}")
    if out is None:
        out = torch.empty((M, N), device=At.device, dtype=out_dtype)
    _require(out.is_cuda and out.dtype == out_dtype and tuple(out.shape) == (M, N), "bad out tensor")
    layout = _lib.B_ROW_MAJOR_NK if b_is_nk else _lib.B_ROW_MAJOR_KN
    od = _lib.OUT_F32 if out_dtype == torch.float32 else _lib.OUT_BF16
    with _OnDevice(At.device):
        check(lib.gemm_b200_gemm_bf16_at(At.data_ptr(), B.data_ptr(), out.data_ptr(), M, N, K, _row_major_ld(At), _row_major_ld(B),
                                         _row_major_ld(out), layout, od, _stream(At)))
    return out


def _batch_layout(t: torch.Tensor) -> tuple[int, int]:
    """(row pitch, batch stride) in elements of a [batch, rows, cols] tensor whose matrices are row-major."""
    _require(t.stride(2) == 1 or t.shape[2] == 1, "the last dimension of every matrix must be contiguous")
    ld = t.stride(1) if t.shape[1] > 1 else max(t.shape[2], 1)
    return ld, t.stride(0)


def gemm_bf16_batched(A: torch.Tensor, B: torch.Tensor, out: torch.Tensor | None = None, *, b_is_nk: bool = False,
                      out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``out[i] = A[i] @ B[i]`` for a batch of equally shaped BF16 problems in one launch.

    ``A`` is ``[batch, M, K]``; ``B`` is ``[batch, K, N]`` (``[batch, N, K]`` with ``b_is_nk``) or a single
    2-D matrix shared by every problem."""
    _require(A.is_cuda and B.is_cuda, "A and B must be CUDA tensors")
    _require(A.dtype == torch.bfloat16 and B.dtype == torch.bfloat16, "expected bfloat16")
    _require(out_dtype in (torch.bfloat16, torch.float32), "out_dtype must be bfloat16 or float32")
    _require(A.dim() == 3 and B.dim() in (2, 3), "A must be 3-D and B 2-D or 3-D")
    batch, M, K = (int(x) for x in A.shape)
    bk, bn = (-1, -2) if b_is_nk else (-2, -1)
    N = int(B.shape[bn])
    _require(B.shape[bk] == K and (B.dim() == 2 or B.shape[0] == batch), f"A is {tuple(A.shape)} but B is {tuple(B.shape)}")
    lda, sa = _batch_layout(A)
    if B.dim() == 3:
        ldb, sb = _batch_layout(B)
        if batch > 1:
            _require(sb != 0, "pass a shared B as a 2-D tensor")
    else:
        ldb, sb = _row_major_ld(B), 0
    if out is None:
        out = torch.empty((batch, M, N), device=A.device, dtype=out_dtype)
    _require(out.is_cuda and out.dtype == out_dtype and tuple(out.shape) == (batch, M, N), "bad out tensor")
    ldc, sc = _batch_layout(out)
    with _OnDevice(A.device):
        check(lib.gemm_b200_gemm_bf16_batched(
            A.data_ptr(), B.data_ptr(), out.data_ptr(), batch, M, N, K, lda, ldb, ldc, sa, sb, sc,
            _lib.B_ROW_MAJOR_NK if b_is_nk else _lib.B_ROW_MAJOR_KN,
            _lib.OUT_F32 if out_dtype == torch.float32 else _lib.OUT_BF16, _stream(A)))
    return out


def sgemm_f32_batched(A: torch.Tensor, B: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out[i] = A[i] @ B[i]`` for a batch of equally shaped FP32 problems in one launch, each
    bit-identical to ``sgemm_f32``.  ``A`` is ``[batch, M, K]``; ``B`` is ``[batch, K, N]`` or a
    single 2-D matrix shared by every problem."""
    _require(A.is_cuda and B.is_cuda, "A and B must be CUDA tensors")
    _require(A.dtype == torch.float32 and B.dtype == torch.float32, "expected float32")
    _require(A.dim() == 3 and B.dim() in (2, 3), "A must be 3-D and B 2-D or 3-D")
    batch, M, K = (int(x) for x in A.shape)
    N = int(B.shape[-1])
    _require(B.shape[-2] == K and (B.dim() == 2 or B.shape[0] == batch), f"A is {tuple(A.shape)} but B is {tuple(B.shape)}")
    lda, sa = _batch_layout(A)
    if B.dim() == 3:
        ldb, sb = _batch_layout(B)
        if batch > 1:
            _require(sb != 0, "pass a shared B as a 2-D tensor")
    else:
        ldb, sb = _row_major_ld(B), 0
    if out is None:
        out = torch.empty((batch, M, N), device=A.device, dtype=torch.float32)
    _require(out.is_cuda and out.dtype == torch.float32 and tuple(out.shape) == (batch, M, N), "bad out tensor")
    ldc, sc = _batch_layout(out)
    with _OnDevice(A.device):
        check(lib.gemm_b200_sgemm_f32_batched(A.data_ptr(), B.data_ptr(), out.data_ptr(), batch, M, N, K, lda, ldb, ldc,
                                              sa, sb, sc, _stream(A)))
    return out


def gemm_bf16_grouped(A: torch.Tensor, B: torch.Tensor, m_sizes, out: torch.Tensor | None = None, *, b_is_nk: bool = False,
                      out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Grouped (ragged) BF16 GEMM: rows of ``A`` [sum(m_sizes), K] belong to consecutive groups,
    group g is multiplied by ``B[g]`` ([groups, K, N], or [groups, N, K] with ``b_is_nk``) into the
    same rows of ``out`` [sum(m_sizes), N].  ``m_sizes``: a sequence of row counts on the host."""
    _require(A.is_cuda and B.is_cuda, "A and B must be CUDA tensors")
    _require(A.dtype == torch.bfloat16 and B.dtype == torch.bfloat16, "expected bfloat16")
    _require(A.dim() == 2 and B.dim() == 3, "A must be 2-D and B 3-D")
    sizes = [int(m) for m in m_sizes]
    groups, rows, K = len(sizes), int(A.shape[0]), int(A.shape[1])
    _require(B.shape[0] == groups and sum(sizes) == rows, f"{groups} groups with {sum(sizes)} rows, but A has {rows} rows and B {B.shape[0]} matrices")
    N = int(B.shape[1] if b_is_nk else B.shape[2])
    _require(int(B.shape[2] if b_is_nk else B.shape[1]) == K, f"A is {tuple(A.shape)} but B is {tuple(B.shape)}")
    ldb, sb = _batch_layout(B)
    if out is None:
        out = torch.empty((rows, N), device=A.device, dtype=out_dtype)
    _require(out.is_cuda and out.dtype == out_dtype and tuple(out.shape) == (rows, N), "bad out tensor")
    arr = (C.c_int64 * max(groups, 1))(*sizes)
    with _OnDevice(A.device):
        check(lib.gemm_b200_gemm_bf16_grouped(A.data_ptr(), B.data_ptr(), out.data_ptr(), groups, arr, N, K, _row_major_ld(A), ldb, sb,
                                              _row_major_ld(out), _lib.B_ROW_MAJOR_NK if b_is_nk else _lib.B_ROW_MAJOR_KN,
                                              _lib.OUT_F32 if out_dtype == torch.float32 else _lib.OUT_BF16, _stream(A)))
    return out


def check_status(device: torch.device | None = None) -> None:
    """Synchronises the current stream and raises if a bounded device-side wait gave up."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    detail = (C.c_int32 * 4)()
    with torch.cuda.device(dev):
        check(lib.gemm_b200_check_status(torch.cuda.current_stream(dev).cuda_stream, detail))


def sgemm_f32_host(A: torch.Tensor, B: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Host-buffer form: A, B, out are CPU tensors (pinned memory overlaps copies and compute)."""
    _require(not A.is_cuda and not B.is_cuda, "host entry point takes CPU tensors")
    _require(A.dtype == torch.float32 and B.dtype == torch.float32, "expected float32")
    _require(A.is_contiguous() and B.is_contiguous(), "host operands must be contiguous")
    M, K = A.shape
    _require(B.shape[0] == K, "shape mismatch")
    N = B.shape[1]
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32)
    _require(out.is_contiguous() and tuple(out.shape) == (M, N) and out.dtype == torch.float32, "bad out tensor")
    check(lib.gemm_b200_sgemm_f32_host(A.data_ptr(), B.data_ptr(), out.data_ptr(), M, N, K))
    return out


def gemm_bf16_host(A: torch.Tensor, B: torch.Tensor, out: torch.Tensor | None = None, *, b_is_nk: bool = False,
                   out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    _require(not A.is_cuda and not B.is_cuda, "host entry point takes CPU tensors")
    _require(A.dtype == torch.bfloat16 and B.dtype == torch.bfloat16, "expected bfloat16")
    _require(A.is_contiguous() and B.is_contiguous(), "host operands must be contiguous")
    M, K = A.shape
    N = B.shape[0] if b_is_nk else B.shape[1]
    _require((B.shape[1] if b_is_nk else B.shape[0]) == K, "shape mismatch")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype)
    _require(out.is_contiguous() and tuple(out.shape) == (M, N) and out.dtype == out_dtype, "bad out tensor")
    check(lib.gemm_b200_gemm_bf16_host(A.data_ptr(), B.data_ptr(), out.data_ptr(), M, N, K,
                                       _lib.B_ROW_MAJOR_NK if b_is_nk else _lib.B_ROW_MAJOR_KN,
                                       _lib.OUT_F32 if out_dtype == torch.float32 else _lib.OUT_BF16))
    return out


def sgemm_f32_configs() -> list[str]:
    return [lib.gemm_b200_sgemm_f32_config_name(i).decode() for i in range(lib.gemm_b200_sgemm_f32_num_configs())]


def gemm_bf16_configs() -> list[str]:
    return [lib.gemm_b200_gemm_bf16_config_name(i).decode() for i in range(lib.gemm_b200_gemm_bf16_num_configs())]


def launch_count() -> int:
    return int(lib.gemm_b200_launch_count())


class MxFp8Tensor:
    """An MXFP8 operand: `data` uint8 [rows, K] (e4m3, K contiguous) and `scales`, the packed UE8M0
    buffer in the layout of gemm_b200_mxfp8_scale_offset()."""

    def __init__(self, data: torch.Tensor, scales: torch.Tensor, rows: int, K: int):
        self.data, self.scales, self.rows, self.K = data, scales, rows, K

    def scale_matrix(self) -> torch.Tensor:
        """The scale bytes as a plain [rows, K/32] uint8 tensor on the host (tests, debugging)."""
        sc = self.scales.cpu()
        r = torch.arange(self.rows).view(-1, 1)
        kb = torch.arange(self.K // 32).view(1, -1)
        kchunks = -(-(self.K // 32) // 4)
        off = ((r // 128) * kchunks + kb // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + (kb % 4)
        return sc[off]


def quantize_mxfp8(X: torch.Tensor, transposed_in: bool = False) -> MxFp8Tensor:
    """bf16 -> MXFP8 along K.  `X` is [rows, K], or with `transposed_in` [K, rows] (e.g. B[K, N])."""
    _require(X.is_cuda and X.dtype == torch.bfloat16 and X.dim() == 2, "expected a 2-D CUDA bfloat16 tensor")
    ldx = _row_major_ld(X)
    K, rows = (X.shape if transposed_in else (X.shape[1], X.shape[0]))
    rows, K = int(rows), int(K)
    data = torch.empty((rows, K), device=X.device, dtype=torch.uint8)
    scales = torch.empty((max(int(lib.gemm_b200_mxfp8_scale_bytes(rows, K)), 1),), device=X.device, dtype=torch.uint8)
    with _OnDevice(X.device):
        check(lib.gemm_b200_quantize_mxfp8(X.data_ptr(), rows, K, ldx, 1 if transposed_in else 0, data.data_ptr(),
                                           scales.data_ptr(), _stream(X)))
    return MxFp8Tensor(data, scales, rows, K)


def gemm_mxfp8(A: MxFp8Tensor, B: MxFp8Tensor, out: torch.Tensor | None = None, *,
               out_dtype: torch.dtype = torch.bfloat16, config: int = -1, cluster_splits: int = 0) -> torch.Tensor:
    """C[M, N] = dequant(A)[M, K] @ dequant(B)[N, K]^T on the block-scaled tensor cores.
    ``cluster_splits`` = 2, 4 or 8 splits K over the CTAs of a cluster (few-tile problems)."""
    _require(A.K == B.K, f"K mismatch: {A.K} vs {B.K}")
    _require(out_dtype in (torch.bfloat16, torch.float32), "out_dtype must be bfloat16 or float32")
    M, N, K = A.rows, B.rows, A.K
    if out is None:
        out = torch.empty((M, N), device=A.data.device, dtype=out_dtype)
    _require(out.is_cuda and out.dtype == out_dtype and tuple(out.shape) == (M, N), "bad out tensor")
    od = _lib.OUT_F32 if out_dtype == torch.float32 else _lib.OUT_BF16
    with _OnDevice(A.data.device):
        if cluster_splits:
            _require(config < 0, "cluster_splits and config cannot both be given")
            check(lib.gemm_b200_gemm_mxfp8_cluster_splitk(A.data.data_ptr(), A.scales.data_ptr(), B.data.data_ptr(),
                                                          B.scales.data_ptr(), out.data_ptr(), M, N, K, _row_major_ld(out), od,
                                                          cluster_splits, _stream(A.data)))
        else:
            check(lib.gemm_b200_gemm_mxfp8_cfg(A.data.data_ptr(), A.scales.data_ptr(), B.data.data_ptr(), B.scales.data_ptr(),
                                               out.data_ptr(), M, N, K, _row_major_ld(out), od, config, _stream(A.data)))
    return out


def quantize_mxfp8_stack(B3: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Quantises a stack of B matrices ``[groups, K, N]`` (bf16) for ``gemm_mxfp8_grouped``: returns the e4m3
    bytes ``[groups, N, K]`` and the packed scale buffers ``[groups, scale_bytes(N, K)]``, one matrix after another."""
    _require(B3.is_cuda and B3.dtype == torch.bfloat16 and B3.dim() == 3, "expected a 3-D CUDA bfloat16 tensor")
    G, K, N = (int(x) for x in B3.shape)
    sb = max(int(lib.gemm_b200_mxfp8_scale_bytes(N, K)), 1)
    data = torch.empty((G, N, K), device=B3.device, dtype=torch.uint8)
    scales = torch.empty((G, sb), device=B3.device, dtype=torch.uint8)
    for g in range(G):
        q = quantize_mxfp8(B3[g], transposed_in=True)
        data[g].copy_(q.data)
        scales[g].copy_(q.scales)
    return data, scales


def gemm_mxfp8_grouped(A: MxFp8Tensor, b_data: torch.Tensor, b_scales: torch.Tensor, m_sizes, out: torch.Tensor | None = None, *,
                       out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Grouped MXFP8 GEMM: rows of group g of ``A`` (quantised as one tall matrix) times ``B_g`` into the same
    rows of ``out``.  ``b_data`` ``[groups, N, K]`` / ``b_scales`` ``[groups, scale_bytes]`` as ``quantize_mxfp8_stack``
    returns them; every entry of ``m_sizes`` a multiple of 256 (pad the groups), their sum ``A.rows``."""
    _require(b_data.is_cuda and b_data.dtype == torch.uint8 and b_data.dim() == 3 and b_data.is_contiguous(), "b_data must be a contiguous [groups, N, K] uint8 tensor")
    _require(b_scales.is_cuda and b_scales.dtype == torch.uint8 and b_scales.dim() == 2 and b_scales.is_contiguous(), "b_scales must be a contiguous [groups, bytes] uint8 tensor")
    _require(out_dtype in (torch.bfloat16, torch.float32), "out_dtype must be bfloat16 or float32")
    sizes = [int(m) for m in m_sizes]
    G, N, K = (int(x) for x in b_data.shape)
    _require(len(sizes) == G, f"{len(sizes)} group sizes for {G} B matrices")
    _require(K == A.K, f"K mismatch: {A.K} vs {K}")
    _require(sum(sizes) == A.rows, f"the group sizes sum to {sum(sizes)}, A has {A.rows} rows")
    _require(b_scales.shape[0] == G and b_scales.shape[1] == max(int(lib.gemm_b200_mxfp8_scale_bytes(N, K)), 1), "b_scales has the wrong shape")
    if out is None:
        out = torch.empty((A.rows, N), device=A.data.device, dtype=out_dtype)
    _require(out.is_cuda and out.dtype == out_dtype and tuple(out.shape) == (A.rows, N), "bad out tensor")
    arr = (C.c_int64 * max(G, 1))(*sizes)
    od = _lib.OUT_F32 if out_dtype == torch.float32 else _lib.OUT_BF16
    with _OnDevice(A.data.device):
        check(lib.gemm_b200_gemm_mxfp8_grouped(A.data.data_ptr(), A.scales.data_ptr(), b_data.data_ptr(), b_scales.data_ptr(),
                                               out.data_ptr(), G, arr, N, K, _row_major_ld(out), od, _stream(A.data)))
    return out


def gemm_mxfp8_quant_out(A: MxFp8Tensor, B: MxFp8Tensor) -> MxFp8Tensor:
    """GEMM whose epilogue emits C already quantised to MXFP8 along its columns (the A operand of a
    following GEMM).  Same bytes as ``quantize_mxfp8(gemm_mxfp8(A, B))``."""
    _require(A.K == B.K, f"K mismatch: {A.K} vs {B.K}")
    M, N, K = A.rows, B.rows, A.K
    _require(N % 32 == 0, "N must be a multiple of 32")
    dev = A.data.device
    data = torch.empty((M, N), device=dev, dtype=torch.uint8)
    scales = torch.empty((max(int(lib.gemm_b200_mxfp8_scale_bytes(M, N)), 1),), device=dev, dtype=torch.uint8)
    with _OnDevice(dev):
        check(lib.gemm_b200_gemm_mxfp8_quant_out(A.data.data_ptr(), A.scales.data_ptr(), B.data.data_ptr(), B.scales.data_ptr(),
                                                 data.data_ptr(), scales.data_ptr(), M, N, K, _stream(A.data)))
    return MxFp8Tensor(data, scales, M, N)


def gemm_mxfp8_splitk(A: MxFp8Tensor, B: MxFp8Tensor, k_splits: int, out: torch.Tensor | None = None, *,
                      out_dtype: torch.dtype = torch.bfloat16, scratch: torch.Tensor | None = None) -> torch.Tensor:
    """Split-K form with a caller-owned scratch tensor (allocated here when not given)."""
    _require(A.K == B.K, f"K mismatch: {A.K} vs {B.K}")
    M, N, K = A.rows, B.rows, A.K
    if out is None:
        out = torch.empty((M, N), device=A.data.device, dtype=out_dtype)
    need = int(lib.gemm_b200_gemm_mxfp8_splitk_scratch_bytes(M, N, k_splits))
    if scratch is None:
        scratch = torch.empty((max(need, 16),), device=A.data.device, dtype=torch.uint8)
    with _OnDevice(A.data.device):
        check(lib.gemm_b200_gemm_mxfp8_splitk(A.data.data_ptr(), A.scales.data_ptr(), B.data.data_ptr(), B.scales.data_ptr(),
                                              out.data_ptr(), M, N, K, _row_major_ld(out),
                                              _lib.OUT_F32 if out_dtype == torch.float32 else _lib.OUT_BF16, k_splits,
                                              scratch.data_ptr(), scratch.numel() * scratch.element_size(), _stream(A.data)))
    return out


def gemm_mxfp8_auto_splits(M: int, N: int, K: int) -> int:
    return int(lib.gemm_b200_gemm_mxfp8_auto_splits(M, N, K))


def gemm_mxfp8_configs() -> list[str]:
    return [lib.gemm_b200_gemm_mxfp8_config_name(i).decode() for i in range(lib.gemm_b200_gemm_mxfp8_num_configs())]
