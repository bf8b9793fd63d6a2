"""TEST INFRASTRUCTURE — the CPU oracle for the GEMM hot path.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference arms of ``bench.py``
may import this module.  The library (``gemm_b200/``) never does.

What is restated here, and from where:

* FP32 GEMM.  The reference's own check is ``torch.matmul`` on the same tensors
  (naive/test.py:23, shared/test.py:28, blocktile_1d/test.py:28) — :func:`matmul_cpu` is that
  check evaluated on the host.  :func:`sgemm_seq` restates the reference KERNELS' arithmetic
  (naive/naive_1.cu:9-13 and the two tiled kernels, which keep the same order): one FP32
  accumulator, k ascending, fused multiply-add, flush-to-zero.  It lives in ``sgemm_seq.c``.
* The reference kernels themselves, compiled unchanged into ``oracle/_ref/`` by the Makefile,
  callable on CUDA tensors through :func:`reference_kernel` (GPU box only).
* BF16 and MXFP8 have no counterpart in the reference (its three kernels are FP32 only).  Their
  oracle is the stated contract: an FP32 matmul of the very same (de)quantised operands.
  The MXFP8 quantiser is restated from the OCP microscaling recipe the benchmark config names:
  blocks of 32 along K, scale = 2^(floor(log2(amax)) - 8) stored as UE8M0, data = e4m3 with
  round-to-nearest-even and saturation at 448.  **Parity of these two paths is unpinned**: the
  reference holds no vectors for them; :func:`e4m3_encode` is pinned against torch's
  ``float8_e4m3fn`` cast in the tests instead.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
_LIB = None


def _lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        path = HERE / "liboracle.so"
        if not path.exists():
            raise ImportError(f"{path} missing: run `make -C oracle`")
        lib = C.CDLL(str(path))
        p, i64 = C.c_void_p, C.c_int64
        lib.oracle_sgemm_seq.argtypes = [p, p, p, i64, i64, i64, i64, i64, i64, C.c_int]
        lib.oracle_sgemm_seq.restype = None
        lib.oracle_sgemm_f64acc.argtypes = [p, p, p, i64, i64, i64, i64, i64, i64]
        lib.oracle_sgemm_f64acc.restype = None
        _LIB = lib
    return _LIB


# --------------------------------------------------------------------------------------
# seeded inputs of the benchmark configurations
# --------------------------------------------------------------------------------------
def gen_uniform_f32(M: int, K: int, N: int, seed: int = 0):
    """A then B, i.i.d. uniform[-1, 1) FP32 from torch.manual_seed(seed) (configs 1 and 2)."""
    g = torch.Generator().manual_seed(seed)
    A = torch.rand(M, K, generator=g, dtype=torch.float32) * 2 - 1
    B = torch.rand(K, N, generator=g, dtype=torch.float32) * 2 - 1
    return A, B


def gen_randn_f32(M: int, K: int, N: int, seed: int = 42):
    """The reference tests' inputs: manual_seed(42), randn A then B (naive/test.py:17-19).
    Generated on the host; the reference draws them on the GPU, so values differ, the
    distribution does not."""
    g = torch.Generator().manual_seed(seed)
    return torch.randn(M, K, generator=g), torch.randn(K, N, generator=g)


def gen_randn_bf16(M: int, K: int, N: int, seed: int = 0):
    """A, B ~ N(0,1) cast to bf16 (configs 3 to 5)."""
    g = torch.Generator().manual_seed(seed)
    A = torch.randn(M, K, generator=g).bfloat16()
    B = torch.randn(K, N, generator=g).bfloat16()
    return A, B


def gen_sharded_a_block(block: int, rows: int, K: int) -> torch.Tensor:
    """Block `block` (of fixed `rows` rows) of the row-sharded A of config 5: seed 1000 + block,
    so A is identical however many ranks it is split over."""
    g = torch.Generator().manual_seed(1000 + block)
    return torch.randn(rows, K, generator=g).bfloat16()


# --------------------------------------------------------------------------------------
# FP32
# --------------------------------------------------------------------------------------
def matmul_cpu(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    """The reference's oracle, torch.matmul (naive/test.py:23), on the host in FP32."""
    return torch.matmul(A.detach().cpu().float(), B.detach().cpu().float())


def sgemm_seq(A, B, ftz: bool = True) -> torch.Tensor:
    """Bit-level restatement of the reference kernels (sgemm_seq.c)."""
    a = np.ascontiguousarray(torch.as_tensor(A).detach().cpu().numpy(), dtype=np.float32)
    b = np.ascontiguousarray(torch.as_tensor(B).detach().cpu().numpy(), dtype=np.float32)
    M, K = a.shape
    K2, N = b.shape
    assert K == K2
    c = np.empty((M, N), dtype=np.float32)
    _lib().oracle_sgemm_seq(a.ctypes.data, b.ctypes.data, c.ctypes.data, M, N, K, max(K, 1), max(N, 1), max(N, 1),
                            1 if ftz else 0)
    return torch.from_numpy(c)


def matmul_f64(A, B) -> torch.Tensor:
    """FP64-accumulated product of FP32-representable operands: the 'truth' that separates a
    kernel's rounding error from the FP32 oracle's own."""
    a = np.ascontiguousarray(torch.as_tensor(A).detach().cpu().float().numpy())
    b = np.ascontiguousarray(torch.as_tensor(B).detach().cpu().float().numpy())
    M, K = a.shape
    _, N = b.shape
    c = np.empty((M, N), dtype=np.float64)
    _lib().oracle_sgemm_f64acc(a.ctypes.data, b.ctypes.data, c.ctypes.data, M, N, K, max(K, 1), max(N, 1), max(N, 1))
    return torch.from_numpy(c)


_REF_SYMBOLS = {
    "naive": ("libref_naive.so", "_Z17launch_naive_gemmPfS_S_iii"),          # naive/naive_1.cu:17
    "shared": ("libref_shared.so", "_Z11launch_gemmPfS_S_iii"),              # shared/shared_2.cu:59
    "blocktile_1d": ("libref_blocktile_1d.so", "_Z11launch_gemmPfS_S_iii"),  # blocktile_1d/blocktile_1d.cu:70
}
_REF_CACHE: dict = {}


def reference_available() -> bool:
    return all((HERE / "_ref" / f).exists() for f, _ in _REF_SYMBOLS.values())


def reference_kernel(variant: str):
    """The reference's own launcher for `variant`, compiled unchanged (oracle/Makefile).
    Returns f(A, B, C) on CUDA float32 tensors; launches on the legacy default stream exactly
    as the reference does, so callers synchronise around it."""
    if variant not in _REF_CACHE:
        fname, sym = _REF_SYMBOLS[variant]
        lib = C.CDLL(str(HERE / "_ref" / fname))
        fn = getattr(lib, sym)
        fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
        fn.restype = None
        _REF_CACHE[variant] = fn
    fn = _REF_CACHE[variant]

    def call(A: torch.Tensor, B: torch.Tensor, Cout: torch.Tensor) -> torch.Tensor:
        assert A.is_cuda and A.dtype == torch.float32 and A.is_contiguous() and B.is_contiguous() and Cout.is_contiguous()
        torch.cuda.current_stream().synchronize()
        fn(A.data_ptr(), B.data_ptr(), Cout.data_ptr(), A.shape[0], B.shape[1], A.shape[1])   # (M, N, K)
        torch.cuda.synchronize()
        return Cout

    return call


def reference_launcher(variant: str):
    """The same launcher without the synchronisation around it, for timing with events recorded on
    the legacy default stream (where the reference launches, naive/naive_1.cu:23): f(A, B, C)."""
    reference_kernel(variant)
    fn = _REF_CACHE[variant]

    def launch(A: torch.Tensor, B: torch.Tensor, Cout: torch.Tensor) -> None:
        fn(A.data_ptr(), B.data_ptr(), Cout.data_ptr(), A.shape[0], B.shape[1], A.shape[1])   # (M, N, K)

    return launch


# --------------------------------------------------------------------------------------
# error metrics
# --------------------------------------------------------------------------------------
def rel_frobenius(c: torch.Tensor, ref: torch.Tensor) -> float:
    c64, r64 = c.detach().cpu().double(), ref.detach().cpu().double()
    den = float(torch.linalg.norm(r64))
    return float(torch.linalg.norm(c64 - r64)) / (den if den > 0 else 1.0)


def assert_close_mismatches(c: torch.Tensor, ref: torch.Tensor, rtol: float = 1.3e-6, atol: float = 1e-5) -> int:
    """Number of elements torch.testing.assert_close (FP32 defaults, as in naive/test.py:26)
    would flag."""
    c64, r64 = c.detach().cpu().double(), ref.detach().cpu().double()
    return int(((c64 - r64).abs() > atol + rtol * r64.abs()).sum())


# --------------------------------------------------------------------------------------
# BF16
# --------------------------------------------------------------------------------------
def bf16_matmul_oracle(A_bf16: torch.Tensor, B_bf16: torch.Tensor) -> torch.Tensor:
    """FP32 matmul of the same BF16 operands (the stated BF16 contract)."""
    return torch.matmul(A_bf16.detach().cpu().float(), B_bf16.detach().cpu().float())


# --------------------------------------------------------------------------------------
# MXFP8: e4m3 data + UE8M0 scale per 32 consecutive K elements
# --------------------------------------------------------------------------------------
E4M3_MAX = 448.0
MX_BLOCK = 32


def e4m3_decode_table() -> np.ndarray:
    """All 256 e4m3 (fn: no infinities, 0x7f/0xff are NaN) values as float32."""
    t = np.zeros(256, dtype=np.float32)
    for b in range(256):
        s = -1.0 if b & 0x80 else 1.0
        e = (b >> 3) & 0xF
        m = b & 0x7
        if e == 0xF and m == 0x7:
            v = np.nan
        elif e == 0:
            v = m * 2.0 ** -9
        else:
            v = (1 + m / 8.0) * 2.0 ** (e - 7)
        t[b] = s * v
    return t


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> e4m3 byte: round to nearest even, saturate finite values at +-448
    (the behaviour of cvt.rn.satfinite.e4m3x2.f32); NaN -> 0x7f."""
    x = np.asarray(x, dtype=np.float32)
    sign = np.signbit(x)
    a = np.minimum(np.abs(x).astype(np.float64), E4M3_MAX)
    nan = np.isnan(x)
    a = np.where(nan, 0.0, a)
    _, e = np.frexp(a)                       # a = m * 2^e, m in [0.5, 1)
    E = np.maximum(e - 1, -6)                # exponent of the binade; subnormals share 2^-6
    step = np.ldexp(1.0, E - 3)
    q = np.rint(a / step) * step             # np.rint rounds half to even
    q = np.minimum(q, E4M3_MAX)
    _, e2 = np.frexp(q)
    E2 = e2 - 1
    sub = (q < 2.0 ** -6)
    mant_sub = np.rint(q / 2.0 ** -9).astype(np.int64)
    mant_norm = np.rint((q / np.ldexp(1.0, E2) - 1.0) * 8).astype(np.int64)
    byte = np.where(sub, mant_sub, ((E2 + 7) << 3) | mant_norm)
    byte = np.where(q == 0, 0, byte)
    byte = np.where(nan, 0x7F, byte)
    return (byte | (sign.astype(np.int64) << 7)).astype(np.uint8)


def mxfp8_quantize(x: torch.Tensor):
    """Quantise `x` [rows, K] (bf16 or float32 holding bf16 values) along K in blocks of 32.

    Returns (q uint8 [rows, K], scale uint8 [rows, K/32]) with
      scale byte = clamp(floor(log2(amax)) - 8, -127, 127) + 127   (amax == 0 -> byte 0)
      q          = e4m3_encode(x * 2^-(byte - 127)).
    """
    xf = x.detach().cpu().float().numpy()
    rows, K = xf.shape
    assert K % MX_BLOCK == 0
    blocks = xf.reshape(rows, K // MX_BLOCK, MX_BLOCK)
    amax = np.abs(blocks).max(axis=2)
    eb = (amax.view(np.uint32) >> 23) & 0xFF           # biased exponent = floor(log2(amax)) + 127
    byte = np.maximum(eb.astype(np.int64) - 8, 0).astype(np.uint8)
    inv_scale = np.ldexp(np.float32(1.0), 127 - byte.astype(np.int64)).astype(np.float32)
    scaled = blocks * inv_scale[:, :, None]
    q = e4m3_encode(scaled).reshape(rows, K)
    return torch.from_numpy(q), torch.from_numpy(byte)


def mxfp8_dequantize(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """float32 [rows, K] = e4m3 value * 2^(scale byte - 127)."""
    table = e4m3_decode_table()
    v = table[q.detach().cpu().numpy()]
    rows, K = v.shape
    s = np.ldexp(np.float32(1.0), scale.detach().cpu().numpy().astype(np.int64) - 127).astype(np.float32)
    return torch.from_numpy((v.reshape(rows, K // MX_BLOCK, MX_BLOCK) * s[:, :, None]).reshape(rows, K))


def mxfp8_scale_offset(rows: int, K: int, r: int, kb: int) -> int:
    """Byte offset of the scale of (row r, K-block kb) in the packed scale buffer the tensor-core
    kernel reads: 512-byte chunks of 128 rows x 4 K-blocks, stored as 32 x 16 bytes with
    byte (r % 32) * 16 + (r // 32 % 4) * 4 + kb % 4; chunks ordered [row block][kb // 4]."""
    kchunks = -(-(K // MX_BLOCK) // 4)
    chunk = (r // 128) * kchunks + kb // 4
    return chunk * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + (kb % 4)


def mxfp8_scale_bytes(rows: int, K: int) -> int:
    return (-(-rows // 128)) * (-(-(K // MX_BLOCK) // 4)) * 512


def mxfp8_pack_scales(scale: torch.Tensor, K: int) -> torch.Tensor:
    """[rows, K/32] scale bytes -> the packed buffer (padding bytes = 0)."""
    s = scale.detach().cpu().numpy()
    rows, kbs = s.shape
    out = np.zeros(mxfp8_scale_bytes(rows, K), dtype=np.uint8)
    r = np.arange(rows)[:, None]
    kb = np.arange(kbs)[None, :]
    kchunks = -(-kbs // 4)
    off = ((r // 128) * kchunks + kb // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + (kb % 4)
    out[off.ravel()] = s.ravel()
    return torch.from_numpy(out)


def mxfp8_matmul_oracle(Aq, SA, Bq, SB) -> torch.Tensor:
    """FP32 matmul of the dequantised operands; Bq is [N, K] (quantised along K)."""
    return torch.matmul(mxfp8_dequantize(Aq, SA), mxfp8_dequantize(Bq, SB).t())


def cpu_threads() -> int:
    return torch.get_num_threads()
