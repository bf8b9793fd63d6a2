"""The allocation-free split-K entry point (gemm_b200_gemm_mxfp8_splitk_static), called through
the C-ABI.

Some callers cannot allocate device memory at the point where they call the GEMM: a serving loop
whose memory pool already owns all of HBM, or a plugin host that forbids allocation inside its
execute callback.  For them the library carries a fixed 16 MiB scratch array in its device image.
This test checks that the entry point gives the same bits as the caller-scratch entry point it is a
variant of, on two calls in a row (the second call sees the first call's leftovers in the shared
array), that it allocates nothing, and that it refuses problems larger than the array.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_BYTES = 16 << 20


def _operands(ops, M, K, N, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    A = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    B = torch.randn(K, N, device="cuda", generator=g).bfloat16()
    return ops.quantize_mxfp8(A), ops.quantize_mxfp8(B, transposed_in=True)


def _call_static(L, Aq, Bq, out, splits):
    M, N, K = Aq.rows, Bq.rows, Aq.K
    od = L.OUT_F32 if out.dtype == torch.float32 else L.OUT_BF16
    return L.lib.gemm_b200_gemm_mxfp8_splitk_static(
        Aq.data.data_ptr(), Aq.scales.data_ptr(), Bq.data.data_ptr(), Bq.scales.data_ptr(), out.data_ptr(),
        M, N, K, N, od, splits, torch.cuda.current_stream().cuda_stream)


def test_static_scratch_matches_caller_scratch_twice_in_a_row(ops, oracle):
    import gemm_b200._lib as L
    cases = [(16, 8192, 28672, 5, torch.bfloat16), (48, 2048, 1000, 4, torch.float32)]
    for (M, K, N, splits, dt) in cases:
        Aq, Bq = _operands(ops, M, K, N, seed=M)
        want = ops.gemm_mxfp8_splitk(Aq, Bq, splits, out_dtype=dt)          # the existing entry point
        ops.check_status()
        # warm the path once so that lazy one-time set-up is not counted as an allocation below
        first = torch.full((M, N), float("nan"), device="cuda", dtype=dt)
        assert _call_static(L, Aq, Bq, first, splits) == 0, L.last_error()
        torch.cuda.synchronize()
        second = torch.full((M, N), float("nan"), device="cuda", dtype=dt)   # torch's own allocation, before the call
        free_mid, _ = torch.cuda.mem_get_info()
        assert _call_static(L, Aq, Bq, second, splits) == 0, L.last_error()
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_mid                                         # the call itself took no device memory
        ops.check_status()
        assert torch.equal(first, want) and torch.equal(second, want)        # same kernels, same order: same bits


def test_static_scratch_against_the_oracle(ops, oracle):
    import gemm_b200._lib as L
    M, K, N = 16, 4096, 2048                                                  # 8 tiles: the library picks > 1 split
    A, B = oracle.gen_randn_bf16(M, K, N, seed=77)
    Aq = ops.quantize_mxfp8(A.cuda()); Bq = ops.quantize_mxfp8(B.cuda(), transposed_in=True)
    qa, sa = oracle.mxfp8_quantize(A); qb, sb = oracle.mxfp8_quantize(B.t().contiguous())
    want = oracle.mxfp8_matmul_oracle(qa, sa, qb, sb)
    for _ in range(2):
        out = torch.full((M, N), float("nan"), device="cuda")
        assert _call_static(L, Aq, Bq, out, 0) == 0, L.last_error()           # 0 = the library picks the split count
        ops.check_status()
        assert oracle.rel_frobenius(out.cpu(), want) <= 1e-3                  # the MXFP8 tolerance of the other tests


def test_static_scratch_rejects_what_does_not_fit(ops):
    import gemm_b200._lib as L
    M, K, N = 128, 1024, 16384                                               # 8 x 128 x 16384 x 4 B = 64 MiB > 16 MiB
    Aq, Bq = _operands(ops, M, K, N, seed=1)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    rc = _call_static(L, Aq, Bq, out, 8)
    assert rc == L.ERR_TOO_LARGE
    assert "scratch" in L.last_error() and str(STATIC_BYTES) in L.last_error()
    assert L.lib.gemm_b200_gemm_mxfp8_splitk_scratch_bytes(M, N, 8) > STATIC_BYTES


def test_static_scratch_second_output_type_loads_nothing(ops):
    """The first call on a device sets up both output types: after a bf16 call, an f32 call (and an
    unsplit one) must not take device memory either."""
    import gemm_b200._lib as L
    M, K, N = 32, 2048, 512
    Aq, Bq = _operands(ops, M, K, N, seed=9)
    out16 = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    out32 = torch.empty(M, N, device="cuda", dtype=torch.float32)
    assert _call_static(L, Aq, Bq, out16, 4) == 0, L.last_error()
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    assert _call_static(L, Aq, Bq, out32, 4) == 0, L.last_error()
    assert _call_static(L, Aq, Bq, out32, 1) == 0, L.last_error()
    assert _call_static(L, Aq, Bq, out16, 1) == 0, L.last_error()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0
    ops.check_status()
    assert torch.equal(out32, ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.float32, config=0))


def test_static_scratch_auto_splits_edge_cases(ops):
    import gemm_b200._lib as L
    # N % 8 != 0 with f32 output: the library's own choice falls back to the unsplit kernel
    M, K, N = 16, 4096, 2052
    Aq, Bq = _operands(ops, M, K, N, seed=4)
    out = torch.empty(M, N, device="cuda", dtype=torch.float32)
    assert _call_static(L, Aq, Bq, out, 0) == 0, L.last_error()
    ops.check_status()
    assert torch.equal(out, ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.float32, config=0))
    # dimensions beyond 2^31 - 1 are refused before any size arithmetic
    rc = L.lib.gemm_b200_gemm_mxfp8_splitk_static(None, None, None, None, None, 1 << 40, 1 << 40, 32, 1 << 40, 0, 2, None)
    assert rc == L.ERR_TOO_LARGE


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_static_scratch_on_a_second_device(ops):
    """Every device has its own copy of the array; its address is looked up with that device current."""
    import gemm_b200._lib as L
    with torch.cuda.device(1):
        M, K, N = 16, 4096, 1024
        Aq, Bq = _operands(ops, M, K, N, seed=2)
        want = ops.gemm_mxfp8_splitk(Aq, Bq, 4, out_dtype=torch.float32)
        for _ in range(2):
            out = torch.full((M, N), float("nan"), device="cuda", dtype=torch.float32)
            assert _call_static(L, Aq, Bq, out, 4) == 0, L.last_error()
            ops.check_status()
            assert torch.equal(out, want)
