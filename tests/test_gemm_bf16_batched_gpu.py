"""Strided-batched BF16 GEMM through the C-ABI (gemm_b200_gemm_bf16_batched).

The reference multiplies one pair of matrices per call (naive/naive.cpp:6-22); the batched entry
must equal that call made once per problem: checked bit-for-bit against the (unsplit) single-problem entry
point and, within the BF16 tolerance, against the FP32 oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL = ATOL = 2e-2


def _operands(batch, M, K, N, seed):
    g = torch.Generator().manual_seed(seed)
    A = torch.randn(batch, M, K, generator=g).bfloat16()
    B = torch.randn(batch, K, N, generator=g).bfloat16()
    return A, B


@pytest.mark.parametrize("batch,M,K,N", [(1, 256, 256, 256), (4, 300, 256, 264), (3, 128, 64, 8), (7, 16, 512, 1024),
                                         (2, 1024, 2048, 1536), (64, 64, 64, 64), (5, 257, 200, 520)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_batched_equals_one_call_per_problem(ops, oracle, batch, M, K, N, out_dtype):
    A, B = _operands(batch, M, K, N, seed=batch + M)
    Ad, Bd = A.cuda(), B.cuda()
    C = torch.full((batch, M, N), float("nan"), device="cuda", dtype=out_dtype)
    out = ops.gemm_bf16_batched(Ad, Bd, C, out_dtype=out_dtype)
    ops.check_status()
    assert out.data_ptr() == C.data_ptr()
    for i in range(batch):
        single = ops.gemm_bf16(Ad[i], Bd[i], out_dtype=out_dtype, k_splits=1)
        assert torch.equal(C[i], single), f"problem {i}"
        want = oracle.bf16_matmul_oracle(A[i], B[i])
        torch.testing.assert_close(C[i].float().cpu(), want, rtol=RTOL, atol=ATOL)


def test_shared_b_and_transposed_b(ops, oracle):
    batch, M, K, N = 6, 200, 320, 392
    A, B = _operands(batch, M, K, N, seed=3)
    Ad = A.cuda()
    # one weight matrix for every problem
    W = B[0].cuda()
    C = ops.gemm_bf16_batched(Ad, W, out_dtype=torch.float32)
    ops.check_status()
    for i in range(batch):
        assert torch.equal(C[i], ops.gemm_bf16(Ad[i], W, out_dtype=torch.float32, k_splits=1))
    # the same result as one tall GEMM over the stacked rows
    tall = ops.gemm_bf16(Ad.reshape(batch * M, K), W, out_dtype=torch.float32, k_splits=1)
    assert torch.equal(C.reshape(batch * M, N), tall)
    # B given per problem as its transpose [batch, N, K]
    Bt = B.transpose(1, 2).contiguous().cuda()
    C2 = ops.gemm_bf16_batched(Ad, Bt, b_is_nk=True, out_dtype=torch.float32)
    ops.check_status()
    for i in range(batch):
        want = oracle.bf16_matmul_oracle(A[i], B[i])
        assert oracle.rel_frobenius(C2[i].cpu(), want) < 1e-5


def test_strided_views(ops, oracle):
    batch, M, K, N = 3, 130, 96, 72
    g = torch.Generator().manual_seed(9)
    big_a = torch.randn(batch, M + 14, K + 40, generator=g).bfloat16().cuda()
    big_b = torch.randn(batch, K + 8, N + 24, generator=g).bfloat16().cuda()
    big_c = torch.full((batch, M + 6, N + 16), -7.0, device="cuda", dtype=torch.bfloat16)
    A, B, C = big_a[:, :M, :K], big_b[:, :K, :N], big_c[:, :M, :N]
    ops.gemm_bf16_batched(A, B, C)
    ops.check_status()
    for i in range(batch):
        want = oracle.bf16_matmul_oracle(A[i].cpu(), B[i].cpu())
        torch.testing.assert_close(C[i].float().cpu(), want, rtol=RTOL, atol=ATOL)
    # nothing outside the C views was written
    assert bool((big_c[:, M:, :] == -7.0).all()) and bool((big_c[:, :, N:] == -7.0).all())


def test_rejects_overlapping_or_misaligned_strides(ops):
    import gemm_b200._lib as L
    A = torch.zeros(4, 64, 64, device="cuda", dtype=torch.bfloat16)
    C = torch.zeros(4, 64, 64, device="cuda", dtype=torch.bfloat16)
    args = lambda sa, sb, sc: (A.data_ptr(), A.data_ptr(), C.data_ptr(), 4, 64, 64, 64, 64, 64, 64, sa, sb, sc,
                               L.B_ROW_MAJOR_KN, L.OUT_BF16, 0)
    assert L.lib.gemm_b200_gemm_bf16_batched(*args(4096, 4096, 100)) == L.ERR_INVALID_ARG     # C matrices overlap
    assert L.lib.gemm_b200_gemm_bf16_batched(*args(4100, 4096, 4096)) == L.ERR_ALIGNMENT      # stride_a % 8 != 0
    assert L.lib.gemm_b200_gemm_bf16_batched(*args(-8, 4096, 4096)) == L.ERR_INVALID_ARG
    assert L.lib.gemm_b200_gemm_bf16_batched(*args(4096, 0, 4096)) == L.OK                    # shared B is fine
    torch.cuda.synchronize()
