"""Operands whose element offsets exceed 2^31 (the reference indexes with 32-bit ints,
naive/naive_1.cu:5-13, and silently overflows there; this library addresses with 64 bits)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_gib():
    free, _ = torch.cuda.mem_get_info()
    return free / 2 ** 30


def test_fp32_rows_beyond_2_31_elements(ops, oracle):
    if _free_gib() < 14:
        pytest.skip("needs ~11 GiB of free device memory")
    M, K, N = 40000, 60000, 64                      # A has 2.4e9 elements: the last rows start past 2^31
    g = torch.Generator(device="cuda").manual_seed(0)
    A = torch.empty(M, K, device="cuda")
    for r0 in range(0, M, 8000):                     # fill in slabs to bound temporary memory
        A[r0:r0 + 8000] = torch.rand(min(8000, M - r0), K, device="cuda", generator=g) * 2 - 1
    B = torch.rand(K, N, device="cuda", generator=g) * 2 - 1
    C = ops.sgemm_f32(A, B)
    torch.cuda.synchronize()
    rows = torch.tensor([0, 1, 35791, 35792, 35800, M - 2, M - 1])    # 35792 * 60000 > 2^31
    want = oracle.sgemm_seq(A[rows].cpu(), B.cpu())
    assert torch.equal(C[rows].cpu(), want)
    del A, B, C
    torch.cuda.empty_cache()


def test_bf16_rows_beyond_2_32_bytes(ops, oracle):
    if _free_gib() < 12:
        pytest.skip("needs ~9 GiB of free device memory")
    M, K, N = 131072, 32768, 256                     # A: 4.3e9 elements, 8 GiB
    g = torch.Generator(device="cuda").manual_seed(1)
    A = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
    for r0 in range(0, M, 16384):
        A[r0:r0 + 16384] = torch.randn(16384, K, device="cuda", generator=g).bfloat16()
    B = torch.randn(K, N, device="cuda", generator=g).bfloat16()
    C = ops.gemm_bf16(A, B, out_dtype=torch.float32)
    ops.check_status()
    rows = torch.tensor([0, 65535, 65536, 65537, 100000, M - 1])       # 65536 * 32768 = 2^31 elements
    want = torch.matmul(A[rows].double().cpu(), B.double().cpu())
    # FP32 accumulation over K = 32768 products; a wrong row address would give an error near 1
    assert oracle.rel_frobenius(C[rows].double().cpu(), want) < 2e-4
    del A, B, C
    torch.cuda.empty_cache()


def test_mxfp8_rows_beyond_2_32_bytes(ops, oracle):
    if _free_gib() < 16:
        pytest.skip("needs ~13 GiB of free device memory")
    M, K, N = 139264, 32768, 256                     # Aq: 4.56e9 bytes; rows past 131072 start beyond 2^32
    g = torch.Generator(device="cuda").manual_seed(2)
    A = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
    for r0 in range(0, M, 8192):
        A[r0:r0 + 8192] = torch.randn(8192, K, device="cuda", generator=g).bfloat16()
    B = torch.randn(K, N, device="cuda", generator=g).bfloat16()
    Aq = ops.quantize_mxfp8(A)
    Bq = ops.quantize_mxfp8(B, transposed_in=True)
    C = ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.float32)
    ops.check_status()
    rows = torch.tensor([0, 65536, 131071, 131072, 131073, 135000, M - 1])
    # the quantiser wrote the selected rows (data and packed scales) where the oracle puts them
    qa, sa = oracle.mxfp8_quantize(A[rows].cpu())
    assert torch.equal(Aq.data[rows].cpu(), qa)
    kb = torch.arange(K // 32).view(1, -1)
    r = rows.view(-1, 1)
    off = ((r // 128) * (K // 128) + kb // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + (kb % 4)
    assert torch.equal(Aq.scales[off.cuda()].cpu(), sa)
    qb, sb = oracle.mxfp8_quantize(B.t().contiguous().cpu())
    want = oracle.mxfp8_matmul_oracle(qa, sa, qb, sb)
    assert oracle.rel_frobenius(C[rows].cpu(), want) <= 1e-3
    del A, B, C, Aq, Bq
    torch.cuda.empty_cache()
