"""The row-sharded benchmark problem at its full size on one GPU: M = 131072, K = N = 8192, BF16 and
MXFP8 operands (A made of eight fixed 16384-row blocks, block b seeded 1000 + b; B seeded 0).

The oracle is run on sampled rows of every one of the eight row blocks (first and last row of the
block, both sides of a 128-row tile boundary, two random rows).  Size-independent property checked
over the whole result: the rows of a block computed inside the full problem equal, bit for bit,
the same block multiplied on its own — which is also what makes the multi-GPU shards equal to the
single-GPU result."""
import pytest
import torch

pytestmark = pytest.mark.gpu

M, K, N = 131072, 8192, 8192
BLOCKS = 8


def _free_gib():
    free, _ = torch.cuda.mem_get_info()
    return free / 2 ** 30


def _operands():
    from gemm_b200 import sharded
    dev = torch.device("cuda", torch.cuda.current_device())
    rows = M // BLOCKS
    A = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
    for b in range(BLOCKS):
        A[b * rows:(b + 1) * rows] = sharded.gen_a_block_cuda(b, rows, K, dev)
    return A, sharded.gen_b_cuda(K, N, dev)


def _sample_rows():
    rows = M // BLOCKS
    g = torch.Generator().manual_seed(5)
    out = []
    for b in range(BLOCKS):
        r0 = b * rows
        rnd = torch.randint(0, rows, (2,), generator=g).tolist()
        out += [r0, r0 + 127, r0 + 128, r0 + rows - 1] + [r0 + r for r in rnd]
    return torch.tensor(sorted(set(out)))


def test_bf16_full_size_sampled_rows_and_block_invariance(ops, oracle):
    if _free_gib() < 12:
        pytest.skip("needs ~8 GiB of free device memory")
    A, B = _operands()
    C = ops.gemm_bf16(A, B)
    ops.check_status()
    rows = _sample_rows()
    want = oracle.bf16_matmul_oracle(A[rows], B)
    torch.testing.assert_close(C[rows].float().cpu(), want, rtol=2e-2, atol=2e-2)          # the stated BF16 tolerance
    # tighter, on FP32 output of the same rows' blocks: only FP32 summation order separates the two
    blk = M // BLOCKS
    for b in (0, 3, 7):
        part = ops.gemm_bf16(A[b * blk:(b + 1) * blk], B)
        ops.check_status()
        assert torch.equal(part, C[b * blk:(b + 1) * blk])
    part32 = ops.gemm_bf16(A[7 * blk:], B, out_dtype=torch.float32)
    ops.check_status()
    sel = rows[rows >= 7 * blk] - 7 * blk
    want64 = torch.matmul(A[7 * blk:][sel].double().cpu(), B.double().cpu())
    assert oracle.rel_frobenius(part32[sel].double().cpu(), want64) <= 1e-5
    assert torch.equal(part32.bfloat16(), C[7 * blk:])


def test_mxfp8_full_size_sampled_rows_and_block_invariance(ops, oracle):
    if _free_gib() < 16:
        pytest.skip("needs ~12 GiB of free device memory")
    A, B = _operands()
    Aq = ops.quantize_mxfp8(A)
    Bq = ops.quantize_mxfp8(B, transposed_in=True)
    C32 = ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.float32)
    ops.check_status()
    rows = _sample_rows()
    qa, sa = oracle.mxfp8_quantize(A[rows].cpu())
    qb, sb = oracle.mxfp8_quantize(B.t().contiguous().cpu())
    assert torch.equal(Aq.data[rows].cpu(), qa)                                            # quantiser, full-size offsets
    assert torch.equal(Bq.data.cpu(), qb) and torch.equal(Bq.scale_matrix(), sb)
    want = oracle.mxfp8_matmul_oracle(qa, sa, qb, sb)
    assert oracle.rel_frobenius(C32[rows].cpu(), want) <= 1e-3                              # the stated MXFP8 tolerance
    C16 = ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.bfloat16)
    ops.check_status()
    assert torch.equal(C16[rows], C32[rows].bfloat16())
    del C32
    blk = M // BLOCKS
    for b in (0, 4, 7):
        Ab = ops.quantize_mxfp8(A[b * blk:(b + 1) * blk])
        assert torch.equal(Ab.data, Aq.data[b * blk:(b + 1) * blk])
        part = ops.gemm_mxfp8(Ab, Bq, out_dtype=torch.bfloat16)
        ops.check_status()
        assert torch.equal(part, C16[b * blk:(b + 1) * blk])
