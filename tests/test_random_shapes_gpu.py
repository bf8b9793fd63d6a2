"""Seeded random shapes (ragged in every dimension) for the three operators, against the oracle."""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu


def _shapes(seed, count, mmax, kmax, nmax, kmul=1, nmul=1):
    rng = random.Random(seed)
    out = []
    for _ in range(count):
        M = rng.randint(1, mmax)
        K = max(kmul, rng.randint(1, kmax) // kmul * kmul)
        N = max(nmul, rng.randint(1, nmax) // nmul * nmul)
        out.append((M, K, N))
    return out


def test_fp32_random_shapes_bit_exact(ops, oracle):
    for (M, K, N) in _shapes(1, 40, 700, 900, 700):
        A, B = oracle.gen_uniform_f32(M, K, N, seed=M + K + N)
        got = ops.sgemm_f32(A.cuda(), B.cuda()).cpu()
        assert torch.equal(got, oracle.sgemm_seq(A, B)), (M, K, N)


def test_bf16_random_shapes(ops, oracle):
    for i, (M, K, N) in enumerate(_shapes(2, 30, 900, 1500, 1400, kmul=8, nmul=8)):
        A, B = oracle.gen_randn_bf16(M, K, N, seed=i)
        want = oracle.bf16_matmul_oracle(A, B)
        nk = bool(i & 1)
        Bd = B.t().contiguous().cuda() if nk else B.cuda()
        got = ops.gemm_bf16(A.cuda(), Bd, b_is_nk=nk, out_dtype=torch.float32)
        ops.check_status()
        assert oracle.rel_frobenius(got.cpu(), want) < 1e-5, (M, K, N, nk)
        got16 = ops.gemm_bf16(A.cuda(), Bd, b_is_nk=nk)
        torch.testing.assert_close(got16.float().cpu(), want, rtol=2e-2, atol=2e-2)


def test_mxfp8_random_shapes(ops, oracle):
    for i, (M, K, N) in enumerate(_shapes(3, 24, 600, 1600, 1200, kmul=32, nmul=8)):
        A, B = oracle.gen_randn_bf16(M, K, N, seed=100 + i)
        Aq = ops.quantize_mxfp8(A.cuda()); Bq = ops.quantize_mxfp8(B.cuda(), transposed_in=True)
        qa, sa = oracle.mxfp8_quantize(A); qb, sb = oracle.mxfp8_quantize(B.t().contiguous())
        assert torch.equal(Aq.data.cpu(), qa) and torch.equal(Bq.data.cpu(), qb), (M, K, N)
        assert torch.equal(Aq.scale_matrix(), sa) and torch.equal(Bq.scale_matrix(), sb), (M, K, N)
        want = oracle.mxfp8_matmul_oracle(qa, sa, qb, sb)
        got = ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.float32)
        ops.check_status()
        assert oracle.rel_frobenius(got.cpu(), want) <= 1e-3, (M, K, N)
