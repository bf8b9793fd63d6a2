"""Grouped MXFP8 GEMM: groups of (256-row padded) tokens, one quantised B per group, one launch.
Every group's rows must equal, bit for bit, the plain entry on that group alone with the same
kernel variant, and meet the MXFP8 tolerance against the FP32 product of the dequantised operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _group_view(ops, A, r0, r1):
    """Rows [r0, r1) (multiples of 128) of a quantised tall matrix as an operand of their own: the
    packed scales are ordered [row block][K chunk], so a run of row blocks is a contiguous slice."""
    kchunks = -(-(A.K // 32) // 4)
    return ops.MxFp8Tensor(A.data[r0:r1], A.scales[(r0 // 128) * kchunks * 512:(r1 // 128) * kchunks * 512], r1 - r0, A.K)


@pytest.mark.parametrize("sizes,K,N", [([256, 512, 0, 768], 1024, 512), ([512, 256], 2048, 264), ([256] * 5, 512, 1000 // 8 * 8),
                                       ([1024, 0, 0, 256, 2048], 4096, 1536), ([0, 0], 256, 256), ([256], 32, 8)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_matches_one_call_per_group(ops, oracle, sizes, K, N, out_dtype):
    G, M = len(sizes), sum(sizes)
    g = torch.Generator(device="cuda").manual_seed(K + N)
    A = torch.randn(max(M, 1), K, device="cuda", generator=g).bfloat16()[:M]
    B3 = torch.randn(G, K, N, device="cuda", generator=g).bfloat16()
    bq, bs = ops.quantize_mxfp8_stack(B3)
    names = ops.gemm_mxfp8_configs()
    cfg = names.index("2cta_256x256x128_s5_maskcommit_tmastore")
    if M == 0:
        out = ops.gemm_mxfp8_grouped(ops.MxFp8Tensor(torch.empty(0, K, device="cuda", dtype=torch.uint8),
                                                     torch.empty(1, device="cuda", dtype=torch.uint8), 0, K), bq, bs, sizes, out_dtype=out_dtype)
        assert out.shape == (0, N)
        return
    Aq = ops.quantize_mxfp8(A)
    canary = torch.full((M + 2, N + 16), -3.0, device="cuda", dtype=out_dtype)
    C = canary[1:M + 1, 8:N + 8]
    ops.gemm_mxfp8_grouped(Aq, bq, bs, sizes, C, out_dtype=out_dtype)
    ops.check_status()
    mask = torch.ones_like(canary, dtype=torch.bool); mask[1:M + 1, 8:N + 8] = False
    assert bool((canary[mask] == -3.0).all())
    r0 = 0
    for gi, m in enumerate(sizes):
        if m == 0:
            continue
        Bg = ops.MxFp8Tensor(bq[gi], bs[gi], N, K)
        want = ops.gemm_mxfp8(_group_view(ops, Aq, r0, r0 + m), Bg, out_dtype=out_dtype, config=cfg)
        assert torch.equal(C[r0:r0 + m], want), f"group {gi}"
        if out_dtype == torch.float32:
            qa, sa = oracle.mxfp8_quantize(A[r0:r0 + m].cpu())
            qb, sb = oracle.mxfp8_quantize(B3[gi].t().contiguous().cpu())
            assert oracle.rel_frobenius(want.cpu(), oracle.mxfp8_matmul_oracle(qa, sa, qb, sb)) <= 1e-3
        r0 += m
    ops.check_status()


def test_more_groups_than_one_launch_takes(ops):
    G, K, N = 70, 256, 256
    sizes = [256 if i % 3 else 0 for i in range(G)]
    M = sum(sizes)
    g = torch.Generator(device="cuda").manual_seed(1)
    A = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    B3 = torch.randn(G, K, N, device="cuda", generator=g).bfloat16()
    bq, bs = ops.quantize_mxfp8_stack(B3)
    Aq = ops.quantize_mxfp8(A)
    C = ops.gemm_mxfp8_grouped(Aq, bq, bs, sizes, out_dtype=torch.float32)
    ops.check_status()
    r0 = 0
    for gi, m in enumerate(sizes):
        if m:
            ref = A[r0:r0 + m].float() @ B3[gi].float()
            rel = (C[r0:r0 + m] - ref).norm() / ref.norm()
            assert rel < 0.06, (gi, float(rel))          # MXFP8 keeps ~3 significant bits per element
            r0 += m


def test_long_k_takes_the_run_time_schedule_and_still_matches(ops):
    sizes, K, N = [2048, 1024, 4096, 1024], 8192, 2048
    M = sum(sizes)
    g = torch.Generator(device="cuda").manual_seed(2)
    A = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    B3 = torch.randn(len(sizes), K, N, device="cuda", generator=g).bfloat16()
    bq, bs = ops.quantize_mxfp8_stack(B3)
    Aq = ops.quantize_mxfp8(A)
    C = ops.gemm_mxfp8_grouped(Aq, bq, bs, sizes)
    ops.check_status()
    cfg = ops.gemm_mxfp8_configs().index("2cta_256x256x128_s5_maskcommit_tmastore")
    r0 = 0
    for gi, m in enumerate(sizes):
        want = ops.gemm_mxfp8(_group_view(ops, Aq, r0, r0 + m), ops.MxFp8Tensor(bq[gi], bs[gi], N, K), config=cfg)
        assert torch.equal(C[r0:r0 + m], want), f"group {gi}"
        r0 += m


def test_argument_errors(ops):
    from gemm_b200 import _lib
    g = torch.Generator(device="cuda").manual_seed(3)
    A = ops.quantize_mxfp8(torch.randn(384, 256, device="cuda", generator=g).bfloat16())
    bq, bs = ops.quantize_mxfp8_stack(torch.randn(2, 256, 256, device="cuda", generator=g).bfloat16())
    with pytest.raises(_lib.GemmB200Error) as e:
        ops.gemm_mxfp8_grouped(A, bq, bs, [256, 128])
    assert e.value.code == _lib.ERR_INVALID_ARG and "multiple of 256" in str(e.value)
