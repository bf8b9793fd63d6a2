"""torch.library registration: the custom ops give the same result as the direct calls and can be
traced with fake tensors."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_custom_ops_match_direct_calls(ops, oracle):
    import gemm_b200.torch_ops  # noqa: F401
    A, B = oracle.gen_uniform_f32(200, 96, 136, seed=1)
    got = torch.ops.gemm_b200.sgemm_f32(A.cuda(), B.cuda())
    assert torch.equal(got.cpu(), oracle.sgemm_seq(A, B))
    Ab, Bb = oracle.gen_randn_bf16(256, 128, 264, seed=2)
    c1 = torch.ops.gemm_b200.gemm_bf16(Ab.cuda(), Bb.cuda())
    assert torch.equal(c1, ops.gemm_bf16(Ab.cuda(), Bb.cuda()))
    c2 = torch.ops.gemm_b200.gemm_bf16(Ab.cuda(), Bb.t().contiguous().cuda(), True, True)
    torch.testing.assert_close(c2.cpu(), oracle.bf16_matmul_oracle(Ab, Bb), rtol=2e-2, atol=2e-2)
    A3 = torch.stack([Ab, Ab * 0.5, -Ab]).cuda()
    c3 = torch.ops.gemm_b200.gemm_bf16_batched(A3, Bb.cuda())
    assert torch.equal(c3, ops.gemm_bf16_batched(A3, Bb.cuda())) and c3.shape == (3, 256, 264)
    At = Ab.t().contiguous().cuda()
    c4 = torch.ops.gemm_b200.gemm_bf16_at(At, Bb.cuda())
    assert torch.equal(c4, ops.gemm_bf16_at(At, Bb.cuda())) and c4.shape == (256, 264)
    torch.testing.assert_close(c4.float().cpu(), oracle.bf16_matmul_oracle(Ab, Bb), rtol=2e-2, atol=2e-2)
    B3 = torch.stack([Bb, -Bb]).cuda()
    c5 = torch.ops.gemm_b200.gemm_bf16_grouped(Ab.cuda(), B3, [100, 156])
    assert torch.equal(c5, ops.gemm_bf16_grouped(Ab.cuda(), B3, [100, 156])) and c5.shape == (256, 264)


def test_mxfp8_custom_ops_match_direct_calls(ops, oracle):
    import gemm_b200.torch_ops  # noqa: F401
    Ab, Bb = oracle.gen_randn_bf16(256, 512, 384, seed=3)
    aq, asf = torch.ops.gemm_b200.quantize_mxfp8(Ab.cuda())
    bq, bsf = torch.ops.gemm_b200.quantize_mxfp8(Bb.cuda(), True)
    A = ops.quantize_mxfp8(Ab.cuda()); B = ops.quantize_mxfp8(Bb.cuda(), transposed_in=True)
    assert torch.equal(aq, A.data) and torch.equal(asf, A.scales) and torch.equal(bq, B.data) and torch.equal(bsf, B.scales)
    got = torch.ops.gemm_b200.gemm_mxfp8(aq, asf, bq, bsf, True)
    ops.check_status()
    assert torch.equal(got, ops.gemm_mxfp8(A, B, out_dtype=torch.float32))
    qa, sa = oracle.mxfp8_quantize(Ab); qb, sb = oracle.mxfp8_quantize(Bb.t().contiguous())
    assert oracle.rel_frobenius(got.cpu(), oracle.mxfp8_matmul_oracle(qa, sa, qb, sb)) <= 1e-3


def test_fake_tensor_shapes():
    import gemm_b200.torch_ops  # noqa: F401
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        A = torch.empty(64, 32, device="cuda"); B = torch.empty(32, 48, device="cuda")
        assert torch.ops.gemm_b200.sgemm_f32(A, B).shape == (64, 48)
        Ab = torch.empty(64, 32, device="cuda", dtype=torch.bfloat16); Bt = torch.empty(48, 32, device="cuda", dtype=torch.bfloat16)
        out = torch.ops.gemm_b200.gemm_bf16(Ab, Bt, True, True)
        assert out.shape == (64, 48) and out.dtype == torch.float32
        A3 = torch.empty(5, 64, 32, device="cuda", dtype=torch.bfloat16)
        assert torch.ops.gemm_b200.gemm_bf16_batched(A3, Bt, True, False).shape == (5, 64, 48)
        At = torch.empty(32, 64, device="cuda", dtype=torch.bfloat16)
        assert torch.ops.gemm_b200.gemm_bf16_at(At, Bt, True, False).shape == (64, 48)
        B3 = torch.empty(2, 32, 48, device="cuda", dtype=torch.bfloat16)
        assert torch.ops.gemm_b200.gemm_bf16_grouped(Ab, B3, [24, 40]).shape == (64, 48)
        aq, asf = torch.ops.gemm_b200.quantize_mxfp8(Ab)
        bq, bsf = torch.ops.gemm_b200.quantize_mxfp8(Bt)
        assert aq.shape == (64, 32) and asf.shape == (512,) and bq.shape == (48, 32)
        assert torch.ops.gemm_b200.gemm_mxfp8(aq, asf, bq, bsf).shape == (64, 48)
