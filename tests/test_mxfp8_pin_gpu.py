"""Independent pin of the MXFP8 path: the same packed e4m3 bytes and UE8M0 scale bytes fed to
torch._scaled_mm (cuBLASLt's block-scaled GEMM; a checker here, never on the product path) must
give the same bf16 output bit for bit.  The reference holds no MXFP8 vectors, so this comparison
and the CPU test of the quantiser against torch's float8 casts are what pins the recipe, the packed
scale layout and the GEMM to an implementation that is not this library."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _scaled_mm(Aq, Bq, out_dtype):
    a8 = Aq.data.view(torch.float8_e4m3fn)
    b8 = Bq.data.view(torch.float8_e4m3fn).t()                       # [K, N] column-major, as cuBLASLt wants
    sa = Aq.scales.view(torch.float8_e8m0fnu)
    sb = Bq.scales.view(torch.float8_e8m0fnu)
    return torch._scaled_mm(a8, b8, scale_a=sa, scale_b=sb, out_dtype=out_dtype)


def _operands(ops, M, K, N, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    A = (torch.randn(M, K, device="cuda", generator=g) * torch.exp(torch.randn(M, 1, device="cuda", generator=g))).bfloat16()
    B = torch.randn(K, N, device="cuda", generator=g).bfloat16()
    return ops.quantize_mxfp8(A), ops.quantize_mxfp8(B, transposed_in=True)


def _skip_if_unsupported(fn):
    try:
        return fn()
    except (RuntimeError, NotImplementedError) as e:                  # a torch build without block-scaled GEMM
        pytest.skip(f"torch._scaled_mm does not take MXFP8 operands here: {str(e)[:120]}")


@pytest.mark.parametrize("M,K,N", [(256, 512, 384), (512, 4096, 4096), (2048, 4096, 4096), (8192, 8192, 8192)])
def test_same_operands_same_result_as_scaled_mm(ops, M, K, N):
    """FP32 output: only the order of the FP32 additions may differ (<= 1e-5 relative).  bf16
    output: equal, or where the checker summed K in another order, different by one bf16 step in
    at most one element per thousand."""
    Aq, Bq = _operands(ops, M, K, N, seed=M + N)
    want32 = _skip_if_unsupported(lambda: _scaled_mm(Aq, Bq, torch.float32))
    got32 = ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.float32)
    ops.check_status()
    rel = float((got32.double() - want32.double()).norm() / want32.double().norm())
    assert rel <= 1e-5
    del want32
    want16 = _scaled_mm(Aq, Bq, torch.bfloat16)
    got16 = ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.bfloat16)
    ops.check_status()
    assert torch.equal(got16, got32.bfloat16())
    if not torch.equal(got16, want16):
        diff = got16 != want16
        assert float(diff.float().mean()) <= 1e-3
        a, b = got16[diff].float(), want16[diff].float()
        assert bool(((a - b).abs() <= 2.0 ** -7 * torch.maximum(a.abs(), b.abs()) + 1e-3).all())   # one bf16 step (absolute allowance near zero)


def test_ffn_shape_bit_equal_to_scaled_mm(ops):
    """The MXFP8 benchmark shape (16384 x 8192 x 28672): both implementations walk K in ascending
    128-element blocks into one FP32 accumulator, so the bf16 results agree bit for bit."""
    M, K, N = 16384, 8192, 28672
    Aq, Bq = _operands(ops, M, K, N, seed=0)
    want = _skip_if_unsupported(lambda: _scaled_mm(Aq, Bq, torch.bfloat16))
    got = ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.bfloat16)
    ops.check_status()
    assert torch.equal(got, want)


def test_skinny_decode_shape_against_scaled_mm(ops):
    # M = 16 runs the narrow-A single-CTA kernel; the checker sums K in another order there, so
    # the bar is the MXFP8 tolerance on FP32 output, not bit equality
    M, K, N = 16, 8192, 28672
    Aq, Bq = _operands(ops, M, K, N, seed=3)
    want = _skip_if_unsupported(lambda: _scaled_mm(Aq, Bq, torch.float32))
    got = ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.float32)
    ops.check_status()
    rel = float((got.double() - want.double()).norm() / want.double().norm())
    assert rel <= 1e-5
