"""BF16 GEMM with A stored transposed ([K, M] row-major): equal, bit for bit, to the plain entry
on a transposed copy when both take the same tile shape, and within BF16 tolerance of the FP32
product of the same operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _operands(M, K, N, seed=0, lda_pad=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    At = torch.randn(K, M + lda_pad, device="cuda", generator=g).bfloat16()[:, :M]
    B = torch.randn(K, N, device="cuda", generator=g).bfloat16()
    return At, B


@pytest.mark.parametrize("M,K,N", [(128, 256, 256), (104, 192, 136), (256, 512, 512), (520, 1000 // 8 * 8, 776),
                                   (2048, 1024, 2048), (4096, 4096, 4096), (8192, 2048, 4096)])
@pytest.mark.parametrize("b_is_nk", [False, True])
def test_matches_plain_entry_on_a_transposed_copy(M, K, N, b_is_nk):
    import gemm_b200.ops as ops
    At, B = _operands(M, K, N)
    Bx = B.t().contiguous() if b_is_nk else B
    A = At.t().contiguous()
    got = ops.gemm_bf16_at(At, Bx, b_is_nk=b_is_nk, out_dtype=torch.float32)
    # the plain entry may split K or take 128-column tiles for few-tile problems: pin it to one launch
    want = ops.gemm_bf16(A, Bx, b_is_nk=b_is_nk, out_dtype=torch.float32, k_splits=1)
    ref = A.float() @ B.float()
    ops.check_status()
    torch.testing.assert_close(got, ref, rtol=2e-2, atol=2e-2)
    rel = (got - want).norm() / want.norm()
    assert rel <= 1e-6, rel          # same products, FP32 accumulation; tile shapes may differ


def test_bit_identical_when_the_tile_shape_is_the_same():
    import gemm_b200.ops as ops
    At, B = _operands(4096, 4096, 4096, seed=3)
    A = At.t().contiguous()
    got = ops.gemm_bf16_at(At, B)
    want = ops.gemm_bf16(A, B)
    ops.check_status()
    assert torch.equal(got, want)


def test_long_k_few_tiles_takes_the_split_path():
    import gemm_b200.ops as ops
    At, B = _operands(1024, 8192, 1024, seed=7)
    got = ops.gemm_bf16_at(At, B, out_dtype=torch.float32)
    ref = At.t().float() @ B.float()
    ops.check_status()
    rel = (got - ref).norm() / ref.norm()
    assert rel <= 1e-5, rel


def test_padded_leading_dimension_and_bf16_output():
    import gemm_b200.ops as ops
    At, B = _operands(1000, 640, 520, seed=5, lda_pad=24)
    assert At.stride(0) == 1024
    got = ops.gemm_bf16_at(At, B)
    ref = (At.t().float() @ B.float())
    ops.check_status()
    torch.testing.assert_close(got.float(), ref, rtol=2e-2, atol=2e-2)


def test_argument_errors():
    import gemm_b200.ops as ops
    from gemm_b200 import _lib
    At, B = _operands(256, 256, 256, lda_pad=4)       # row pitch 260 elements: not a multiple of 8
    with pytest.raises(_lib.GemmB200Error) as e:
        ops.gemm_bf16_at(At, B)
    assert e.value.code == _lib.ERR_ALIGNMENT
