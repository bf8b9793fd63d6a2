"""Grouped (ragged) BF16 GEMM through the C-ABI (gemm_b200_gemm_bf16_grouped): groups of different
row counts that share N and K, their rows one after another in one A and one C.  Bar: bit-identical
to one single-problem call per group with the same kernel variant; that call is held to the oracle
elsewhere, and one case is checked against it here."""
import pytest
import torch

pytestmark = pytest.mark.gpu

VARIANT = "1cta_128x256x64_s4_direct"


def _case(ops, sizes, K, N, b_is_nk, out_dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    rows = sum(sizes)
    A = torch.randn(rows, K, device="cuda", generator=g).bfloat16()
    B = torch.randn(len(sizes), K, N, device="cuda", generator=g).bfloat16()
    Bd = B.transpose(1, 2).contiguous() if b_is_nk else B
    out = torch.full((rows + 3, N + 8), -5.0, device="cuda", dtype=out_dtype)      # canary rows / columns around C
    ops.gemm_bf16_grouped(A, Bd, sizes, out[1:rows + 1, :N], b_is_nk=b_is_nk, out_dtype=out_dtype)
    ops.check_status()
    cfg = ops.gemm_bf16_configs().index(VARIANT)
    r0 = 0
    for gi, m in enumerate(sizes):
        if m:
            want = ops.gemm_bf16(A[r0:r0 + m], Bd[gi], b_is_nk=b_is_nk, out_dtype=out_dtype, config=cfg)
            assert torch.equal(out[1 + r0:1 + r0 + m, :N], want), (gi, m)
        r0 += m
    assert bool((out[0] == -5.0).all()) and bool((out[rows + 1:] == -5.0).all()) and bool((out[:, N:] == -5.0).all())
    return A, B, out[1:rows + 1, :N]


@pytest.mark.parametrize("b_is_nk", [False, True])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_ragged_groups_match_one_call_per_group(ops, oracle, b_is_nk, out_dtype):
    sizes = [300, 0, 128, 1, 777, 64, 0, 129]
    A, B, C = _case(ops, sizes, 512, 520, b_is_nk, out_dtype, seed=3)
    # and against the oracle for one group
    r0 = sum(sizes[:4])
    want = oracle.bf16_matmul_oracle(A[r0:r0 + 777], B[4])
    torch.testing.assert_close(C[r0:r0 + 777].float().cpu(), want, rtol=2e-2, atol=2e-2)


def test_more_groups_than_one_launch_takes(ops):
    # 150 groups: three launches of at most 64 groups, rows and B matrices offset between them
    sizes = [(7 * i) % 50 for i in range(150)]
    _case(ops, sizes, 256, 264, False, torch.bfloat16, seed=5)


def test_mixture_of_experts_shape(ops):
    # 8 experts, 4096 tokens routed unevenly, hidden 2048 -> 4096
    sizes = [900, 310, 505, 12, 1024, 0, 777, 568]
    _case(ops, sizes, 2048, 4096, False, torch.bfloat16, seed=7)


def test_grouped_argument_errors(ops):
    import ctypes as C
    import gemm_b200._lib as L
    A = torch.zeros(256, 64, device="cuda", dtype=torch.bfloat16)
    B = torch.zeros(2, 64, 64, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(256, 64, device="cuda", dtype=torch.bfloat16)
    bad = (C.c_int64 * 2)(128, -1)
    rc = L.lib.gemm_b200_gemm_bf16_grouped(A.data_ptr(), B.data_ptr(), out.data_ptr(), 2, bad, 64, 64, 64, 64, 64 * 64, 64, 0, 0, None)
    assert rc == L.ERR_INVALID_ARG and "negative group size" in L.last_error()
    ok = (C.c_int64 * 2)(128, 128)
    rc = L.lib.gemm_b200_gemm_bf16_grouped(A.data_ptr(), B.data_ptr(), out.data_ptr(), 2, ok, 64, 64, 64, 64, 100, 64, 0, 0, None)
    assert rc == L.ERR_INVALID_ARG                                                   # stride_b smaller than a matrix
    assert L.lib.gemm_b200_gemm_bf16_grouped(None, None, None, 0, None, 64, 64, 64, 64, 0, 64, 0, 0, None) == L.OK
    with pytest.raises(ValueError):
        ops.gemm_bf16_grouped(A, B, [100, 100])                                       # row counts do not add up
