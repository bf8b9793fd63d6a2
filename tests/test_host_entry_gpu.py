"""Host-buffer entry points (gemm_b200_sgemm_f32_host / gemm_b200_gemm_bf16_host): operands start
and end in host memory; large problems are cut into row slabs whose copies and GEMMs overlap."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,K,N", [(1, 1, 1), (200, 77, 130), (1024, 512, 768)])
def test_f32_host_bit_exact(ops, oracle, M, K, N):
    A, B = oracle.gen_uniform_f32(M, K, N, seed=M)
    C = ops.sgemm_f32_host(A, B)
    assert torch.equal(C, oracle.sgemm_seq(A, B))


def test_f32_host_pinned_and_slabbed(ops, oracle):
    # 20480 x 512 x 512: A + C = 80 MB -> several row slabs through the three-stream pipeline
    M, K, N = 20480, 512, 512
    A, B = oracle.gen_uniform_f32(M, K, N, seed=3)
    Ap, Bp = A.pin_memory(), B.pin_memory()
    Cp = torch.empty(M, N).pin_memory()
    out = ops.sgemm_f32_host(Ap, Bp, Cp)
    assert out.data_ptr() == Cp.data_ptr()
    rows = torch.tensor([0, 1, 255, 256, 4095, 4096, 10000, M - 1])
    assert torch.equal(Cp[rows], oracle.sgemm_seq(A[rows], B))
    # every slab was written: compare whole-matrix checksums against the device path
    dev = ops.sgemm_f32(A.cuda(), B.cuda()).cpu()
    assert torch.equal(Cp, dev)


@pytest.mark.parametrize("b_is_nk", [False, True])
def test_bf16_host(ops, oracle, b_is_nk):
    M, K, N = 24576, 1024, 1024      # A + C = 96 MB -> slabs
    A, B = oracle.gen_randn_bf16(M, K, N, seed=5)
    Bh = B.t().contiguous() if b_is_nk else B
    C = ops.gemm_bf16_host(A.pin_memory(), Bh.pin_memory(), b_is_nk=b_is_nk)
    rows = torch.tensor([0, 127, 128, 5000, 12287, 12288, M - 1])
    torch.testing.assert_close(C[rows].float(), oracle.bf16_matmul_oracle(A[rows], B), rtol=2e-2, atol=2e-2)
    dev = ops.gemm_bf16(A.cuda(), Bh.cuda(), b_is_nk=b_is_nk).cpu()
    assert torch.equal(C, dev)


def test_host_entry_argument_errors(ops):
    import gemm_b200._lib as L
    assert L.lib.gemm_b200_sgemm_f32_host(None, None, None, 4, 4, 4) == L.ERR_INVALID_ARG
    assert L.lib.gemm_b200_sgemm_f32_host(None, None, None, 0, 4, 4) == L.OK
    with pytest.raises(ValueError):
        ops.sgemm_f32_host(torch.zeros(4, 4, device="cuda"), torch.zeros(4, 4, device="cuda"))
    assert L.lib.gemm_b200_release_workspace() == L.OK


def test_host_entry_error_leaves_nothing_in_flight(ops, oracle):
    """A launch the device entry point refuses (K not a multiple of 8 for BF16) comes back as that
    error with every queued copy finished: the caller may overwrite or free its buffers at once,
    and the next call works on the same workspace."""
    import gemm_b200._lib as L
    M, K, N = 24576, 1028, 1024                      # several slabs; K % 8 != 0 -> GEMM_B200_ERR_ALIGNMENT
    A = torch.ones(M, K, dtype=torch.bfloat16).pin_memory()
    B = torch.ones(K, N, dtype=torch.bfloat16).pin_memory()
    C = torch.full((M, N), 7.0, dtype=torch.bfloat16).pin_memory()
    rc = L.lib.gemm_b200_gemm_bf16_host(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, L.B_ROW_MAJOR_KN, L.OUT_BF16)
    assert rc == L.ERR_ALIGNMENT
    A.fill_(3.0); B.fill_(3.0)                        # nothing reads them any more
    assert bool((C == 7.0).all())                     # and nothing was written
    M, K, N = 4096, 1024, 512
    A2, B2 = oracle.gen_randn_bf16(M, K, N, seed=8)
    got = ops.gemm_bf16_host(A2.pin_memory(), B2.pin_memory())
    assert torch.equal(got, ops.gemm_bf16(A2.cuda(), B2.cuda()).cpu())
