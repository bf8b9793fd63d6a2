"""BF16 tensor-core parity on the GPU through the C-ABI (gemm_b200_gemm_bf16).

Bar (stated BF16 tolerance): rtol = atol = 2e-2 against an FP32 matmul of the same BF16
operands.  With FP32 output the kernel is also held to a much tighter bound, because only the
summation order differs from the oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL = ATOL = 2e-2


def _check(ops, oracle, M, K, N, *, b_is_nk=False, out_dtype=torch.bfloat16, config=-1, seed=0):
    A, B = oracle.gen_randn_bf16(M, K, N, seed=seed)
    want = oracle.bf16_matmul_oracle(A, B)
    Bdev = B.t().contiguous().cuda() if b_is_nk else B.cuda()
    C = torch.full((M, N), float("nan"), device="cuda", dtype=out_dtype)
    out = ops.gemm_bf16(A.cuda(), Bdev, C, b_is_nk=b_is_nk, out_dtype=out_dtype, config=config)
    ops.check_status()
    assert out.data_ptr() == C.data_ptr()
    got = C.float().cpu()
    torch.testing.assert_close(got, want, rtol=RTOL, atol=ATOL)
    if out_dtype == torch.float32:
        assert oracle.rel_frobenius(got, want) < 1e-5
    else:
        # within one BF16 rounding of the FP32 result
        assert oracle.rel_frobenius(got, want) < 3e-3


@pytest.mark.parametrize("shape", [(256, 256, 256), (512, 1024, 768), (1024, 4096, 1024)])
@pytest.mark.parametrize("b_is_nk", [False, True])
def test_square_and_rect(ops, oracle, shape, b_is_nk):
    M, K, N = shape
    _check(ops, oracle, M, K, N, b_is_nk=b_is_nk)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_every_config_both_layouts(ops, oracle, out_dtype):
    for cfg, name in enumerate(ops.gemm_bf16_configs()):
        for b_is_nk in (False, True):
            _check(ops, oracle, 768, 640, 1280, b_is_nk=b_is_nk, out_dtype=out_dtype, config=cfg, seed=cfg)


# ragged: M, N not multiples of the tile, K not a multiple of 64, single row, skinny
EDGE = [(1, 64, 8), (16, 8192, 256), (100, 72, 40), (129, 136, 264), (255, 8, 520), (300, 200, 1000), (2000, 1000, 24)]


@pytest.mark.parametrize("M,K,N", EDGE)
@pytest.mark.parametrize("b_is_nk", [False, True])
def test_edge_shapes(ops, oracle, M, K, N, b_is_nk):
    for cfg in range(len(ops.gemm_bf16_configs())):
        _check(ops, oracle, M, K, N, b_is_nk=b_is_nk, out_dtype=torch.float32, config=cfg, seed=M + N)


def test_k_zero_and_empty(ops):
    C = torch.full((8, 16), 3.0, device="cuda", dtype=torch.bfloat16)
    ops.gemm_bf16(torch.empty(8, 0, device="cuda", dtype=torch.bfloat16),
                  torch.empty(0, 16, device="cuda", dtype=torch.bfloat16), C)
    assert torch.count_nonzero(C) == 0
    ops.gemm_bf16(torch.empty(0, 8, device="cuda", dtype=torch.bfloat16),
                  torch.empty(8, 16, device="cuda", dtype=torch.bfloat16))


def test_canaries_around_c(ops, oracle):
    M, K, N = 200, 128, 264
    A, B = oracle.gen_randn_bf16(M, K, N, seed=5)
    for cfg in range(len(ops.gemm_bf16_configs())):
        Cbig = torch.full((M + 2, N + 16), -3.0, device="cuda", dtype=torch.bfloat16)
        ops.gemm_bf16(A.cuda(), B.cuda(), Cbig[1:M + 1, 8:N + 8], config=cfg)
        ops.check_status()
        got = Cbig.float().cpu()
        torch.testing.assert_close(got[1:M + 1, 8:N + 8], oracle.bf16_matmul_oracle(A, B), rtol=RTOL, atol=ATOL)
        mask = torch.ones_like(got, dtype=torch.bool); mask[1:M + 1, 8:N + 8] = False
        assert torch.all(got[mask] == -3.0)


def test_deterministic(ops, oracle):
    A, B = oracle.gen_randn_bf16(1024, 2048, 1024, seed=9)
    a, b = A.cuda(), B.cuda()
    c1 = ops.gemm_bf16(a, b).clone()
    for _ in range(3):
        assert torch.equal(ops.gemm_bf16(a, b), c1)


def test_config3_shapes_sampled(ops, oracle):
    # full benchmark sizes; the oracle is evaluated on a sample of rows (first/last tile rows included)
    for (M, K, N) in [(8192, 8192, 8192), (8192, 16384, 4096)]:
        g = torch.Generator(device="cuda").manual_seed(0)
        A = torch.randn(M, K, device="cuda", generator=g).bfloat16()
        B = torch.randn(K, N, device="cuda", generator=g).bfloat16()
        C = ops.gemm_bf16(A, B)
        ops.check_status()
        rows = torch.tensor([0, 1, 127, 128, 255, 256, 4095, 4096, M - 129, M - 128, M - 1])
        want = torch.matmul(A[rows].float().cpu(), B.float().cpu())
        torch.testing.assert_close(C[rows].float().cpu(), want, rtol=RTOL, atol=ATOL)
        # linearity in A (exact: scaling by 2 commutes with every rounding step)
        C2 = ops.gemm_bf16(A * 2, B)
        assert torch.equal(C2.float(), C.float() * 2)


def test_alignment_errors(ops):
    import gemm_b200._lib as L
    A = torch.zeros(16, 20, device="cuda", dtype=torch.bfloat16)      # lda = 20, not a multiple of 8
    B = torch.zeros(20, 16, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(L.GemmB200Error) as e:
        ops.gemm_bf16(A, B)
    assert e.value.code == L.ERR_ALIGNMENT


@pytest.mark.parametrize("M,K,N,splits", [(256, 8192, 256, 8), (128, 4096, 264, 3), (16, 2048, 512, 5), (300, 1000, 520, 4),
                                          (1, 512, 8, 2), (256, 65536, 256, 64), (1024, 4096, 1032, 4), (520, 2048, 256, 3)])
@pytest.mark.parametrize("b_is_nk", [False, True])
def test_splitk_matches_the_oracle(ops, oracle, M, K, N, splits, b_is_nk):
    """K cut into ranges whose FP32 partial sums are added in split order: within the FP32 bound of
    the unsplit kernel, and the bf16 output is the rounding of the FP32 one."""
    A, B = oracle.gen_randn_bf16(M, K, N, seed=splits)
    want = oracle.bf16_matmul_oracle(A, B)
    Bdev = B.t().contiguous().cuda() if b_is_nk else B.cuda()
    got32 = ops.gemm_bf16(A.cuda(), Bdev, b_is_nk=b_is_nk, out_dtype=torch.float32, k_splits=splits)
    ops.check_status()
    assert oracle.rel_frobenius(got32.cpu(), want) < 1e-5
    got16 = ops.gemm_bf16(A.cuda(), Bdev, b_is_nk=b_is_nk, k_splits=splits)
    ops.check_status()
    assert torch.equal(got16, got32.bfloat16())


def test_few_tiles_long_k_takes_the_split_path_by_itself(ops, oracle):
    import gemm_b200._lib as L
    M, K, N = 256, 32768, 512
    assert L.lib.gemm_b200_gemm_bf16_auto_splits(M, N, K) > 1
    assert L.lib.gemm_b200_gemm_bf16_auto_splits(8192, 8192, 8192) == 1
    A, B = oracle.gen_randn_bf16(M, K, N, seed=11)
    want = oracle.bf16_matmul_oracle(A, B)
    got = ops.gemm_bf16(A.cuda(), B.cuda(), out_dtype=torch.float32)          # library decides
    unsplit = ops.gemm_bf16(A.cuda(), B.cuda(), out_dtype=torch.float32, k_splits=1)
    ops.check_status()
    # one FP32 accumulator over 32768 products drifts further than 16 shorter partial sums
    assert oracle.rel_frobenius(got.cpu(), want) < 1e-5
    assert oracle.rel_frobenius(unsplit.cpu(), want) < 1e-4


def test_splitk_rejects_a_small_scratch(ops):
    import gemm_b200._lib as L
    A = torch.zeros(128, 1024, device="cuda", dtype=torch.bfloat16)
    B = torch.zeros(1024, 256, device="cuda", dtype=torch.bfloat16)
    C = torch.zeros(128, 256, device="cuda", dtype=torch.bfloat16)
    scratch = torch.zeros(1024, device="cuda", dtype=torch.uint8)
    rc = L.lib.gemm_b200_gemm_bf16_splitk(A.data_ptr(), B.data_ptr(), C.data_ptr(), 128, 256, 1024, 1024, 256, 256,
                                          L.B_ROW_MAJOR_KN, L.OUT_BF16, 4, scratch.data_ptr(), 1024, 0)
    assert rc == L.ERR_INVALID_ARG and b"scratch" in L.lib.gemm_b200_last_error()


@pytest.mark.parametrize("name", ["2cta_256x256x64_s6_tmastore_maskcommit", "2cta_256x512x64_s3_tmastore2_maskcommit"])
def test_runtime_unit_handout_matches_the_static_schedule(ops, oracle, name):
    """Many short units per cluster (2048 of 256 x 256, K = 128: about 28 per cluster), so the ring
    that carries the adopted unit indices wraps; every unit must be computed exactly once."""
    M, K, N = 16384, 128, 8192
    g = torch.Generator(device="cuda").manual_seed(4)
    A = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    B = torch.randn(K, N, device="cuda", generator=g).bfloat16()
    names = ops.gemm_bf16_configs()
    static = ops.gemm_bf16(A, B, config=names.index(name))
    for _ in range(3):
        dyn = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
        ops.gemm_bf16(A, B, dyn, config=names.index(name + "_dynamic"))
        ops.check_status()
        assert torch.equal(dyn, static)
    rows = torch.tensor([0, 255, 256, 8191, M - 1])
    torch.testing.assert_close(static[rows].float().cpu(), oracle.bf16_matmul_oracle(A[rows], B), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("M,K,N", [(768, 640, 1280), (2048, 4096, 4096), (8192, 8192, 8192)])
def test_against_an_independent_bf16_gemm(ops, M, K, N):
    """Independent pin: cuBLAS (torch.matmul on the GPU, a checker here, never on the product path)
    on the same bf16 operands.  Both accumulate in FP32 and round once to bf16, so the results can
    differ only where the order of the FP32 additions moves a sum across a rounding boundary: FP32
    outputs within 1e-5 relative (the FP32 rounding of a K-long sum), bf16 outputs one bf16 step
    apart in at most 1 element in 100."""
    g = torch.Generator(device="cuda").manual_seed(M + K)
    A = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    B = torch.randn(K, N, device="cuda", generator=g).bfloat16()
    got32 = ops.gemm_bf16(A, B, out_dtype=torch.float32)
    ops.check_status()
    want32 = torch.matmul(A.float(), B.float())            # FP32 SGEMM of the same values (TF32 is off by default)
    rel = float((got32.double() - want32.double()).norm() / want32.double().norm())
    assert rel <= 1e-5
    got16 = ops.gemm_bf16(A, B)
    want16 = torch.matmul(A, B)
    ops.check_status()
    diff = got16 != want16
    assert float(diff.float().mean()) <= 1e-2
    a, b = got16[diff].float(), want16[diff].float()
    # one bf16 step; sums that nearly cancel (|c| << sqrt(K)) get an absolute allowance instead
    assert bool(((a - b).abs() <= 2.0 ** -7 * torch.maximum(a.abs(), b.abs()) + 1e-3).all())


@pytest.mark.parametrize("splits", [2, 4, 8])
@pytest.mark.parametrize("M,K,N", [(128, 4096, 4096), (16, 8192, 1024), (300, 1024, 520), (100, 1504, 136), (512, 2048, 384)])
@pytest.mark.parametrize("b_is_nk", [False, True])
def test_cluster_splitk_matches_the_oracle(ops, oracle, M, K, N, splits, b_is_nk):
    """K split over the CTAs of a cluster, partial sums combined through distributed shared memory."""
    A, B = oracle.gen_randn_bf16(M, K, N, seed=M + splits)
    Bd = B.t().contiguous().cuda() if b_is_nk else B.cuda()
    want = oracle.bf16_matmul_oracle(A, B)
    C32 = torch.full((M, N), float("nan"), device="cuda")
    ops.gemm_bf16(A.cuda(), Bd, C32, b_is_nk=b_is_nk, out_dtype=torch.float32, cluster_splits=splits)
    ops.check_status()
    assert oracle.rel_frobenius(C32.cpu(), want) <= 1e-5           # FP32 sums of exact bf16 products: order only
    C16 = ops.gemm_bf16(A.cuda(), Bd, b_is_nk=b_is_nk, cluster_splits=splits)
    ops.check_status()
    assert torch.equal(C16, C32.bfloat16())                        # same sums, rounded once
    torch.testing.assert_close(C16.float().cpu(), want, rtol=2e-2, atol=2e-2)
    # the order of the additions is fixed: a second run gives the same bits
    again = ops.gemm_bf16(A.cuda(), Bd, b_is_nk=b_is_nk, out_dtype=torch.float32, cluster_splits=splits)
    assert torch.equal(again, C32)


def test_cluster_splitk_is_taken_by_itself_and_checks_its_arguments(ops, oracle):
    import gemm_b200._lib as L
    M, K, N = 128, 4096, 4096                       # 32 tiles of 128 x 128: the library splits K over clusters of 4
    A, B = oracle.gen_randn_bf16(M, K, N, seed=1)
    auto = ops.gemm_bf16(A.cuda(), B.cuda(), out_dtype=torch.float32)
    ops.check_status()
    assert torch.equal(auto, ops.gemm_bf16(A.cuda(), B.cuda(), out_dtype=torch.float32, cluster_splits=4))
    canary = torch.full((M + 2, N + 16), -3.0, device="cuda", dtype=torch.bfloat16)
    ops.gemm_bf16(A.cuda(), B.cuda(), canary[1:M + 1, 8:N + 8], cluster_splits=8)
    ops.check_status()
    mask = torch.ones_like(canary, dtype=torch.bool); mask[1:M + 1, 8:N + 8] = False
    assert bool((canary[mask] == -3.0).all())
    a = A.cuda()
    rc = L.lib.gemm_b200_gemm_bf16_cluster_splitk(a.data_ptr(), a.data_ptr(), a.data_ptr(), 128, 128, 128, 128, 128, 128, 0, 0, 3, None)
    assert rc == L.ERR_INVALID_ARG and "2, 4 or 8" in L.last_error()
    rc = L.lib.gemm_b200_gemm_bf16_cluster_splitk(a.data_ptr(), a.data_ptr(), a.data_ptr(), 128, 128, 128, 128, 128, 128, 0, 0, 8, None)
    assert rc == L.ERR_INVALID_ARG and "without K blocks" in L.last_error()      # K = 128 is two blocks of 64
