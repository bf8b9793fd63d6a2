"""MXFP8 (e4m3 + UE8M0 per 32 k) on the GPU through the C-ABI.

Quantiser bar: bit-exact (bytes and scales) against the oracle's restatement of the recipe.
GEMM bar (stated MXFP8 tolerance): relative error <= 1e-3 against an FP32 matmul of the
dequantised operands, measured on FP32 output (bf16 rounding of the output alone is ~1.7e-3);
bf16 output is held to the bf16 rounding of that FP32 result."""
import pytest
import torch

pytestmark = pytest.mark.gpu

REL_TOL = 1e-3


@pytest.mark.parametrize("rows,K", [(1, 32), (16, 8192), (128, 128), (130, 96), (257, 416), (1000, 2048)])
@pytest.mark.parametrize("transposed_in", [False, True])
def test_quantiser_bit_exact(ops, oracle, rows, K, transposed_in):
    g = torch.Generator().manual_seed(rows * 7 + K)
    X = (torch.randn(rows, K, generator=g) * torch.exp(torch.randn(rows, 1, generator=g) * 3)).bfloat16()
    X[0, :32] = 0                                   # an all-zero block
    if rows > 1:
        X[1, :32] = 1e-40                           # a block of denormals
    q_want, s_want = oracle.mxfp8_quantize(X)
    Xd = X.t().contiguous().cuda() if transposed_in else X.cuda()
    got = ops.quantize_mxfp8(Xd, transposed_in=transposed_in)
    torch.cuda.synchronize()
    assert torch.equal(got.scale_matrix(), s_want)
    assert torch.equal(got.data.cpu(), q_want)
    # the packed buffer matches the oracle's packer byte for byte (padding = 0)
    assert torch.equal(got.scales.cpu(), oracle.mxfp8_pack_scales(s_want, K))


def test_saturation_and_extremes(ops, oracle):
    # scale 2^(floor(log2 amax) - 8) puts |x / s| in [256, 512): values above 448 must saturate
    X = torch.zeros(4, 64).bfloat16()
    X[0, :32] = torch.linspace(1.0, 1.99, 32).bfloat16()
    X[1, :32] = 3.3895e38                           # near the bf16 maximum
    X[2, 0] = -1.75
    X[3, :] = torch.tensor([2.0 ** -120]).bfloat16()
    q_want, s_want = oracle.mxfp8_quantize(X)
    got = ops.quantize_mxfp8(X.cuda())
    assert torch.equal(got.data.cpu(), q_want) and torch.equal(got.scale_matrix(), s_want)
    assert int(q_want[0].max()) == 0x7E             # 448, the e4m3 maximum


NARROW = "1cta_32x256x128_s5_narrowA"


def _configs_for(ops, M):
    """Every kernel variant that accepts M rows (the narrow-A variant takes at most 32)."""
    return [i for i, name in enumerate(ops.gemm_mxfp8_configs()) if "narrowA" not in name or M <= 32]


def _gemm_check(ops, oracle, M, K, N, config=-1, seed=0):
    A, B = oracle.gen_randn_bf16(M, K, N, seed=seed)
    Aq = ops.quantize_mxfp8(A.cuda())
    Bq = ops.quantize_mxfp8(B.cuda(), transposed_in=True)
    qa, sa = oracle.mxfp8_quantize(A)
    qb, sb = oracle.mxfp8_quantize(B.t().contiguous())
    want = oracle.mxfp8_matmul_oracle(qa, sa, qb, sb)
    C32 = torch.full((M, N), float("nan"), device="cuda")
    ops.gemm_mxfp8(Aq, Bq, C32, out_dtype=torch.float32, config=config)
    ops.check_status()
    assert oracle.rel_frobenius(C32.cpu(), want) <= REL_TOL
    torch.testing.assert_close(C32.cpu(), want, rtol=1e-3, atol=1e-3 * float(want.abs().max()))
    C16 = ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.bfloat16, config=config)
    ops.check_status()
    assert torch.equal(C16.cpu(), C32.bfloat16().cpu())      # same accumulator, rounded once


@pytest.mark.parametrize("shape", [(128, 128, 256), (256, 512, 256), (512, 1024, 768), (1024, 4096, 1024)])
def test_gemm_every_config(ops, oracle, shape):
    M, K, N = shape
    for cfg in _configs_for(ops, M):
        _gemm_check(ops, oracle, M, K, N, config=cfg, seed=cfg)


@pytest.mark.parametrize("M,K,N", [(1, 32, 8), (16, 8192, 512), (100, 96, 40), (129, 160, 264), (300, 224, 1000), (2000, 992, 24)])
def test_gemm_edge_shapes(ops, oracle, M, K, N):
    for cfg in _configs_for(ops, M):
        _gemm_check(ops, oracle, M, K, N, config=cfg, seed=M + N)


@pytest.mark.parametrize("M,K,N", [(1, 128, 256), (16, 8192, 1024), (17, 640, 520), (32, 4096, 768), (32, 96, 8), (16, 1152, 304)])
def test_narrow_a_variant(ops, oracle, M, K, N):
    """M <= 32: stages load 32 rows of A and overlap in shared memory; rows >= M of the
    accumulator see other stages' bytes and must never reach C."""
    cfg = ops.gemm_mxfp8_configs().index(NARROW)
    _gemm_check(ops, oracle, M, K, N, config=cfg, seed=M * 7 + N)
    # the default path picks it, and agrees bit for bit with the full-height single-CTA variant
    A, B = oracle.gen_randn_bf16(M, K, N, seed=5)
    Aq = ops.quantize_mxfp8(A.cuda())
    Bq = ops.quantize_mxfp8(B.cuda(), transposed_in=True)
    got = ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.float32, config=cfg)
    full = ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.float32, config=0)
    ops.check_status()
    assert torch.equal(got, full)


def test_narrow_a_variant_rejects_taller_problems(ops):
    import gemm_b200._lib as L
    cfg = ops.gemm_mxfp8_configs().index(NARROW)
    X = torch.zeros(64, 128, device="cuda", dtype=torch.bfloat16)
    q = ops.quantize_mxfp8(X)
    with pytest.raises(Exception, match="at most 32 rows"):
        ops.gemm_mxfp8(q, q, config=cfg)


def test_scales_matter(ops, oracle):
    # rows of A with very different magnitudes: wrong scale placement would show at once
    M, K, N = 256, 256, 256
    g = torch.Generator().manual_seed(3)
    A = (torch.randn(M, K, generator=g) * (2.0 ** torch.randint(-20, 20, (M, 1), generator=g))).bfloat16()
    B = (torch.randn(K, N, generator=g) * (2.0 ** torch.randint(-10, 10, (1, N), generator=g))).bfloat16()
    # and per-K-block variation
    A[:, 32:64] *= 64
    B[96:128, :] *= 1 / 128
    Aq = ops.quantize_mxfp8(A.cuda()); Bq = ops.quantize_mxfp8(B.cuda(), transposed_in=True)
    qa, sa = oracle.mxfp8_quantize(A); qb, sb = oracle.mxfp8_quantize(B.t().contiguous())
    want = oracle.mxfp8_matmul_oracle(qa, sa, qb, sb)
    for cfg in _configs_for(ops, M):
        got = ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.float32, config=cfg)
        ops.check_status()
        err = ((got.cpu() - want).abs() / (want.abs() + 1e-30))
        assert oracle.rel_frobenius(got.cpu(), want) <= REL_TOL
        # row-wise relative error, so small-magnitude rows are checked as strictly as large ones
        rowerr = torch.linalg.norm((got.cpu() - want).double(), dim=1) / torch.linalg.norm(want.double(), dim=1)
        assert float(rowerr.max()) <= REL_TOL


def test_config4_shapes_sampled(ops, oracle):
    # the FFN shape and the skinny decode shape at full size; oracle on sampled rows
    for (M, K, N) in [(16384, 8192, 28672), (16, 8192, 28672)]:
        g = torch.Generator(device="cuda").manual_seed(0)
        A = torch.randn(M, K, device="cuda", generator=g).bfloat16()
        B = torch.randn(K, N, device="cuda", generator=g).bfloat16()
        Aq = ops.quantize_mxfp8(A); Bq = ops.quantize_mxfp8(B, transposed_in=True)
        C = ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.float32)
        ops.check_status()
        rows = torch.tensor(sorted({0, 1, min(127, M - 1), min(128, M - 1), M // 2, M - 1}))
        qa, sa = oracle.mxfp8_quantize(A[rows].cpu())
        assert torch.equal(Aq.data[rows].cpu(), qa)
        cols = torch.arange(0, N, 7)
        qb, sb = oracle.mxfp8_quantize(B[:, cols].t().contiguous().cpu())
        want = oracle.mxfp8_matmul_oracle(qa, sa, qb, sb)
        assert oracle.rel_frobenius(C[rows][:, cols].cpu(), want) <= REL_TOL
        del A, B, Aq, Bq, C
        torch.cuda.empty_cache()


@pytest.mark.parametrize("M,K,N,splits", [(16, 8192, 512, 5), (16, 2048, 264, 2), (100, 1024, 1000, 7), (128, 4096, 256, 16), (1, 1024, 8, 3)])
def test_splitk_matches_the_oracle(ops, oracle, M, K, N, splits):
    A, B = oracle.gen_randn_bf16(M, K, N, seed=splits)
    Aq = ops.quantize_mxfp8(A.cuda()); Bq = ops.quantize_mxfp8(B.cuda(), transposed_in=True)
    qa, sa = oracle.mxfp8_quantize(A); qb, sb = oracle.mxfp8_quantize(B.t().contiguous())
    want = oracle.mxfp8_matmul_oracle(qa, sa, qb, sb)
    got32 = ops.gemm_mxfp8_splitk(Aq, Bq, splits, out_dtype=torch.float32)
    ops.check_status()
    assert oracle.rel_frobenius(got32.cpu(), want) <= REL_TOL
    got16 = ops.gemm_mxfp8_splitk(Aq, Bq, splits, out_dtype=torch.bfloat16)
    assert torch.equal(got16.cpu(), got32.bfloat16().cpu())
    # same bits on a second run (partials are summed in a fixed order)
    assert torch.equal(ops.gemm_mxfp8_splitk(Aq, Bq, splits, out_dtype=torch.float32), got32)


def test_skinny_default_takes_the_splitk_path(ops, oracle):
    # 16 column tiles on 148 SMs: the library splits K by itself; 112 tiles (N = 28672) run unsplit
    assert ops.gemm_mxfp8_auto_splits(16, 28672, 8192) == 1
    M, K, N = 16, 16384, 4096
    splits = ops.gemm_mxfp8_auto_splits(M, N, K)
    assert splits > 1
    g = torch.Generator(device="cuda").manual_seed(0)
    A = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    B = torch.randn(K, N, device="cuda", generator=g).bfloat16()
    Aq = ops.quantize_mxfp8(A); Bq = ops.quantize_mxfp8(B, transposed_in=True)
    auto = ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.float32)
    explicit = ops.gemm_mxfp8_splitk(Aq, Bq, splits, out_dtype=torch.float32)
    ops.check_status()
    assert torch.equal(auto, explicit)
    unsplit = ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.float32, config=0)
    assert oracle.rel_frobenius(auto.cpu(), unsplit.cpu()) <= 1e-5      # only the summation order differs


def test_splitk_rejects_a_small_scratch(ops):
    import gemm_b200._lib as L
    A = torch.zeros(16, 1024, device="cuda", dtype=torch.bfloat16)
    B = torch.zeros(1024, 256, device="cuda", dtype=torch.bfloat16)
    Aq = ops.quantize_mxfp8(A); Bq = ops.quantize_mxfp8(B, transposed_in=True)
    with pytest.raises(L.GemmB200Error) as e:
        ops.gemm_mxfp8_splitk(Aq, Bq, 4, scratch=torch.empty(1024, device="cuda", dtype=torch.uint8))
    assert e.value.code == L.ERR_INVALID_ARG


@pytest.mark.parametrize("M,K,N", [(256, 512, 256), (100, 96, 160), (129, 160, 288), (16, 1024, 512), (1000, 992, 1056)])
def test_quantising_epilogue_equals_gemm_then_quantise(ops, oracle, M, K, N):
    A, B = oracle.gen_randn_bf16(M, K, N, seed=M + N)
    A = (A.float() * torch.exp(torch.randn(M, 1, generator=torch.Generator().manual_seed(M)) * 2)).bfloat16()
    Aq = ops.quantize_mxfp8(A.cuda()); Bq = ops.quantize_mxfp8(B.cuda(), transposed_in=True)
    fused = ops.gemm_mxfp8_quant_out(Aq, Bq)
    ops.check_status()
    C16 = ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.bfloat16, config=(0 if M <= 128 else ops.gemm_mxfp8_configs().index("2cta_256x256x128_s5_maskcommit_tmastore")))
    unfused = ops.quantize_mxfp8(C16)
    assert torch.equal(fused.data, unfused.data)
    assert torch.equal(fused.scales, unfused.scales)                    # packed buffers, padding included
    # and against the oracle's quantiser applied to the same bf16 result
    q, s = oracle.mxfp8_quantize(C16.cpu())
    assert torch.equal(fused.data.cpu(), q) and torch.equal(fused.scale_matrix(), s)


def test_chained_gemms_through_the_quantising_epilogue(ops, oracle):
    # Y = (X W1) W2 with the intermediate kept in MXFP8 end to end
    M, K, H, N = 256, 512, 1024, 256
    g = torch.Generator().manual_seed(9)
    X = torch.randn(M, K, generator=g).bfloat16(); W1 = (torch.randn(K, H, generator=g) / 16).bfloat16()
    W2 = (torch.randn(H, N, generator=g) / 16).bfloat16()
    Xq = ops.quantize_mxfp8(X.cuda()); W1q = ops.quantize_mxfp8(W1.cuda(), transposed_in=True)
    W2q = ops.quantize_mxfp8(W2.cuda(), transposed_in=True)
    Hq = ops.gemm_mxfp8_quant_out(Xq, W1q)
    Y = ops.gemm_mxfp8(Hq, W2q, out_dtype=torch.float32)
    ops.check_status()
    # oracle: dequantise the very same intermediate bytes
    Hd = oracle.mxfp8_dequantize(Hq.data.cpu(), Hq.scale_matrix())
    qb, sb = oracle.mxfp8_quantize(W2.t().contiguous())
    want = torch.matmul(Hd, oracle.mxfp8_dequantize(qb, sb).t())
    assert oracle.rel_frobenius(Y.cpu(), want) <= REL_TOL


@pytest.mark.parametrize("M,K,N", [(256, 2048, 4096), (300, 1024, 1000), (512, 512, 2048)])
def test_half_round_problems_take_the_128_column_tiles(ops, oracle, M, K, N):
    """Few 256-column tiles: the library switches to 256 x 128 tiles by itself; same bits as the
    256-column variant."""
    A, B = oracle.gen_randn_bf16(M, K, N, seed=M + K)
    Aq = ops.quantize_mxfp8(A.cuda())
    Bq = ops.quantize_mxfp8(B.cuda(), transposed_in=True)
    auto = ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.float32)
    wide = ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.float32, config=ops.gemm_mxfp8_configs().index("2cta_256x256x128_s5_maskcommit_tmastore"))
    ops.check_status()
    assert torch.equal(auto, wide)
    _gemm_check(ops, oracle, M, K, N, config=ops.gemm_mxfp8_configs().index("2cta_256x128x128_s7_maskcommit_tmastore"), seed=1)


def test_handful_of_tiles_and_long_k_splits_by_itself(ops, oracle):
    """M > 128 with two tiles and K = 32768: the library cuts K on its own scratch; only the
    summation order differs from the unsplit kernel."""
    M, K, N = 256, 32768, 264
    A, B = oracle.gen_randn_bf16(M, K, N, seed=21)
    Aq = ops.quantize_mxfp8(A.cuda())
    Bq = ops.quantize_mxfp8(B.cuda(), transposed_in=True)
    auto = ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.float32)
    unsplit = ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.float32, config=ops.gemm_mxfp8_configs().index("2cta_256x256x128_s5_maskcommit_tmastore"))
    ops.check_status()
    assert oracle.rel_frobenius(auto.cpu(), unsplit.cpu()) <= 1e-5
    qa, sa = oracle.mxfp8_quantize(A)
    qb, sb = oracle.mxfp8_quantize(B.t().contiguous())
    assert oracle.rel_frobenius(auto.cpu(), oracle.mxfp8_matmul_oracle(qa, sa, qb, sb)) <= REL_TOL


def test_runtime_unit_handout_matches_the_static_schedule(ops, oracle):
    """2048 units of 256 x 256 with K = 128 (about 28 per cluster): the unit ring wraps; same bits as
    the static schedule."""
    M, K, N = 16384, 128, 8192
    g = torch.Generator(device="cuda").manual_seed(6)
    Aq = ops.quantize_mxfp8(torch.randn(M, K, device="cuda", generator=g).bfloat16())
    Bq = ops.quantize_mxfp8(torch.randn(K, N, device="cuda", generator=g).bfloat16(), transposed_in=True)
    names = ops.gemm_mxfp8_configs()
    static = ops.gemm_mxfp8(Aq, Bq, config=names.index("2cta_256x256x128_s5_maskcommit_tmastore"))
    for _ in range(3):
        dyn = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
        ops.gemm_mxfp8(Aq, Bq, dyn, config=names.index("2cta_256x256x128_s5_maskcommit_tmastore_dynamic"))
        ops.check_status()
        assert torch.equal(dyn, static)


@pytest.mark.parametrize("splits", [2, 4, 8])
@pytest.mark.parametrize("M,K,N", [(128, 4096, 2048), (16, 8192, 1024), (300, 2048, 520), (100, 3040, 136), (1, 1024, 8)])
def test_cluster_splitk_matches_the_oracle(ops, oracle, M, K, N, splits):
    """K split over the CTAs of a cluster, partial sums combined through distributed shared memory."""
    A, B = oracle.gen_randn_bf16(M, K, N, seed=M + splits)
    A = (A.float() * torch.exp(torch.randn(M, 1, generator=torch.Generator().manual_seed(M)) * 2)).bfloat16()
    Aq = ops.quantize_mxfp8(A.cuda()); Bq = ops.quantize_mxfp8(B.cuda(), transposed_in=True)
    qa, sa = oracle.mxfp8_quantize(A); qb, sb = oracle.mxfp8_quantize(B.t().contiguous())
    want = oracle.mxfp8_matmul_oracle(qa, sa, qb, sb)
    C32 = torch.full((M, N), float("nan"), device="cuda")
    ops.gemm_mxfp8(Aq, Bq, C32, out_dtype=torch.float32, cluster_splits=splits)
    ops.check_status()
    assert oracle.rel_frobenius(C32.cpu(), want) <= REL_TOL
    unsplit = ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.float32, config=0)
    assert oracle.rel_frobenius(C32.cpu(), unsplit.cpu()) <= 1e-5     # only the summation order differs
    C16 = ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.bfloat16, cluster_splits=splits)
    ops.check_status()
    assert torch.equal(C16, C32.bfloat16())
    assert torch.equal(ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.float32, cluster_splits=splits), C32)   # fixed order: same bits again


def test_cluster_splitk_is_taken_by_itself(ops, oracle):
    import gemm_b200._lib as L
    M, K, N = 64, 4096, 2048                        # 16 tiles of 128 x 128: clusters of 4
    A, B = oracle.gen_randn_bf16(M, K, N, seed=2)
    Aq = ops.quantize_mxfp8(A.cuda()); Bq = ops.quantize_mxfp8(B.cuda(), transposed_in=True)
    auto = ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.float32)
    ops.check_status()
    assert torch.equal(auto, ops.gemm_mxfp8(Aq, Bq, out_dtype=torch.float32, cluster_splits=4))
    rc = L.lib.gemm_b200_gemm_mxfp8_cluster_splitk(Aq.data.data_ptr(), Aq.scales.data_ptr(), Bq.data.data_ptr(), Bq.scales.data_ptr(),
                                                   auto.data_ptr(), M, N, K, N, 1, 3, None)
    assert rc == L.ERR_INVALID_ARG and "2, 4 or 8" in L.last_error()
    rc = L.lib.gemm_b200_gemm_mxfp8_cluster_splitk(Aq.data.data_ptr(), Aq.scales.data_ptr(), Bq.data.data_ptr(), Bq.scales.data_ptr(),
                                                   auto.data_ptr(), M, N, 256, N, 1, 8, None)
    assert rc == L.ERR_INVALID_ARG and "without K blocks" in L.last_error()
