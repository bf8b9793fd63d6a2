"""FP32 parity on the GPU, through the C-ABI (gemm_b200_sgemm_f32 via ctypes).

Bar: bit-exact against the CPU restatement of the reference kernels' arithmetic
(oracle.sgemm_seq) and against the reference's own kernels compiled unchanged
(oracle/_ref); relative Frobenius error <= 1e-5 against torch.matmul on the CPU, the
reference's oracle (naive/test.py:23) as the benchmark config places it."""
import pytest
import torch

pytestmark = pytest.mark.gpu

REL_FRO_TOL = 1e-5   # stated FP32 tolerance


def _run(ops, A, B, config=-1):
    C = torch.full((A.shape[0], B.shape[1]), float("nan"), device="cuda")
    out = ops.sgemm_f32(A.cuda(), B.cuda(), C, config=config)
    assert out.data_ptr() == C.data_ptr()      # written in place and returned (naive/naive.cpp:17-21)
    torch.cuda.synchronize()
    return C.cpu()


# the reference tests' shapes (naive/test.py:13) + the config-1 shape
@pytest.mark.parametrize("n", [128, 512, 1024])
def test_reference_test_shapes_bit_exact(ops, oracle, n):
    A, B = oracle.gen_randn_f32(n, n, n, seed=42)
    C = _run(ops, A, B)
    want = oracle.sgemm_seq(A, B)
    assert torch.equal(C, want)
    assert oracle.rel_frobenius(C, oracle.matmul_cpu(A, B)) <= REL_FRO_TOL


def test_config1_uniform_1024(ops, oracle):
    A, B = oracle.gen_uniform_f32(1024, 1024, 1024, seed=0)
    C = _run(ops, A, B)
    assert torch.equal(C, oracle.sgemm_seq(A, B))
    assert oracle.rel_frobenius(C, oracle.matmul_cpu(A, B)) <= REL_FRO_TOL


# ragged / edge shapes the reference handles through its guards (shared/shared_2.cu:24-41)
EDGE_SHAPES = [
    (1, 1, 1), (1, 7, 1), (3, 5, 2), (16, 16, 16), (17, 33, 65), (64, 64, 64), (100, 100, 100),
    (127, 129, 63), (128, 4, 128), (129, 8, 257), (255, 1024, 3), (1, 4096, 1), (16, 512, 300),
    (300, 20, 16), (513, 12, 516), (260, 260, 260), (1000, 36, 1000),
]


@pytest.mark.parametrize("M,K,N", EDGE_SHAPES)
def test_edge_shapes_bit_exact(ops, oracle, M, K, N):
    A, B = oracle.gen_uniform_f32(M, K, N, seed=M * 131 + K * 17 + N)
    assert torch.equal(_run(ops, A, B), oracle.sgemm_seq(A, B))


def test_every_config_bit_exact(ops, oracle):
    # aligned shape -> 16-byte path; odd shape -> 4-byte path; both must match for every tile config
    for (M, K, N) in [(384, 200, 320), (130, 37, 99)]:
        A, B = oracle.gen_uniform_f32(M, K, N, seed=7)
        want = oracle.sgemm_seq(A, B)
        for cfg, name in enumerate(ops.sgemm_f32_configs()):
            assert torch.equal(_run(ops, A, B, config=cfg), want), name


def test_k_zero_writes_zeros(ops):
    A = torch.empty(8, 0, device="cuda")
    B = torch.empty(0, 12, device="cuda")
    C = torch.full((8, 12), 5.0, device="cuda")
    ops.sgemm_f32(A, B, C)
    assert torch.count_nonzero(C) == 0


def test_empty_m_or_n_is_a_no_op(ops):
    ops.sgemm_f32(torch.empty(0, 4, device="cuda"), torch.empty(4, 3, device="cuda"))
    ops.sgemm_f32(torch.empty(3, 4, device="cuda"), torch.empty(4, 0, device="cuda"))


def test_beta_zero_overwrites_c(ops, oracle):
    A, B = oracle.gen_uniform_f32(96, 40, 72, seed=3)
    C = torch.full((96, 72), 1e30, device="cuda")
    ops.sgemm_f32(A.cuda(), B.cuda(), C)
    assert torch.equal(C.cpu(), oracle.sgemm_seq(A, B))


def test_strided_rows_and_canaries(ops, oracle):
    # row-major views with a leading dimension larger than the row; bytes outside C stay untouched
    M, K, N = 70, 52, 44
    A, B = oracle.gen_uniform_f32(M, K, N, seed=11)
    Abig = torch.zeros(M, K + 12, device="cuda"); Abig[:, :K] = A.cuda()
    Bbig = torch.zeros(K, N + 20, device="cuda"); Bbig[:, :N] = B.cuda()
    Cbig = torch.full((M + 2, N + 8), -7.0, device="cuda")
    ops.sgemm_f32(Abig[:, :K], Bbig[:, :N], Cbig[1:M + 1, 4:N + 4])
    got = Cbig.cpu()
    assert torch.equal(got[1:M + 1, 4:N + 4], oracle.sgemm_seq(A, B))
    mask = torch.ones_like(got, dtype=torch.bool); mask[1:M + 1, 4:N + 4] = False
    assert torch.all(got[mask] == -7.0)


def test_denormals_are_flushed_like_the_reference(ops, oracle):
    # --use_fast_math implies -ftz=true in the reference build (naive/test.py:8)
    A = torch.full((4, 8), 1e-30); B = torch.full((8, 4), 1e-10)
    got = _run(ops, A, B)
    assert torch.equal(got, oracle.sgemm_seq(A, B, ftz=True))
    assert torch.count_nonzero(got) == 0


def test_linearity_at_full_size(ops):
    # size-independent property at the largest sweep shape: (2A) @ B == 2 (A @ B) exactly in FP32
    n = 4096
    g = torch.Generator(device="cuda").manual_seed(0)
    A = torch.rand(n, n, device="cuda", generator=g) * 2 - 1
    B = torch.rand(n, n, device="cuda", generator=g) * 2 - 1
    C1 = ops.sgemm_f32(A, B)
    C2 = ops.sgemm_f32(A * 2, B)
    assert torch.equal(C1 * 2, C2)
    # and a sampled exact check of 64 rows against the CPU restatement
    from oracle import oracle as O
    rows = torch.randint(0, n, (64,), generator=torch.Generator().manual_seed(1))
    want = O.sgemm_seq(A[rows].cpu(), B.cpu())
    assert torch.equal(C1[rows].cpu(), want)


def _tile_edge_rows(n, extra=48, seed=1):
    """First and last rows of C, the rows either side of every 64/128-row tile boundary near both
    ends, and `extra` random rows."""
    edge = [0, 1, 63, 64, 127, 128, n // 2 - 1, n // 2, n - 129, n - 128, n - 65, n - 64, n - 2, n - 1]
    rnd = torch.randint(0, n, (extra,), generator=torch.Generator().manual_seed(seed)).tolist()
    return torch.tensor(sorted(set(edge + rnd)))


def test_sweep_2048_full_frobenius_and_sampled_bits(ops, oracle):
    # sweep point 2048^3 (uniform[-1,1), seed 0): the whole result against torch.matmul on the CPU,
    # sampled rows bit for bit against the restated reference arithmetic
    n = 2048
    A, B = oracle.gen_uniform_f32(n, n, n, seed=0)
    C = _run(ops, A, B)
    assert oracle.rel_frobenius(C, oracle.matmul_cpu(A, B)) <= REL_FRO_TOL
    rows = _tile_edge_rows(n)
    assert torch.equal(C[rows], oracle.sgemm_seq(A[rows], B))


def test_sweep_8192_sampled(ops, oracle):
    # sweep point 8192^3: sampled rows (tile edges included) bit for bit, and the same rows within
    # the Frobenius tolerance of torch.matmul on the CPU
    n = 8192
    A, B = oracle.gen_uniform_f32(n, n, n, seed=0)
    C = _run(ops, A, B)
    rows = _tile_edge_rows(n, extra=50, seed=2)
    got = C[rows]
    assert torch.equal(got, oracle.sgemm_seq(A[rows], B))
    assert oracle.rel_frobenius(got, oracle.matmul_cpu(A[rows], B)) <= REL_FRO_TOL
    # no row of the result was left unwritten (C starts as NaN)
    assert not bool(torch.isnan(C).any())


@pytest.mark.parametrize("variant", ["naive", "shared", "blocktile_1d"])
@pytest.mark.parametrize("shape", [(128, 128, 128), (512, 512, 512), (200, 77, 130)])
def test_bit_identical_to_reference_kernels(ops, oracle, variant, shape):
    if not oracle.reference_available():
        pytest.skip("oracle/_ref not built")
    M, K, N = shape
    A, B = oracle.gen_randn_f32(M, K, N, seed=42)
    ref = oracle.reference_kernel(variant)(A.cuda(), B.cuda(), torch.zeros(M, N, device="cuda")).cpu()
    assert torch.equal(_run(ops, A, B), ref)
    assert torch.equal(oracle.sgemm_seq(A, B), ref)     # pins the CPU restatement to the real reference


def test_argument_errors(ops):
    import gemm_b200._lib as L
    with pytest.raises(ValueError):
        ops.sgemm_f32(torch.zeros(4, 5, device="cuda"), torch.zeros(6, 3, device="cuda"))
    rc = L.lib.gemm_b200_sgemm_f32(None, None, None, 4, 4, 4, 4, 4, 4, None)
    assert rc == L.ERR_INVALID_ARG and "null" in L.last_error()
    A = torch.zeros(4, 4, device="cuda")
    rc = L.lib.gemm_b200_sgemm_f32(A.data_ptr(), A.data_ptr(), A.data_ptr(), 4, 4, 4, 2, 4, 4, None)
    assert rc == L.ERR_INVALID_ARG
    rc = L.lib.gemm_b200_sgemm_f32(A.data_ptr(), A.data_ptr(), A.data_ptr(), -1, 4, 4, 4, 4, 4, None)
    assert rc == L.ERR_INVALID_ARG


def test_log_and_forced_config_knobs(oracle):
    # the knobs are read once per process, so exercise them in a child process
    import os, subprocess, sys
    code = ("import torch, gemm_b200.ops as ops; A = torch.ones(256, 64, device='cuda'); B = torch.ones(64, 256, device='cuda');"
            "C = ops.sgemm_f32(A, B); torch.cuda.synchronize(); assert float(C[0, 0]) == 64.0")
    env = dict(os.environ, GEMM_B200_LOG="1", GEMM_B200_F32_CONFIG="0")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, cwd=str(__import__("pathlib").Path(__file__).resolve().parent.parent))
    assert r.returncode == 0, r.stderr
    assert "[gemm_b200] sgemm_f32 256x64x256 -> 64x128x32_s3_f32x2" in r.stderr


@pytest.mark.parametrize("batch,M,K,N", [(3, 70, 52, 44), (5, 128, 64, 256), (2, 1, 9, 3), (7, 200, 33, 130)])
def test_strided_batched_equals_one_call_per_problem(ops, oracle, batch, M, K, N):
    g = torch.Generator().manual_seed(batch * 100 + M)
    A = torch.rand(batch, M, K, generator=g) * 2 - 1
    B = torch.rand(batch, K, N, generator=g) * 2 - 1
    got = ops.sgemm_f32_batched(A.cuda(), B.cuda()).cpu()
    for i in range(batch):
        assert torch.equal(got[i], oracle.sgemm_seq(A[i], B[i]))
    shared = ops.sgemm_f32_batched(A.cuda(), B[0].cuda()).cpu()         # one B for every problem
    for i in range(batch):
        assert torch.equal(shared[i], oracle.sgemm_seq(A[i], B[0]))
    # padded pitches and batch strides; bytes between the matrices stay untouched
    Cbig = torch.full((batch, M + 3, N + 5), -7.0, device="cuda")
    ops.sgemm_f32_batched(A.cuda(), B.cuda(), Cbig[:, 1:M + 1, 2:N + 2])
    assert torch.equal(Cbig[:, 1:M + 1, 2:N + 2].cpu(), got)
    mask = torch.ones_like(Cbig, dtype=torch.bool); mask[:, 1:M + 1, 2:N + 2] = False
    assert bool((Cbig[mask] == -7.0).all())


def test_strided_batched_argument_errors(ops):
    import gemm_b200._lib as L
    A = torch.zeros(2, 4, 4, device="cuda")
    rc = L.lib.gemm_b200_sgemm_f32_batched(A.data_ptr(), A.data_ptr(), A.data_ptr(), 2, 4, 4, 4, 4, 4, 4, 8, 16, 16, None)
    assert rc == L.ERR_INVALID_ARG and "stride" in L.last_error()
    assert L.lib.gemm_b200_sgemm_f32_batched(None, None, None, 0, 4, 4, 4, 4, 4, 4, 16, 16, 16, None) == L.OK
