"""The operators under CUDA-graph capture: a launch-bound loop of small GEMMs is what a caller
captures once and replays (the reference's own benchmark sizes start at 128^3,
naive/benchmark.py:18).  Each operator is warmed up, captured on a side stream, and the replay is
compared bit for bit with the eager result on NEW input values (the graph holds pointers, not
data)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _capture(fn):
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            fn()                                   # warm-up: first-use set-up happens outside the capture
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    return graph


@pytest.mark.parametrize("n", [128, 512])
def test_fp32_small_problem_replays(ops, n):
    g = torch.Generator(device="cuda").manual_seed(n)
    A = torch.rand(n, n, device="cuda", generator=g) * 2 - 1
    B = torch.rand(n, n, device="cuda", generator=g) * 2 - 1
    C = torch.zeros(n, n, device="cuda")
    graph = _capture(lambda: ops.sgemm_f32(A, B, C))
    A.copy_(torch.rand(n, n, device="cuda", generator=g) * 2 - 1)
    C.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(C, ops.sgemm_f32(A, B))
    ops.check_status()


def test_variant_module_replays():
    from gemm_b200.variants import load_variant
    mod = load_variant("blocktile_1d")
    g = torch.Generator(device="cuda").manual_seed(7)
    A = torch.randn(256, 256, device="cuda", generator=g)
    B = torch.randn(256, 256, device="cuda", generator=g)
    C = torch.zeros(256, 256, device="cuda")
    graph = _capture(lambda: mod.gemm_cuda(A, B, C))
    B.copy_(torch.randn(256, 256, device="cuda", generator=g))
    C.zero_()
    graph.replay()
    torch.cuda.synchronize()
    want = torch.zeros_like(C)
    mod.gemm_cuda(A, B, want)
    assert torch.equal(C, want)


@pytest.mark.parametrize("M,K,N", [(512, 1024, 512), (128, 4096, 4096), (1024, 8192, 1024), (4096, 4096, 4096)])
def test_bf16_replays_including_the_split_paths(ops, M, K, N):
    """(128, 4096, 4096) takes the in-cluster K split, (1024, 8192, 1024) the two-launch split on
    library-owned scratch (allocated by the warm-up calls, on the capturing stream)."""
    g = torch.Generator(device="cuda").manual_seed(M + N)
    A = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    B = torch.randn(K, N, device="cuda", generator=g).bfloat16()
    C = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    graph = _capture(lambda: ops.gemm_bf16(A, B, C))
    A.copy_(torch.randn(M, K, device="cuda", generator=g).bfloat16())
    C.zero_()
    graph.replay()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(C, ops.gemm_bf16(A, B))
    ops.check_status()


def test_mxfp8_quantise_and_gemm_replay_as_one_graph(ops):
    M, K, N = 256, 2048, 1024
    g = torch.Generator(device="cuda").manual_seed(3)
    A = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    Bq = ops.quantize_mxfp8(torch.randn(K, N, device="cuda", generator=g).bfloat16(), transposed_in=True)
    out = {}

    def step():
        out["C"] = ops.gemm_mxfp8(ops.quantize_mxfp8(A), Bq)

    graph = _capture(step)
    A.copy_(torch.randn(M, K, device="cuda", generator=g).bfloat16())
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out["C"], ops.gemm_mxfp8(ops.quantize_mxfp8(A), Bq))
    ops.check_status()
