"""Chains of dependent launches without host synchronisation.  Every tensor-core kernel is a
programmatic dependent launch: it may be scheduled, and set itself up, while the kernel before it
still runs, and must wait for that kernel before it touches memory.  A consumer that started too
early would read a half-written operand, so each chain is compared bit for bit with the same chain
run with a device synchronisation after every step."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _chain(ops, A, Bs, sync, **kw):
    X = A
    for B in Bs:
        X = ops.gemm_bf16(X, B, **kw)
        if sync:
            torch.cuda.synchronize()
    return X


@pytest.mark.parametrize("M,D,depth", [(256, 512, 12), (128, 4096, 6), (1024, 1024, 8), (4096, 2048, 4), (1024, 8192, 3)])
def test_bf16_chain_matches_the_synchronised_chain(ops, M, D, depth):
    """(128, 4096) takes the in-cluster K split, (1024, 8192) the two-launch split (GEMM -> reduction ->
    next GEMM on the same scratch), the others the plain kernels."""
    g = torch.Generator(device="cuda").manual_seed(M + D)
    A = torch.randn(M, D, device="cuda", generator=g).bfloat16()
    Bs = [(torch.randn(D, D, device="cuda", generator=g) / D ** 0.5).bfloat16() for _ in range(depth)]
    want = _chain(ops, A, Bs, sync=True)
    for _ in range(3):
        got = _chain(ops, A, Bs, sync=False)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    ops.check_status()


def test_reused_output_buffer_is_not_overwritten_early(ops):
    """C = A @ B into one buffer, a torch copy of it, then the next GEMM into the same buffer: the second
    GEMM may not store before the copy has read."""
    g = torch.Generator(device="cuda").manual_seed(5)
    A1 = torch.randn(2048, 1024, device="cuda", generator=g).bfloat16()
    A2 = torch.randn(2048, 1024, device="cuda", generator=g).bfloat16()
    B = torch.randn(1024, 2048, device="cuda", generator=g).bfloat16()
    C = torch.empty(2048, 2048, device="cuda", dtype=torch.bfloat16)
    w1 = ops.gemm_bf16(A1, B); w2 = ops.gemm_bf16(A2, B)
    torch.cuda.synchronize()
    for _ in range(5):
        ops.gemm_bf16(A1, B, C)
        k1 = C.clone()
        ops.gemm_bf16(A2, B, C)
        ops.gemm_bf16(A1, B, C)          # GEMM straight behind a GEMM on the same output
        k2 = C.clone()
        ops.gemm_bf16(A2, B, C)
        torch.cuda.synchronize()
        assert torch.equal(k1, w1) and torch.equal(k2, w1) and torch.equal(C, w2)


def test_mxfp8_quantise_gemm_chain(ops):
    g = torch.Generator(device="cuda").manual_seed(9)
    D = 2048
    X0 = torch.randn(512, D, device="cuda", generator=g).bfloat16()
    Bqs = [ops.quantize_mxfp8((torch.randn(D, D, device="cuda", generator=g) / D ** 0.5).bfloat16(), transposed_in=True) for _ in range(6)]

    def run(sync):
        X = X0
        for Bq in Bqs:
            X = ops.gemm_mxfp8(ops.quantize_mxfp8(X), Bq)
            if sync:
                torch.cuda.synchronize()
        return X

    want = run(True)
    for _ in range(3):
        got = run(False)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    ops.check_status()


def test_two_streams_with_an_event_between_them(ops):
    g = torch.Generator(device="cuda").manual_seed(11)
    A = torch.randn(1024, 1024, device="cuda", generator=g).bfloat16()
    B1 = (torch.randn(1024, 1024, device="cuda", generator=g) / 32).bfloat16()
    B2 = (torch.randn(1024, 1024, device="cuda", generator=g) / 32).bfloat16()
    want = ops.gemm_bf16(ops.gemm_bf16(A, B1), B2)
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    for _ in range(5):
        with torch.cuda.stream(s1):
            X = ops.gemm_bf16(A, B1)
            done = torch.cuda.Event(); done.record(s1)
        with torch.cuda.stream(s2):
            s2.wait_event(done)
            Y = ops.gemm_bf16(X, B2)
        s2.synchronize(); s1.synchronize()
        assert torch.equal(Y, want)
