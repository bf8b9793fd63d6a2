"""The library-owned split-K scratch is kept per (device, stream): two automatically split
problems launched on two streams at the same time give the bits of the serial run."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_auto_split_on_two_streams_matches_the_serial_run(ops):
    g = torch.Generator(device="cuda").manual_seed(0)
    # few output tiles and a long K: both entry points cut K by themselves
    M, K, N = 256, 32768, 256
    assert ops.gemm_mxfp8_auto_splits(M, N, K) > 1
    A1 = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    B1 = torch.randn(K, N, device="cuda", generator=g).bfloat16()
    A2 = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    B2 = torch.randn(K, N, device="cuda", generator=g).bfloat16()
    A1q, B1q = ops.quantize_mxfp8(A1), ops.quantize_mxfp8(B1, transposed_in=True)
    A2q, B2q = ops.quantize_mxfp8(A2), ops.quantize_mxfp8(B2, transposed_in=True)
    serial = [ops.gemm_bf16(A1, B1, out_dtype=torch.float32), ops.gemm_bf16(A2, B2, out_dtype=torch.float32),
              ops.gemm_mxfp8(A1q, B1q, out_dtype=torch.float32), ops.gemm_mxfp8(A2q, B2q, out_dtype=torch.float32)]
    ops.check_status()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    outs = [torch.empty(M, N, device="cuda") for _ in range(4)]
    torch.cuda.synchronize()
    for rep in range(20):                      # many back-to-back pairs: the kernels of the two streams overlap
        with torch.cuda.stream(s1):
            ops.gemm_bf16(A1, B1, outs[0], out_dtype=torch.float32)
            ops.gemm_mxfp8(A1q, B1q, outs[2], out_dtype=torch.float32)
        with torch.cuda.stream(s2):
            ops.gemm_bf16(A2, B2, outs[1], out_dtype=torch.float32)
            ops.gemm_mxfp8(A2q, B2q, outs[3], out_dtype=torch.float32)
    torch.cuda.synchronize()
    ops.check_status()
    for got, want in zip(outs, serial):
        assert torch.equal(got, want)
