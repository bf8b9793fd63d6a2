"""The bounded-wait / status path.  No GPU is hung or faulted: the self-test kernel waits 200 µs on
a barrier nothing arrives on, gives up by itself, records where, and returns normally; the host
then reads GEMM_B200_ERR_TIMEOUT from the status word, and the library keeps working."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_runs_out_and_is_reported(ops, oracle):
    import gemm_b200._lib as L
    ops.check_status()                                         # clean to begin with
    flag = torch.zeros(1, device="cuda", dtype=torch.int32)
    stream = torch.cuda.current_stream().cuda_stream
    assert L.lib.gemm_b200_selftest_wait_timeout(200, flag.data_ptr(), stream) == 0, L.last_error()
    detail = (C.c_int32 * 4)()
    rc = L.lib.gemm_b200_check_status(stream, detail)
    assert rc == L.ERR_TIMEOUT
    assert detail[0] == L.ERR_TIMEOUT and detail[1] == 0 and detail[2] == 4 and detail[3] == 777
    assert "role 4" in L.last_error()
    assert int(flag.item()) == 1                               # the kernel reached its normal end
    # the status word was cleared by the read, and real kernels run normally afterwards
    assert L.lib.gemm_b200_check_status(stream, detail) == 0
    A, B = oracle.gen_randn_bf16(256, 256, 512, seed=4)
    Cd = ops.gemm_bf16(A.cuda(), B.cuda())
    ops.check_status()
    torch.testing.assert_close(Cd.float().cpu(), oracle.bf16_matmul_oracle(A, B), rtol=2e-2, atol=2e-2)


def test_selftest_argument_checks():
    import gemm_b200._lib as L
    assert L.lib.gemm_b200_selftest_wait_timeout(0, None, None) == L.ERR_INVALID_ARG
    assert L.lib.gemm_b200_selftest_wait_timeout(10**7, None, None) == L.ERR_INVALID_ARG
    assert L.lib.gemm_b200_selftest_wait_timeout(100, None, None) == L.ERR_INVALID_ARG


def test_tma_stream_probe_runs_and_validates():
    """The bandwidth probe (a library of its own under gemm_b200/profiling) streams a matrix through
    TMA, leaves its status word clean and checks its arguments."""
    from gemm_b200.profiling.run_stream import load_probe
    P = load_probe()
    X = torch.ones(2048, 4096, device="cuda", dtype=torch.uint8)
    st = torch.cuda.current_stream().cuda_stream
    for pattern in range(4):
        assert P.gemm_b200_probe_tma_stream(X.data_ptr(), 2048, 4096, 256, pattern, st) == 0
    assert P.gemm_b200_probe_check_status(st) == 0
    assert P.gemm_b200_probe_tma_stream(X.data_ptr(), 2048, 4096, 256, 9, st) == -1
    assert P.gemm_b200_probe_tma_stream(X.data_ptr(), 2048, 4096, 100, 0, st) == -1
    assert P.gemm_b200_probe_tma_stream(0, 2048, 4096, 256, 0, st) == -1
