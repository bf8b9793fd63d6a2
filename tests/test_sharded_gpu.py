"""Row-sharded BF16 and MXFP8 GEMM on two GPUs (NCCL): every rank's rows equal the single-GPU
result bit for bit.  Skipped on machines with fewer than two GPUs."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q, mx=False):
    import torch.distributed as dist
    import gemm_b200.ops as ops
    from gemm_b200 import sharded
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        dev = torch.device("cuda", rank)
        M, K, N = 4096, 1024, 1536
        shard = sharded.shard_rows(M, world, rank)
        rows_per_block = M // sharded.BLOCKS
        A = torch.cat([sharded.gen_a_block_cuda(b, rows_per_block, K, dev) for b in shard.blocks])
        B = sharded.gen_b_cuda(K, N, dev) if rank == 0 else torch.empty(K, N, device=dev, dtype=torch.bfloat16)
        sharded.broadcast_b(B, src=0)
        if mx:
            # rank 0's quantised B is the one every rank multiplies by
            Bq = ops.quantize_mxfp8(B if rank == 0 else torch.zeros_like(B), transposed_in=True)
            sharded.broadcast_mxfp8(Bq, src=0)
            Cd = ops.gemm_mxfp8(ops.quantize_mxfp8(A), Bq)
        else:
            Cd = ops.gemm_bf16(A, B)
        ops.check_status(dev)
        t = sharded.max_over_ranks(float(rank + 1), device=dev)
        q.put((rank, shard.row0, shard.rows, Cd.cpu(), t))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("mx", [False, True], ids=["bf16", "mxfp8"])
def test_two_ranks_match_one_gpu(ops, mx):
    import torch.multiprocessing as mp
    from gemm_b200 import sharded
    import socket
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, mx)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted([q.get(timeout=300) for _ in range(world)], key=lambda x: x[0])
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    M, K, N = 4096, 1024, 1536
    dev = torch.device("cuda", 0)
    A = torch.cat([sharded.gen_a_block_cuda(b, M // sharded.BLOCKS, K, dev) for b in range(sharded.BLOCKS)])
    B = sharded.gen_b_cuda(K, N, dev)
    if mx:
        full = ops.gemm_mxfp8(ops.quantize_mxfp8(A), ops.quantize_mxfp8(B, transposed_in=True)).cpu()
    else:
        full = ops.gemm_bf16(A, B).cpu()
    for rank, row0, rows, Cd, t in results:
        assert torch.equal(Cd, full[row0:row0 + rows])
        assert t == 2.0
