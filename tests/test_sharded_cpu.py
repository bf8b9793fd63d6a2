"""Row sharding: partition arithmetic and the N > 1 bookkeeping on two gloo ranks (CPU)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gemm_b200 import sharded


def test_shard_rows_partitions_every_row_once():
    M = 131072
    for world in (1, 2, 4, 8):
        shards = [sharded.shard_rows(M, world, r) for r in range(world)]
        assert shards[0].row0 == 0 and shards[-1].row0 + shards[-1].rows == M
        for a, b in zip(shards, shards[1:]):
            assert a.row0 + a.rows == b.row0
        assert all(s.rows == M // world for s in shards)
        blocks = [b for s in shards for b in s.blocks]
        assert blocks == list(range(sharded.BLOCKS))


def test_shard_rows_rejects_bad_arguments():
    with pytest.raises(ValueError):
        sharded.shard_rows(131072, 3, 0)
    with pytest.raises(ValueError):
        sharded.shard_rows(100, 8, 0)
    with pytest.raises(ValueError):
        sharded.shard_rows(1024, 2, 2)


def test_helpers_are_identity_without_a_process_group():
    B = torch.arange(6.0).view(2, 3)
    assert sharded.broadcast_b(B) is B
    assert sharded.max_over_ranks(1.5) == 1.5 and sharded.sum_over_ranks(2.0) == 2.0


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, K, N = 64, 24, 16
        shard = sharded.shard_rows(M, world, rank)
        g = torch.Generator().manual_seed(0)
        B = torch.randn(K, N, generator=g) if rank == 0 else torch.zeros(K, N)
        sharded.broadcast_b(B, src=0)
        rows_per_block = M // sharded.BLOCKS
        A = torch.cat([torch.randn(rows_per_block, K, generator=torch.Generator().manual_seed(1000 + b)) for b in shard.blocks])
        C = A @ B                                        # stands in for the GPU operator on this rank's rows
        t = sharded.max_over_ranks(0.25 * (rank + 1))
        n = sharded.sum_over_ranks(3.0)
        q.put((rank, shard.row0, shard.rows, C, float(B.sum()), t, n))
    finally:
        dist.destroy_process_group()


def _free_port() -> int:
    import socket
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as sk:
        sk.bind(("127.0.0.1", 0))
        return sk.getsockname()[1]


def test_two_gloo_ranks_reproduce_the_single_rank_result():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted([q.get(timeout=120) for _ in range(world)], key=lambda x: x[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    M, K, N = 64, 24, 16
    B = torch.randn(K, N, generator=torch.Generator().manual_seed(0))
    A = torch.cat([torch.randn(M // sharded.BLOCKS, K, generator=torch.Generator().manual_seed(1000 + b))
                   for b in range(sharded.BLOCKS)])
    full = A @ B
    for rank, row0, rows, C, bsum, t, n in results:
        assert torch.equal(C, full[row0:row0 + rows])     # same rows, same bits, whatever the rank count
        assert bsum == float(B.sum())                     # every rank holds the broadcast B
        assert t == 0.5 and n == 6.0                      # max / sum over ranks


# ----------------------------------------------------------------------------------------------
# failure detection on the host: a rank that leaves between steps, and one that stops answering
# ----------------------------------------------------------------------------------------------
def _live_worker(rank, world, port, q, mode):
    import datetime
    import time
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=30))
    live = sharded.Liveness(store, rank, world, timeout_s=1.0)
    done, outcome = 0, "finished"
    try:
        for step in range(4):
            if rank == 1 and step == 2:
                if mode == "leaves":
                    live.leave()              # between steps, nothing in flight
                    outcome = "left"
                else:
                    time.sleep(3.0)           # stops answering: never checks in for step 2
                    outcome = "silent"
                break
            live.check_in(step)
            done += 1                         # the step itself (this rank's rows) would run here
    except sharded.PeerLeft as e:
        outcome = "peer-left: " + str(e)
    except sharded.PeerLost as e:
        outcome = "peer-lost: " + str(e)
    q.put((rank, done, outcome))
    if rank == 0:
        time.sleep(0.5 if mode == "leaves" else 3.5)   # the store's host outlives its clients


@pytest.mark.parametrize("mode", ["leaves", "silent"])
def test_a_rank_that_goes_away_is_noticed_before_the_next_step(mode):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_live_worker, args=(r, world, port, q, mode)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict((r, (d, o)) for r, d, o in [q.get(timeout=60) for _ in range(world)])
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    assert results[1][0] == 2                                   # rank 1 ran steps 0 and 1
    done0, outcome0 = results[0]
    assert done0 == 2                                            # rank 0 launched nothing for step 2
    if mode == "leaves":
        assert outcome0.startswith("peer-left: rank 1 left before step 2")
    else:
        assert outcome0.startswith("peer-lost: rank 1 did not check in for step 2")
