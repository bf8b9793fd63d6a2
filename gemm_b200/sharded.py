"""Row-sharded GEMM across the GPUs of one box: C[rows of rank r] = A[rows of rank r] @ B.

Rows of C depend only on the same rows of A and on all of B, so ranks never exchange data
during the GEMM.  B is broadcast once (NCCL over NVLink, or gloo in CPU tests) into each rank's
own memory before any kernel reads it; C stays sharded.  No kernel reads a peer's memory.

The reference is single-GPU (its launchers take one device's pointers,
naive/naive_1.cu:17-24); this module only adds the partition bookkeeping around the same
operator."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

BLOCKS = 8   # A is defined as 8 fixed row blocks so its contents do not depend on the rank count


@dataclass(frozen=True)
class RowShard:
    rank: int
    world: int
    row0: int
    rows: int
    blocks: tuple      # indices of the fixed row blocks this rank owns


def shard_rows(M: int, world: int, rank: int, blocks: int = BLOCKS) -> RowShard:
    """Rank `rank` of `world` owns blocks/world consecutive row blocks of M/blocks rows each."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    if blocks % world != 0:
        raise ValueError(f"{blocks} row blocks do not split over {world} ranks")
    if M % blocks != 0:
        raise ValueError(f"M={M} is not a multiple of {blocks} row blocks")
    per = blocks // world
    rows_per_block = M // blocks
    owned = tuple(range(rank * per, (rank + 1) * per))
    return RowShard(rank, world, owned[0] * rows_per_block, per * rows_per_block, owned)


def broadcast_b(B: torch.Tensor, src: int = 0) -> torch.Tensor:
    """Broadcast B from `src` into every rank's own copy (no-op without a process group)."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.broadcast(B, src=src)
    return B


def max_over_ranks(seconds: float, device=None) -> float:
    """Whole-job time of a step = the slowest rank's device time."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([seconds], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return seconds


def sum_over_ranks(value: float, device=None) -> float:
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([value], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())
    return value


def gen_a_block_cuda(block: int, rows: int, K: int, device) -> torch.Tensor:
    """Row block `block` of A ~ N(0,1) in bf16, seeded 1000 + block (same bits for any rank count)."""
    g = torch.Generator(device=device).manual_seed(1000 + block)
    return torch.randn(rows, K, device=device, generator=g).bfloat16()


def gen_b_cuda(K: int, N: int, device, seed: int = 0) -> torch.Tensor:
    g = torch.Generator(device=device).manual_seed(seed)
    return torch.randn(K, N, device=device, generator=g).bfloat16()
