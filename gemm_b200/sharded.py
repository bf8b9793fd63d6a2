"""Row-sharded GEMM across the GPUs of one box: C[rows of rank r] = A[rows of rank r] @ B.

Rows of C depend only on the same rows of A and on all of B, so ranks never exchange data
during the GEMM.  B is broadcast once (NCCL over NVLink, or gloo in CPU tests) into each rank's
own memory before any kernel reads it; C stays sharded.  No kernel reads a peer's memory.

The reference is single-GPU (its launchers take one device's pointers,
naive/naive_1.cu:17-24); this module only adds the partition bookkeeping around the same
operator."""
from __future__ import annotations

import datetime
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


def broadcast_mxfp8(Bq, src: int = 0):
    """Broadcast a quantised operand (e4m3 bytes and packed UE8M0 scales) from `src`: every rank
    then multiplies by exactly the bytes rank `src` produced."""
    broadcast_b(Bq.data, src=src)
    broadcast_b(Bq.scales, src=src)
    return Bq


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


class PeerLeft(RuntimeError):
    """A rank announced that it leaves the job (between two steps)."""


class PeerLost(RuntimeError):
    """A rank did not check in for a step within the time limit."""


class Liveness:
    """Host-side check-in before every step, over the process group's key-value store.

    The ranks of a row-sharded job never exchange data inside a step, so a rank that has gone away
    is only noticed at the next collective (the timing all-reduce, a re-broadcast of B), where the
    others would block until the process-group timeout.  With this check-in every rank learns on
    the host, before it launches anything for step `s`, whether all its peers are still there:

        live = Liveness(store, rank, world, timeout_s=1.0)
        for s in range(steps):
            live.check_in(s)        # raises PeerLeft / PeerLost
            ... launch the step ...
        live.leave()                # only between steps, with nothing of this rank in flight

    Nothing here touches a GPU: a rank leaves between steps, and a rank that stopped answering is
    detected by the store wait running out."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 5.0):
        self.store, self.rank, self.world = store, rank, world
        self.timeout = datetime.timedelta(seconds=timeout_s)
        self.step = -1

    def _key(self, rank: int, step: int) -> str:
        return f"gemm_b200/live/{step}/{rank}"

    def check_in(self, step: int) -> None:
        self.step = step
        self.store.set(self._key(self.rank, step), "here")
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                self.store.wait([self._key(r, step)], self.timeout)
            except Exception as e:   # the store raises its own timeout error type
                raise PeerLost(f"rank {r} did not check in for step {step} within {self.timeout.total_seconds():.1f} s") from e
            if self.store.get(self._key(r, step)) == b"left":
                raise PeerLeft(f"rank {r} left before step {step}")

    def leave(self) -> None:
        """Announce that this rank takes no part in the next step.  Call it between steps only."""
        self.store.set(self._key(self.rank, self.step + 1), "left")
