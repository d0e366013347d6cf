"""Multi-GPU plumbing for the decode step: one process per GPU, sequences sharded, no data-path collective.

The decode step of independent sequences needs no exchange between GPUs: every rank holds a full
replica of the int4 weights (2.2 GB) and decodes its own sequences with its own cache and CUDA graph.
``torch.distributed`` is used only to line the ranks up (barrier) and to combine their timings and
token counts. The same functions run on CPU ranks over ``gloo`` (the tests) and on GPU ranks over NCCL.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Rank:
    rank: int
    world: int
    local_rank: int

    @property
    def is_main(self) -> bool:
        return self.rank == 0


def rank_from_env() -> Rank:
    """RANK / WORLD_SIZE / LOCAL_RANK as torchrun sets them; a single process when they are absent."""
    return Rank(int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0")))


def init(backend: str, r: Rank | None = None) -> Rank:
    """Join the process group named by the environment (MASTER_ADDR/MASTER_PORT) when there is more than one rank."""
    r = r or rank_from_env()
    if r.world > 1 and not dist.is_initialized():
        kwargs = {}
        if backend == "nccl":
            torch.cuda.set_device(r.local_rank)
            kwargs["device_id"] = torch.device("cuda", r.local_rank)
        dist.init_process_group(backend, rank=r.rank, world_size=r.world, **kwargs)
    return r


def shard_range(n_items: int, rank: int, world: int) -> range:
    """Contiguous, balanced slice of ``n_items`` independent sequences for ``rank``: sizes differ by at most one,
    earlier ranks take the larger ones, every item belongs to exactly one rank."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"rank {rank} is not in a world of {world}")
    if n_items < 0:
        raise ValueError("n_items must be non-negative")
    base, extra = divmod(n_items, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def barrier() -> None:
    if dist.is_initialized():
        dist.barrier()


def max_over_ranks(value: float, device="cpu") -> float:
    """The slowest rank's value: multi-GPU timings are reported as the maximum over ranks."""
    t = torch.tensor([value], dtype=torch.float64, device=device)
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value: float, device="cpu") -> float:
    t = torch.tensor([value], dtype=torch.float64, device=device)
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def aggregate_throughput(tokens_this_rank: int, seconds_this_rank: float, device="cpu") -> float:
    """Whole-job tokens per second: all ranks' tokens over the slowest rank's time."""
    return sum_over_ranks(float(tokens_this_rank), device) / max_over_ranks(seconds_this_rank, device)
