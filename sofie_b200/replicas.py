"""One replica per GPU: rank discovery, batch sharding and max-over-ranks timing.

Inferences are independent (a reference Session holds all state and owns one device,
core/src/RModel_ALPAKA.cxx:1123-1132), so the batch is split across ranks and no collective sits
on the data path; torch.distributed is used only for the start barrier and for reducing the
timing.  Works with the `nccl` backend on GPUs and with `gloo` on CPU (used by the tests).
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class Replica:
    rank: int
    local_rank: int
    world: int

    @property
    def is_root(self) -> bool:
        return self.rank == 0


def init_from_env(backend: str | None = None) -> Replica:
    """Reads RANK / LOCAL_RANK / WORLD_SIZE (torchrun's variables); single process if absent."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        be = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        if be == "nccl":
            torch.cuda.set_device(local)
        dist.init_process_group(backend=be, rank=rank, world_size=world)
    return Replica(rank, local, world)


def shard_range(total: int, rank: int, world: int) -> tuple[int, int]:
    """[begin, end) of `total` independent units owned by `rank`: contiguous, sizes differ by at most 1."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world}")
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def barrier(rep: Replica) -> None:
    if rep.world > 1:
        dist.barrier()


def max_over_ranks(rep: Replica, value: float, device: str | None = None) -> float:
    """The slowest rank's value (every multi-GPU time is reported as the max over ranks)."""
    if rep.world == 1:
        return float(value)
    dev = device or ("cuda" if dist.get_backend() == "nccl" else "cpu")
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(rep: Replica, value: float, device: str | None = None) -> float:
    if rep.world == 1:
        return float(value)
    dev = device or ("cuda" if dist.get_backend() == "nccl" else "cpu")
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def shutdown(rep: Replica) -> None:
    if rep.world > 1 and dist.is_initialized():
        dist.destroy_process_group()
