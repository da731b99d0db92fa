"""Multi-GPU plumbing for the W4A4 linear path.

The path shards along the token/batch dimension M with no exchange: quantisation groups are
per row, GEMM rows are independent, the low-rank branch and every fused epilogue are per row.
So the scale-out is one process per GPU, each running the whole path on its rows; the only
collectives are control-plane ones (a barrier around timing, a MAX over ranks of the measured
time, an optional gather of outputs for checks).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def row_shard(total_rows: int, world_size: int, rank: int, align: int = 256) -> tuple[int, int]:
    """Contiguous, ``align``-aligned split of ``total_rows`` rows; the last non-empty shard takes
    the ragged tail.  Returns [start, stop)."""
    if not 0 <= rank < world_size:
        raise ValueError("rank out of range")
    blocks = (total_rows + align - 1) // align
    base, extra = divmod(blocks, world_size)
    b0 = rank * base + min(rank, extra)
    b1 = b0 + base + (1 if rank < extra else 0)
    return min(b0 * align, total_rows), min(b1 * align, total_rows)


def init_from_env(backend: str | None = None) -> tuple[int, int, int]:
    """Initialise torch.distributed from the torchrun environment.  Returns (rank, world, local_rank);
    (0, 1, 0) without initialising anything when WORLD_SIZE is absent or 1."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(local)
            dist.init_process_group(backend=backend, rank=rank, world_size=world, device_id=torch.device("cuda", local))
        else:
            dist.init_process_group(backend=backend, rank=rank, world_size=world)
    return rank, world, local


def shutdown() -> None:
    """Tear the process group down (NCCL warns when a process exits with it alive)."""
    if dist.is_initialized():
        dist.destroy_process_group()


def barrier() -> None:
    if dist.is_initialized():
        dist.barrier()


def max_over_ranks(value: float, device: torch.device | str = "cpu") -> float:
    if not dist.is_initialized():
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_rows(local: torch.Tensor, total_rows: int, align: int = 256) -> torch.Tensor:
    """All-gather row shards produced with :func:`row_shard` back into [total_rows, ...]."""
    if not dist.is_initialized():
        return local
    world = dist.get_world_size()
    sizes = [row_shard(total_rows, world, r, align) for r in range(world)]
    cap = max(b - a for a, b in sizes)
    pad = torch.zeros((cap,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    pad[: local.shape[0]] = local
    bufs = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(bufs, pad)
    return torch.cat([b[: e - s] for b, (s, e) in zip(bufs, sizes)], dim=0)
