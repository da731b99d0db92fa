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


# ---------------------------------------------------------------------------------------------
# N-split variant: for a single image there are too few rows to shard, so the output columns are.
# ---------------------------------------------------------------------------------------------
def column_shard(total_cols: int, world_size: int, rank: int, align: int = 128) -> tuple[int, int]:
    """Contiguous split of the N output columns in units of ``align`` (128 = one block of the packed
    weight layouts, which are all N-block-major).  Returns [start, stop)."""
    if total_cols % align:
        raise ValueError(f"N ({total_cols}) must be a multiple of {align}")
    return row_shard(total_cols, world_size, rank, align)


def shard_linear_columns(module, world_size: int, rank: int):
    """The ``SVDQW4A4Linear`` that computes columns ``column_shard(N, world_size, rank)`` of ``module``.

    Every per-column tensor of the reference's packed layouts is N-block-major (``qweight``
    [N/128][K/64]..., ``wscales`` [N/128][K/G]..., ``proj_up`` [N/16][R/16]..., ``bias`` / ``wcscales``
    [N/128][128]; nunchaku/lora/flux/packer.py:187-398), so a shard is a contiguous byte range of each;
    ``smooth_factor``, ``proj_down`` and ``wtscale`` are replicated."""
    from .models.linear import SVDQW4A4Linear

    N, K = module.out_features, module.in_features
    n0, n1 = column_shard(N, world_size, rank)
    n = n1 - n0
    if n == 0:
        raise ValueError(f"rank {rank} of {world_size} gets no columns of N={N}")
    shard = SVDQW4A4Linear(
        K, n, rank=module.rank, bias=module.bias is not None, precision=module.precision,
        act_unsigned=module.act_unsigned, torch_dtype=module.torch_dtype, device=module.qweight.device,
    )
    G = K // module.group_size
    with torch.no_grad():
        shard.qweight.copy_(module.qweight.reshape(-1)[n0 * (K // 2): n1 * (K // 2)].view(n, K // 2))
        shard.wscales.view(torch.uint8).copy_(
            module.wscales.reshape(-1).view(torch.uint8).view(N, -1)[n0:n1].reshape(shard.wscales.view(torch.uint8).shape))
        shard.proj_up.copy_(module.proj_up[n0:n1])
        if module.bias is not None:
            shard.bias.copy_(module.bias[n0:n1])
        if module.wcscales is not None:
            shard.wcscales.copy_(module.wcscales[n0:n1])
            shard.wtscale.copy_(module.wtscale)
        shard.smooth_factor.copy_(module.smooth_factor)
        shard.smooth_factor_orig.copy_(module.smooth_factor_orig)
        shard.proj_down.copy_(module.proj_down)
    assert G * n == shard.wscales.numel()
    return shard


def gather_columns(local: torch.Tensor, total_cols: int, align: int = 128, group=None) -> torch.Tensor:
    """All-gather column shards ``[M, n_r]`` made with :func:`column_shard` into ``[M, total_cols]``.

    One collective (NCCL all-gather over NVLink on GPUs) into a ``[world, M, cap]`` buffer, then one strided copy
    that interleaves the ranks' slabs into rows; ``cap`` is the widest shard, narrower ones are padded."""
    if not dist.is_initialized():
        return local
    world = dist.get_world_size(group)
    spans = [column_shard(total_cols, world, r, align) for r in range(world)]
    cap = max(b - a for a, b in spans)
    M = local.shape[0]
    if local.shape[1] != cap:
        padded = local.new_zeros(M, cap)
        padded[:, : local.shape[1]] = local
        local = padded
    flat = torch.empty(world * M, cap, dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat, local.contiguous(), group=group)
    slab = flat.view(world, M, cap)
    if all(b - a == cap for a, b in spans):
        return slab.permute(1, 0, 2).reshape(M, total_cols)
    return torch.cat([slab[r, :, : b - a] for r, (a, b) in enumerate(spans)], dim=1)


class ColumnParallelW4A4Linear(torch.nn.Module):
    """N-split W4A4 linear for single-image calls: every rank quantises the (replicated) activations, runs the
    4-bit GEMM on its own column range of the weights and the ranks all-gather the bf16 result.  The quantiser
    output (8.6 MB at M=4608, K=3072) is cheaper to recompute than to broadcast."""

    def __init__(self, full, world_size: int | None = None, rank: int | None = None, group=None):
        super().__init__()
        if world_size is None:
            world_size = dist.get_world_size(group) if dist.is_initialized() else 1
        if rank is None:
            rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.group = group
        self.out_features = full.out_features
        self.in_features = full.in_features
        self.world_size, self.rank = world_size, rank
        self.local = shard_linear_columns(full, world_size, rank)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b, s, _ = x.shape
        y = self.local(x).view(b * s, -1)
        return gather_columns(y, self.out_features, group=self.group).view(b, s, self.out_features)
