"""Partitioning of the quantized GEMM path over the GPUs of one node (one process per GPU).

Rows of A / dst (and convolution batches) are independent, so they are split with no exchange at all.  The
large linear layer is split by columns of B instead: every rank produces dst[:, n0:n1] and the column blocks
are all-gathered (NCCL on GPUs, gloo in the CPU tests).  torch.distributed is used as plumbing only.
"""
from __future__ import annotations


def split_even(total: int, world: int, rank: int, align: int = 1):
    """[begin, end) of rank's share of `total` items, in multiples of `align` (the last rank takes the rest).
    Shares differ by at most one alignment unit."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad world / rank")
    units = -(-total // align)
    base, extra = divmod(units, world)
    begin_u = rank * base + min(rank, extra)
    end_u = begin_u + base + (1 if rank < extra else 0)
    return min(begin_u * align, total), min(end_u * align, total)


def row_shard(M: int, world: int, rank: int):
    """Rows of A / dst owned by `rank` (configs 2-4: no collective)."""
    return split_even(M, world, rank, 1)


def batch_shard(B: int, world: int, rank: int):
    """Images of a convolution / network batch owned by `rank`."""
    return split_even(B, world, rank, 1)


def column_shard(N: int, world: int, rank: int, align: int = 256):
    """Columns of B / dst owned by `rank` (config 5), aligned to the 256-column tile of the GEMM kernel."""
    return split_even(N, world, rank, align)


def allgather_columns(local, N: int, world: int, rank: int, group=None, align: int = 256):
    """All-gather of column blocks: `local` is this rank's [M, n_local] block (a torch tensor on the backend's
    device); returns the full [M, N] matrix on every rank.  Blocks may have different widths: they are padded
    to the widest one for the collective and trimmed when re-tiled."""
    import torch
    import torch.distributed as dist
    M = local.shape[0]
    widths = [column_shard(N, world, r, align) for r in range(world)]
    wmax = max(e - b for b, e in widths)
    staging = local
    if local.shape[1] != wmax:
        staging = torch.zeros((M, wmax), dtype=local.dtype, device=local.device)
        staging[:, :local.shape[1]] = local
    flat = torch.empty((world * M, wmax), dtype=local.dtype, device=local.device)  # blocks stacked along rows
    dist.all_gather_into_tensor(flat, staging.contiguous(), group=group)
    gathered = flat.view(world, M, wmax)
    out = torch.empty((M, N), dtype=local.dtype, device=local.device)
    for r, (b, e) in enumerate(widths):
        out[:, b:e] = gathered[r, :, :e - b]
    return out
