"""Row sharding of an evaluation across the GPUs of one box, and assembly of the sharded result.

Every benchmark graph is a set of independent output rows (rows of x and y for the fused reduce,
softmax lines, rows of A / X for the contractions, batch x heads for attention), so each rank
evaluates the same graph recorded at its shard's shape on its slice of the row-sharded inputs;
replicated operands (B, W, bias, scales) go to every rank. There is no collective on the data path.
`assemble` is the optional all-gather that puts the pieces back together over NCCL (or gloo on CPU);
the reference has no multi-device code, so this file has no counterpart there.
"""
from __future__ import annotations

import numpy as np


def row_range(n_rows: int, rank: int, world: int) -> tuple:
    """Contiguous block of rows owned by `rank`: sizes differ by at most one, earlier ranks get the extra row."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(n_rows, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_rows(arr: np.ndarray, rank: int, world: int, axis: int = 0) -> np.ndarray:
    lo, hi = row_range(arr.shape[axis], rank, world)
    idx = [slice(None)] * arr.ndim
    idx[axis] = slice(lo, hi)
    return np.ascontiguousarray(arr[tuple(idx)])


def assemble(local, n_rows: int, group=None):
    """All-gather row shards (a torch tensor whose dim 0 is this rank's rows) into the full tensor on
    every rank. Uneven shards are padded to the largest one for the collective and trimmed after."""
    import torch
    import torch.distributed as dist
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    sizes = [row_range(n_rows, r, world)[1] - row_range(n_rows, r, world)[0] for r in range(world)]
    if local.shape[0] != sizes[rank]:
        raise ValueError(f"rank {rank} holds {local.shape[0]} rows, its shard of {n_rows} is {sizes[rank]}")
    biggest = max(sizes)
    padded = local
    if local.shape[0] < biggest:
        pad = torch.zeros((biggest - local.shape[0],) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        padded = torch.cat([local, pad], 0)
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded.contiguous(), group=group)
    return torch.cat([p[:n] for p, n in zip(parts, sizes)], 0)
