"""Sharding of one evaluation across the GPUs of a box: rank r of `world` evaluates the part graph of
ku_graph_row_split (kurumi_b200/csrc/core/split.cc) on its slices of the row-wise inputs and on all of the
replicated ones (B, W, bias, scales). There is no collective on the data path; `assemble_cpu` is the host-side
all-gather used by the CPU tests (on a GPU the library's own ku_cuda_all_gather_rows runs over NCCL).
The reference has no multi-device code, so this file has no counterpart there."""
from __future__ import annotations

import numpy as np

from . import api


def slice_of(arr: np.ndarray, axis, rank: int, world: int) -> np.ndarray:
    """This rank's slice of an input: `axis` None = every rank needs all of it."""
    if axis is None:
        return arr
    if arr.shape[axis] % world:
        raise ValueError(f"extent {arr.shape[axis]} does not divide over {world} ranks")
    step = arr.shape[axis] // world
    idx = [slice(None)] * arr.ndim
    idx[axis] = slice(rank * step, (rank + 1) * step)
    return np.ascontiguousarray(arr[tuple(idx)])


def part_feeds(lib: api.Library, inputs, arrays: dict, rank: int, world: int) -> api.Feeds:
    """Feeds of the part graph from the whole host arrays {original input node: (array, dtype)}."""
    f = api.Feeds(lib)
    for orig, part, axis in inputs:
        arr, dt = arrays[orig]
        f.set(part, slice_of(arr, axis, rank, world), dt)
    return f


def assemble_cpu(local, group=None):
    """All-gather equal row shards (a torch tensor whose dim 0 is this rank's rows) into the whole, on every rank."""
    import torch
    import torch.distributed as dist
    parts = [torch.empty_like(local) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, local.contiguous(), group=group)
    return torch.cat(parts, 0)
