"""Ownership partition of a parameter set over the GPUs of one box (ZeRO-1 style) and the all-gather of
the updated weights that follows a step.

The reference is single-process (no collective anywhere in came_pytorch); this module is the one
distributed component around the step.  Tensors are independent units of the CAME step (clip RMS, row/col
means and absmax blocks are all per tensor, came_pytorch/CAME8bit.py:739-861), so each rank steps the whole
tensors it owns and no collective is needed inside the step.  Afterwards every rank needs every updated
weight: parameters live in ONE flat buffer ordered by owner, each owner's slice padded to the same length,
so a single in-place `all_gather_into_tensor` (ncclAllGather with sendbuff inside recvbuff) moves them.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

ALIGN_ELEMS = 128   # every tensor starts on a 256-byte boundary (bf16), keeping the 16-byte vector paths


def assign_owners(numels, world_size: int):
    """Greedy longest-processing-time assignment of tensors to ranks by element count.
    Deterministic: ties go to the lower tensor index, then to the lower rank."""
    if world_size <= 0:
        raise ValueError("world_size must be positive")
    order = sorted(range(len(numels)), key=lambda i: (-int(numels[i]), i))
    load = [0] * world_size
    owners = [0] * len(numels)
    for i in order:
        r = min(range(world_size), key=lambda k: (load[k], k))
        owners[i] = r
        load[r] += int(numels[i])
    return owners


def imbalance(numels, owners, world_size: int) -> float:
    """max rank load / mean rank load."""
    load = [0] * world_size
    for n, r in zip(numels, owners):
        load[r] += int(n)
    mean = sum(load) / world_size
    return max(load) / mean if mean > 0 else 1.0


class ShardedParams:
    """All parameters of a model as views into one flat buffer laid out for an in-place all-gather."""

    def __init__(self, shapes, dtype: torch.dtype, device, world_size: int, rank: int, owners=None):
        self.shapes = [tuple(s) for s in shapes]
        self.world_size, self.rank = int(world_size), int(rank)
        numels = [math.prod(s) for s in self.shapes]
        self.owners = list(owners) if owners is not None else assign_owners(numels, world_size)
        if len(self.owners) != len(self.shapes) or any(not 0 <= r < world_size for r in self.owners):
            raise ValueError("owners must give one rank in [0, world_size) per tensor")
        # offsets inside each owner's slice
        fill = [0] * world_size
        local_off = []
        for n, r in zip(numels, self.owners):
            local_off.append(fill[r])
            fill[r] += (n + ALIGN_ELEMS - 1) // ALIGN_ELEMS * ALIGN_ELEMS
        self.slice_len = max(max(fill), ALIGN_ELEMS)
        self.flat = torch.zeros(self.slice_len * world_size, dtype=dtype, device=device)
        self.views = []
        for shape, n, r, off in zip(self.shapes, numels, self.owners, local_off):
            start = r * self.slice_len + off
            self.views.append(self.flat[start:start + n].view(shape))
        self.owned = [i for i, r in enumerate(self.owners) if r == rank]

    def my_slice(self) -> torch.Tensor:
        return self.flat[self.rank * self.slice_len:(self.rank + 1) * self.slice_len]

    def all_gather(self, group=None, async_op: bool = False):
        """Every rank sends its slice and receives everybody else's, in place."""
        if self.world_size == 1:
            return None
        return dist.all_gather_into_tensor(self.flat, self.my_slice(), group=group, async_op=async_op)

    def gathered_bytes_per_rank(self) -> int:
        """Bytes each rank receives from its peers in one all-gather."""
        return (self.world_size - 1) * self.slice_len * self.flat.element_size()
