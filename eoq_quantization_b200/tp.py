"""Row sharding of an entropy-coded linear layer over the GPUs of one node.

Every output row is an independent dot product and every tile an independent set of rANS
streams, so a layer shards by output rows with nothing to exchange while it computes: rank
r keeps only the tiles (and scales) of rows [r*N/g, (r+1)*N/g), x is replicated, and the
output slices meet once per layer in an all-gather (NCCL over NVLink on GPUs, gloo in the
CPU tests).  No reduction is needed.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def shard_rows(n_rows: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, equal row ranges; the row count must divide evenly so that the gather is a
    plain all-gather of equal slices."""
    if n_rows % world:
        raise ValueError(f"{n_rows} rows do not split evenly over {world} ranks")
    per = n_rows // world
    return rank * per, (rank + 1) * per


def gather_rows(local: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """local: (..., N/g) slice of this rank -> (..., N) on every rank, slices in rank order."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return local
    flat = local.reshape(-1, local.shape[-1]).contiguous()
    out = torch.empty((world * flat.shape[0], flat.shape[1]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, flat, group=group)            # rank-major concatenation along dim 0
    out = out.view(world, flat.shape[0], flat.shape[1])
    if flat.shape[0] == 1:
        return out.reshape(*local.shape[:-1], world * local.shape[-1])
    return out.permute(1, 0, 2).reshape(*local.shape[:-1], world * local.shape[-1])


class RowShardedLinear:
    """One rank's share of y = x W^T: a local weight (anything with ``gemv(x) -> (..., N/g)``)
    plus the layer-boundary all-gather."""

    def __init__(self, local_weight, n_rows: int, group: Optional[dist.ProcessGroup] = None):
        self.local = local_weight
        self.n_rows = n_rows
        self.group = group

    def forward_local(self, x: torch.Tensor) -> torch.Tensor:
        return self.local.gemv(x)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return gather_rows(self.local.gemv(x), self.group)
