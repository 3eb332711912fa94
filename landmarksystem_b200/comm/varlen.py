"""Variable-length all-gather without per-rank host syncs: sizes travel in one small all-gather,
payloads in one padded ``all_gather_into_tensor`` (the reference does a list all-gather preceded by
``.sum()`` host syncs per block mask, landmark/nerf_components/data/samples.py:283-309)."""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist


def all_gather_varlen(local: torch.Tensor, group=None) -> List[torch.Tensor]:
    """``local [n_r, W]`` on each rank -> list of ``[n_p, W]`` tensors, one per rank of the group."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return [local]
    world = dist.get_world_size(group)
    sizes = torch.zeros(world, dtype=torch.long, device=local.device)
    mine = torch.tensor([local.shape[0]], dtype=torch.long, device=local.device)
    dist.all_gather_into_tensor(sizes, mine, group=group)
    counts = sizes.tolist()
    cap = max(max(counts), 1)
    padded = torch.zeros((cap, *local.shape[1:]), dtype=local.dtype, device=local.device)
    padded[: local.shape[0]] = local.detach()
    out = torch.empty((world * cap, *local.shape[1:]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, padded, group=group)
    return [out[r * cap: r * cap + counts[r]] for r in range(world)]
