"""Model-parallel / data-parallel group algebra for training (reference:
landmark/nerf_components/components_convertor/comm_groups.py:19-97).

``mp_degree = nx * ny`` (branch parallel) or ``channel_parallel_size``; model-parallel groups are
contiguous rank blocks, data-parallel groups are strided by ``mp_degree``.
"""
from __future__ import annotations

from typing import List, Tuple

import torch.distributed as dist


def mp_degree_of(config) -> int:
    if getattr(config, "branch_parallel", False):
        nx, ny = config.plane_division
        return int(nx) * int(ny)
    if getattr(config, "channel_parallel", False):
        return int(config.channel_parallel_size or 1)
    return 1


def group_layout(world_size: int, mp_degree: int) -> Tuple[List[List[int]], List[List[int]]]:
    """Pure rank lists: ``(mp_groups, dp_groups)``."""
    assert world_size % mp_degree == 0, "world size must be a multiple of the model-parallel degree"
    n_mp_groups = world_size // mp_degree
    mp_groups = [list(range(g * mp_degree, (g + 1) * mp_degree)) for g in range(n_mp_groups)]
    dp_groups = [[off + j * mp_degree for j in range(n_mp_groups)] for off in range(mp_degree)]
    return mp_groups, dp_groups


def init_train_groups(config) -> None:
    """Create the groups collectively and record this rank's membership on ``config``:
    ``dp_group, dp_rank, num_mp_groups, mp_group, mp_rank`` (and ``dp_size``, ``mp_size``)."""
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    degree = mp_degree_of(config)
    if world > 1 and degree > 1 and not getattr(config, "model_parallel_and_DDP", False):
        assert world == degree, f"model parallel degree {degree} needs world size {degree}, got {world}"
    mp_groups, dp_groups = group_layout(world, degree)
    config.num_mp_groups = len(mp_groups)
    config.mp_size, config.dp_size = degree, len(mp_groups)
    config.mp_group = config.dp_group = None
    config.mp_rank, config.dp_rank = rank % degree, rank // degree
    if not dist.is_initialized() or world == 1:
        return
    for ranks in mp_groups:
        group = dist.new_group(ranks)
        if rank in ranks:
            config.mp_group, config.mp_rank = group, ranks.index(rank)
    for ranks in dp_groups:
        group = dist.new_group(ranks)
        if rank in ranks:
            config.dp_group, config.dp_rank = group, ranks.index(rank)
