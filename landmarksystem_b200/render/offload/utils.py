"""Helpers of the dynamic-loading stack (reference: landmark/render/parameter_loader/utils.py:13-435)."""
from __future__ import annotations

import fnmatch
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ...utils import MERGE_TYPE_STR
from ..types import MergeType


def calculate_block_neighbours(block_idx: int, plane_split: Sequence[int], local_plane_split: Sequence[int]) -> List[int]:
    """Global ids (row-major, ``bx * ny + by``) of the ``local_plane_split`` window around ``block_idx``,
    shifted where necessary so that it stays inside the ``plane_split`` grid."""
    nx, ny = int(plane_split[0]), int(plane_split[1])
    lx, ly = min(int(local_plane_split[0]), nx), min(int(local_plane_split[1]), ny)
    bx, by = int(block_idx) // ny, int(block_idx) % ny
    x0 = min(max(bx - lx // 2, 0), nx - lx)
    y0 = min(max(by - ly // 2, 0), ny - ly)
    return [(x0 + i) * ny + (y0 + j) for i in range(lx) for j in range(ly)]


def assign_block_to_pose(pose: torch.Tensor, aabb: torch.Tensor, plane_split: Sequence[int]) -> int:
    """Block under a camera-to-world pose's translation."""
    xy = pose[:2, 3] if pose.dim() == 2 else pose[:2]
    width = (aabb[1, :2] - aabb[0, :2]) / torch.tensor(list(plane_split), dtype=aabb.dtype, device=aabb.device)
    idx = torch.floor((xy.to(aabb.device) - aabb[0, :2]) / width)
    bx = int(idx[0].clamp(0, plane_split[0] - 1))
    by = int(idx[1].clamp(0, plane_split[1] - 1))
    return bx * int(plane_split[1]) + by


def match(key: str, table: Dict[str, object]) -> Optional[str]:
    """Find the merge-config entry for a state-dict key (entries may contain ``*`` wildcards)."""
    if key in table:
        return key
    for pattern in table:
        if "*" in pattern and fnmatch.fnmatchcase(key, pattern):
            return pattern
    return None


def get_merge_type(key: str, merge_config: Dict[str, object]) -> MergeType:
    """Merge type that applies to ``key``: the ``merge_type`` entry of the owning component."""
    parts = key.split(".")
    for depth in range(len(parts) - 1, -1, -1):
        name = ".".join(parts[:depth] + [MERGE_TYPE_STR])
        if name in merge_config:
            return MergeType(merge_config[name])
    return MergeType.Evenly


def mergeable_keys(merge_config: Dict[str, object], state_dict: Dict[str, torch.Tensor]) -> Dict[str, Tuple[str, object]]:
    """``{state key: (pattern, merge dim)}`` for every key the merge config covers."""
    table = {k: v for k, v in merge_config.items() if not k.endswith(MERGE_TYPE_STR)}
    out = {}
    for key in state_dict:
        pattern = match(key, table)
        if pattern is not None:
            out[key] = (pattern, table[pattern])
    return out


def split_tensor_into_block(key: str, dim, tensor: torch.Tensor, merge_type: MergeType, block_num: int,
                            split_sizes: Optional[Sequence[int]] = None) -> List[torch.Tensor]:
    if merge_type is MergeType.Evenly:
        assert tensor.shape[dim] % block_num == 0, f"{key}: dim {dim} of {tuple(tensor.shape)} is not {block_num} blocks"
        return list(torch.chunk(tensor, block_num, dim=dim))
    if merge_type is MergeType.Unevenly:
        assert split_sizes is not None, f"{key}: uneven merge needs per-block sizes"
        return list(torch.split(tensor, list(split_sizes), dim=dim))
    raise ValueError(f"{key}: list-merged parameters are addressed by key, not split")


def list_key_for_block(key: str, block_idx: int) -> Optional[str]:
    """For list-merged parameters (``...{i}.params``) return the canonical per-window key of block i."""
    parts = key.split(".")
    for i, p in enumerate(parts):
        if p.isdigit():
            return ".".join(parts[:i] + ["{}"] + parts[i + 1:]) if int(p) == block_idx else None
    return None


def search_maximum_memory_used_per_param(blocks, plane_split, local_plane_split) -> Dict[str, int]:
    """Largest per-parameter element count over all windows (uneven blocks differ in size)."""
    nx, ny = plane_split
    best: Dict[str, int] = {}
    for b in range(nx * ny):
        window = calculate_block_neighbours(b, plane_split, local_plane_split)
        sizes: Dict[str, int] = {}
        for w in window:
            for key, t in blocks[w].state_dict.items():
                sizes[key] = sizes.get(key, 0) + t.numel()
        for key, n in sizes.items():
            best[key] = max(best.get(key, 0), n)
    return best
