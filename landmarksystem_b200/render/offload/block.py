"""One spatial block of the scene held in pinned host memory (reference:
landmark/render/parameter_loader/block.py:1-26)."""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import torch

from ..types import MergeType
from .utils import get_merge_type, mergeable_keys, split_tensor_into_block


class Block:
    def __init__(self, block_idx: int, coord, aabb=None, state_dict: Optional[Dict[str, torch.Tensor]] = None):
        self.block_idx, self.coord, self.aabb = block_idx, coord, aabb
        self.state_dict: Dict[str, torch.Tensor] = state_dict or {}

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.state_dict.values())


def create_blocks(merge_config, merged_state_dict, plane_split: Sequence[int], to_internal: Optional[Callable] = None,
                  dtype: Optional[torch.dtype] = None, pin_memory: bool = True) -> List[Block]:
    """Split a merged (block-stacked) checkpoint into per-block host tensors.

    ``to_internal(key, tensor)`` converts a one-block slice from the checkpoint layout to the layout the
    model keeps in memory (e.g. channels-last planes), so that swapping a buffer in is a pointer update.
    Keys of list-merged parameters are normalised to ``...{}....`` (the slot index is filled in later)."""
    nx, ny = int(plane_split[0]), int(plane_split[1])
    n = nx * ny
    blocks = [Block(b, (b // ny, b % ny)) for b in range(n)]
    for key, (pattern, dim) in mergeable_keys(merge_config, merged_state_dict).items():
        mtype = get_merge_type(key, merge_config)
        tensor = merged_state_dict[key]
        if mtype is MergeType.List:
            parts = key.split(".")
            pos = next(i for i, p in enumerate(parts) if p.isdigit())
            b = int(parts[pos])
            if b >= n:
                continue
            pieces = {b: tensor}
            norm_key = ".".join(parts[:pos] + ["{}"] + parts[pos + 1:])
        else:
            pieces = dict(enumerate(split_tensor_into_block(key, dim, tensor, mtype, n)))
            norm_key = key
        for b, piece in pieces.items():
            piece = to_internal(key, piece) if to_internal is not None else piece
            piece = piece.contiguous()
            if dtype is not None and piece.is_floating_point():
                piece = piece.to(dtype)
            if pin_memory and torch.cuda.is_available():
                piece = piece.pin_memory()
            blocks[b].state_dict[norm_key] = piece
    return blocks
