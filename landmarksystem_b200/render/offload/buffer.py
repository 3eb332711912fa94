"""Device-resident window of blocks (reference: landmark/render/parameter_loader/buffer.py:1-54).
For every streamed parameter the buffer holds one tensor whose leading dimension is the slot inside
the window."""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch

BUFFER_SIZE = 2  # double buffering: render from one window while the next one streams in


class Buffer:
    def __init__(self, local_plane_split: Sequence[int], state_dict: Dict[str, torch.Tensor]):
        self.local_plane_split = [int(v) for v in local_plane_split]
        self.local_block_idxes: List[int] = []
        self.state_dict = state_dict

    @property
    def n_slots(self) -> int:
        return self.local_plane_split[0] * self.local_plane_split[1]


def create_buffers(blocks, local_plane_split, device, count: int = BUFFER_SIZE, symmetric_group=None) -> List[Buffer]:
    """``symmetric_group``: allocate every window as one peer-mapped allocation (same layout on every rank of the
    group) so that ranks can store pieces of a block straight into each other's windows over NVLink; the buffer then
    carries ``symm`` (the allocation) and ``offsets`` (byte offset of every tensor inside it)."""
    n_slots = int(local_plane_split[0]) * int(local_plane_split[1])
    proto = blocks[0].state_dict
    shapes = {}
    for key, t in proto.items():
        lead = t.shape[0] if t.dim() > 1 and t.shape[0] == 1 else None
        shapes[key] = (n_slots, *t.shape[1:]) if lead == 1 else (n_slots, *t.shape)
    out = []
    for _ in range(count):
        state = {}
        if symmetric_group is None:
            for key, t in proto.items():
                state[key] = torch.empty(shapes[key], dtype=t.dtype, device=device)
            out.append(Buffer(local_plane_split, state))
            continue
        from ...comm.symmetric import SymmetricBuffer

        offsets, total = {}, 0
        for key, t in proto.items():
            offsets[key] = total
            nbytes = t.element_size() * int(torch.tensor(shapes[key]).prod())
            total += (nbytes + 255) // 256 * 256
        symm = SymmetricBuffer(total, symmetric_group)
        for key, t in proto.items():
            state[key] = symm.view(offsets[key], shapes[key], t.dtype)
        buf = Buffer(local_plane_split, state)
        buf.symm, buf.offsets = symm, offsets
        out.append(buf)
    return out
