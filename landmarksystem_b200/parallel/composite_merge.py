"""Cross-GPU ordered alpha-composite for model-parallel rendering.

Each rank renders, for ALL rays of the frame, only the samples that fall into its resident spatial
blocks and writes one partial per ray ``(rgb, T, depth, acc, t_entry)`` into a symmetric buffer.
``merge`` then runs one kernel per rank (``csrc/fused_comm.cu: composite_merge_p2p``): rank r pulls the
P partials of its slice of rays from peer memory, orders them by entry distance, composites them and
stores the finished pixels into the root's (or every rank's) image buffer.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..comm.symmetric import PeerBarrier, SymmetricBuffer
from ..ops import native
from .zero_adam import _table

native.register_signature("lmb_composite_merge_p2p", [native.P, native.P, ctypes.c_longlong, ctypes.c_int, ctypes.c_int,
                                                       ctypes.c_int, ctypes.c_float, native.P])


def merge_reference(partials: torch.Tensor, bg: float = 0.0) -> torch.Tensor:
    """``partials [P, R, 8]`` -> ``[R, 6]`` (rgb, T, depth, acc): plain PyTorch statement."""
    order = torch.argsort(partials[..., 6], dim=0)                       # [P, R]
    sorted_p = torch.gather(partials, 0, order[..., None].expand_as(partials))
    T = torch.ones(partials.shape[1], device=partials.device)
    out = torch.zeros(partials.shape[1], 6, device=partials.device)
    for k in range(partials.shape[0]):
        seg = sorted_p[k]
        out[:, 0:3] += T[:, None] * seg[:, 0:3]
        out[:, 4] += T * seg[:, 4]
        out[:, 5] += T * seg[:, 5]
        T = T * seg[:, 3]
    out[:, 0:3] += T[:, None] * bg
    out[:, 3] = T
    return out


def pack_partial(rgb, trans, depth, acc, t_entry) -> torch.Tensor:
    """Assemble the ``[R, 8]`` partial record; rays that miss every local block use ``t_entry = +inf``."""
    pad = torch.zeros_like(trans)
    return torch.stack((rgb[:, 0], rgb[:, 1], rgb[:, 2], trans, depth, acc, t_entry, pad), dim=-1).contiguous()


class CompositeMerger:
    def __init__(self, max_rays: int, group=None):
        self.max_rays = max_rays
        self.buf = SymmetricBuffer(max_rays * (8 + 6) * 4, group)
        self.partial = self.buf.view(0, (max_rays, 8), torch.float32)
        self.out = self.buf.view(max_rays * 32, (max_rays, 6), torch.float32)
        self.partial_table = _table(self.buf.peer_table(0))
        self.out_table = _table(self.buf.peer_table(max_rays * 32))
        self.barrier = PeerBarrier(group)
        self.rank, self.world = self.buf.rank, self.buf.world

    def merge(self, partial: torch.Tensor, bg: float = 0.0, root: int = -1) -> torch.Tensor:
        """``partial [R, 8]`` of this rank -> merged ``[R, 6]`` (valid on ``root``, or everywhere if -1)."""
        R = partial.shape[0]
        assert R <= self.max_rays
        self.partial[:R].copy_(partial)
        self.barrier()                                   # all partials are in place
        native.check(native.lib().lmb_composite_merge_p2p(self.partial_table, self.out_table, R, self.rank, self.world,
                                                          root, float(bg), native.stream_ptr()), "composite_merge_p2p")
        self.barrier()                                   # all slices have been written
        return self.out[:R]
