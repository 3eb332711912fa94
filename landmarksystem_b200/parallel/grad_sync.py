"""Gradient synchronisation for replicated parameters.

The reference wraps models in ``DistributedDataParallel(find_unused_parameters=True)`` and re-creates
the wrapper whenever parameters are replaced (grid upsampling; benchmarks/nerf/gridnerf/
gridnerf_trainer.py:120-123, 447-460).  Here synchronisation is an explicit step between backward
and the optimiser: it works on whatever parameters exist at that moment (nothing to re-wrap), on
fp32 ``.grad`` tensors as well as on the persistent gradient sinks of the fused optimiser, and
supports SUM (branch parallel: each rank holds a partial sum over its own samples) or MEAN
(data parallel) semantics.  Small tensors are coalesced into one flat bucket.
"""
from __future__ import annotations

from typing import Iterable, List

import torch
import torch.distributed as dist


def _grad_of(p: torch.Tensor):
    sink = getattr(p, "_lmb_grad_sink", None)
    return sink if sink is not None else p.grad


class _P2PSmallAllReduce:
    """All-reduce of a flat fp32 vector through peer-mapped staging buffers: one kernel copies the vector into this
    rank's staging buffer and raises its flag on every peer, a second kernel waits for all flags and sums the staging
    buffers with plain peer loads.  No library collective and no barrier launch is involved, so the call is a fixed
    pair of kernel launches that can be recorded in a CUDA graph."""

    def __init__(self, capacity: int, group=None):
        from ctypes import c_float, c_int, c_longlong

        from ..comm.symmetric import SymmetricBuffer
        from ..ops import native
        from .zero_adam import _table

        P = native.P
        native.register_signature("lmb_allreduce_small_p2p", [P, P, P, P, P, P, c_int, c_int, c_longlong, c_longlong, P,
                                                               c_float, P, P])
        self.capacity = (capacity + 3) // 4 * 4
        self.off_flags = self.capacity * 4 * 2                    # two staging buffers (epoch parity), then the flag words
        self.buf = SymmetricBuffer(self.off_flags + 256, group)
        self.table = _table(self.buf.peer_table(0))
        self.flags_table = _table(self.buf.peer_table(self.off_flags))
        self.state = torch.zeros(4, dtype=torch.int32, device=self.buf.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.buf.device)
        self.native = native
        if self.buf.world > 1:
            dist.barrier(group)              # every rank has mapped the staging buffers before the first flag is raised

    def __call__(self, flat: torch.Tensor, scale: float) -> torch.Tensor:
        n = flat.numel()
        n4 = (n + 3) // 4 * 4
        assert n4 <= self.capacity
        src = flat.contiguous().float()
        if n4 > n:
            src = torch.nn.functional.pad(src, (0, n4 - n))
        out = torch.empty(n4, device=flat.device, dtype=torch.float32)
        nat = self.native
        nat.check(nat.lib().lmb_allreduce_small_p2p(src.data_ptr(), self.table, self.flags_table, self.buf.local_ptr,
                                                    self.buf.local_ptr + self.off_flags, self.state.data_ptr(), self.buf.rank,
                                                    self.buf.world, n4, self.capacity, out.data_ptr(), float(scale),
                                                    self.status.data_ptr(), nat.stream_ptr()), "allreduce_small_p2p")
        return out[:n]

    def check(self) -> None:
        code = int(self.status.item())
        if code:
            raise RuntimeError(f"small all-reduce: the wait for rank {code - 500} ran out")

    def close(self) -> None:
        """Collective teardown (every rank of the group calls it at the same point): no peer may still address the
        staging buffer when it is unmapped and freed."""
        if self.buf is None:
            return
        if dist.is_initialized() and self.buf.world > 1:
            dist.barrier(self.buf.group)
        torch.cuda.synchronize()
        if dist.is_initialized() and self.buf.world > 1:
            dist.barrier(self.buf.group)
        self.buf.close()
        self.buf = None


class GradSynchronizer:
    """``p2p_small``: on CUDA, coalesced small gradients go through :class:`_P2PSmallAllReduce` instead of the
    process group's collective (same result; graph-capturable, no library launch)."""

    def __init__(self, group=None, average: bool = True, bucket_elems: int = 1 << 22, p2p_small: bool = False):
        self.group, self.average, self.bucket_elems = group, average, bucket_elems
        self.p2p_small = p2p_small
        self._p2p = None

    def world(self) -> int:
        return dist.get_world_size(self.group) if dist.is_initialized() else 1

    @torch.no_grad()
    def sync(self, params: Iterable[torch.Tensor]) -> None:
        world = self.world()
        if world == 1:
            return
        small: List[torch.Tensor] = []
        for p in params:
            g = _grad_of(p)
            if g is None:
                # a parameter unused on this rank still has to take part in the collective
                g = torch.zeros_like(p, dtype=torch.float32)
                if getattr(p, "_lmb_grad_sink", None) is None:
                    p.grad = g
            if g.numel() >= self.bucket_elems:
                dist.all_reduce(g, group=self.group)
                if self.average:
                    g.div_(world)
            else:
                small.append(g)
        if small:
            flat = torch.cat([g.reshape(-1) for g in small])
            if self.p2p_small and flat.is_cuda:
                if self._p2p is None or self._p2p.capacity < flat.numel():
                    if self._p2p is not None:
                        self._p2p.close()            # same parameter sizes on every rank: all ranks regrow together
                    self._p2p = _P2PSmallAllReduce(max(flat.numel(), 1 << 16), self.group)
                flat = self._p2p(flat.float(), 1.0 / world if self.average else 1.0)
            else:
                dist.all_reduce(flat, group=self.group)
                if self.average:
                    flat.div_(world)
            off = 0
            for g in small:
                g.copy_(flat[off:off + g.numel()].view_as(g))
                off += g.numel()
