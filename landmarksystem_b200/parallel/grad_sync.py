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


class GradSynchronizer:
    def __init__(self, group=None, average: bool = True, bucket_elems: int = 1 << 22):
        self.group, self.average, self.bucket_elems = group, average, bucket_elems

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
            dist.all_reduce(flat, group=self.group)
            if self.average:
                flat.div_(world)
            off = 0
            for g in small:
                g.copy_(flat[off:off + g.numel()].view_as(g))
                off += g.numel()
