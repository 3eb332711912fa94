"""Differentiable collectives (reference: landmark/nerf_components/utils/comm_utils.py:5-40).

No host synchronisation is issued around the collectives (the reference calls
``torch.cuda.synchronize()`` after every all-gather)."""
from __future__ import annotations

import torch
import torch.distributed as dist


class AllGather(torch.autograd.Function):
    """Concatenate equal-shaped tensors of the group on dim 0; backward keeps the local slice."""

    @staticmethod
    def forward(ctx, tensor, group=None):
        world = dist.get_world_size(group)
        ctx.rank, ctx.n = dist.get_rank(group), tensor.shape[0]
        out = torch.empty((world * tensor.shape[0], *tensor.shape[1:]), dtype=tensor.dtype, device=tensor.device)
        dist.all_gather_into_tensor(out, tensor.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        return grad[ctx.rank * ctx.n:(ctx.rank + 1) * ctx.n], None


class AllReduce(torch.autograd.Function):
    """Sum over the group; backward sums the gradients as well."""

    @staticmethod
    def forward(ctx, tensor, group=None):
        ctx.group = group
        out = tensor.clone()
        dist.all_reduce(out, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        grad = grad.clone()
        dist.all_reduce(grad, group=ctx.group)
        return grad, None


class _AllReduceLocalGrad(torch.autograd.Function):
    """Sum over the group in forward; identity in backward.  Used where every element is produced by
    exactly one rank (zeros elsewhere) and every rank computes the same downstream loss: the local
    contribution then receives exactly its own gradient."""

    @staticmethod
    def forward(ctx, tensor, group=None):
        out = tensor.clone()
        dist.all_reduce(out, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        return grad, None


def all_reduce_sum_local_grad(tensor: torch.Tensor, group=None) -> torch.Tensor:
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return tensor
    return _AllReduceLocalGrad.apply(tensor, group)
