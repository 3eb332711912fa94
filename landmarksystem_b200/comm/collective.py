"""Collective wrappers keyed by parallel mode (reference: landmark/communicator/collective.py:13-155)."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from .comm_context import CommContext
from .modes import CommMode


def _group(mode: CommMode):
    return CommContext().get_group(mode)


def _global_rank(mode: CommMode, group_rank: int) -> int:
    return CommContext().get_ranks_in_group(mode)[group_rank]


def scatter(tensor, scatter_list: Optional[List[torch.Tensor]] = None, src: int = 0,
            comm_mode: CommMode = CommMode.GLOBAL, async_op: bool = False):
    """Scatter ``scatter_list`` from group-rank ``src`` into ``tensor``."""
    return dist.scatter(tensor, scatter_list, src=_global_rank(comm_mode, src), group=_group(comm_mode),
                        async_op=async_op)


def broadcast_object_list(object_list, src: int = 0, comm_mode: CommMode = CommMode.MESSAGE_TRANSFER, device=None):
    return dist.broadcast_object_list(object_list, src=_global_rank(comm_mode, src), group=_group(comm_mode),
                                      device=device)


def all_gather(output_tensor, input_tensor, comm_mode: CommMode = CommMode.GLOBAL, async_op: bool = False):
    """Gather equal-size tensors from the group into one pre-allocated ``output_tensor``."""
    return dist.all_gather_into_tensor(output_tensor, input_tensor, group=_group(comm_mode), async_op=async_op)


def all_reduce(tensor, op=dist.ReduceOp.SUM, comm_mode: CommMode = CommMode.GLOBAL, async_op: bool = False):
    return dist.all_reduce(tensor, op=op, group=_group(comm_mode), async_op=async_op)


def broadcast(tensor, src: int = 0, comm_mode: CommMode = CommMode.GLOBAL, async_op: bool = False):
    return dist.broadcast(tensor, src=_global_rank(comm_mode, src), group=_group(comm_mode), async_op=async_op)


def gather(tensor, gather_list=None, dst: int = 0, comm_mode: CommMode = CommMode.GLOBAL, async_op: bool = False):
    return dist.gather(tensor, gather_list, dst=_global_rank(comm_mode, dst), group=_group(comm_mode),
                       async_op=async_op)


def _broadcast_user_inputs_message(inputs=None, src: int = 0):
    """Broadcast the rank-0 user arguments (a picklable python object) over the gloo group."""
    box = [inputs]
    broadcast_object_list(box, src=src, comm_mode=CommMode.MESSAGE_TRANSFER)
    return box[0]
