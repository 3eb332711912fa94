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


class _WireTensor:
    """A CPU tensor on its way through the message broadcast, carried as a numpy array (numpy arrays pickle an order of
    magnitude faster than tensors, and a render call's pose is all the message usually holds)."""
    __slots__ = ("array",)

    def __init__(self, array):
        self.array = array


def _to_wire(obj):
    if torch.is_tensor(obj) and obj.device.type == "cpu" and not obj.requires_grad and obj.dtype != torch.bfloat16:
        return _WireTensor(obj.numpy())
    if type(obj) is tuple:                 # plain containers only: subclasses (named tuples, ...) travel as they are
        return tuple(_to_wire(o) for o in obj)
    if type(obj) is list:
        return [_to_wire(o) for o in obj]
    if type(obj) is dict:
        return {k: _to_wire(v) for k, v in obj.items()}
    return obj


def _from_wire(obj):
    if isinstance(obj, _WireTensor):
        return torch.from_numpy(obj.array)
    if type(obj) is tuple:
        return tuple(_from_wire(o) for o in obj)
    if type(obj) is list:
        return [_from_wire(o) for o in obj]
    if type(obj) is dict:
        return {k: _from_wire(v) for k, v in obj.items()}
    return obj


_MESSAGE_BYTES = 4096           # user arguments of a render call (a pose, a few numbers) pickle to under a kilobyte
_MESSAGE_BUF = None             # reused staging buffer: 8-byte length + payload


def _broadcast_user_inputs_message(inputs=None, src: int = 0):
    """Broadcast the rank-0 user arguments (a picklable python object) over the gloo group.

    One fixed-size byte broadcast carries an 8-byte length and the pickled arguments; ``broadcast_object_list`` costs two
    collectives, a size negotiation and tensor pickling per call (1.1 ms between two ranks, 1.6 ms between eight, against
    0.25 / 0.57 ms this way), which is a large part of a multi-GPU frame.  Arguments that do not fit take the object broadcast; every rank
    learns that from the length field."""
    import pickle

    import numpy as np

    global _MESSAGE_BUF
    if _MESSAGE_BUF is None:
        _MESSAGE_BUF = torch.zeros(8 + _MESSAGE_BYTES, dtype=torch.uint8)
    buf = _MESSAGE_BUF
    raw = buf.numpy()                               # shares memory with the tensor
    ctx = CommContext()
    me = ctx.get_local_rank(CommMode.MESSAGE_TRANSFER)
    if me == src:
        data = pickle.dumps(_to_wire(inputs), protocol=pickle.HIGHEST_PROTOCOL)
        n = len(data) if len(data) <= _MESSAGE_BYTES else -1
        raw[:8].view(np.int64)[0] = n
        if n >= 0:
            raw[8:8 + n] = np.frombuffer(data, dtype=np.uint8)
    dist.broadcast(buf, src=_global_rank(CommMode.MESSAGE_TRANSFER, src), group=_group(CommMode.MESSAGE_TRANSFER))
    n = int(raw[:8].view(np.int64)[0])
    if n < 0:
        box = [inputs]
        broadcast_object_list(box, src=src, comm_mode=CommMode.MESSAGE_TRANSFER)
        return box[0]
    if me == src:
        return inputs
    return _from_wire(pickle.loads(raw[8:8 + n].tobytes()))
