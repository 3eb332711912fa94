"""Spatial-block all-to-all over peer memory.

``BlockDispatcher.query(payload, owner, fn, out_width)`` sends each row of ``payload`` to the rank that
owns it, runs ``fn`` there on the compacted rows (a differentiable callable - grid lookup + head - that
honours a device-side row count), and returns the results in the caller's row order.  Gradients w.r.t. the results travel the
reverse route and ``fn``'s backward runs on the owner, so grid gradients stay local to the owner.
CPU / single-rank calls degenerate to ``fn(payload)``.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_longlong
from typing import Callable

import torch
import torch.distributed as dist

from ..comm.symmetric import PeerBarrier, SymmetricBuffer
from ..ops import native
from .zero_adam import _table

P = native.P
native.register_signature("lmb_a2a_dispatch", [P, P, P, c_longlong, c_int, P, P, c_int, c_int, c_longlong, P, P, P, P])
native.register_signature("lmb_a2a_collect", [P, P, c_int, c_longlong, c_int, P, P, P, P, P, P])
native.register_signature("lmb_a2a_combine", [P, P, P, P, c_longlong, c_int, P, c_int, P])
native.register_signature("lmb_a2a_grad_dispatch", [P, P, P, P, c_longlong, c_int, P, c_int, c_int, c_longlong, P])
native.register_signature("lmb_a2a_grad_collect", [P, P, c_int, c_longlong, c_int, P, P])


class BlockDispatcher:
    """``cap`` = max rows one source may send to one owner; ``max_w`` / ``max_v`` = widest payload / result.

    Nothing on the host ever learns a row count: the owner-side buffers have the static worst-case size
    ``world * cap`` and every consumer takes the device-side count, so a query is a fixed sequence of
    launches (and can be recorded in a CUDA graph together with the rest of the step)."""

    def __init__(self, cap: int, max_w: int = 8, max_v: int = 4, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.cap, self.max_w, self.max_v = int(cap), max_w, max_v
        w = self.world
        self.off_inbox = 0
        record = (max_w + 1 + 3) // 4 * 4              # floats per inbox record: payload + slot, whole 16-byte words
        self.off_ginbox = self.off_inbox + w * cap * record * 4
        self.off_out = self.off_ginbox + w * cap * ((max_v + 3) // 4 * 4) * 4
        self.off_incoming = self.off_out + cap * max_v * 4
        total = self.off_incoming + 256
        self.buf = SymmetricBuffer(total, group)
        self.inbox_table = _table(self.buf.peer_table(self.off_inbox))
        self.ginbox_table = _table(self.buf.peer_table(self.off_ginbox))
        self.out_table = _table(self.buf.peer_table(self.off_out))
        self.incoming_table = _table(self.buf.peer_table(self.off_incoming))
        self.incoming = self.buf.view(self.off_incoming, (w,), torch.int32)
        dev = self.buf.device
        self.counts = torch.zeros(w, dtype=torch.int32, device=dev)
        self.overflow = torch.zeros(1, dtype=torch.int32, device=dev)
        self.barrier = PeerBarrier(group)

    @property
    def owner_rows(self) -> int:
        """Static row capacity of the owner-side tensors handed to ``fn``."""
        return self.world * self.cap

    def query(self, payload: torch.Tensor, owner: torch.Tensor, fn: Callable, out_width: int,
              count: torch.Tensor = None) -> torch.Tensor:
        """``payload [n, W]`` (first three columns: block-local xyz), ``owner [n]`` (rank or -1); only the first
        ``count`` rows (device int, ``None`` = all) are sent.  ``fn(coords [M_cap, 4], extra [M_cap, W-3] or None,
        m)`` runs on the owner with ``m`` a device int and must return ``[M_cap, out_width]`` whose first ``m`` rows
        are valid; its backward must only read the first ``m`` gradient rows."""
        return _Query.apply(payload, owner, count, self, fn, out_width, *_fn_params(fn))


def _fn_params(fn):
    params = getattr(fn, "parameters_for_autograd", None)
    return tuple(params()) if params is not None else ()


class _Query(torch.autograd.Function):
    @staticmethod
    def forward(ctx, payload, owner, count, disp: BlockDispatcher, fn, out_width, *params):
        lib, st = native.lib(), native.stream_ptr()
        n, W = payload.shape
        assert 3 <= W <= disp.max_w and out_width <= disp.max_v and n <= disp.cap
        payload = payload.contiguous().float()
        owner = owner.to(torch.int32).contiguous()
        dev = payload.device
        pos = torch.empty(n, dtype=torch.int32, device=dev)
        # Two device barriers per forward.  The inbox needs none before it is written: every rank read its previous
        # contents (collect) before the closing barrier of the query that filled it, and this rank passed that barrier.
        # The output buffer is cleared here, ahead of the first barrier, so that barrier also tells the owners that
        # every output buffer is ready for their stores (its previous contents were copied out in stream order).
        out = disp.buf.view(disp.off_out, (n, out_width), torch.float32)
        out.zero_()
        native.check(lib.lmb_a2a_dispatch(payload.data_ptr(), owner.data_ptr(), native.ptr(count), n, W, disp.inbox_table,
                                          disp.incoming_table, disp.rank, disp.world, disp.cap, disp.counts.data_ptr(),
                                          pos.data_ptr(), disp.overflow.data_ptr(), st), "a2a_dispatch")
        disp.barrier()                                           # records and counts have landed everywhere; outputs are cleared
        incoming = disp.incoming.clone()
        M = disp.owner_rows
        coords = torch.empty(M, 4, device=dev)
        extra = torch.empty(M, W - 3, device=dev) if W > 3 else None
        route_src = torch.empty(M, dtype=torch.int32, device=dev)
        route_slot = torch.empty(M, dtype=torch.int32, device=dev)
        m_dev = torch.empty(1, dtype=torch.int32, device=dev)
        inbox = disp.buf.local_ptr + disp.off_inbox
        native.check(lib.lmb_a2a_collect(inbox, incoming.data_ptr(), disp.world, disp.cap, W, coords.data_ptr(),
                                         native.ptr(extra), route_src.data_ptr(), route_slot.data_ptr(), m_dev.data_ptr(), st),
                     "a2a_collect")
        with torch.enable_grad():
            values = fn(coords, extra, m_dev).float().reshape(M, out_width)
        native.check(lib.lmb_a2a_combine(values.detach().contiguous().data_ptr(), route_src.data_ptr(), route_slot.data_ptr(),
                                         m_dev.data_ptr(), M, out_width, disp.out_table, disp.world, st), "a2a_combine")
        disp.barrier()                                           # all results are in place
        ctx.disp, ctx.values, ctx.V, ctx.n, ctx.count = disp, values, out_width, n, count
        ctx.save_for_backward(owner, pos, incoming)
        ctx.n_params = len(params)
        return out.clone()

    @staticmethod
    def backward(ctx, dout):
        owner, pos, incoming = ctx.saved_tensors
        disp, lib, st = ctx.disp, native.lib(), native.stream_ptr()
        V, n = ctx.V, ctx.n
        dout = dout.contiguous().float()
        disp.barrier()
        native.check(lib.lmb_a2a_grad_dispatch(dout.data_ptr(), owner.data_ptr(), pos.data_ptr(), native.ptr(ctx.count), n, V,
                                               disp.ginbox_table, disp.rank, disp.world, disp.cap, st), "a2a_grad_dispatch")
        disp.barrier()
        dvals = torch.empty(disp.owner_rows, V, device=dout.device)
        native.check(lib.lmb_a2a_grad_collect(disp.buf.local_ptr + disp.off_ginbox, incoming.data_ptr(), disp.world,
                                              disp.cap, V, dvals.data_ptr(), st), "a2a_grad_collect")
        if ctx.values.requires_grad:
            ctx.values.backward(dvals.view_as(ctx.values))        # owner-side backward: grads land in local params
        return (None, None, None, None, None, None) + (None,) * ctx.n_params
