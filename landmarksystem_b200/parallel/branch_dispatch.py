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

from ..comm.symmetric import SymmetricBuffer
from ..ops import native
from .zero_adam import _table

P = native.P
U = ctypes.c_void_p
native.register_signature("lmb_a2a_dispatch", [P, c_int, P, P, c_int, P, c_longlong, c_int, P, c_int, c_int, c_longlong, P, P, P, P, P])
native.register_signature("lmb_a2a_collect", [P, P, P, P, P, P, c_int, c_int, c_longlong, c_int, P, P, P, P, P, P, P, P])
native.register_signature("lmb_a2a_combine", [P, P, P, P, c_longlong, c_int, P, c_int, P])
native.register_signature("lmb_a2a_result", [P, P, P, P, c_longlong, c_int, P, P, P, c_int, c_int, P, P, P])
native.register_signature("lmb_a2a_grad_dispatch", [P, P, P, P, c_longlong, c_int, P, c_int, c_int, c_longlong, P])
native.register_signature("lmb_a2a_grad_collect", [P, P, P, P, P, c_int, c_int, c_longlong, c_int, P, P, P])

_FLAG_WORDS = 3 * 8          # ready / done / gradients-ready, eight peers each (kA2AMaxPeers)


class _Channel:
    """Peer-mapped buffers and device-side state of one kind of query (payload width ``W``, result width ``V``).
    Every kind gets its own channel, so two queries of one step never share an inbox or a gradient inbox."""

    def __init__(self, cap: int, W: int, V: int, group):
        self.cap, self.W, self.V = int(cap), int(W), int(V)
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        record = (W + 1 + 3) // 4 * 4                   # floats per inbox record: payload + slot, whole 16-byte words
        gstride = 1 if V == 1 else (V + 3) // 4 * 4
        self.off_inbox = 0
        self.off_ginbox = self.off_inbox + world * cap * record * 4
        self.off_out = self.off_ginbox + world * cap * gstride * 4
        self.off_incoming = (self.off_out + cap * V * 4 + 255) // 256 * 256
        self.off_flags = self.off_incoming + 256
        self.buf = SymmetricBuffer(self.off_flags + _FLAG_WORDS * 4, group)
        self.inbox_table = _table(self.buf.peer_table(self.off_inbox))
        self.ginbox_table = _table(self.buf.peer_table(self.off_ginbox))
        self.out_table = _table(self.buf.peer_table(self.off_out))
        self.incoming_table = _table(self.buf.peer_table(self.off_incoming))
        self.flags_table = _table(self.buf.peer_table(self.off_flags))
        self.flags_local = self.buf.local_ptr + self.off_flags
        dev = self.buf.device
        self.state = torch.zeros(16, dtype=torch.int32, device=dev)      # epochs, block tickets, per-owner counts
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)      # a bounded wait that ran out: 200/300/400 + peer

    def check(self) -> None:
        code = int(self.status.item())
        if code:
            kind = {2: "records of", 3: "results from", 4: "gradients of"}.get(code // 100, "data of")
            raise RuntimeError(f"all-to-all: the wait for the {kind} rank {code % 100} ran out")


class BlockDispatcher:
    """``cap`` = max rows one source may send to one owner.

    Nothing on the host ever learns a row count: the owner-side buffers have the static worst-case size
    ``world * cap`` and every consumer takes the device-side count, so a query is a fixed sequence of
    launches (and can be recorded in a CUDA graph together with the rest of the step).  The hand-over between the
    ranks is a device-side barrier folded into the prologue of each consuming kernel (``csrc/peer_sync.cuh``): no
    barrier launches."""

    def __init__(self, cap: int, max_w: int = 8, max_v: int = 4, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.cap, self.max_w, self.max_v = int(cap), max_w, max_v
        self.channels = {}
        self.overflow = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", torch.cuda.current_device()))

    def channel(self, name: str, W: int, V: int) -> _Channel:
        ch = self.channels.get(name)
        if ch is None or ch.W != W or ch.V != V:
            if ch is not None:
                raise ValueError(f"channel {name!r} was created for payload width {ch.W} / result width {ch.V}")
            ch = self.channels[name] = _Channel(self.cap, W, V, self.group)
            if self.world > 1:
                dist.barrier(self.group)      # every rank has mapped the new buffers before anyone writes into them
        return ch

    @property
    def owner_rows(self) -> int:
        """Static row capacity of the owner-side tensors handed to ``fn``."""
        return self.world * self.cap

    def close(self) -> None:
        """Collective teardown of every channel's peer-mapped buffers (all ranks call it at the same point)."""
        if self.world > 1:
            dist.barrier(self.group)
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(self.group)
        for ch in self.channels.values():
            ch.buf.close()
        self.channels = {}

    def check(self) -> None:
        """Host-side read of the status words (off the hot path): raises if a wait gave up or rows were dropped."""
        for ch in self.channels.values():
            ch.check()
        if int(self.overflow.item()):
            raise RuntimeError("all-to-all: more rows for one owner than the inbox capacity; rows were dropped")

    def query(self, payload: torch.Tensor, owner: torch.Tensor, fn: Callable, out_width: int,
              count: torch.Tensor = None, channel: str = None, payload_width: int = None, owner_column: int = None) -> torch.Tensor:
        """``payload [n, W]`` (first three columns: block-local xyz), ``owner [n]`` (rank or -1); only the first
        ``count`` rows (device int, ``None`` = all) are sent.  ``fn(coords [M_cap, 4], extra [M_cap, W-3] or None,
        m)`` runs on the owner with ``m`` a device int and must return ``[M_cap, out_width]`` whose first ``m`` rows
        are valid; its backward must only read the first ``m`` gradient rows.  ``channel`` names the buffer set; two
        queries that are in flight in the same step (forward or backward) must use different channels.
        ``payload_width`` / ``owner_column``: send only the first columns of wider rows and read the owner from a float
        column of the same rows (``owner=None``) - the sampler's ``[n, 4]`` output goes out without a copy."""
        W = int(payload_width or payload.shape[1])
        name = channel or f"w{W}v{out_width}"
        return _Query.apply(payload, owner, count, self, self.channel(name, W, out_width), fn, out_width, owner_column,
                            *_fn_params(fn))


def _fn_params(fn):
    params = getattr(fn, "parameters_for_autograd", None)
    return tuple(params()) if params is not None else ()


class _Query(torch.autograd.Function):
    @staticmethod
    def forward(ctx, payload, owner, count, disp: BlockDispatcher, ch: _Channel, fn, out_width, owner_column, *params):
        lib, st = native.lib(), native.stream_ptr()
        n, W = payload.shape[0], ch.W
        assert payload.shape[1] >= W and out_width == ch.V and n <= disp.cap
        payload = payload.contiguous().float()
        dev = payload.device
        pos = torch.empty(n, dtype=torch.int32, device=dev)
        state = ch.state.data_ptr()
        if owner is None:                      # owner = a float column of the payload rows; the kernel writes it out as int
            assert owner_column is not None and owner_column < payload.shape[1]
            owner = torch.empty(n, dtype=torch.int32, device=dev)
            own_i, own_f, own_out = None, payload.data_ptr() + 4 * int(owner_column), owner.data_ptr()
        else:
            owner = owner.to(torch.int32).contiguous()
            own_i, own_f, own_out = owner.data_ptr(), None, None
        # records go straight into the owners' inboxes (peer stores)
        native.check(lib.lmb_a2a_dispatch(payload.data_ptr(), payload.shape[1], own_i, own_f, payload.shape[1], native.ptr(count),
                                          n, W, ch.inbox_table, disp.rank, disp.world, disp.cap, state, pos.data_ptr(), own_out,
                                          disp.overflow.data_ptr(), st), "a2a_dispatch")
        M = disp.owner_rows
        coords = torch.empty(M, 4, device=dev)
        extra = torch.empty(M, W - 3, device=dev) if W > 3 else None
        route_src = torch.empty(M, dtype=torch.int32, device=dev)
        route_slot = torch.empty(M, dtype=torch.int32, device=dev)
        m_dev = torch.empty(1, dtype=torch.int32, device=dev)
        incoming = torch.empty(disp.world, dtype=torch.int32, device=dev)
        base = ch.buf.local_ptr
        # prologue: publish this rank's counts + "dispatch complete", wait for every source; then compact the inbox segments
        native.check(lib.lmb_a2a_collect(base + ch.off_inbox, base + ch.off_incoming, ch.incoming_table, ch.flags_table,
                                         ch.flags_local, state, disp.rank, disp.world, disp.cap, W, coords.data_ptr(),
                                         native.ptr(extra), route_src.data_ptr(), route_slot.data_ptr(), m_dev.data_ptr(),
                                         incoming.data_ptr(), ch.status.data_ptr(), st), "a2a_collect")
        with torch.enable_grad():
            if getattr(fn, "accepts_route", False) and out_width == 1:
                # the owner's kernel may store each result into its source's landing buffer itself
                values = fn(coords, extra, m_dev, route=(route_src, route_slot, ch.out_table, disp.world))
            else:
                values = fn(coords, extra, m_dev)
            values = values.float().reshape(M, out_width)
        if not getattr(fn, "combined", False):
            # results go straight into the sources' landing buffers (peer stores)
            native.check(lib.lmb_a2a_combine(values.detach().contiguous().data_ptr(), route_src.data_ptr(),
                                             route_slot.data_ptr(), m_dev.data_ptr(), M, out_width, ch.out_table, disp.world, st),
                         "a2a_combine")
        out = torch.empty(n, out_width, device=dev)
        # prologue: "combine complete" out, wait for every owner; then read this rank's rows back (unsent rows read as zero)
        native.check(lib.lmb_a2a_result(base + ch.off_out, owner.data_ptr(), pos.data_ptr(), native.ptr(count), n, out_width,
                                        ch.flags_table, ch.flags_local, state, disp.rank, disp.world, out.data_ptr(),
                                        ch.status.data_ptr(), st), "a2a_result")
        ctx.disp, ctx.ch, ctx.values, ctx.V, ctx.n, ctx.count = disp, ch, values, out_width, n, count
        ctx.save_for_backward(owner, pos, incoming)
        ctx.n_params = len(params)
        return out

    @staticmethod
    def backward(ctx, dout):
        owner, pos, incoming = ctx.saved_tensors
        disp, ch, lib, st = ctx.disp, ctx.ch, native.lib(), native.stream_ptr()
        V, n = ctx.V, ctx.n
        dout = dout.contiguous().float()
        state = ch.state.data_ptr()
        native.check(lib.lmb_a2a_grad_dispatch(dout.data_ptr(), owner.data_ptr(), pos.data_ptr(), native.ptr(ctx.count), n, V,
                                               ch.ginbox_table, disp.rank, disp.world, disp.cap, st), "a2a_grad_dispatch")
        dvals = torch.empty(disp.owner_rows, V, device=dout.device)
        native.check(lib.lmb_a2a_grad_collect(ch.buf.local_ptr + ch.off_ginbox, incoming.data_ptr(), ch.flags_table,
                                              ch.flags_local, state, disp.rank, disp.world, disp.cap, V, dvals.data_ptr(),
                                              ch.status.data_ptr(), st), "a2a_grad_collect")
        if ctx.values.requires_grad:
            ctx.values.backward(dvals.view_as(ctx.values))        # owner-side backward: grads land in local params
        return (None, None, None, None, None, None, None, None) + (None,) * ctx.n_params
