"""Data-parallel optimiser step fused with its collectives.

Parameters, gradients (and optional bf16 shadows) of all replicated tensors live in flat symmetric
buffers that every rank of the data-parallel group maps.  One kernel per step
(``csrc/fused_comm.cu: zero_adam_p2p``) does the gradient reduce-scatter (peer loads), the Adam
update of the rank's own shard (moments exist only on the owner: ZeRO-1 style) and the parameter
all-gather (peer stores).  Two device-side barriers bracket it.  ``NcclZeroAdam`` is the same algorithm
on NCCL collectives - the baseline and the fallback where peer mapping is unavailable.
"""
from __future__ import annotations

import ctypes
from typing import Iterable, List

import torch
import torch.distributed as dist

from ..comm.symmetric import PeerBarrier, SymmetricBuffer
from ..ops import native
from ..ops import optim as _optim

native.register_signature("lmb_zero_adam_p2p", [native.P, native.P, native.P, native.P, native.P, ctypes.c_longlong,
                                                 ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_float,
                                                 ctypes.c_float, ctypes.c_float, ctypes.c_int, ctypes.c_float, native.P])


native.register_signature("lmb_zero_adam_clear_remote_shards", [native.P, ctypes.c_longlong, ctypes.c_int, ctypes.c_int,
                                                                 native.P])


def _table(t: torch.Tensor):
    vals = t.tolist()
    return (ctypes.c_longlong * len(vals))(*vals)


class FlatParams:
    """Re-homes ``params`` into one flat symmetric buffer (params | grads | bf16 shadows) and gives
    every parameter views into it (``p.data`` and the persistent gradient sink)."""

    def __init__(self, params: Iterable[torch.Tensor], group=None, shadow: bool = False):
        self.params: List[torch.Tensor] = [p for p in params]
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        unit = 4 * self.world
        self.offsets, n = [], 0
        for p in self.params:
            self.offsets.append(n)
            n += (p.numel() + 3) // 4 * 4
        self.n = (n + unit - 1) // unit * unit
        self.shadow = shadow
        nbytes = self.n * 4 * 2 + (self.n * 2 if shadow else 0)
        self.buf = SymmetricBuffer(nbytes, group)
        self.flat_param = self.buf.view(0, (self.n,), torch.float32)
        self.flat_grad = self.buf.view(self.n * 4, (self.n,), torch.float32)
        self.flat_shadow = self.buf.view(self.n * 8, (self.n,), torch.bfloat16) if shadow else None
        self.flat_grad.zero_()
        for p, off in zip(self.params, self.offsets):
            view = self.flat_param[off:off + p.numel()].view_as(p)
            view.copy_(p.detach())
            p.data = view
            p._lmb_grad_sink = self.flat_grad[off:off + p.numel()].view_as(p)
            if shadow:
                p._lmb_shadow = self.flat_shadow[off:off + p.numel()].view_as(p)
                p._lmb_shadow.copy_(p.detach())
        self.param_table = _table(self.buf.peer_table(0))
        self.grad_table = _table(self.buf.peer_table(self.n * 4))
        self.shadow_table = _table(self.buf.peer_table(self.n * 8)) if shadow else None

    def close(self):
        """Move the parameters back to ordinary memory and free the symmetric buffer.  The caller has made sure (peer
        barrier / group barrier) that no peer still reads or writes this rank's buffer."""
        if self.buf is None:
            return
        for p in self.params:
            p.data = p.data.clone()
            for name in ("_lmb_grad_sink", "_lmb_shadow"):
                if hasattr(p, name):
                    delattr(p, name)
        self.flat_param = self.flat_grad = self.flat_shadow = None
        self.buf.close()
        self.buf = None

    def absorb_autograd_grads(self):
        """Parameters whose backward produced an ordinary ``.grad`` (PyTorch ops) are folded into the sink."""
        for p in self.params:
            if p.grad is not None:
                p._lmb_grad_sink.add_(p.grad)
                p.grad = None


class P2PZeroAdam:
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, group=None, shadow=False, average=True):
        self.flat = FlatParams(params, group, shadow)
        self.group, self.lr, self.betas, self.eps, self.average = group, lr, betas, eps, average
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = self.flat.world
        shard = self.flat.n // self.world
        dev = self.flat.buf.device
        self.m = torch.zeros(shard, device=dev)
        self.v = torch.zeros(shard, device=dev)
        self.barrier = PeerBarrier(group)
        self.step_count = 0
        self.param_groups = [{"lr": lr, "params": self.flat.params}]

    @torch.no_grad()
    def step(self):
        self.flat.absorb_autograd_grads()
        self.step_count += 1
        _optim.GENERATION += 1
        f = self.flat
        self.barrier()                                   # every rank's backward has finished
        native.check(native.lib().lmb_zero_adam_p2p(f.grad_table, f.param_table, f.shadow_table, self.m.data_ptr(),
                                                    self.v.data_ptr(), f.n, self.rank, self.world,
                                                    self.param_groups[0]["lr"], self.betas[0], self.betas[1], self.eps,
                                                    self.step_count, (1.0 / self.world) if self.average else 1.0,
                                                    native.stream_ptr()), "zero_adam_p2p")
        self.barrier()                                   # every shard has landed in every replica
        native.check(native.lib().lmb_zero_adam_clear_remote_shards(f.flat_grad.data_ptr(), f.n, self.rank, self.world,
                                                                    native.stream_ptr()), "zero_adam_clear")

    def zero_grad(self, set_to_none=True):
        for p in self.flat.params:
            p.grad = None

    def close(self):
        """Collective teardown: a group barrier (all kernels that touch peer memory have been enqueued by every rank),
        a device synchronise (they have finished), a second group barrier (they have finished everywhere), then the
        mappings and the allocation are released."""
        if self.flat.buf is None:
            return
        if dist.is_initialized() and self.world > 1:
            dist.barrier(self.group)
        torch.cuda.synchronize()
        if dist.is_initialized() and self.world > 1:
            dist.barrier(self.group)
        self.flat.close()
        self.barrier.close()
        self.m = self.v = None


class NcclZeroAdam:
    """Same partitioned update with ``reduce_scatter_tensor`` / ``all_gather_into_tensor`` (baseline)."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, group=None, average=True):
        self.params = [p for p in params]
        self.group, self.lr, self.betas, self.eps, self.average = group, lr, betas, eps, average
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        n = sum(p.numel() for p in self.params)
        self.n = (n + self.world - 1) // self.world * self.world
        dev = self.params[0].device
        self.m = torch.zeros(self.n // self.world, device=dev)
        self.v = torch.zeros(self.n // self.world, device=dev)
        self.step_count = 0
        self.param_groups = [{"lr": lr, "params": self.params}]

    @torch.no_grad()
    def step(self):
        self.step_count += 1
        dev = self.params[0].device
        flat_g = torch.zeros(self.n, device=dev)
        flat_p = torch.zeros(self.n, device=dev)
        off = 0
        for p in self.params:
            g = getattr(p, "_lmb_grad_sink", None)
            g = g if g is not None else p.grad
            if g is not None:
                flat_g[off:off + p.numel()] = g.reshape(-1)
            flat_p[off:off + p.numel()] = p.detach().reshape(-1)
            off += p.numel()
        shard = self.n // self.world
        g_shard = torch.empty(shard, device=dev)
        if self.world > 1:
            dist.reduce_scatter_tensor(g_shard, flat_g, group=self.group)
        else:
            g_shard.copy_(flat_g)
        if self.average:
            g_shard /= self.world
        p_shard = flat_p[self.rank * shard:(self.rank + 1) * shard].clone()
        b1, b2 = self.betas
        self.m.mul_(b1).add_(g_shard, alpha=1 - b1)
        self.v.mul_(b2).addcmul_(g_shard, g_shard, value=1 - b2)
        denom = (self.v / (1 - b2 ** self.step_count)).sqrt_().add_(self.eps)
        p_shard.addcdiv_(self.m, denom, value=-self.param_groups[0]["lr"] / (1 - b1 ** self.step_count))
        if self.world > 1:
            dist.all_gather_into_tensor(flat_p, p_shard, group=self.group)
        else:
            flat_p.copy_(p_shard)
        off = 0
        for p in self.params:
            p.copy_(flat_p[off:off + p.numel()].view_as(p))
            sink = getattr(p, "_lmb_grad_sink", None)
            if sink is not None:
                sink.zero_()
            p.grad = None
            off += p.numel()

    def zero_grad(self, set_to_none=True):
        for p in self.params:
            p.grad = None


class GroupedP2PZeroAdam:
    """One :class:`P2PZeroAdam` per distinct learning rate, behind the ``param_groups`` / ``step`` /
    ``zero_grad`` / ``state_dict`` surface the trainers use."""

    def __init__(self, groups, betas=(0.9, 0.999), eps=1e-8, group=None, shadow=False):
        merged = {}
        for g in groups:
            # groups that share a learning rate (and the trainer's "follows the schedule" switch) share one flat buffer
            key = (float(g["lr"]), bool(g.get("scheduled", True)))
            merged.setdefault(key, []).extend(list(g["params"]))
        self.opts = [P2PZeroAdam(params, lr=lr, betas=betas, eps=eps, group=group, shadow=shadow)
                     for (lr, _), params in merged.items()]
        self.param_groups = [o.param_groups[0] for o in self.opts]
        for pg, (_, scheduled) in zip(self.param_groups, merged.keys()):
            pg["scheduled"] = scheduled

    def step(self):
        for o in self.opts:
            o.step()

    def zero_grad(self, set_to_none=True):
        for o in self.opts:
            o.zero_grad(set_to_none)

    #: the moments are this rank's 1/world shard: a checkpoint of this optimiser is per rank
    partitioned = True

    def state_dict(self):
        """This rank's shard of the moments plus the partition it belongs to (checked by ``load_state_dict``)."""
        return {"partition": {"rank": self.opts[0].rank, "world": self.opts[0].world, "elems": [o.flat.n for o in self.opts]},
                "groups": [{"m": o.m, "v": o.v, "step": o.step_count, "lr": o.param_groups[0]["lr"]} for o in self.opts]}

    def load_state_dict(self, state):
        part = state.get("partition")
        if part is None:
            raise ValueError("optimiser state carries no partition record: it was not written by a partitioned optimiser")
        mine = {"rank": self.opts[0].rank, "world": self.opts[0].world, "elems": [o.flat.n for o in self.opts]}
        if part != mine:
            raise ValueError(f"optimiser shard of partition {part} cannot be loaded into partition {mine}: every rank "
                             "must read the file its own rank wrote, with the same group size and parameters")
        for o, s in zip(self.opts, state["groups"]):
            o.m.copy_(s["m"]); o.v.copy_(s["v"]); o.step_count = s["step"]; o.param_groups[0]["lr"] = s["lr"]

    def group_lr(self, params) -> float:
        """Learning rate of the group that holds ``params[0]`` (groups are merged by rate, so indices of the
        caller's original group list do not apply)."""
        want = params[0] if isinstance(params, (list, tuple)) else params
        for o in self.opts:
            if any(p is want for p in o.flat.params):
                return o.param_groups[0]["lr"]
        raise KeyError("parameter is not managed by this optimiser")

    def close(self):
        """Release the peer-mapped buffers (collective: every rank of the group calls it at the same point)."""
        for o in self.opts:
            o.close()
        self.opts = []
