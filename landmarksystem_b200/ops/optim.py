"""Fused Adam with fp32 master weights, optional bf16 shadow copies and in-kernel gradient reset.

Replaces ``torch.optim.Adam`` + ``zero_grad`` of the reference trainers
(benchmarks/nerf/gridnerf/gridnerf_trainer.py:127-154, 296-322) with one HBM pass per tensor.
On CPU tensors the same update is written with torch ops so that tests can compare the two.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional

import torch

from ctypes import c_float, c_int

from . import native

native.register_signature("lmb_adam_plane_reg", [native.P, native.P, native.P, native.P, native.P, native.P, c_int, c_int, c_int,
                                                  c_int, native.P, c_float, c_int, c_float, c_float, c_float, c_float, native.P,
                                                  c_float, c_float, c_float, native.P, native.P])


# Bumped by every fused step: the kernel updates parameters through raw pointers, which autograd's
# per-tensor version counters do not see, so consumers that cache derived data (packed MLP weights)
# key their caches on this generation as well.
GENERATION = 0


def radam_step_size(lr: float, beta1: float, beta2: float, step: int):
    """Step size of rectified Adam at ``step`` and whether the adaptive denominator ``sqrt(v) + eps`` applies
    (the variance is tractable once rho_t > 5); same arithmetic as ``lmb_radam_step``."""
    b1, b2t = 1.0 - beta1 ** step, beta2 ** step
    rho_inf = 2.0 / (1.0 - beta2) - 1.0
    rho_t = rho_inf - 2.0 * step * b2t / (1.0 - b2t)
    if rho_t > 5.0:
        rect = ((rho_t - 4.0) * (rho_t - 2.0) * rho_inf / ((rho_inf - 4.0) * (rho_inf - 2.0) * rho_t)) ** 0.5
        return lr * rect * (1.0 - b2t) ** 0.5 / b1, True
    return lr / b1, False


class FusedAdam(torch.optim.Optimizer):
    """Adam (no amsgrad).  Per-group options: ``lr, betas, eps, weight_decay``.

    A parameter may carry two optional attributes that the fused path honours:

    * ``_lmb_grad_sink`` - persistent fp32 gradient accumulator written directly by backward kernels
      (then ``.grad`` is unused and never allocated);
    * ``_lmb_shadow`` - bf16 copy of the parameter, refreshed in the same kernel that updates it.
    """

    rectified = False      # FusedRAdam: variance-rectified step size (same device pass)

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, capturable: bool = False):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        assert not (capturable and self.rectified), "the rectified variant keeps its schedule on the host"
        # capturable: every group's {learning rate, step number} lives on the device and is advanced by a
        # kernel at the end of step() (lr *= group["lr_decay"]), so a step recorded in a CUDA graph follows
        # the schedule on replay.  The optimiser owns the schedule in this mode: group["lr"] mirrors the device value
        # (step() and host_advance() keep it in step; callers must not decay it themselves); call ``sync_dyn`` after
        # changing it by hand and ``host_advance`` after every graph replay.
        self.capturable = capturable
        if capturable:
            self.sync_dyn()

    def sync_dyn(self) -> None:
        """Push every group's host-side learning rate and step count to its device-resident schedule."""
        for group in self.param_groups:
            dev = next((p.device for p in group["params"] if p.is_cuda), None)
            if dev is None:
                continue
            steps = [self.state[p].get("step", 0) for p in group["params"] if p in self.state and self.state[p]]
            steps += [p._lmb_lazy.steps_done for p in group["params"] if getattr(p, "_lmb_lazy", None) is not None]
            nxt = float(max(steps) + 1 if steps else 1)
            if group.get("_dyn") is None:
                group["_dyn"] = torch.tensor([group["lr"], nxt], device=dev, dtype=torch.float32)
            else:
                group["_dyn"].copy_(torch.tensor([group["lr"], nxt], dtype=torch.float32))
            for p in group["params"]:
                if getattr(p, "_lmb_lazy", None) is not None:
                    p._lmb_lazy.dyn = group["_dyn"]

    # -- checkpointing: the deferred-update state of planes lives outside ``self.state`` -----------------------------
    def _lazy_params(self):
        out, k = [], 0
        for group in self.param_groups:
            for p in group["params"]:
                if getattr(p, "_lmb_lazy", None) is not None:
                    out.append((k, p))
                k += 1
        return out

    def state_dict(self):
        """Standard optimiser state plus, for planes with the deferred update, their moments and step count (every texel
        is brought up to date first, so the saved moments are those a dense Adam would hold)."""
        sd = super().state_dict()
        lazy = {}
        for k, p in self._lazy_params():
            st = p._lmb_lazy
            st.flush(p)
            lazy[k] = {"exp_avg": st.m, "exp_avg_sq": st.v, "step": st.steps_done}
        if lazy:
            sd["lazy"] = lazy
        return sd

    def load_state_dict(self, state_dict):
        state_dict = dict(state_dict)
        lazy = state_dict.pop("lazy", None)
        for g in state_dict.get("param_groups", []):
            g.pop("_dyn", None)                     # device-resident schedules are rebuilt below
        super().load_state_dict(state_dict)
        if lazy:
            for k, p in self._lazy_params():
                rec = lazy.get(k, lazy.get(str(k)))
                if rec is None:
                    continue
                st = p._lmb_lazy
                st.m.copy_(rec["exp_avg"])
                st.v.copy_(rec["exp_avg_sq"])
                st.steps_done = int(rec["step"])
                st.last_step.fill_(st.steps_done)
                st.need.zero_()
                st.dirty = False
        if self.capturable:
            for group in self.param_groups:
                group["_dyn"] = None
            self.sync_dyn()

    def host_advance(self) -> None:
        """Mirror one graph-replayed step in the host-side bookkeeping (no kernel is launched)."""
        for group in self.param_groups:
            group["lr"] *= float(group.get("lr_decay", 1.0))
            for p in group["params"]:
                lazy = getattr(p, "_lmb_lazy", None)
                if lazy is not None:
                    lazy.steps_done += 1
                    lazy.dirty = True
                elif p in self.state and self.state[p]:
                    self.state[p]["step"] += 1
                    if self._plane_reg_active(p):
                        p.data, p._lmb_pong = p._lmb_pong, p.data      # the replayed step wrote the other buffer

    @staticmethod
    def attach_sink(param: torch.Tensor, shadow: bool = False, lazy: bool = False) -> None:
        """Give ``param`` a persistent zeroed fp32 accumulator (and a bf16 shadow if asked).  ``lazy``
        (4-D channels-last planes on CUDA only) additionally enables the deferred update."""
        param._lmb_grad_sink = torch.zeros_like(param, dtype=torch.float32)
        if shadow:
            param._lmb_shadow = param.detach().to(torch.bfloat16)
        if lazy and shadow and param.is_cuda and param.dim() == 4:
            from .lazy_adam import LazyPlaneState

            param._lmb_lazy = LazyPlaneState(param)

    @staticmethod
    def attach_plane_regulariser(param: torch.Tensor, tv_weight=None, tv_index: int = 0, l1_weight: float = 0.0,
                                 loss_scale: float = 1.0, loss_out: Optional[torch.Tensor] = None) -> None:
        """Fold the total-variation / L1 regularisers of a channels-last plane ``[B, H, W, C]`` into its Adam step
        (``csrc/adam.cu: adam_plane_reg_kernel``).  ``tv_weight``: a device tensor whose element ``tv_index`` is the
        (decaying) weight, a float, or ``None``; ``loss_scale``: the factor the caller applies to its total loss;
        ``loss_out``: optional device ``float[2]`` that accumulates the TV and L1 loss values.  Needs the gradient sink
        and the bf16 shadow (``attach_sink(param, shadow=True)``); a second parameter buffer is allocated (the step
        ping-pongs between the two so that neighbours are read at their old values)."""
        tv_dev = tv_weight[tv_index:tv_index + 1] if torch.is_tensor(tv_weight) else None
        tv_host = 0.0 if (tv_weight is None or torch.is_tensor(tv_weight)) else float(tv_weight)
        param._lmb_reg = {"tv_dev": tv_dev, "tv": tv_host, "l1": float(l1_weight), "scale": float(loss_scale), "loss": loss_out}
        if getattr(param, "_lmb_pong", None) is None or param._lmb_pong.shape != param.shape:
            param._lmb_pong = torch.empty_like(param.data)

    @staticmethod
    def _plane_reg_active(p) -> bool:
        reg = getattr(p, "_lmb_reg", None)
        return (reg is not None and (reg["tv_dev"] is not None or reg["tv"] > 0 or reg["l1"] > 0) and p.is_cuda and p.dim() == 4
                and p.shape[-1] % 4 == 0 and getattr(p, "_lmb_grad_sink", None) is not None
                and getattr(p, "_lmb_shadow", None) is not None and getattr(p, "_lmb_lazy", None) is None)

    @torch.no_grad()
    def step(self, closure=None, grad_scale: float = 1.0):
        global GENERATION
        GENERATION += 1
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            dyn = group.get("_dyn") if self.capturable else None
            stepped = False
            for p in group["params"]:
                sink = getattr(p, "_lmb_grad_sink", None)
                if sink is not None and p.grad is not None:
                    # a loss term evaluated with PyTorch ops (a regulariser, say) left an ordinary gradient next to the
                    # kernels' accumulator: fold it in, or it would be ignored and pile up
                    sink.add_(p.grad)
                    p.grad = None
                grad = sink if sink is not None else p.grad
                if grad is None:
                    continue
                lazy = getattr(p, "_lmb_lazy", None)
                if lazy is not None and sink is not None and not self.rectified:
                    # deferred update: only the texels this step's samples touched are visited
                    decay = float(group.get("lr_decay", 1.0))
                    lazy.sched.update(lr_ref=group["lr"], t_ref=lazy.steps_done + 1, decay=decay, beta1=beta1, beta2=beta2,
                                      eps=group["eps"])
                    lazy.step(p, sink, grad_scale)
                    stepped = True
                    continue
                state = self.state[p]
                if not state:
                    state["step"] = 0
                    state["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    state["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                state["step"] += 1
                shadow = getattr(p, "_lmb_shadow", None)
                if sink is None and p.is_cuda and not grad.is_contiguous():
                    grad = grad.contiguous()          # e.g. a transposed view handed back by a fused backward
                if dyn is not None and p.is_cuda and not (p.dtype == torch.float32 and p.is_contiguous()
                                                          and grad.dtype == torch.float32):
                    raise RuntimeError("capturable FusedAdam needs contiguous fp32 CUDA parameters and gradients: the PyTorch "
                                       "fallback would bake the host-side learning rate and step count into a recorded graph")
                stepped = True
                if self._plane_reg_active(p) and not self.rectified and p.dtype == torch.float32 and p.is_contiguous():
                    reg = p._lmb_reg
                    B, H, W, C = p.shape
                    cur, other = p.data, p._lmb_pong
                    odd, even = (cur, other) if state["step"] % 2 == 1 else (other, cur)     # `cur` is read at this step number
                    native.check(native.lib().lmb_adam_plane_reg(
                        odd.data_ptr(), even.data_ptr(), grad.data_ptr(), state["exp_avg"].data_ptr(),
                        state["exp_avg_sq"].data_ptr(), shadow.data_ptr(), B, H, W, C, native.ptr(dyn), group["lr"], state["step"],
                        beta1, beta2, group["eps"], grad_scale, native.ptr(reg["tv_dev"]), reg["tv"], reg["l1"], reg["scale"],
                        native.ptr(reg["loss"]), native.stream_ptr()), "adam_plane_reg")
                    p.data, p._lmb_pong = other, cur             # the updated values are in the other buffer now
                    continue
                if p.is_cuda and p.dtype == torch.float32 and p.is_contiguous() and grad.is_contiguous() \
                        and grad.dtype == torch.float32 and dyn is not None:
                    native.check(native.lib().lmb_adam_step_dyn(
                        p.data_ptr(), grad.data_ptr(), state["exp_avg"].data_ptr(), state["exp_avg_sq"].data_ptr(),
                        native.ptr(shadow), p.numel(), dyn.data_ptr(), beta1, beta2, group["eps"], grad_scale,
                        group["weight_decay"], native.stream_ptr()), "adam_step_dyn")
                elif p.is_cuda and p.dtype == torch.float32 and p.is_contiguous() and grad.is_contiguous() \
                        and grad.dtype == torch.float32:
                    fn = native.lib().lmb_radam_step if self.rectified else native.lib().lmb_adam_step
                    native.check(fn(
                        p.data_ptr(), grad.data_ptr(), state["exp_avg"].data_ptr(), state["exp_avg_sq"].data_ptr(),
                        native.ptr(shadow), p.numel(), group["lr"], beta1, beta2, group["eps"], state["step"],
                        grad_scale, group["weight_decay"], native.stream_ptr()), "adam_step")
                else:
                    g = grad.float() * grad_scale + group["weight_decay"] * p
                    state["exp_avg"].mul_(beta1).add_(g, alpha=1 - beta1)
                    state["exp_avg_sq"].mul_(beta2).addcmul_(g, g, value=1 - beta2)
                    b1 = 1 - beta1 ** state["step"]
                    b2 = 1 - beta2 ** state["step"]
                    if self.rectified:
                        step_size, adaptive = radam_step_size(group["lr"], beta1, beta2, state["step"])
                        if adaptive:
                            p.addcdiv_(state["exp_avg"], state["exp_avg_sq"].sqrt().add_(group["eps"]), value=-step_size)
                        else:
                            p.add_(state["exp_avg"], alpha=-step_size)
                    else:
                        denom = (state["exp_avg_sq"] / b2).sqrt_().add_(group["eps"])
                        p.addcdiv_(state["exp_avg"], denom, value=-group["lr"] / b1)
                    grad.zero_()
                    if shadow is not None:
                        shadow.copy_(p)
            if dyn is not None and stepped:
                native.check(native.lib().lmb_adam_dyn_advance(dyn.data_ptr(), float(group.get("lr_decay", 1.0)),
                                                               native.stream_ptr()), "adam_dyn_advance")
                group["lr"] *= float(group.get("lr_decay", 1.0))      # host mirror of the device-side schedule
        return loss

    def zero_grad(self, set_to_none: bool = True):  # gradients are cleared inside step()
        for group in self.param_groups:
            for p in group["params"]:
                if getattr(p, "_lmb_grad_sink", None) is None and p.grad is not None:
                    if set_to_none:
                        p.grad = None
                    else:
                        p.grad.zero_()


class FusedRAdam(FusedAdam):
    """Rectified Adam with the same fused device pass (``torch.optim.RAdam`` of the reference's Nerfacto trainer,
    benchmarks/nerf/nerfacto/nerfacto_trainer.py:139)."""

    rectified = True
