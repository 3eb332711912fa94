"""Distortion and inter-level (proposal) losses as one-warp-per-ray kernels (``csrc/ray_losses.cu``); the kernels return
the gradient with the loss, so the backward is a broadcast multiply."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong

import torch

from . import native

P = native.P
native.register_signature("lmb_distortion_loss", [P, P, P, c_longlong, c_int, P, P, P])
native.register_signature("lmb_interlevel_loss", [P, P, P, P, c_longlong, c_int, c_int, c_float, P, P, P])


def kernels_usable(*tensors: torch.Tensor) -> bool:
    return all(t.is_cuda for t in tensors) and native.available()


class _Distortion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, w, m, d):
        R, S = w.shape
        loss = torch.empty(R, device=w.device, dtype=torch.float32)
        dw = torch.empty_like(w) if w.requires_grad else None
        native.check(native.lib().lmb_distortion_loss(w.data_ptr(), m.data_ptr(), d.data_ptr(), R, S, loss.data_ptr(),
                                                      native.ptr(dw), native.stream_ptr()), "distortion_loss")
        ctx.dw = dw
        return loss

    @staticmethod
    def backward(ctx, g):
        return (ctx.dw * g[:, None] if ctx.dw is not None else None), None, None


def distortion_per_ray(w: torch.Tensor, m: torch.Tensor, interval: torch.Tensor) -> torch.Tensor:
    """``sum_ij w_i w_j |m_i - m_j| + 1/3 sum_i w_i^2 interval_i`` for every ray (``[R, S]`` inputs, ``m`` sorted along
    the ray); differentiable in ``w`` only - ``m`` and ``interval`` come from the sampler."""
    assert not (m.requires_grad or interval.requires_grad), "sample positions are constants of this loss"
    lead = w.shape[:-1]
    w2 = w.reshape(-1, w.shape[-1]).contiguous().float()
    out = _Distortion.apply(w2, m.reshape(w2.shape).contiguous().float(), interval.reshape(w2.shape).contiguous().float())
    return out.view(lead)


class _Interlevel(torch.autograd.Function):
    @staticmethod
    def forward(ctx, w_env, t_env, t, w, eps):
        R, E = w_env.shape
        S = w.shape[1]
        loss = torch.empty(R, device=w.device, dtype=torch.float32)
        dw = torch.empty_like(w_env) if w_env.requires_grad else None
        native.check(native.lib().lmb_interlevel_loss(t.data_ptr(), w.data_ptr(), t_env.data_ptr(), w_env.data_ptr(), R, S, E,
                                                      float(eps), loss.data_ptr(), native.ptr(dw), native.stream_ptr()),
                     "interlevel_loss")
        ctx.dw = dw
        return loss

    @staticmethod
    def backward(ctx, g):
        return (ctx.dw * g[:, None] if ctx.dw is not None else None), None, None, None, None


def interlevel_per_ray(t: torch.Tensor, w: torch.Tensor, t_env: torch.Tensor, w_env: torch.Tensor, eps: float = 1e-7) -> torch.Tensor:
    """``sum_i max(0, w_i - outer_i)^2 / (w_i + eps)`` for every ray, ``outer_i`` = the proposal histogram
    ``(t_env [R, E+1], w_env [R, E])`` summed over the bins that overlap fine interval ``i`` of ``(t [R, S+1], w [R, S])``.
    Differentiable in ``w_env`` only (the fine level is the target)."""
    R = w.shape[0]
    f = lambda x: x.detach().reshape(R, -1).contiguous().float()  # noqa: E731
    return _Interlevel.apply(w_env.reshape(R, -1).contiguous().float(), f(t_env), f(t), f(w), eps)
