"""Deferred ("lazy") Adam for feature planes: see ``csrc/lazy_adam.cu`` for the algorithm.

``LazyPlaneState`` is attached to a plane parameter (``param._lmb_lazy``).  The encoding calls
:meth:`prepare` with the step's sample coordinates before each lookup; :class:`FusedAdam` calls
:meth:`step` instead of its dense kernel; :meth:`flush` makes every texel current (checkpoints,
evaluation, resizing).  The state needs the optimiser's schedule, which ``FusedAdam`` publishes into
``LazyPlaneState.sched`` at the end of every step.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong
from typing import Optional

import torch

from . import native

P = native.P
native.register_signature("lmb_vm_mark", [P, P, c_longlong, c_int, c_int, c_int, P, P])
native.register_signature("lmb_lazy_adam_prepare", [P, P, P, P, P, P, c_int, c_longlong, c_float, c_int, c_float, c_float,
                                                     c_float, c_float, c_int, P, P])
native.register_signature("lmb_lazy_adam_step", [P, P, P, P, P, P, P, c_int, c_longlong, c_float, c_int, c_float, c_float,
                                                  c_float, c_float, c_int, c_float, P, P])
native.register_signature("lmb_lazy_adam_flush", [P, P, P, P, P, c_int, c_longlong, c_float, c_int, c_float, c_float,
                                                   c_float, c_float, c_int, P])


class LazyPlaneState:
    def __init__(self, param: torch.Tensor):
        B, H, W, C = param.shape
        assert C % 4 == 0
        self.shape = (B, H, W, C)
        dev = param.device
        n = B * H * W
        self.need = torch.zeros(n, dtype=torch.uint8, device=dev)         # 0 idle, 1 marked, 2 prepared
        self.last_step = torch.zeros(n, dtype=torch.int32, device=dev)    # last optimiser step applied to the texel
        self.m = torch.zeros_like(param, dtype=torch.float32)
        self.v = torch.zeros_like(param, dtype=torch.float32)
        self.steps_done = 0
        self.marked = False
        # schedule published by the optimiser: lr of step `t_ref`, geometric decay, Adam constants
        self.sched = {"lr_ref": 0.0, "t_ref": 1, "decay": 1.0, "beta1": 0.9, "beta2": 0.999, "eps": 1e-8}
        # device-resident {lr, step} of a capturable optimiser (None: the host values above are passed by value)
        self.dyn: Optional[torch.Tensor] = None
        self.dirty = False

    def _sched_args(self):
        s = self.sched
        return (float(s["lr_ref"]), int(s["t_ref"]), float(s["decay"]), float(s["beta1"]), float(s["beta2"]), float(s["eps"]))

    def prepare(self, param, coords: torch.Tensor, count: Optional[torch.Tensor] = None) -> None:
        """Flag the texels ``coords [N, 4]`` will read and bring their bf16 shadows up to date."""
        B, H, W, C = self.shape
        lib, st = native.lib(), native.stream_ptr()
        native.check(lib.lmb_vm_mark(coords.data_ptr(), native.ptr(count), coords.shape[0], B, H, W, self.need.data_ptr(), st),
                     "vm_mark")
        self.marked = True
        if self.steps_done > 0:
            native.check(lib.lmb_lazy_adam_prepare(self.need.data_ptr(), self.last_step.data_ptr(), param.data_ptr(),
                                                   self.m.data_ptr(), self.v.data_ptr(), param._lmb_shadow.data_ptr(), C,
                                                   B * H * W, *self._sched_args(), self.steps_done + 1, native.ptr(self.dyn), st),
                         "lazy_prepare")

    def step(self, param, grad, grad_scale: float = 1.0) -> None:
        B, H, W, C = self.shape
        t = self.steps_done + 1
        if self.marked:
            native.check(native.lib().lmb_lazy_adam_step(self.need.data_ptr(), self.last_step.data_ptr(), param.data_ptr(),
                                                         grad.data_ptr(), self.m.data_ptr(), self.v.data_ptr(),
                                                         native.ptr(getattr(param, "_lmb_shadow", None)), C, B * H * W,
                                                         *self._sched_args(), t, float(grad_scale), native.ptr(self.dyn),
                                                         native.stream_ptr()), "lazy_step")
        self.marked = False
        self.steps_done = t
        self.dirty = True

    def flush(self, param) -> None:
        """Bring every texel to ``steps_done`` (zero-gradient replay of whatever it skipped)."""
        if not self.dirty or self.steps_done == 0:
            return
        if self.dyn is not None:                 # steps replayed from a CUDA graph advance only the device copy
            lr, nxt = self.dyn.tolist()
            self.steps_done = int(round(nxt)) - 1
            self.sched.update(lr_ref=lr, t_ref=int(round(nxt)))
        B, H, W, C = self.shape
        native.check(native.lib().lmb_lazy_adam_flush(self.last_step.data_ptr(), param.data_ptr(), self.m.data_ptr(),
                                                      self.v.data_ptr(), native.ptr(getattr(param, "_lmb_shadow", None)), C,
                                                      B * H * W, *self._sched_args(), self.steps_done, native.stream_ptr()),
                     "lazy_flush")
        self.dirty = False
