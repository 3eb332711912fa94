"""Sync-free row selection (``csrc/select.cu``): mask compaction with a device-side count and the
gather / scatter pair that moves 3-wide rows between the compacted and the full sample layout."""
from __future__ import annotations

from ctypes import c_int, c_longlong
from typing import Tuple

import torch

from . import native

P = native.P
native.register_signature("lmb_compact_rows", [P, c_longlong, P, P, P, P, P])
native.register_signature("lmb_scatter_rows3", [P, P, P, P, c_longlong, P, P])
native.register_signature("lmb_gather_rows3", [P, P, P, P, c_longlong, P, P])
native.register_signature("lmb_build_payload6", [P, P, P, P, c_longlong, c_int, P, P, P])


def compact_rows(mask: torch.Tensor, xyzb: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``mask [N]`` bool, ``xyzb [N, 4]`` -> ``(idx int32 [N], coords [N, 4], count int32 [1])``; only the first
    ``count`` entries of ``idx`` / ``coords`` are defined.  No host synchronisation."""
    n = mask.shape[0]
    mask = mask.contiguous()
    xyzb = xyzb.contiguous().float()
    idx = torch.empty(n, dtype=torch.int32, device=mask.device)
    coords = torch.empty(n, 4, dtype=torch.float32, device=mask.device)
    count = torch.empty(1, dtype=torch.int32, device=mask.device)
    native.check(native.lib().lmb_compact_rows(mask.data_ptr(), n, xyzb.data_ptr(), idx.data_ptr(), coords.data_ptr(),
                                               count.data_ptr(), native.stream_ptr()), "compact_rows")
    return idx, coords, count


def build_payload6(coords: torch.Tensor, dirs: torch.Tensor, idx: torch.Tensor, count: torch.Tensor, samples_per_ray: int):
    """Compacted colour samples -> ``(payload [n, 6] = xyz + view direction, owner int32 [n] = block id)``; only the
    first ``count`` rows are written."""
    n = coords.shape[0]
    dirs = dirs.contiguous().float()
    payload = torch.empty(n, 6, device=coords.device, dtype=torch.float32)
    owner = torch.empty(n, device=coords.device, dtype=torch.int32)
    native.check(native.lib().lmb_build_payload6(coords.data_ptr(), dirs.data_ptr(), idx.data_ptr(), count.data_ptr(), n,
                                                 samples_per_ray, payload.data_ptr(), owner.data_ptr(), native.stream_ptr()),
                 "build_payload6")
    return payload, owner


class ScatterRows3(torch.autograd.Function):
    """``vals [cap, 3]`` (first ``count`` rows valid) -> ``[n_full, 3]`` with zeros elsewhere; rows whose compacted
    coordinate carries block id ``-1`` are dropped.  Backward gathers the same rows."""

    @staticmethod
    def forward(ctx, vals, idx, coords, count, n_full):
        vals = vals.contiguous().float()
        out = torch.zeros(n_full, 3, device=vals.device, dtype=torch.float32)
        native.check(native.lib().lmb_scatter_rows3(vals.data_ptr(), idx.data_ptr(), coords.data_ptr(), count.data_ptr(),
                                                    vals.shape[0], out.data_ptr(), native.stream_ptr()), "scatter_rows3")
        ctx.save_for_backward(idx, coords, count)
        ctx.cap = vals.shape[0]
        return out

    @staticmethod
    def backward(ctx, dout):
        idx, coords, count = ctx.saved_tensors
        dout = dout.contiguous().float()
        dvals = torch.empty(ctx.cap, 3, device=dout.device, dtype=torch.float32)
        native.check(native.lib().lmb_gather_rows3(dout.data_ptr(), idx.data_ptr(), coords.data_ptr(), count.data_ptr(),
                                                   ctx.cap, dvals.data_ptr(), native.stream_ptr()), "gather_rows3")
        return dvals, None, None, None, None
