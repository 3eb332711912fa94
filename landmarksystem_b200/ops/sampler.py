"""Fused uniform ray sampler + spatial-block assignment (``csrc/sampler.cu``)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong
from typing import Optional, Tuple

import torch

from . import native

P = native.P
native.register_signature("lmb_uniform_sampler", [P, c_int, c_longlong, c_int, P, P, c_float, c_float, c_float, c_float, c_float,
                                                   c_int, c_int, c_int, c_int, c_int, c_int, c_int, P, P, P, P, P])


def uniform_sample_blocks(rays: torch.Tensor, n_samples: int, aabb: torch.Tensor, near: float, far: float, step: float,
                          norm_lo: float, norm_size: float, partition: Tuple[int, int], window_origin: Tuple[int, int],
                          window: Tuple[int, int], jitter: Optional[torch.Tensor] = None, hull: bool = False):
    """``rays [R, >=6]`` -> ``(z [R,S], dists [R,S], xyzb [R*S,4], valid [R*S] bool)``; see the kernel header.
    ``jitter [R]`` in ``[0, 1)`` shifts all samples of a ray (stratified training sampling).  ``hull``: the samples
    are spaced linearly from ``near`` to the ray's ground-plane hit (``far`` for rays that look up) instead of
    ``step`` apart from the box entry - the render-time sampling of ``UniformSampler.compute_z_vals``."""
    rays = rays.contiguous().float()
    R = rays.shape[0]
    dev = rays.device
    z = torch.empty(R, n_samples, device=dev)
    dists = torch.empty(R, n_samples, device=dev)
    xyzb = torch.empty(R * n_samples, 4, device=dev)
    valid = torch.empty(R * n_samples, dtype=torch.uint8, device=dev)
    aabb = aabb.contiguous().float()
    native.check(native.lib().lmb_uniform_sampler(rays.data_ptr(), rays.shape[1], R, n_samples, native.ptr(jitter), aabb.data_ptr(),
                                                  float(near), float(far), float(step), float(norm_lo), float(norm_size),
                                                  int(partition[0]), int(partition[1]), int(window_origin[0]),
                                                  int(window_origin[1]), int(window[0]), int(window[1]), int(bool(hull)), z.data_ptr(),
                                                  dists.data_ptr(), xyzb.data_ptr(), valid.data_ptr(), native.stream_ptr()),
                 "uniform_sampler")
    return z, dists, xyzb, valid.view(torch.bool)
