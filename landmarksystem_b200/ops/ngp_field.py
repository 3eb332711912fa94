"""Kernels for the per-sample glue of the hash-grid radiance fields (``csrc/ngp_field.cu``): SH direction encoding,
sample positions -> hash-grid coordinates, the colour head's input rows with their backward, and the occupancy grid's
periodic refresh.  Every function has a PyTorch statement of the same math beside it (the CPU path and the oracle of
the GPU tests).

Reference counterparts: tiny-cuda-nn's SH encoding behind
landmark/nerf_components/model_components/fields/encodings/sh_encoding.py:31-38; the tensor-op field evaluation of
benchmarks/nerf/instant_ngp/instant_ngp.py:225-289; nerfacc's occupancy-grid update called from
instant_ngp.py:316-326.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_uint
from typing import Optional, Tuple

import torch

from . import native
from ..components.utils.sh_utils import sh_basis

P = native.P
native.register_signature("lmb_sh_encode", [c_longlong, P, c_int, c_int, P, P])
native.register_signature("lmb_ngp_positions", [c_longlong, P, c_int, P, P, P, P, P, c_int, c_int, c_int, P, P, P])
native.register_signature("lmb_ngp_head_rows", [c_longlong, P, c_int, P, P, c_int, P, P, c_int, c_int, P, P, P])
native.register_signature("lmb_ngp_head_rows_bwd", [c_longlong, P, c_int, P, P, P, c_int, P, c_int, c_int, P, P, P])
native.register_signature("lmb_occ_cells", [c_longlong, P, c_int, P, c_int, c_uint, c_int, P, c_float, P, P, P])
native.register_signature("lmb_occ_update", [c_longlong, P, P, P, P, P])
native.register_signature("lmb_occ_binarise", [c_longlong, P, c_float, P, P, P])
native.register_signature("lmb_ngp_gather_cached", [c_longlong, P, c_int, P, P, P, c_int, P, c_int, P, P, P])
native.register_signature("lmb_occ_cull", [c_int, c_int, P, P, P, P, c_float, c_float, P, P])

SH_WIDTH = 16


def _use_kernel(t: torch.Tensor) -> bool:
    return t.is_cuda and native.available()


# -- SH direction encoding ----------------------------------------------------------------------------------------------
def sh_encode(dirs: torch.Tensor, levels: int, unit_range: bool) -> torch.Tensor:
    """``dirs [..., 3]`` (in ``[0, 1]`` when ``unit_range``) -> ``[..., levels^2]`` fp32.  Directions are inputs of the
    models, so no gradient flows to them; a tensor that does require one takes the PyTorch path."""
    if not _use_kernel(dirs) or dirs.requires_grad:
        d = dirs * 2.0 - 1.0 if unit_range else dirs
        return sh_basis(d.float(), levels - 1)
    flat = dirs.reshape(-1, 3).contiguous().float()
    out = torch.empty(flat.shape[0], levels * levels, device=dirs.device, dtype=torch.float32)
    native.check(native.lib().lmb_sh_encode(flat.shape[0], flat.data_ptr(), int(unit_range), levels, out.data_ptr(),
                                            native.stream_ptr()), "sh_encode")
    return out.view(*dirs.shape[:-1], levels * levels)


# -- sample positions -----------------------------------------------------------------------------------------------------
def positions_reference(idx, samples_per_ray, origins, dirs, z_flat, aabb, nx, ny, only_block=-1):
    flat = idx if idx is not None else torch.arange(z_flat.numel(), device=z_flat.device)
    ray = flat // samples_per_ray
    pos = origins[ray] + dirs[ray] * z_flat[flat][:, None]
    norm = (pos - aabb[0]) / (aabb[1] - aabb[0])
    inside = ((norm > 0.0) & (norm < 1.0)).all(dim=-1)
    if nx * ny == 1:
        return torch.cat((norm * inside[:, None], torch.zeros_like(norm[:, :1])), -1), inside
    u, v = norm[:, 0] * nx, norm[:, 1] * ny
    bx, by = u.floor().clamp(0, nx - 1), v.floor().clamp(0, ny - 1)
    block = bx * ny + by
    if only_block >= 0:
        inside = inside & (block == float(only_block))
        block = torch.zeros_like(block)
    local = torch.stack((u - bx, v - by, norm[:, 2]), -1) * inside[:, None]
    return torch.cat((local, block[:, None]), -1), inside


@torch.no_grad()
def sample_positions(idx: Optional[torch.Tensor], samples_per_ray: int, origins: torch.Tensor, dirs: torch.Tensor,
                     z_flat: torch.Tensor, aabb: torch.Tensor, aabb_host, nx: int, ny: int,
                     only_block: int = -1) -> Tuple[torch.Tensor, torch.Tensor]:
    """Valid-sample indices (``None``: all ``R x S`` samples) -> ``([M, 4] block-local xyz + block id, inside [M] bool)``.
    ``aabb_host``: the six bounds as Python floats (lo, hi) so that no device read happens here."""
    if not _use_kernel(z_flat):
        return positions_reference(idx, samples_per_ray, origins, dirs, z_flat, aabb, nx, ny, only_block)
    m = idx.numel() if idx is not None else z_flat.numel()
    xyzb = torch.empty(m, 4, device=z_flat.device, dtype=torch.float32)
    inside = torch.empty(m, device=z_flat.device, dtype=torch.uint8)
    lo, hi = (c_float * 3)(*aabb_host[:3]), (c_float * 3)(*aabb_host[3:])
    native.check(native.lib().lmb_ngp_positions(m, native.ptr(idx), samples_per_ray, origins.data_ptr(), dirs.data_ptr(),
                                                z_flat.data_ptr(), lo, hi, nx, ny, only_block, xyzb.data_ptr(),
                                                inside.data_ptr(), native.stream_ptr()), "ngp_positions")
    return xyzb, inside.view(torch.bool)


# -- colour-head input rows -------------------------------------------------------------------------------------------------
def head_rows_reference(idx, samples_per_ray, dirs, h, inside, app_ray, width):
    """PyTorch statement: ``(rows [M, width] bf16, sigma [M])``."""
    from ..components.utils.activation_utils import trunc_exp

    m, geo = h.shape[0], h.shape[1] - 1
    flat = idx if idx is not None else torch.arange(m, device=h.device)
    ray = flat // samples_per_ray
    keep = inside.to(h.dtype)[:, None]
    unit = torch.nn.functional.normalize(dirs[ray].float(), dim=-1)
    parts = [sh_basis(unit, 3), h[:, 1:] * keep]
    if app_ray is not None:
        parts.append(app_ray[ray])
    row = torch.cat(parts, -1)
    rows = torch.zeros(m, width, device=h.device, dtype=torch.bfloat16)
    rows[:, : row.shape[1]] = row.to(torch.bfloat16)
    return rows, (trunc_exp(h[:, :1]) * keep)[:, 0]


class _HeadRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, app_ray, idx, samples_per_ray, dirs, inside, width, app_width):
        m, geo = h.shape[0], h.shape[1] - 1
        h = h.contiguous()
        rows = torch.empty(m, width, device=h.device, dtype=torch.bfloat16)
        sigma = torch.empty(m, device=h.device, dtype=torch.float32)
        app = None if app_ray is None else app_ray.contiguous().float()
        native.check(native.lib().lmb_ngp_head_rows(m, native.ptr(idx), samples_per_ray, dirs.data_ptr(), h.data_ptr(), geo,
                                                    inside.data_ptr(), native.ptr(app), app_width, width, rows.data_ptr(),
                                                    sigma.data_ptr(), native.stream_ptr()), "ngp_head_rows")
        ctx.save_for_backward(h, idx, inside)
        ctx.meta = (samples_per_ray, width, app_width, None if app_ray is None else tuple(app_ray.shape))
        return rows, sigma

    @staticmethod
    def backward(ctx, d_rows, d_sigma):
        h, idx, inside = ctx.saved_tensors
        samples_per_ray, width, app_width, app_shape = ctx.meta
        m, geo = h.shape[0], h.shape[1] - 1
        d_rows = d_rows.contiguous() if d_rows is not None else torch.zeros(m, width, device=h.device, dtype=torch.bfloat16)
        d_sigma = d_sigma.contiguous().float() if d_sigma is not None else torch.zeros(m, device=h.device)
        d_h = torch.empty_like(h)
        want_app = app_shape is not None and ctx.needs_input_grad[1]
        d_app = torch.zeros(app_shape, device=h.device, dtype=torch.float32) if want_app else None
        native.check(native.lib().lmb_ngp_head_rows_bwd(m, native.ptr(idx), samples_per_ray, d_rows.data_ptr(),
                                                        d_sigma.data_ptr(), h.data_ptr(), geo, inside.data_ptr(), app_width,
                                                        width, d_h.data_ptr(), native.ptr(d_app), native.stream_ptr()),
                     "ngp_head_rows_bwd")
        return d_h, d_app, None, None, None, None, None, None


def head_rows_supported(h: torch.Tensor, app_width: int, width: int) -> bool:
    return (_use_kernel(h) and h.dtype == torch.float32 and width % 8 == 0 and width <= 64
            and SH_WIDTH + h.shape[1] - 1 + app_width <= width)


def head_rows(idx: Optional[torch.Tensor], samples_per_ray: int, dirs: torch.Tensor, h: torch.Tensor, inside: torch.Tensor,
              app_ray: Optional[torch.Tensor], app_width: int, width: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Density-head output ``h [M, 1+G]`` (fp32) -> ``(rows [M, width] bf16, sigma [M] fp32)`` where a row is
    ``[SH16(unit dir of the sample's ray) | h[:, 1:] * inside | app_ray[ray] | 0...]`` and ``sigma = exp(h[:, 0]) *
    inside`` with the truncated exponential's backward.  ``app_ray``: ``[R, app_width]`` or ``None`` (zeros)."""
    if not head_rows_supported(h, app_width, width):
        return head_rows_reference(idx, samples_per_ray, dirs, h, inside, app_ray, width)
    inside_u8 = inside.view(torch.uint8) if inside.dtype == torch.bool else inside
    return _HeadRows.apply(h, app_ray, idx, samples_per_ray, dirs.contiguous().float(), inside_u8.contiguous(), width, app_width)


# -- occupancy grid refresh ---------------------------------------------------------------------------------------------------
@torch.no_grad()
def occ_cells(idx: Optional[torch.Tensor], n_cells: int, resolution: int, roi_host, level: int, seed: int, jitter: bool,
              occs_level: torch.Tensor, decay: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sampled cells -> ``(world positions [n, 3], decayed previous occupancy [n])``."""
    n = idx.numel() if idx is not None else n_cells
    xyz = torch.empty(n, 3, device=occs_level.device, dtype=torch.float32)
    decayed = torch.empty(n, device=occs_level.device, dtype=torch.float32)
    roi = (c_float * 6)(*roi_host)
    native.check(native.lib().lmb_occ_cells(n, native.ptr(idx), resolution, roi, level, seed & 0xFFFFFFFF, int(jitter),
                                            occs_level.data_ptr(), float(decay), xyz.data_ptr(), decayed.data_ptr(),
                                            native.stream_ptr()), "occ_cells")
    return xyz, decayed


@torch.no_grad()
def occ_update(idx: Optional[torch.Tensor], decayed: torch.Tensor, fresh: torch.Tensor, occs_level: torch.Tensor) -> None:
    """``occs[idx] = max(decayed, fresh)`` (a cell sampled twice keeps the larger estimate)."""
    fresh = fresh.contiguous().float()
    native.check(native.lib().lmb_occ_update(decayed.numel(), native.ptr(idx), decayed.data_ptr(), fresh.data_ptr(),
                                             occs_level.data_ptr(), native.stream_ptr()), "occ_update")


@torch.no_grad()
def occ_binarise(occs: torch.Tensor, threshold: float, binaries_u8: torch.Tensor, scratch: torch.Tensor) -> None:
    """``binaries = occs > min(mean(occs), threshold)`` without a host read; ``scratch``: one float64 on the device."""
    native.check(native.lib().lmb_occ_binarise(occs.numel(), occs.data_ptr(), float(threshold), scratch.data_ptr(),
                                               binaries_u8.data_ptr(), native.stream_ptr()), "occ_binarise")


@torch.no_grad()
def occ_cull(sigma: torch.Tensor, ts: torch.Tensor, te: torch.Tensor, counts: torch.Tensor, alpha_thre: float,
             early_stop_eps: float, want_source: bool = False) -> Optional[torch.Tensor]:
    """In place: per ray keep the samples with opacity ``1 - exp(-sigma * (te - ts)) >= alpha_thre`` and transmittance in
    front of them ``>= early_stop_eps``, moved to the front of the row in order; ``counts`` becomes the survivors' count.
    ``sigma``, ``ts``, ``te``: fp32 ``[R, S]`` contiguous; ``counts``: int32 ``[R]``.  ``want_source``: also return int32
    ``[R, S]`` with the slot every survivor had before the compaction (entries past ``counts`` undefined)."""
    R, S = ts.shape
    src = torch.empty(R, S, dtype=torch.int32, device=ts.device) if want_source else None
    native.check(native.lib().lmb_occ_cull(R, S, sigma.data_ptr(), ts.data_ptr(), te.data_ptr(), counts.data_ptr(),
                                           float(alpha_thre), float(early_stop_eps), native.ptr(src), native.stream_ptr()),
                 "occ_cull")
    return src


@torch.no_grad()
def gather_cached_rows(idx: torch.Tensor, samples_per_ray: int, source: torch.Tensor, where: Optional[torch.Tensor],
                       a: torch.Tensor, b: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Rows of ``a`` and ``b`` (results of a query over marched samples) for the survivors ``idx`` of a culling whose
    compaction recorded ``source`` (see :func:`occ_cull`); ``where``: flat slot -> row of the query, ``None`` if the
    query covered every slot."""
    n = idx.numel()
    if not _use_kernel(a):
        before = (idx // samples_per_ray) * samples_per_ray + source.reshape(-1)[idx].long()
        rows = before if where is None else where[before]
        return a[rows], b[rows]
    a, b = a.contiguous(), b.contiguous()
    out_a = torch.empty((n, *a.shape[1:]), device=a.device, dtype=a.dtype)
    out_b = torch.empty((n, *b.shape[1:]), device=b.device, dtype=b.dtype)
    native.check(native.lib().lmb_ngp_gather_cached(n, idx.data_ptr(), samples_per_ray, source.data_ptr(), native.ptr(where),
                                                    a.data_ptr(), a[0].numel() * a.element_size(), b.data_ptr(),
                                                    b[0].numel() * b.element_size(), out_a.data_ptr(), out_b.data_ptr(),
                                                    native.stream_ptr()), "ngp_gather_cached")
    return out_a, out_b
