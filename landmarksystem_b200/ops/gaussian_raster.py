"""3D Gaussian splatting rasteriser: public module API, CUDA path and PyTorch oracle.

API mirrors what the reference imports from its rasteriser extension
(``GaussianRasterizationSettings`` / ``GaussianRasterizer(...)(means3D, means2D, shs, colors_precomp,
opacities, scales, rotations, cov3D_precomp) -> (image [3,H,W], radii [N], extra)`` and
``.visible_filter(...) -> radii``; call sites benchmarks/nerf/origin_gs/gs_model.py:82-97,148-162,
211-220).  CUDA tensors run ``csrc/gs_raster.cu`` + ``csrc/sort_scan.cu``; CPU tensors run
:func:`rasterize_reference`, a dense differentiable PyTorch statement of the same math that serves as
the numerics oracle (small scenes only).
"""
from __future__ import annotations

import math
from ctypes import POINTER, Structure, byref, c_float, c_int, c_longlong
from typing import NamedTuple, Optional

import torch
from torch import nn

from . import native

TILE = 16


class GaussianRasterizationSettings(NamedTuple):
    image_height: int
    image_width: int
    tanfovx: float
    tanfovy: float
    bg: torch.Tensor
    scale_modifier: float
    viewmatrix: torch.Tensor      # [4,4] transposed world-to-view (row-vector convention)
    projmatrix: torch.Tensor      # [4,4] viewmatrix @ projection
    sh_degree: int
    campos: torch.Tensor
    prefiltered: bool = False
    debug: bool = False


class GSCamera(Structure):
    _fields_ = [("view", c_float * 16), ("proj", c_float * 16), ("campos", c_float * 3), ("tanfovx", c_float),
                ("tanfovy", c_float), ("W", c_int), ("H", c_int), ("scale_modifier", c_float), ("sh_degree", c_int),
                ("sh_coeffs", c_int)]


P = native.P
native.register_signature("lmb_gs_preprocess", [c_int, P, P, P, P, P, P, P, P, POINTER(GSCamera), P, P, P, P, P, P, P, P,
                                                 c_int, P])
native.register_signature("lmb_gs_make_keys", [c_int, P, P, P, P, P, c_int, c_int, c_longlong, P, P, P, P, P])
native.register_signature("lmb_gs_tile_ranges", [P, P, c_longlong, P, c_int, P])
native.register_signature("lmb_gs_render_fwd", [P, P, c_int, c_int, P, P, P, P, P, P, P, P])
native.register_signature("lmb_gs_render_bwd", [P, P, c_int, c_int, P, P, P, P, P, P, P, P, P, P, P, P])
native.register_signature("lmb_gs_preprocess_bwd", [c_int, P, P, P, P, P, P, P, POINTER(GSCamera), P, P, P, P, P, P, P, P,
                                                     c_int, P])
native.register_signature("lmb_exclusive_scan_u32", [P, P, c_longlong, P, P])
native.register_signature("lmb_radix_sort_pairs", [P, P, P, c_longlong, c_int, c_int, P, P])


def _lib_ll(name):
    fn = getattr(native.lib(), name)
    fn.restype = c_longlong
    fn.argtypes = [c_longlong]
    return fn


def _camera_struct(s: GaussianRasterizationSettings, sh_coeffs: int) -> GSCamera:
    cam = GSCamera()
    view = s.viewmatrix.detach().float().cpu().reshape(-1).tolist()
    proj = s.projmatrix.detach().float().cpu().reshape(-1).tolist()
    pos = s.campos.detach().float().cpu().reshape(-1).tolist()
    for i in range(16):
        cam.view[i], cam.proj[i] = view[i], proj[i]
    for i in range(3):
        cam.campos[i] = pos[i]
    cam.tanfovx, cam.tanfovy, cam.W, cam.H = s.tanfovx, s.tanfovy, s.image_width, s.image_height
    cam.scale_modifier, cam.sh_degree, cam.sh_coeffs = s.scale_modifier, s.sh_degree, sh_coeffs
    return cam


# ---------------------------------------------------------------------------------------------------
# PyTorch oracle
# ---------------------------------------------------------------------------------------------------
def _quat_to_rot(q):
    r, x, y, z = q.unbind(-1)
    return torch.stack((1 - 2 * (y * y + z * z), 2 * (x * y - r * z), 2 * (x * z + r * y),
                        2 * (x * y + r * z), 1 - 2 * (x * x + z * z), 2 * (y * z - r * x),
                        2 * (x * z - r * y), 2 * (y * z + r * x), 1 - 2 * (x * x + y * y)), -1).reshape(-1, 3, 3)


def project_reference(means3D, scales, rotations, cov3D_precomp, s: GaussianRasterizationSettings):
    """Per-Gaussian screen quantities: ``(xy [N,2], depth [N], conic [N,3], radii [N], valid [N])``."""
    N = means3D.shape[0]
    V, Pm = s.viewmatrix.to(means3D), s.projmatrix.to(means3D)
    hom = torch.cat((means3D, torch.ones(N, 1, dtype=means3D.dtype, device=means3D.device)), -1)
    t = (hom @ V)[:, :3]
    ph = hom @ Pm
    ndc = ph[:, :2] / (ph[:, 3:4] + 1e-7)
    if cov3D_precomp is not None:
        c = cov3D_precomp
        Sigma = torch.stack((c[:, 0], c[:, 1], c[:, 2], c[:, 1], c[:, 3], c[:, 4], c[:, 2], c[:, 4], c[:, 5]), -1).reshape(-1, 3, 3)
    else:
        R = _quat_to_rot(rotations)
        M = R * (scales * s.scale_modifier)[:, None, :]
        Sigma = M @ M.transpose(1, 2)
    W, H = s.image_width, s.image_height
    fx, fy = W / (2 * s.tanfovx), H / (2 * s.tanfovy)
    tz = t[:, 2]
    limx, limy = 1.3 * s.tanfovx, 1.3 * s.tanfovy
    txz = torch.clamp(t[:, 0] / tz, -limx, limx) * tz
    tyz = torch.clamp(t[:, 1] / tz, -limy, limy) * tz
    zeros = torch.zeros_like(tz)
    J = torch.stack((fx / tz, zeros, -fx * txz / (tz * tz), zeros, fy / tz, -fy * tyz / (tz * tz)), -1).reshape(-1, 2, 3)
    Wr = V[:3, :3].t()
    T = J @ Wr
    cov = T @ Sigma @ T.transpose(1, 2)
    a, b, c = cov[:, 0, 0] + 0.3, cov[:, 0, 1], cov[:, 1, 1] + 0.3
    det = a * c - b * b
    conic = torch.stack((c / det, -b / det, a / det), -1)
    mid = 0.5 * (a + c)
    lam = mid + torch.sqrt(torch.clamp(mid * mid - det, min=0.1))
    radii = torch.ceil(3.0 * torch.sqrt(lam)).int()
    xy = torch.stack((((ndc[:, 0] + 1) * W - 1) * 0.5, ((ndc[:, 1] + 1) * H - 1) * 0.5), -1)
    valid = (tz > 0.2) & (det != 0)
    return xy, tz, conic, radii, valid


def _tile_rect(xy, radii, W, H):
    tx, ty = (W + TILE - 1) // TILE, (H + TILE - 1) // TILE
    r = radii.to(xy.dtype)
    x0 = torch.clamp(((xy[:, 0] - r) / TILE).int(), 0, tx)
    y0 = torch.clamp(((xy[:, 1] - r) / TILE).int(), 0, ty)
    x1 = torch.clamp(((xy[:, 0] + r + TILE - 1) / TILE).int(), 0, tx)
    y1 = torch.clamp(((xy[:, 1] + r + TILE - 1) / TILE).int(), 0, ty)
    return x0, y0, x1, y1


def rasterize_reference(means3D, opacities, s: GaussianRasterizationSettings, shs=None, colors_precomp=None, scales=None,
                        rotations=None, cov3D_precomp=None, visible=None):
    """Dense differentiable oracle: every pixel blends all Gaussians whose tile rectangle covers it."""
    from ..components.utils.sh_utils import eval_sh

    W, H = s.image_width, s.image_height
    xy, depth, conic, radii, valid = project_reference(means3D, scales, rotations, cov3D_precomp, s)
    x0, y0, x1, y1 = _tile_rect(xy.detach(), radii, W, H)
    valid = valid & ((x1 - x0) * (y1 - y0) > 0)
    if visible is not None:
        valid = valid & visible.bool()
    if colors_precomp is None:
        dirs = means3D - s.campos.to(means3D)
        dirs = dirs / dirs.norm(dim=-1, keepdim=True)
        colors = torch.clamp_min(eval_sh(s.sh_degree, shs.transpose(1, 2), dirs) + 0.5, 0.0)
    else:
        colors = colors_precomp
    order = torch.argsort(depth.detach() + (~valid) * 1e10, stable=True)
    order = order[valid[order]]
    ys, xs = torch.meshgrid(torch.arange(H, device=means3D.device), torch.arange(W, device=means3D.device), indexing="ij")
    pix = torch.stack((xs, ys), -1).reshape(-1, 2).to(means3D.dtype)          # [P, 2]
    tile_x, tile_y = (xs // TILE).reshape(-1), (ys // TILE).reshape(-1)
    T = torch.ones(H * W, dtype=means3D.dtype, device=means3D.device)
    C = torch.zeros(H * W, 3, dtype=means3D.dtype, device=means3D.device)
    done = torch.zeros(H * W, dtype=torch.bool, device=means3D.device)
    for g in order.tolist():
        cover = (tile_x >= x0[g]) & (tile_x < x1[g]) & (tile_y >= y0[g]) & (tile_y < y1[g]) & ~done
        d = xy[g][None] - pix
        power = -0.5 * (conic[g, 0] * d[:, 0] ** 2 + conic[g, 2] * d[:, 1] ** 2) - conic[g, 1] * d[:, 0] * d[:, 1]
        alpha = torch.clamp(opacities[g].reshape(()) * torch.exp(power), max=0.99)
        use = cover & (power <= 0) & (alpha >= 1.0 / 255.0)
        test_T = T * (1 - alpha)
        stop = use & (test_T < 1e-4)
        done = done | stop
        use = use & ~stop
        w = torch.where(use, alpha * T, torch.zeros_like(T))
        C = C + w[:, None] * colors[g][None]
        T = torch.where(use, test_T, T)
    img = C + T[:, None] * s.bg.to(means3D)[None]
    out_radii = torch.where(valid, radii, torch.zeros_like(radii))
    return img.t().reshape(3, H, W), out_radii, (1.0 - T).reshape(H, W).detach()


# ---------------------------------------------------------------------------------------------------
# CUDA path
# ---------------------------------------------------------------------------------------------------
class _Workspace:
    """Per-device growable buffers so that steady-state frames allocate nothing."""
    _cache = {}

    @classmethod
    def get(cls, device, name, nbytes):
        key = (device, name)
        buf = cls._cache.get(key)
        if buf is None or buf.numel() < nbytes:
            buf = torch.empty(int(nbytes * 1.25) + 256, dtype=torch.uint8, device=device)
            cls._cache[key] = buf
        return buf


def _preprocess(means3D, scales, rotations, opacities, shs, colors_precomp, cov3D_precomp, visible, cam, radius_only):
    N, dev = means3D.shape[0], means3D.device
    radii = torch.empty(N, dtype=torch.int32, device=dev)
    if radius_only:
        native.check(native.lib().lmb_gs_preprocess(N, means3D.data_ptr(), native.ptr(scales), native.ptr(rotations), None,
                                                    None, None, native.ptr(cov3D_precomp), native.ptr(visible), byref(cam),
                                                    radii.data_ptr(), None, None, None, None, None, None, None, 1,
                                                    native.stream_ptr()), "gs_preprocess")
        return radii
    xy = torch.empty(N, 2, device=dev)
    depth = torch.empty(N, device=dev)
    cov3d = torch.empty(N, 6, device=dev)
    conic_op = torch.empty(N, 4, device=dev)
    rgb = torch.empty(N, 3, device=dev)
    clamped = torch.zeros(N, 3, dtype=torch.uint8, device=dev)
    touched = torch.empty(N, dtype=torch.int32, device=dev)
    native.check(native.lib().lmb_gs_preprocess(N, means3D.data_ptr(), native.ptr(scales), native.ptr(rotations),
                                                opacities.data_ptr(), native.ptr(shs), native.ptr(colors_precomp),
                                                native.ptr(cov3D_precomp), native.ptr(visible), byref(cam), radii.data_ptr(),
                                                xy.data_ptr(), depth.data_ptr(), cov3d.data_ptr(), conic_op.data_ptr(),
                                                rgb.data_ptr(), clamped.data_ptr(), touched.data_ptr(), 0,
                                                native.stream_ptr()), "gs_preprocess")
    return radii, xy, depth, cov3d, conic_op, rgb, clamped, touched


class _Rasterize(torch.autograd.Function):
    @staticmethod
    def forward(ctx, means3D, means2D, shs, colors_precomp, opacities, scales, rotations, cov3D_precomp, visible, settings):
        s = settings
        N, dev = means3D.shape[0], means3D.device
        W, H = s.image_width, s.image_height
        sh_coeffs = 0 if shs is None else shs.shape[1]
        cam = _camera_struct(s, sh_coeffs)
        f = lambda t: None if t is None else t.contiguous().float()  # noqa: E731
        means3D, shs, colors_precomp, opacities = f(means3D), f(shs), f(colors_precomp), f(opacities)
        scales, rotations, cov3D_precomp = f(scales), f(rotations), f(cov3D_precomp)
        vis = None if visible is None else visible.to(torch.uint8).contiguous()
        radii, xy, depth, cov3d, conic_op, rgb, clamped, touched = _preprocess(
            means3D, scales, rotations, opacities, shs, colors_precomp, cov3D_precomp, vis, cam, False)
        lib = native.lib()
        offsets = torch.empty(N, dtype=torch.int32, device=dev)
        scan_ws = _Workspace.get(dev, "scan", _lib_ll("lmb_scan_scratch_bytes")(N))
        native.check(lib.lmb_exclusive_scan_u32(touched.data_ptr(), offsets.data_ptr(), N, scan_ws.data_ptr(),
                                                native.stream_ptr()), "scan")
        total = int(offsets[-1].item()) + int(touched[-1].item())          # one host sync per frame
        n_tiles = ((W + TILE - 1) // TILE) * ((H + TILE - 1) // TILE)
        ranges = torch.empty(n_tiles, 2, dtype=torch.int32, device=dev)
        cap = max(total, 1)
        keys = torch.empty(cap, dtype=torch.int64, device=dev)
        vals = torch.empty(cap, dtype=torch.int32, device=dev)
        counters = torch.zeros(2, dtype=torch.int32, device=dev)
        native.check(lib.lmb_gs_make_keys(N, xy.data_ptr(), depth.data_ptr(), radii.data_ptr(), offsets.data_ptr(),
                                          touched.data_ptr(), W, H, cap, keys.data_ptr(), vals.data_ptr(),
                                          counters.data_ptr(), counters[1:].data_ptr(), native.stream_ptr()), "gs_make_keys")
        if total > 0:
            tile_bits = max(int(math.ceil(math.log2(max(n_tiles, 2)))), 1)
            sort_ws = _Workspace.get(dev, "sort", _lib_ll("lmb_radix_sort_scratch_bytes")(cap))
            native.check(lib.lmb_radix_sort_pairs(keys.data_ptr(), vals.data_ptr(), None, total, 0, 32 + tile_bits,
                                                  sort_ws.data_ptr(), native.stream_ptr()), "radix_sort")
        native.check(lib.lmb_gs_tile_ranges(keys.data_ptr(), None, total, ranges.data_ptr(), n_tiles, native.stream_ptr()),
                     "gs_tile_ranges")
        color = torch.empty(3, H, W, device=dev)
        final_T = torch.empty(H, W, device=dev)
        n_contrib = torch.empty(H, W, dtype=torch.int32, device=dev)
        bg = s.bg.to(dev).float().contiguous()
        native.check(lib.lmb_gs_render_fwd(ranges.data_ptr(), vals.data_ptr(), W, H, xy.data_ptr(), rgb.data_ptr(),
                                           conic_op.data_ptr(), bg.data_ptr(), color.data_ptr(), final_T.data_ptr(),
                                           n_contrib.data_ptr(), native.stream_ptr()), "gs_render_fwd")
        ctx.settings, ctx.cam = s, cam
        ctx.have = (shs is not None, colors_precomp is not None, scales is not None, cov3D_precomp is not None)
        ctx.save_for_backward(means3D, scales, rotations, shs, cov3d, radii, clamped, xy, conic_op, rgb, final_T, n_contrib,
                              ranges, vals, bg)
        alpha = 1.0 - final_T
        ctx.mark_non_differentiable(radii, alpha)
        return color, radii, alpha

    @staticmethod
    def backward(ctx, dcolor, _dradii, _dalpha):
        (means3D, scales, rotations, shs, cov3d, radii, clamped, xy, conic_op, rgb, final_T, n_contrib, ranges, vals,
         bg) = ctx.saved_tensors
        s, cam = ctx.settings, ctx.cam
        have_shs, have_cols, have_scales, have_cov = ctx.have
        N, dev = means3D.shape[0], means3D.device
        W, H = s.image_width, s.image_height
        lib = native.lib()
        dcolor = dcolor.contiguous().float()
        d_mean2D = torch.zeros(N, 2, device=dev)
        d_conic = torch.zeros(N, 3, device=dev)
        d_opacity = torch.zeros(N, 1, device=dev)
        d_rgb = torch.zeros(N, 3, device=dev)
        native.check(lib.lmb_gs_render_bwd(ranges.data_ptr(), vals.data_ptr(), W, H, bg.data_ptr(), xy.data_ptr(),
                                           conic_op.data_ptr(), rgb.data_ptr(), final_T.data_ptr(), n_contrib.data_ptr(),
                                           dcolor.data_ptr(), d_mean2D.data_ptr(), d_conic.data_ptr(), d_opacity.data_ptr(),
                                           d_rgb.data_ptr(), native.stream_ptr()), "gs_render_bwd")
        d_means = torch.zeros(N, 3, device=dev)
        d_scales = torch.zeros(N, 3, device=dev) if have_scales else None
        d_rots = torch.zeros(N, 4, device=dev) if have_scales else None
        d_shs = torch.zeros_like(shs) if have_shs else None
        d_cols = torch.zeros(N, 3, device=dev) if have_cols else None
        native.check(lib.lmb_gs_preprocess_bwd(N, means3D.data_ptr(), native.ptr(scales), native.ptr(rotations),
                                               native.ptr(shs), cov3d.data_ptr(), radii.data_ptr(), clamped.data_ptr(),
                                               byref(cam), d_mean2D.data_ptr(), d_conic.data_ptr(), d_rgb.data_ptr(),
                                               d_means.data_ptr(), native.ptr(d_scales), native.ptr(d_rots),
                                               native.ptr(d_shs), native.ptr(d_cols), int(have_scales),
                                               native.stream_ptr()), "gs_preprocess_bwd")
        # means2D receives the NDC-space screen gradient (what densification statistics accumulate)
        d_means2D = torch.cat((d_mean2D, torch.zeros(N, 1, device=dev)), -1)
        return d_means, d_means2D, d_shs, d_cols, d_opacity, d_scales, d_rots, None, None, None


class GaussianRasterizer(nn.Module):
    def __init__(self, raster_settings: GaussianRasterizationSettings):
        super().__init__()
        self.raster_settings = raster_settings

    def visible_filter(self, means3D, scales=None, rotations=None, cov3D_precomp=None):
        """Radii of the Gaussians for this view without rendering (0 = culled)."""
        s = self.raster_settings
        with torch.no_grad():
            if not means3D.is_cuda:
                xy, _, _, radii, valid = project_reference(means3D, scales, rotations, cov3D_precomp, s)
                x0, y0, x1, y1 = _tile_rect(xy, radii, s.image_width, s.image_height)
                return torch.where(valid & ((x1 - x0) * (y1 - y0) > 0), radii, torch.zeros_like(radii))
            cam = _camera_struct(s, 0)
            f = lambda t: None if t is None else t.contiguous().float()  # noqa: E731
            return _preprocess(f(means3D), f(scales), f(rotations), None, None, None, f(cov3D_precomp), None, cam, True)

    def forward(self, means3D, means2D, opacities, shs=None, colors_precomp=None, scales=None, rotations=None,
                cov3D_precomp=None, visible_mask=None):
        s = self.raster_settings
        assert (shs is None) != (colors_precomp is None), "provide exactly one of shs / colors_precomp"
        assert ((scales is None or rotations is None) != (cov3D_precomp is None)), \
            "provide exactly one of (scales, rotations) / cov3D_precomp"
        if not means3D.is_cuda:
            img, radii, alpha = rasterize_reference(means3D, opacities, s, shs, colors_precomp, scales, rotations,
                                                    cov3D_precomp, visible_mask)
            return img, radii, alpha
        if means2D is None:
            means2D = torch.zeros_like(means3D, requires_grad=means3D.requires_grad)
        return _Rasterize.apply(means3D, means2D, shs, colors_precomp, opacities, scales, rotations, cov3D_precomp,
                                visible_mask, s)
