"""PyTorch restatement of the 3D Gaussian splatting render / training step (baseline arm, labelled "restatement").

The reference renders Gaussians with its ``opt_gaussian_rasterization`` CUDA extension
(call sites: benchmarks/nerf/origin_gs/gs_model.py:211-220, 297-331); that submodule is empty in the reference
checkout and cannot be fetched offline, so the reference's own rasteriser cannot be built.  This file states the same
math with plain PyTorch operators only - no kernel of this framework is imported - and is timed on the same GPU as the
baseline of the 3DGS figures: projection + 2-D covariance + radius, degree-3 spherical harmonics, (tile, depth) key
sort, per-tile front-to-back alpha blending, differentiated by autograd, optimised by ``torch.optim.Adam``.

It follows the published 3DGS algorithm: a Gaussian is duplicated into every 16x16 tile its 3-sigma square overlaps,
pairs are sorted by (tile, depth), every tile blends its list front to back with alpha = min(0.99, o * exp(-q / 2)),
contributions below 1/255 are skipped and a pixel stops once its transmittance drops below 1e-4.
"""
from __future__ import annotations

import math

import torch

C0 = 0.28209479177387814
C1 = 0.4886025119029199
C2 = (1.0925484305920792, -1.0925484305920792, 0.31539156525252005, -1.0925484305920792, 0.5462742152960396)
C3 = (-0.5900435899266435, 2.890611442640554, -0.4570457994644658, 0.3731763325901154, -0.4570457994644658,
      1.445305721320277, -0.5900435899266435)


def orbit_camera(k: int, device, W: int = 1920, H: int = 1080, focal: float = 1400.0, radius: float = 260.0,
                 height: float = 120.0, znear: float = 0.01, zfar: float = 2000.0):
    """Pose ``k`` of the benchmark's 300-pose orbit around the origin (z up): ``(view, proj, campos, tanfovx, tanfovy)``
    with the matrices in the row-vector convention of the reference cameras (graphics_utils.py:43-77):
    ``view = W2C^T`` with x right, y down, z forward; ``proj = view @ P^T``."""
    ang = 2 * math.pi * (k % 300) / 300.0
    eye = torch.tensor([radius * math.cos(ang), radius * math.sin(ang), height], dtype=torch.float64)
    fwd = -eye / eye.norm()
    right = torch.linalg.cross(fwd, torch.tensor([0.0, 0.0, 1.0], dtype=torch.float64))
    right = right / right.norm()
    down = torch.linalg.cross(fwd, right)
    c2w = torch.eye(4, dtype=torch.float64)
    c2w[:3, 0], c2w[:3, 1], c2w[:3, 2], c2w[:3, 3] = right, down, fwd, eye
    view = torch.linalg.inv(c2w).t().float()
    tanx, tany = W / (2.0 * focal), H / (2.0 * focal)
    P = torch.zeros(4, 4)
    P[0, 0], P[1, 1], P[3, 2] = 1.0 / tanx, 1.0 / tany, 1.0
    P[2, 2], P[2, 3] = zfar / (zfar - znear), -(zfar * znear) / (zfar - znear)
    proj = view @ P.t()
    return view.to(device), proj.to(device), eye.float().to(device), tanx, tany


def eval_sh3(sh: torch.Tensor, d: torch.Tensor) -> torch.Tensor:
    """``sh [N, 16, 3]``, unit directions ``d [N, 3]`` -> rgb ``[N, 3]`` (degree 3, +0.5, clamped at 0)."""
    x, y, z = d[:, 0:1], d[:, 1:2], d[:, 2:3]
    xx, yy, zz, xy, yz, xz = x * x, y * y, z * z, x * y, y * z, x * z
    r = C0 * sh[:, 0] - C1 * y * sh[:, 1] + C1 * z * sh[:, 2] - C1 * x * sh[:, 3]
    r = r + C2[0] * xy * sh[:, 4] + C2[1] * yz * sh[:, 5] + C2[2] * (2 * zz - xx - yy) * sh[:, 6] \
        + C2[3] * xz * sh[:, 7] + C2[4] * (xx - yy) * sh[:, 8]
    r = r + C3[0] * y * (3 * xx - yy) * sh[:, 9] + C3[1] * xy * z * sh[:, 10] + C3[2] * y * (4 * zz - xx - yy) * sh[:, 11] \
        + C3[3] * z * (2 * zz - 3 * xx - 3 * yy) * sh[:, 12] + C3[4] * x * (4 * zz - xx - yy) * sh[:, 13] \
        + C3[5] * z * (xx - yy) * sh[:, 14] + C3[6] * x * (xx - 3 * yy) * sh[:, 15]
    return torch.clamp_min(r + 0.5, 0.0)


def quat_to_rot(q: torch.Tensor) -> torch.Tensor:
    q = torch.nn.functional.normalize(q, dim=-1)
    r, x, y, z = q.unbind(-1)
    return torch.stack((1 - 2 * (y * y + z * z), 2 * (x * y - r * z), 2 * (x * z + r * y),
                        2 * (x * y + r * z), 1 - 2 * (x * x + z * z), 2 * (y * z - r * x),
                        2 * (x * z - r * y), 2 * (y * z + r * x), 1 - 2 * (x * x + y * y)), -1).view(-1, 3, 3)


def render(means, log_scales, quats, opacity_logit, sh, view, proj, campos, W: int, H: int, tanfovx: float, tanfovy: float,
           bg: torch.Tensor, tile: int = 16) -> torch.Tensor:
    """``view`` / ``proj``: world->camera and full projection matrices in the row-vector convention of the reference
    cameras (``p_cam = [p, 1] @ view``).  Returns the image ``[3, H, W]``."""
    N = means.shape[0]
    ones = torch.ones(N, 1, device=means.device)
    p_view = torch.cat((means, ones), -1) @ view
    depth = p_view[:, 2]
    p_hom = torch.cat((means, ones), -1) @ proj
    ndc = p_hom[:, :2] / (p_hom[:, 3:4] + 1e-7)
    px = ((ndc[:, 0] + 1.0) * W - 1.0) * 0.5
    py = ((ndc[:, 1] + 1.0) * H - 1.0) * 0.5
    # 3-D covariance and its EWA projection
    R = quat_to_rot(quats)
    M = R * torch.exp(log_scales)[:, None, :]
    cov3 = M @ M.transpose(1, 2)
    fx, fy = W / (2.0 * tanfovx), H / (2.0 * tanfovy)
    tz = depth.clamp_min(1e-6)
    tx = (p_view[:, 0] / tz).clamp(-1.3 * tanfovx, 1.3 * tanfovx) * tz
    ty = (p_view[:, 1] / tz).clamp(-1.3 * tanfovy, 1.3 * tanfovy) * tz
    zero = torch.zeros_like(tz)
    J = torch.stack((fx / tz, zero, -fx * tx / (tz * tz), zero, fy / tz, -fy * ty / (tz * tz)), -1).view(N, 2, 3)
    Wm = view[:3, :3].t()
    T = J @ Wm
    cov2 = T @ cov3 @ T.transpose(1, 2)
    a, b, c = cov2[:, 0, 0] + 0.3, cov2[:, 0, 1], cov2[:, 1, 1] + 0.3
    det = a * c - b * b
    conic = torch.stack((c, -b, a), -1) / det[:, None]
    mid = 0.5 * (a + c)
    lam = mid + torch.sqrt(torch.clamp_min(mid * mid - det, 0.1))
    radius = torch.ceil(3.0 * torch.sqrt(lam))
    dirs = torch.nn.functional.normalize(means - campos[None], dim=-1)
    rgb = eval_sh3(sh, dirs)
    opac = torch.sigmoid(opacity_logit).reshape(-1)
    # tile rectangles
    tx_n, ty_n = (W + tile - 1) // tile, (H + tile - 1) // tile
    with torch.no_grad():
        x0 = ((px - radius) / tile).floor().clamp(0, tx_n).long()
        x1 = ((px + radius + tile - 1) / tile).floor().clamp(0, tx_n).long()
        y0 = ((py - radius) / tile).floor().clamp(0, ty_n).long()
        y1 = ((py + radius + tile - 1) / tile).floor().clamp(0, ty_n).long()
        ok = (depth > 0.2) & (det > 0) & (x1 > x0) & (y1 > y0)
        nx, ny = (x1 - x0) * ok, (y1 - y0) * ok
        count = nx * ny
        gid = torch.repeat_interleave(torch.arange(N, device=means.device), count)
        start = torch.cumsum(count, 0) - count
        local = torch.arange(gid.shape[0], device=means.device) - start[gid]
        tile_x = x0[gid] + local % nx[gid].clamp_min(1)
        tile_y = y0[gid] + local // nx[gid].clamp_min(1)
        tile_id = tile_y * tx_n + tile_x
        # sort by depth, then (stably) by tile: lists per tile in front-to-back order
        order = torch.argsort(depth[gid], stable=True)
        order = order[torch.argsort(tile_id[order], stable=True)]
        gid, tile_id = gid[order], tile_id[order]
        bounds = torch.searchsorted(tile_id, torch.arange(tx_n * ty_n + 1, device=means.device))
        bounds_host = bounds.tolist()
    image = bg.view(3, 1, 1).expand(3, ty_n * tile, tx_n * tile).clone()
    ys, xs = torch.meshgrid(torch.arange(tile, device=means.device, dtype=torch.float32),
                            torch.arange(tile, device=means.device, dtype=torch.float32), indexing="ij")
    for t in range(tx_n * ty_n):
        lo, hi = bounds_host[t], bounds_host[t + 1]
        if hi <= lo:
            continue
        g = gid[lo:hi]
        oy, ox = (t // tx_n) * tile, (t % tx_n) * tile
        dx = (ox + xs).reshape(1, -1) - px[g, None]
        dy = (oy + ys).reshape(1, -1) - py[g, None]
        power = -0.5 * (conic[g, 0:1] * dx * dx + conic[g, 2:3] * dy * dy) - conic[g, 1:2] * dx * dy
        alpha = torch.clamp_max(opac[g, None] * torch.exp(power), 0.99)
        alpha = torch.where((power <= 0) & (alpha >= 1.0 / 255.0), alpha, torch.zeros_like(alpha))
        trans = torch.cumprod(1.0 - alpha, 0)
        trans_before = torch.cat((torch.ones_like(trans[:1]), trans[:-1]), 0)
        alpha = alpha * (trans_before >= 1e-4)
        w = alpha * trans_before
        col = (w[:, None, :] * rgb[g, :, None]).sum(0) + trans[-1][None] * bg.view(3, 1)
        image[:, oy:oy + tile, ox:ox + tile] = col.view(3, tile, tile)
    return image[:, :H, :W]


def l1_ssim_loss(img: torch.Tensor, target: torch.Tensor, lam: float = 0.2) -> torch.Tensor:
    """``(1 - lam) * L1 + lam * (1 - SSIM)`` with the 11x11 Gaussian window of the reference
    (landmark/nerf_components/utils/loss_utils.py:14-61)."""
    import torch.nn.functional as F

    g = torch.tensor([math.exp(-(x - 5) ** 2 / (2 * 1.5 ** 2)) for x in range(11)], device=img.device)
    g = (g / g.sum())[:, None]
    win = (g @ g.t())[None, None].expand(3, 1, 11, 11).contiguous()
    a, b = img[None], target[None]
    mu1, mu2 = F.conv2d(a, win, padding=5, groups=3), F.conv2d(b, win, padding=5, groups=3)
    s1 = F.conv2d(a * a, win, padding=5, groups=3) - mu1 * mu1
    s2 = F.conv2d(b * b, win, padding=5, groups=3) - mu2 * mu2
    s12 = F.conv2d(a * b, win, padding=5, groups=3) - mu1 * mu2
    ssim = ((2 * mu1 * mu2 + 1e-4) * (2 * s12 + 9e-4)) / ((mu1 * mu1 + mu2 * mu2 + 1e-4) * (s1 + s2 + 9e-4))
    return (1 - lam) * (img - target).abs().mean() + lam * (1 - ssim.mean())
