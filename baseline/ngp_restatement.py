"""PyTorch restatement of one Instant-NGP training step (baseline arm, labelled "restatement").

The reference trains Instant-NGP through tiny-cuda-nn (hash grid, fully fused MLPs, SH encoding) and nerfacc (occupancy
grid marching): benchmarks/nerf/instant_ngp/instant_ngp.py:120-170 (field), :225-289 (forward), :316-326 (grid refresh),
instant_ngp_trainer.py:124-125 (DistributedDataParallel).  Neither extension is in this image and neither can be
fetched offline, so the reference's own Instant-NGP cannot run here.  This file states the same training step with plain
PyTorch operators only - no kernel of this framework is imported - and is timed on the same GPU as the baseline of the
Instant-NGP figure: multiresolution hash grid (dense index where the level fits, XOR-of-primes hash above), trilinear
blend, 1x64 density head with truncated-exp density, SH degree-4 view encoding, 2x64 colour head with an appearance
embedding, occupancy-grid marching with a fixed step, opacity culling under ``no_grad``, alpha compositing, MSE loss,
``torch.optim.Adam``; bf16 autocast for the heads (tiny-cuda-nn runs them in half precision).

The samples of a ray batch do not fit the autograd graph of tensor ops at once (8 corner gathers x 16 levels per
sample), so the step walks the rays in chunks and accumulates gradients - what a PyTorch user has to do.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

PRIMES = (1, 2654435761, 805459861)
C0 = 0.28209479177387814
C1 = 0.4886025119029199
C2 = (1.0925484305920792, -1.0925484305920792, 0.31539156525252005, -1.0925484305920792, 0.5462742152960396)
C3 = (-0.5900435899266435, 2.890611442640554, -0.4570457994644658, 0.3731763325901154, -0.4570457994644658,
      1.445305721320277, -0.5900435899266435)


def sh16(d: torch.Tensor) -> torch.Tensor:
    x, y, z = d.unbind(-1)
    xx, yy, zz, xy, yz, xz = x * x, y * y, z * z, x * y, y * z, x * z
    return torch.stack((torch.full_like(x, C0), -C1 * y, C1 * z, -C1 * x,
                        C2[0] * xy, C2[1] * yz, C2[2] * (2 * zz - xx - yy), C2[3] * xz, C2[4] * (xx - yy),
                        C3[0] * y * (3 * xx - yy), C3[1] * xy * z, C3[2] * y * (4 * zz - xx - yy),
                        C3[3] * z * (2 * zz - 3 * xx - 3 * yy), C3[4] * x * (4 * zz - xx - yy), C3[5] * z * (xx - yy),
                        C3[6] * x * (xx - 3 * yy)), -1)


class HashGrid(nn.Module):
    def __init__(self, levels=16, features=2, log2_size=22, base_res=16, max_res=8192):
        super().__init__()
        growth = math.exp((math.log(max_res) - math.log(base_res)) / (levels - 1))
        self.features = features
        self.scales, self.res, self.offsets = [], [], [0]
        for l in range(levels):
            scale = growth ** l * base_res - 1.0
            res = int(math.ceil(scale)) + 1
            entries = min((res ** 3 + 7) // 8 * 8, 1 << log2_size)
            self.scales.append(scale)
            self.res.append(res)
            self.offsets.append(self.offsets[-1] + entries)
        self.table = nn.Parameter((torch.rand(self.offsets[-1], features) * 2 - 1) * 1e-4)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        outs = []
        for l, (scale, res) in enumerate(zip(self.scales, self.res)):
            entries = self.offsets[l + 1] - self.offsets[l]
            tab = self.table[self.offsets[l]:self.offsets[l + 1]]
            p = x * scale + 0.5
            p0 = p.floor()
            w = p - p0
            p0 = p0.long().clamp_min(0)
            acc = 0
            for c in range(8):
                dx, dy, dz = c & 1, (c >> 1) & 1, (c >> 2) & 1
                ix, iy, iz = ((p0[:, k] + o).clamp_max(res - 1) for k, o in enumerate((dx, dy, dz)))
                if res ** 3 <= entries:
                    index = ix + iy * res + iz * res * res
                else:
                    index = (((ix * PRIMES[0]) ^ (iy * PRIMES[1]) ^ (iz * PRIMES[2])) & 0xFFFFFFFF) % entries
                wt = (w[:, 0] if dx else 1 - w[:, 0]) * (w[:, 1] if dy else 1 - w[:, 1]) * (w[:, 2] if dz else 1 - w[:, 2])
                acc = acc + tab[index] * wt[:, None]
            outs.append(acc)
        return torch.cat(outs, -1)


class TruncExp(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        ctx.save_for_backward(x)
        return torch.exp(x)

    @staticmethod
    def backward(ctx, g):
        return g * torch.exp(ctx.saved_tensors[0].clamp(-15, 15))


class Field(nn.Module):
    def __init__(self, geo=15, app_dim=32, n_cameras=1024, hidden=64, **grid):
        super().__init__()
        self.grid = HashGrid(**grid)
        width = self.grid.features * len(self.grid.res)
        self.base = nn.Sequential(nn.Linear(width, hidden, bias=False), nn.ReLU(), nn.Linear(hidden, 1 + geo, bias=False))
        self.head = nn.Sequential(nn.Linear(16 + geo + app_dim, hidden, bias=False), nn.ReLU(),
                                  nn.Linear(hidden, hidden, bias=False), nn.ReLU(), nn.Linear(hidden, 3, bias=False), nn.Sigmoid())
        self.embedding = nn.Embedding(n_cameras, app_dim)

    def density(self, x01: torch.Tensor):
        inside = ((x01 > 0) & (x01 < 1)).all(-1)
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=x01.is_cuda):
            h = self.base(self.grid(x01 * inside[:, None])).float()
        return TruncExp.apply(h[:, :1]) * inside[:, None], h[:, 1:] * inside[:, None]

    def colour(self, dirs: torch.Tensor, geo: torch.Tensor, app: torch.Tensor) -> torch.Tensor:
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=dirs.is_cuda):
            return self.head(torch.cat((sh16(F.normalize(dirs, dim=-1)), geo, app), -1)).float()


class Trainer:
    """``aabb``: ``[[lo], [hi]]``; ``step``: marching step in world units; one occupancy cascade of ``grid_res^3`` cells."""

    def __init__(self, aabb, step: float, max_samples: int, device, alpha_thre: float = 0.01, grid_res: int = 128,
                 lr: float = 1e-2, chunk_rays: int = 1 << 14, **grid):
        self.aabb = torch.as_tensor(aabb, dtype=torch.float32, device=device)
        self.step, self.max_samples, self.alpha_thre, self.chunk = step, max_samples, alpha_thre, chunk_rays
        self.field = Field(**grid).to(device)
        self.opt = torch.optim.Adam(self.field.parameters(), lr=lr, eps=1e-15)
        self.grid_res = grid_res
        self.occ = torch.zeros(grid_res ** 3, device=device)
        self.binary = torch.ones(grid_res, grid_res, grid_res, dtype=torch.bool, device=device)
        self.iteration = 0

    def _norm(self, p):
        return (p - self.aabb[0]) / (self.aabb[1] - self.aabb[0])

    @torch.no_grad()
    def refresh_grid(self, decay: float = 0.95, thre: float = 0.01):
        r = self.grid_res
        idx = torch.arange(r ** 3, device=self.occ.device)
        ijk = torch.stack((idx // (r * r), (idx // r) % r, idx % r), -1).float()
        x01 = (ijk + torch.rand_like(ijk)) / r
        sigma = torch.cat([self.field.density(c)[0] for c in x01.split(1 << 20)])[:, 0]
        self.occ = torch.maximum(self.occ * decay, sigma * self.step)
        self.binary = (self.occ > min(float(self.occ.mean()), thre)).view(r, r, r)

    @torch.no_grad()
    def march(self, o, d):
        """Fixed-step marching between the ray's entry and exit of the box: ``(t_mid [R, S], valid [R, S])``."""
        inv = 1.0 / torch.where(d.abs() > 1e-12, d, torch.full_like(d, 1e-12))
        a, b = (self.aabb[0] - o) * inv, (self.aabb[1] - o) * inv
        t0 = torch.minimum(a, b).amax(-1).clamp_min(0.0)
        t1 = torch.maximum(a, b).amin(-1)
        k = torch.arange(self.max_samples, device=o.device)[None] + torch.rand(o.shape[0], 1, device=o.device)
        t = t0[:, None] + (k + 0.5) * self.step
        valid = (t < t1[:, None]) & (t1 > t0)[:, None]
        x01 = self._norm(o[:, None] + d[:, None] * t[..., None])
        cell = (x01 * self.grid_res).long().clamp(0, self.grid_res - 1)
        valid &= self.binary[cell[..., 0], cell[..., 1], cell[..., 2]]
        return t, valid

    def train_step(self, rays: torch.Tensor, target: torch.Tensor, camera: torch.Tensor) -> float:
        if self.iteration % 16 == 0:
            self.refresh_grid()
        self.iteration += 1
        self.opt.zero_grad(set_to_none=True)
        total, n_rays = torch.zeros((), device=rays.device), rays.shape[0]
        for lo in range(0, n_rays, self.chunk):
            o, d = rays[lo:lo + self.chunk, :3], rays[lo:lo + self.chunk, 3:6]
            t, valid = self.march(o, d)
            R, S = t.shape
            idx = valid.reshape(-1).nonzero(as_tuple=True)[0]
            ray = idx // S
            x01 = self._norm(o[ray] + d[ray] * t.reshape(-1)[idx][:, None])
            with torch.no_grad():                                   # opacity culling, as nerfacc does before the real pass
                sig = torch.zeros(R * S, device=rays.device)
                sig[idx] = self.field.density(x01)[0][:, 0]
                alpha = 1.0 - torch.exp(-sig.view(R, S) * self.step)
                trans = torch.cumprod(torch.cat((torch.ones_like(alpha[:, :1]), 1.0 - alpha), -1), -1)[:, :-1]
                keep = (valid & (alpha >= self.alpha_thre) & (trans >= 1e-4)).reshape(-1)[idx]
            idx, ray, x01 = idx[keep], ray[keep], x01[keep]
            sigma, geo = self.field.density(x01)
            app = self.field.embedding(camera[lo:lo + self.chunk].long())[ray]
            rgb = self.field.colour(d[ray], geo, app)
            sig_full = torch.zeros(R * S, device=rays.device).index_put((idx,), sigma[:, 0]).view(R, S)
            rgb_full = torch.zeros(R * S, 3, device=rays.device).index_put((idx,), rgb).view(R, S, 3)
            alpha = 1.0 - torch.exp(-sig_full * self.step)
            trans = torch.cumprod(torch.cat((torch.ones_like(alpha[:, :1]), 1.0 - alpha + 1e-10), -1), -1)[:, :-1]
            w = alpha * trans
            image = (w[..., None] * rgb_full).sum(1).clamp(0, 1)
            loss = ((image - target[lo:lo + self.chunk]) ** 2).sum() / (3 * n_rays)
            loss.backward()
            total += loss.detach()
        self.opt.step()
        return float(total)
