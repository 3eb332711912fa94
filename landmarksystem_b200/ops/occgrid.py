"""Multi-level occupancy grid: estimator state, grid update and ray marching.

Stands in for ``nerfacc.OccGridEstimator`` as the reference uses it
(benchmarks/nerf/instant_ngp/instant_ngp.py:146-150,316-326 and
landmark/nerf_components/ray_samplers/volumetric_sampler.py:92-104): ``resolution^3`` cells x ``levels``
cascades (cascade ``l`` spans the region of interest scaled by ``2^l``), an exponential moving maximum
of sampled densities per cell, a binary grid thresholded at ``min(mean, occ_thre)``, and marching that
emits samples ``[t, t+dt]`` in occupied cells with ``dt = max(t * cone_angle, step)``.

Marching writes the padded ``[R, max_samples]`` layout directly (``counts[r]`` valid samples per ray).
"""
from __future__ import annotations

from ctypes import c_float, c_int
from typing import Callable, Optional, Tuple

import torch

from . import native

P = native.P
native.register_signature("lmb_occ_march", [c_int, P, P, P, P, P, c_int, c_int, c_float, c_float, c_float, c_float, c_int,
                                             P, P, P, P])


def march_reference(rays_o, rays_d, jitter, binaries, roi, near, far, step, cone_angle, max_samples):
    """Plain-python statement of the marching rule (per ray loops; tiny inputs only)."""
    levels, res = binaries.shape[0], binaries.shape[1]
    lo, hi = roi[:3], roi[3:]
    c, h = 0.5 * (lo + hi), 0.5 * (hi - lo)
    R = rays_o.shape[0]
    counts = torch.zeros(R, dtype=torch.int32)
    ts = torch.zeros(R, max_samples)
    te = torch.zeros(R, max_samples)
    grow = float(1 << (levels - 1))
    for r in range(R):
        o, d = rays_o[r], rays_d[r]
        dd = torch.where(d.abs() > 1e-12, d, torch.where(d >= 0, torch.tensor(1e-12), torch.tensor(-1e-12)))
        a, b = (c - h * grow - o) / dd, (c + h * grow - o) / dd
        t0 = max(float(torch.minimum(a, b).max()), near)
        t1 = min(float(torch.maximum(a, b).min()), far)
        if float(torch.minimum(a, b).max()) >= float(torch.maximum(a, b).min()):
            continue
        t = t0
        if jitter is not None:
            t += float(jitter[r]) * max(t * cone_angle, step)
        n = 0
        while t < t1 and n < max_samples:
            dt = max(t * cone_angle, step)
            p = o + (t + 0.5 * dt) * d
            m = float(((p - c).abs() / h).max())
            l = 0
            while l < levels - 1 and m > (1 << l):
                l += 1
            if m > (1 << l):
                t += dt
                continue
            s = float(1 << l)
            u = ((p - c) / (h * s) * 0.5 + 0.5) * res
            idx = u.long().clamp(0, res - 1)
            if binaries[l, idx[0], idx[1], idx[2]]:
                ts[r, n], te[r, n] = t, t + dt
                n += 1
                t += dt
            else:
                texit = float("inf")
                for k in range(3):
                    if abs(float(d[k])) < 1e-12:
                        continue
                    edge = float(idx[k] + 1) if d[k] > 0 else float(idx[k])
                    world = float(c[k]) + ((edge / res - 0.5) * 2.0) * float(h[k]) * s
                    texit = min(texit, (world - float(o[k])) / float(d[k]))
                while True:
                    t += max(t * cone_angle, step)
                    if not (t + 0.5 * max(t * cone_angle, step) < texit and t < t1):
                        break
        counts[r] = n
    return counts, ts, te


class OccGridEstimator(torch.nn.Module):
    def __init__(self, roi_aabb, resolution: int = 128, levels: int = 1):
        super().__init__()
        roi = torch.as_tensor(roi_aabb, dtype=torch.float32).reshape(6)
        self.register_buffer("roi_aabb", roi)
        self.resolution, self.levels = int(resolution), int(levels)
        n = self.levels * self.resolution ** 3
        self.register_buffer("occs", torch.zeros(n))
        self.register_buffer("binaries", torch.ones(self.levels, resolution, resolution, resolution, dtype=torch.bool))
        self._roi_host = roi.tolist()

    # -- marching ---------------------------------------------------------------------------------
    @torch.no_grad()
    def sampling(self, rays_o, rays_d, sigma_fn: Optional[Callable] = None, near_plane: float = 0.0,
                 far_plane: float = 1e10, render_step_size: float = 1e-3, stratified: bool = False,
                 cone_angle: float = 0.0, alpha_thre: float = 0.0, max_samples: int = 1024,
                 early_stop_eps: float = 1e-4) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Returns ``(counts [R], t_starts [R, S], t_ends [R, S])`` with ``S = max_samples``.
        With ``sigma_fn`` and ``alpha_thre > 0`` samples whose opacity is below the threshold, or that
        lie behind an (almost) opaque prefix, are dropped and the survivors are compacted to the front."""
        R = rays_o.shape[0]
        dev = rays_o.device
        self.last_cull = None
        jitter = torch.rand(R, device=dev) if stratified else None
        if rays_o.is_cuda:
            counts = torch.empty(R, dtype=torch.int32, device=dev)
            ts = torch.zeros(R, max_samples, device=dev)
            te = torch.zeros(R, max_samples, device=dev)
            roi = (c_float * 6)(*self._roi_host)
            cells = self.binaries.to(torch.uint8).contiguous()
            native.check(native.lib().lmb_occ_march(R, rays_o.contiguous().float().data_ptr(),
                                                    rays_d.contiguous().float().data_ptr(), native.ptr(jitter),
                                                    cells.data_ptr(), roi, self.resolution, self.levels, float(near_plane),
                                                    float(far_plane), float(render_step_size), float(cone_angle),
                                                    int(max_samples), counts.data_ptr(), ts.data_ptr(), te.data_ptr(),
                                                    native.stream_ptr()), "occ_march")
        else:
            counts, ts, te = march_reference(rays_o.float(), rays_d.float(), jitter, self.binaries, self.roi_aabb,
                                             near_plane, far_plane, render_step_size, cone_angle, max_samples)
        if sigma_fn is not None and alpha_thre > 0.0 and rays_o.is_cuda:
            # kernel path: densities of the marched samples (the callback may take the padded block directly and build the
            # positions with its own kernel), then one warp per ray culls and compacts in place
            from . import ngp_field

            valid = torch.arange(max_samples, device=dev)[None] < counts[:, None]
            idx = valid.reshape(-1).nonzero(as_tuple=True)[0]
            if idx.numel():
                full = idx.numel() == R * max_samples
                if hasattr(sigma_fn, "from_samples"):
                    dens = sigma_fn.from_samples(None if full else idx, max_samples, ts, te).reshape(-1).float()
                else:
                    dens = sigma_fn(ts.reshape(-1)[idx], te.reshape(-1)[idx], idx // max_samples).reshape(-1).float()
                sig = dens if full else torch.zeros(R * max_samples, device=dev).index_put_((idx,), dens)
                src = ngp_field.occ_cull(sig.contiguous(), ts, te, counts, alpha_thre, early_stop_eps, want_source=True)
                # which marched sample every survivor was: a field that cached per-sample results of the density query
                # can reuse them for the survivors (``queried``: flat indices the query covered, None = all R x S)
                self.last_cull = {"queried": None if full else idx, "source": src, "n_queried": idx.numel()}
        elif sigma_fn is not None and alpha_thre > 0.0:
            valid = torch.arange(max_samples, device=dev)[None] < counts[:, None]
            idx = valid.reshape(-1).nonzero(as_tuple=True)[0]
            if idx.numel():
                ray = idx // max_samples
                sig = torch.zeros(R * max_samples, device=dev)
                sig[idx] = sigma_fn(ts.reshape(-1)[idx], te.reshape(-1)[idx], ray).reshape(-1).float()
                sig = sig.view(R, max_samples)
                alpha = 1.0 - torch.exp(-sig * (te - ts))
                trans = torch.cumprod(torch.cat((torch.ones_like(alpha[:, :1]), 1.0 - alpha), -1), -1)[:, :-1]
                keep = valid & (alpha >= alpha_thre) & (trans >= early_stop_eps)
                order = torch.argsort((~keep).to(torch.int8), dim=1, stable=True)   # survivors first, order kept
                ts, te = torch.gather(ts, 1, order), torch.gather(te, 1, order)
                counts = keep.sum(1).to(torch.int32)
        return counts, ts, te

    # -- grid update ---------------------------------------------------------------------------------------
    def _cell_centers(self, level: int, idx: torch.Tensor, jitter: bool = True) -> torch.Tensor:
        res = self.resolution
        lo, hi = self.roi_aabb[:3], self.roi_aabb[3:]
        c, h = 0.5 * (lo + hi), 0.5 * (hi - lo) * float(1 << level)
        ijk = torch.stack((idx // (res * res), (idx // res) % res, idx % res), -1).float()
        u = (ijk + (torch.rand_like(ijk) if jitter else 0.5)) / res
        return c + (u * 2.0 - 1.0) * h

    @torch.no_grad()
    def update_every_n_steps(self, step: int, occ_eval_fn: Callable, occ_thre: float = 1e-2, ema_decay: float = 0.95,
                             warmup_steps: int = 256, n: int = 16) -> None:
        if not self.training or step % n != 0:
            return
        res3 = self.resolution ** 3
        dev = self.occs.device
        on_gpu = self.occs.is_cuda and native.available()
        if on_gpu:
            from . import ngp_field

            self._refresh_count = getattr(self, "_refresh_count", 0) + 1
        for level in range(self.levels):
            if step < warmup_steps:
                idx = None if on_gpu else torch.arange(res3, device=dev)
            else:
                m = res3 // 4
                uniform = torch.randint(res3, (m,), device=dev)
                occupied = self.binaries[level].reshape(-1).nonzero(as_tuple=True)[0]
                if occupied.numel() > m:
                    occupied = occupied[torch.randint(occupied.numel(), (m,), device=dev)]
                idx = torch.cat((uniform, occupied))
            view = self.occs[level * res3:(level + 1) * res3]
            if on_gpu:
                # cell centres + decayed old value, the density query, then the two-pass maximum: three launches around
                # the field evaluation instead of the index arithmetic, gather and scatter as tensor ops
                seed = (step * 131 + level * 7919 + self._refresh_count * 104729) & 0x7FFFFFFF
                xyz, decayed = ngp_field.occ_cells(idx, res3, self.resolution, self._roi_host, level, seed, True, view,
                                                   ema_decay)
                ngp_field.occ_update(idx, decayed, occ_eval_fn(xyz).reshape(-1), view)
                continue
            occ = occ_eval_fn(self._cell_centers(level, idx)).reshape(-1).float()
            view[idx] = torch.maximum(view[idx] * ema_decay, occ)
        if on_gpu:
            if getattr(self, "_sum_scratch", None) is None or self._sum_scratch.device != dev:
                self._sum_scratch = torch.zeros(1, device=dev, dtype=torch.float64)
            if not self.binaries.is_contiguous():
                self.binaries = self.binaries.contiguous()
            ngp_field.occ_binarise(self.occs, occ_thre, self.binaries.view(torch.uint8), self._sum_scratch)
            return
        thre = min(float(self.occs.mean()), occ_thre)
        self.binaries = (self.occs > thre).view(self.binaries.shape)
