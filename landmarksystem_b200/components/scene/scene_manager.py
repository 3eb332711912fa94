"""Scene geometry: global AABB, XY block partition and coordinate normalisation
(reference: landmark/nerf_components/scene/scene_manager.py:10-133).

``block_partition = [nx, ny]`` splits the AABB footprint into ``nx*ny`` blocks, block id
``bx*ny + by``.  For dynamic loading only a window (``local_block_partition`` blocks whose first
block is ``relative_block_idx``) is resident; ids are then relative to that window.
"""
from __future__ import annotations

from typing import Sequence

import torch

from ..data.samples import Samples


class SceneManager:
    def __init__(self, config):
        self.config = config
        device = getattr(config, "device", "cpu")
        if isinstance(device, str) and device.startswith("cuda") and not torch.cuda.is_available():
            device = "cpu"
        self.device = torch.device(device) if not isinstance(device, torch.device) else device
        lb = torch.as_tensor(config.lb, dtype=torch.float32)
        ub = torch.as_tensor(config.ub, dtype=torch.float32)
        self.aabb = torch.stack((lb, ub)).to(self.device)
        rng = getattr(config, "aabb_norm_range", None) or [-1.0, 1.0]
        self.aabb_norm_range = torch.tensor(rng, dtype=torch.float32, device=self.device)
        self.aabb_norm_size = float(rng[1] - rng[0])
        self._norm_lo = float(rng[0])
        part = getattr(config, "plane_division", None) or [1, 1]
        self.block_partition = torch.tensor(list(part), dtype=torch.long, device=self.device)
        self._partition = (int(part[0]), int(part[1]))     # host copy: reading the tensor would synchronise
        self._refresh()
        local = getattr(config, "local_block_partition", None)
        self.local_block_partition = list(local) if local is not None else [int(v) for v in part]
        self.assign_relative_block_idx(getattr(config, "relative_block_idx", 0))

    def _refresh(self) -> None:
        self.aabb_size = self.aabb[1] - self.aabb[0]
        self.invaabbSize = self.aabb_norm_size / self.aabb_size
        self.block_width = self.aabb_size[:2] / self.block_partition
        self.norm_block_width = self.aabb_norm_size / self.block_partition.float()

    @property
    def n_blocks(self) -> int:
        return self._partition[0] * self._partition[1]

    @property
    def n_local_blocks(self) -> int:
        return int(self.local_block_partition[0] * self.local_block_partition[1])

    def to(self, device):
        self.device = torch.device(device)
        self.aabb = self.aabb.to(device)
        self.aabb_norm_range = self.aabb_norm_range.to(device)
        self.block_partition = self.block_partition.to(device)
        self._refresh()
        return self

    # -- partition bookkeeping ---------------------------------------------------
    def assign_block_partition(self, block_partition: Sequence[int]) -> None:
        self.block_partition = torch.tensor(list(block_partition), dtype=torch.long, device=self.device)
        self._partition = (int(block_partition[0]), int(block_partition[1]))
        self._refresh()

    def assign_local_block_partition(self, local_block_partition: Sequence[int]) -> None:
        self.local_block_partition = [int(v) for v in local_block_partition]

    def assign_relative_block_idx(self, relative_block_idx: int = 0) -> None:
        ny = self._partition[1]
        self.relative_block_idx = int(relative_block_idx)
        self.relative_block_idx_x = self.relative_block_idx // ny
        self.relative_block_idx_y = self.relative_block_idx % ny

    def select_block_idx(self, rays) -> torch.Tensor:
        """Global id of the block under the first ray's origin (the camera position)."""
        data = rays.data if hasattr(rays, "data") and not torch.is_tensor(rays) else rays
        xy = torch.floor((data[0, :2] - self.aabb[0, :2]) / self.block_width)
        xy = torch.minimum(torch.clamp(xy, min=0), (self.block_partition - 1).to(xy.dtype))
        return (xy[0] * self.block_partition[1] + xy[1]).to(torch.int)

    # -- coordinates ----------------------------------------------------------------
    def normalize_coord(self, xyz: torch.Tensor) -> torch.Tensor:
        if xyz.shape[-1] == 3:
            return (xyz - self.aabb[0]) * self.invaabbSize + self.aabb_norm_range[0]
        assert xyz.shape[-1] == 4, "expected xyz or xyzb"
        out = xyz.clone().detach()
        out[..., :3] = (xyz[..., :3] - self.aabb[0]) * self.invaabbSize + self.aabb_norm_range[0]
        return out

    @torch.no_grad()
    def block_local_coords(self, xyz_norm: torch.Tensor):
        """Map globally-normalised xyz to ``(block-local xyz in [-1, 1], window-relative block id)``.
        Samples outside the resident window get id ``-1``."""
        lo = self.aabb_norm_range[0]
        nx, ny = self._partition
        lx, ly = self.local_block_partition
        u = (xyz_norm[..., 0] - lo) / self.norm_block_width[0]
        v = (xyz_norm[..., 1] - lo) / self.norm_block_width[1]
        bx = torch.floor(u).clamp(0, nx - 1)
        by = torch.floor(v).clamp(0, ny - 1)
        rx, ry = bx - self.relative_block_idx_x, by - self.relative_block_idx_y
        inside = (rx >= 0) & (rx < lx) & (ry >= 0) & (ry < ly)
        block = torch.where(inside, rx * ly + ry, torch.full_like(rx, -1.0))
        # block-local coordinates are always expressed in [-1, 1] (what the lookup kernels expect)
        local = torch.stack(((u - bx) * 2.0 - 1.0, (v - by) * 2.0 - 1.0,
                             (xyz_norm[..., 2] - lo) / self.aabb_norm_size * 2.0 - 1.0), dim=-1)
        return local, block

    @torch.no_grad()
    def assign_blockIdx(self, samples: Samples, norm_coord: bool = False) -> Samples:
        """In place: set ``samples.block_idx`` (window-relative) and per-block ``masks``; with
        ``norm_coord`` also rewrite xyz to block-local ``[-1, 1]`` coordinates."""
        local, block = self.block_local_coords(samples.xyz)
        samples.block_idx = block
        n_local = self.n_local_blocks
        samples.masks = torch.stack([block == b for b in range(n_local)], dim=0)
        if norm_coord:
            samples._data[..., 9:12] = local
        return samples

    def filter_valid_samples(self, samples: Samples):
        inside = ~((samples.xyz < self.aabb[0]) | (samples.xyz > self.aabb[1])).any(dim=-1)
        return inside, samples[inside]
