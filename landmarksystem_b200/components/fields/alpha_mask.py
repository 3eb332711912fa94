"""Binary occupancy volume used to cull empty-space samples (reference:
landmark/nerf_components/model_components/fields/alpha_mask.py:6-129)."""
from __future__ import annotations

import torch
import torch.nn.functional as F


class AlphaGridMask(torch.nn.Module):
    def __init__(self, device, aabb: torch.Tensor, alpha_volume: torch.Tensor):
        super().__init__()
        self.device = device
        self.aabb = aabb.to(device)
        self.alpha_volume = alpha_volume.reshape(1, 1, *alpha_volume.shape[-3:]).to(device)
        self._refresh()

    def _refresh(self) -> None:
        self.aabbSize = self.aabb[1] - self.aabb[0]
        self.invgridSize = 2.0 / self.aabbSize
        d, h, w = self.alpha_volume.shape[-3:]
        self.gridSize = torch.tensor([w, h, d], dtype=torch.long, device=self.aabb.device)

    def update_device(self, device) -> None:
        self.device = device
        self.aabb = self.aabb.to(device)
        self.alpha_volume = self.alpha_volume.to(device)
        self._refresh()

    def normalize_coord(self, xyz: torch.Tensor) -> torch.Tensor:
        return (xyz - self.aabb[0]) * self.invgridSize - 1.0

    def sample_alpha(self, xyz: torch.Tensor) -> torch.Tensor:
        grid = self.normalize_coord(xyz).view(1, -1, 1, 1, 3)
        return F.grid_sample(self.alpha_volume.float(), grid, align_corners=True).view(-1)

    def generate_alpha_mask(self, xyz, filter_thresh=0, mask=None):
        if mask is None:
            return self.sample_alpha(xyz) > filter_thresh
        alpha_mask = self.sample_alpha(xyz[mask]) > filter_thresh
        valid = mask.clone()
        valid[mask] = alpha_mask
        return alpha_mask, valid

    def forward(self, xyz, filter_thresh, mask=None):
        """Return the validity mask of ``xyz`` (restricted to ``mask`` when given)."""
        if mask is None:
            return self.sample_alpha(xyz) > filter_thresh
        return self.generate_alpha_mask(xyz, filter_thresh, mask)[1]
