"""Ray bundle packed as ``[..., 7]`` = origin(3) + direction(3) + camera index(1)
(reference: landmark/nerf_components/data/rays.py:8-120)."""
from __future__ import annotations

from typing import Optional

import torch

from .tensor_dataclass import TensorDataClass


class Rays(TensorDataClass):
    def __init__(self, origin: Optional[torch.Tensor] = None, dirs: Optional[torch.Tensor] = None,
                 camera_idx: Optional[torch.Tensor] = None, near=None, far=None, data: Optional[torch.Tensor] = None,
                 rank=None, group=None, device=None, _data: Optional[torch.Tensor] = None):
        """``device`` (move the packed tensor there) and ``_data`` (alias of ``data``) are the reference's keywords
        (rays.py:8-40)."""
        data = data if data is not None else _data
        if data is None:
            assert origin is not None and dirs is not None, "Rays needs origin and dirs (or packed data)"
            if camera_idx is None:
                camera_idx = torch.zeros_like(origin[..., :1])
            elif camera_idx.dim() == origin.dim() - 1:
                camera_idx = camera_idx[..., None]
            data = torch.cat((origin, dirs, camera_idx.to(origin.dtype)), dim=-1)
        elif data.shape[-1] == 6:
            data = torch.cat((data, torch.zeros_like(data[..., :1])), dim=-1)
        assert data.shape[-1] == 7, "packed rays are [..., 7]"
        super().__init__(data if device is None else data.to(device), rank, group)
        self.near, self.far = near, far

    @property
    def origin(self) -> torch.Tensor:
        return self._data[..., 0:3]

    @property
    def dirs(self) -> torch.Tensor:
        return self._data[..., 3:6]

    @property
    def camera_idx(self) -> torch.Tensor:
        return self._data[..., 6].long()

    @property
    def nears(self):
        return self.near

    @property
    def fars(self):
        return self.far
