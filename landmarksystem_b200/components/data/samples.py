"""Point samples along rays packed as ``[..., 13]`` fp32:
``sigma(1) rgb(3) camera_idx(1) z_vals(1) dirs(3) xyz(3) block_idx(1)``
(column order of the reference, landmark/nerf_components/data/samples.py:104).

Differences by design: the block index stays an integer-valued float (the lookup kernels index the
block directly; :attr:`block_coord` gives the reference's ``[-1, 1]`` depth coordinate), and the
cross-rank ``sync_sigma`` / ``sync_rgb`` exchange goes through the communication layer's
variable-length gather instead of list all-gathers preceded by host syncs
(reference: samples.py:283-309).
"""
from __future__ import annotations

from typing import Optional

import torch

from .tensor_dataclass import TensorDataClass

_SIGMA, _RGB, _CAM, _Z, _DIRS, _XYZ, _BLK = 0, slice(1, 4), 4, 5, slice(6, 9), slice(9, 12), 12


class Samples(TensorDataClass):
    WIDTH = 13

    def __init__(self, xyz: Optional[torch.Tensor] = None, dirs: Optional[torch.Tensor] = None,
                 z_vals: Optional[torch.Tensor] = None, camera_idx: Optional[torch.Tensor] = None,
                 block_idx: Optional[torch.Tensor] = None, sigma: Optional[torch.Tensor] = None,
                 rgb: Optional[torch.Tensor] = None, data: Optional[torch.Tensor] = None, rank=None, group=None,
                 device=None, _data: Optional[torch.Tensor] = None):
        data = data if data is not None else _data          # ``_data`` / ``device``: the reference's keywords
        self._has_z_vals = z_vals is not None
        self._has_camera_idx = camera_idx is not None
        self._has_block_idx = block_idx is not None
        self.masks = None
        if data is None:
            assert xyz is not None, "Samples needs xyz (or packed data)"
            lead = xyz.shape[:-1]
            data = torch.zeros(*lead, self.WIDTH, device=xyz.device, dtype=torch.float32)
            data[..., _XYZ] = xyz
            if dirs is not None:
                data[..., _DIRS] = dirs
            if z_vals is not None:
                data[..., _Z] = z_vals
            if camera_idx is not None:
                data[..., _CAM] = camera_idx.reshape(lead).to(torch.float32)
            if block_idx is not None:
                data[..., _BLK] = block_idx.reshape(lead).to(torch.float32)
            if sigma is not None:
                data[..., _SIGMA] = sigma
            if rgb is not None:
                data[..., _RGB] = rgb
        else:
            self._has_z_vals = self._has_camera_idx = self._has_block_idx = True
        super().__init__(data if device is None else data.to(device), rank, group)

    # -- field views ------------------------------------------------------------
    @property
    def xyz(self):
        return self._data[..., _XYZ]

    @xyz.setter
    def xyz(self, value):
        self._assign(_XYZ, value)

    @property
    def xyzb(self):
        assert self._has_block_idx, "the block index of the samples has not been assigned"
        return self._data[..., 9:13]

    @property
    def dirs(self):
        return self._data[..., _DIRS]

    @property
    def z_vals(self):
        return self._data[..., _Z] if self._has_z_vals else None

    @property
    def camera_idx(self):
        return self._data[..., _CAM].long() if self._has_camera_idx else None

    @property
    def block_idx(self):
        return self._data[..., _BLK].long() if self._has_block_idx else None

    @block_idx.setter
    def block_idx(self, value):
        self._set(_BLK, value.to(torch.float32))
        self._has_block_idx = True

    @property
    def block_coord(self):
        """Reference-style depth coordinate of the block in the stacked plane tensor."""
        n_blocks = 1 if self.masks is None else self.masks.shape[0]
        return -1.0 + 2.0 * self._data[..., _BLK] / (n_blocks - 1 + 1e-6)

    @property
    def sigma(self):
        return self._data[..., _SIGMA]

    @sigma.setter
    def sigma(self, value):
        self._assign(_SIGMA, value)

    @property
    def rgb(self):
        return self._data[..., _RGB]

    @rgb.setter
    def rgb(self, value):
        self._assign(_RGB, value)

    @property
    def dists(self):
        z = self.z_vals
        return torch.cat((z[..., 1:] - z[..., :-1], torch.zeros_like(z[..., :1])), dim=-1)

    def _set(self, cols, value):
        self._data[..., cols] = value
        return self._data

    def _assign(self, cols, value):
        """Write a field; when ``value`` carries autograd history the packed tensor is rebuilt
        out-of-place so gradients flow (the reference uses ``scatter`` for the same purpose,
        samples.py:152-198)."""
        if torch.is_tensor(value) and value.requires_grad:
            parts = list(self._data.unbind(-1))
            if isinstance(cols, slice):
                for i, c in enumerate(range(cols.start, cols.stop)):
                    parts[c] = value[..., i]
            else:
                parts[cols] = value
            self._data = torch.stack(parts, dim=-1)
        else:
            self._set(cols, value)

    def __getitem__(self, item):
        new = super().__getitem__(item)
        new.masks = None
        return new

    def __setitem__(self, item, value):
        assert isinstance(value, Samples), "the value to be set must be a Samples object"
        super().__setitem__(item, value)
        self._has_z_vals, self._has_camera_idx, self._has_block_idx = (
            value._has_z_vals, value._has_camera_idx, value._has_block_idx)

    # -- model-parallel exchange ----------------------------------------------------
    @property
    def mask(self):
        assert self.rank is not None and self.masks is not None
        return self.masks[self.rank]

    def _sync(self, cols, width: int) -> None:
        from ...comm.varlen import all_gather_varlen  # late import: comm needs torch.distributed

        own = self._data[..., cols][self.mask].reshape(-1, width)
        pieces = all_gather_varlen(own, group=self.group)
        flat = self._data.reshape(-1, self.WIDTH)
        for r, (mask, piece) in enumerate(zip(self.masks, pieces)):
            if r == self.rank:
                continue  # own slot already holds the (differentiable) local values
            idx = mask.reshape(-1).nonzero(as_tuple=True)[0]
            if width == 1:
                flat[idx, cols] = piece[:, 0]
            else:
                flat[idx, cols] = piece

    def sync_sigma(self) -> None:
        self._sync(_SIGMA, 1)

    def sync_rgb(self) -> None:
        self._sync(_RGB, 3)
