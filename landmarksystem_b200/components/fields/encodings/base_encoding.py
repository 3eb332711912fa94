"""Encoding base classes (reference:
landmark/nerf_components/model_components/fields/encodings/base_encoding.py:10-67)."""
from __future__ import annotations

from ...model.base_module import BaseModule


class VolumeEncoding(BaseModule):
    """Maps sample positions to feature vectors."""

    def forward(self, xyzb):
        raise NotImplementedError

    def feature2density(self, feature):
        raise NotImplementedError


class BaseGaussianEncoding(BaseModule):
    """Parameter store of a point-based (Gaussian / anchor) representation."""

    def create_from_pcd(self, pcd, spatial_lr_scale: float = 1.0):
        raise NotImplementedError

    def save_ply(self, path: str):
        raise NotImplementedError

    def load_ply_to_state_dict(self, path: str, map_location="cpu"):
        raise NotImplementedError

    def load_encoding_state(self, state):
        raise NotImplementedError
