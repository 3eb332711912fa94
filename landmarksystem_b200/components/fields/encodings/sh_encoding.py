"""Spherical-harmonics direction encoding, degree <= 4 -> 16 outputs (reference:
landmark/nerf_components/model_components/fields/encodings/sh_encoding.py:6-59, which wraps
``tcnn.Encoding("SphericalHarmonics")``).  Directions are given in ``[0, 1]`` (tiny-cuda-nn's
convention) when ``unit_range`` is set, else as unit vectors.  CUDA tensors go through ``sh_encode_kernel``
(``ops/csrc/ngp_field.cu``), CPU tensors through the PyTorch statement of the basis."""
import torch

from ...model.base_module import BaseModule


class SHEncoding(BaseModule):
    def __init__(self, levels: int = 4, unit_range: bool = True) -> None:
        super().__init__()
        assert 1 <= levels <= 5, "SH encoding supports 1..5 levels (degree 0..4)"
        self.levels, self.unit_range = levels, unit_range
        self.save_init_kwargs(locals())

    def get_out_dim(self) -> int:
        return self.levels ** 2

    def forward(self, dirs: torch.Tensor) -> torch.Tensor:
        from ....ops.ngp_field import sh_encode

        return sh_encode(dirs, self.levels, self.unit_range)
