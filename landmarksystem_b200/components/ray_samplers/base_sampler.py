"""Sampler interface (reference: landmark/nerf_components/ray_samplers/base_sampler.py:1-17)."""
from ..model.base_module import BaseModule


class BaseSampler(BaseModule):
    def __init__(self, num_samples=None):
        super().__init__()
        self.num_samples = num_samples

    def forward(self, *args, **kwargs):
        raise NotImplementedError
