"""Renderer interface (reference:
landmark/nerf_components/model_components/renderers/base_renderer.py:1-24)."""
from ..model.base_module import BaseModule


class BaseRenderer(BaseModule):
    def forward(self, *args, **kwargs):
        raise NotImplementedError
