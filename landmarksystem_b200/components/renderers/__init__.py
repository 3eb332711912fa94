from .base_renderer import BaseRenderer
from .gaussian_splatting_rasterizer import GassianSplattingRasterizer, GaussianSplattingRasterizer
from .volume_renderer import FusedVolumeRenderer, VolumeRenderer

__all__ = ["BaseRenderer", "VolumeRenderer", "FusedVolumeRenderer", "GaussianSplattingRasterizer",
           "GassianSplattingRasterizer"]
