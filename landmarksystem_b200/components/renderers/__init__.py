from .base_renderer import BaseRenderer
from .volume_renderer import FusedVolumeRenderer, VolumeRenderer

__all__ = ["BaseRenderer", "VolumeRenderer", "FusedVolumeRenderer"]
