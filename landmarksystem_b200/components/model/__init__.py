from .base_model import BaseGaussian, BaseNeRF, Model
from .base_module import BaseModule

__all__ = ["BaseGaussian", "BaseNeRF", "Model", "BaseModule"]
