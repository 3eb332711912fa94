from .rays import Rays
from .samples import Samples
from .tensor_dataclass import TensorDataClass

__all__ = ["Rays", "Samples", "TensorDataClass"]
