"""Hand-written sm_100a operators with PyTorch reference implementations for CPU tensors."""
from .composite import composite_render, composite_weights
from .optim import FusedAdam
from .vm import vm_encode, vm_encode_reference

__all__ = ["composite_render", "composite_weights", "FusedAdam", "vm_encode", "vm_encode_reference"]
