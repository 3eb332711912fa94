"""Hand-written sm_100a operators with PyTorch reference implementations for CPU tensors."""
from .composite import composite_render, composite_weights
from .optim import FusedAdam, FusedRAdam
from .vm import vm_encode, vm_encode_reference

__all__ = ["composite_render", "composite_weights", "FusedAdam", "FusedRAdam", "vm_encode", "vm_encode_reference"]
