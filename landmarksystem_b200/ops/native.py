"""ctypes binding of ``liblmb200.so`` (the sm_100a kernel library built by :mod:`.build`).

The library is loaded lazily.  On a machine with a GPU a missing library is a hard error: the
CUDA path must never silently degrade to the PyTorch reference implementation.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build as _build

_LIB: Optional[ctypes.CDLL] = None
MAX_LEVELS = 4


class VMLevels(Structure):
    _fields_ = [
        ("plane", c_void_p * MAX_LEVELS),
        ("line", c_void_p * MAX_LEVELS),
        ("gplane", c_void_p * MAX_LEVELS),
        ("gline", c_void_p * MAX_LEVELS),
        ("H", c_int * MAX_LEVELS),
        ("W", c_int * MAX_LEVELS),
        ("Z", c_int * MAX_LEVELS),
        ("L", c_int),
        ("C", c_int),
        ("B", c_int),
    ]


def available() -> bool:
    return _build.library_path().exists()


def lib() -> ctypes.CDLL:
    """Return the loaded kernel library, building it on first use if sources are newer."""
    global _LIB
    if _LIB is None:
        path = _build.library_path()
        if not path.exists():
            path = _build.build_all()
        _LIB = ctypes.CDLL(str(path))
        _declare(_LIB)
    return _LIB


def _declare(L: ctypes.CDLL) -> None:
    for name in dir(L):  # nothing to iterate; kept for symmetry
        pass
    default_int = [n for n in _SIGNATURES]
    for name in default_int:
        fn = getattr(L, name, None)
        if fn is None:
            continue
        fn.restype = c_int
        fn.argtypes = _SIGNATURES[name]


P = c_void_p
_SIGNATURES = {
    "lmb_vm_encode_fwd": [P, P, c_longlong, POINTER(VMLevels), c_int, P, c_int, c_int, P, P, c_int, c_int, P],
    "lmb_vm_encode_bwd": [P, P, c_longlong, POINTER(VMLevels), c_int, P, c_int, c_int, P],
    "lmb_weights_fwd": [P, P, c_int, c_int, P, P, P],
    "lmb_weights_bwd": [P, P, P, P, c_int, c_int, P, P],
    "lmb_render_fwd": [P, P, P, c_int, c_int, c_float, P, P, P, P],
    "lmb_render_bwd": [P, P, P, c_int, c_int, c_float, P, P, P],
    "lmb_adam_step": [P, P, P, P, P, c_longlong, c_float, c_float, c_float, c_float, c_int, c_float, c_float, P],
    "lmb_radam_step": [P, P, P, P, P, c_longlong, c_float, c_float, c_float, c_float, c_int, c_float, c_float, P],
    "lmb_adam_step_dyn": [P, P, P, P, P, c_longlong, P, c_float, c_float, c_float, c_float, c_float, P],
    "lmb_adam_dyn_advance": [P, c_float, P],
    "lmb_cast_bf16": [P, P, c_longlong, P],
}


def register_signature(name: str, argtypes) -> None:
    """Let other op modules add entry points of the same library."""
    _SIGNATURES[name] = argtypes
    if _LIB is not None and hasattr(_LIB, name):
        fn = getattr(_LIB, name)
        fn.restype = c_int
        fn.argtypes = argtypes


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


LAUNCH_CALLS = 0


def check(code: int, what: str) -> None:
    """Every kernel launcher call is funnelled through here: count it and raise on a CUDA error."""
    global LAUNCH_CALLS
    LAUNCH_CALLS += 1
    if code != 0:
        raise RuntimeError(f"{what} failed with CUDA error {code}")


DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
