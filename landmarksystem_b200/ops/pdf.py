"""Inverse-CDF resampling kernel binding (``csrc/pdf.cu``)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong
from typing import Optional

import torch

from . import native

P = native.P
native.register_signature("lmb_pdf_resample", [P, P, P, c_longlong, c_int, c_int, c_float, P, P])


def pdf_resample(bins: torch.Tensor, weights: torch.Tensor, n_samples: int, u: Optional[torch.Tensor] = None,
                 eps: float = 1e-5) -> torch.Tensor:
    """``bins [R, B+1]``, ``weights [R, B]`` -> ``[R, n_samples]``; ``u [R, n_samples]`` uniform numbers, or ``None`` for the
    deterministic ``linspace(0, 1, n_samples)``."""
    bins = bins.detach().contiguous().float()
    weights = weights.detach().contiguous().float()
    R, B = weights.shape
    assert bins.shape == (R, B + 1)
    out = torch.empty(R, n_samples, device=weights.device, dtype=torch.float32)
    if u is not None:
        u = u.contiguous().float()
    native.check(native.lib().lmb_pdf_resample(bins.data_ptr(), weights.data_ptr(), native.ptr(u), R, B, n_samples, float(eps),
                                               out.data_ptr(), native.stream_ptr()), "pdf_resample")
    return out
