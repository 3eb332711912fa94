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


native.register_signature("lmb_prop_resample", [P, P, P, c_longlong, c_int, c_int, c_float, c_float, c_int, P, P])


def prop_resample(weights: torch.Tensor, existing: torch.Tensor, u: torch.Tensor, hist_pad: float, eps: float,
                  include_original: bool) -> torch.Tensor:
    """Proposal resampling: ``weights [R, E]`` over the intervals of ``existing [R, E+1]`` (ascending), ``u [R, B]``
    ascending in [0, 1) -> the ``B`` inverse-CDF positions, merged in order with ``existing`` when
    ``include_original`` (``[R, B + E + 1]``).  Not differentiable (the sampler detaches its bins)."""
    weights = weights.detach().contiguous().float()
    existing = existing.detach().contiguous().float()
    u = u.contiguous().float()
    R, E = weights.shape
    B = u.shape[1]
    out = torch.empty(R, B + E + 1 if include_original else B, device=weights.device, dtype=torch.float32)
    native.check(native.lib().lmb_prop_resample(weights.data_ptr(), existing.data_ptr(), u.data_ptr(), R, E, B, float(hist_pad),
                                                float(eps), int(include_original), out.data_ptr(), native.stream_ptr()),
                 "prop_resample")
    return out
