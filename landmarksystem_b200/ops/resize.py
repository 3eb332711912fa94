"""Channels-last bilinear resize (``csrc/resize.cu``)."""
from __future__ import annotations

from ctypes import c_int

import torch

from . import native

P = native.P
native.register_signature("lmb_resize_bilinear_nhwc", [P, P, c_int, c_int, c_int, c_int, c_int, c_int, P])


def resize_bilinear_nhwc(src: torch.Tensor, H2: int, W2: int) -> torch.Tensor:
    """``src [B, H, W, C]`` fp32 -> ``[B, H2, W2, C]`` (align_corners bilinear).  CPU tensors use ``F.interpolate``."""
    B, H, W, C = src.shape
    if not src.is_cuda or C % 4 or src.dtype != torch.float32:
        out = torch.nn.functional.interpolate(src.permute(0, 3, 1, 2).float(), size=(H2, W2), mode="bilinear", align_corners=True)
        return out.permute(0, 2, 3, 1).contiguous().to(src.dtype)
    src = src.contiguous()
    dst = torch.empty(B, H2, W2, C, device=src.device, dtype=torch.float32)
    native.check(native.lib().lmb_resize_bilinear_nhwc(src.data_ptr(), dst.data_ptr(), B, H, W, H2, W2, C, native.stream_ptr()),
                 "resize_bilinear_nhwc")
    return dst


def resize_linear_nlc(src: torch.Tensor, Z2: int) -> torch.Tensor:
    """``src [B, Z, C]`` -> ``[B, Z2, C]`` (align_corners linear)."""
    return resize_bilinear_nhwc(src[:, :, None, :], Z2, 1)[:, :, 0, :].contiguous()
