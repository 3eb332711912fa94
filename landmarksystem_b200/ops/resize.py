"""Channels-last bilinear resize (``csrc/resize.cu``)."""
from __future__ import annotations

from ctypes import c_float, c_int

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


native.register_signature("lmb_alpha_pool", [P, c_int, c_int, c_int, c_float, P, P, P])


def alpha_mask_pool(alpha: torch.Tensor, thre: float):
    """``alpha [X, Y, Z]`` -> (``mask [Z, Y, X]`` of 0/1 after a 3x3x3 max-pool of the clamped alpha and the
    threshold, ``bbox`` int32 ``[6]`` = min / max voxel index (x, y, z) of the occupied cells, ``max < 0`` if none)."""
    X, Y, Z = alpha.shape
    if alpha.is_cuda and native.available():
        alpha = alpha.contiguous().float()
        mask = torch.empty(Z, Y, X, device=alpha.device, dtype=torch.float32)
        bbox = torch.tensor([X, Y, Z, -1, -1, -1], device=alpha.device, dtype=torch.int32)
        native.check(native.lib().lmb_alpha_pool(alpha.data_ptr(), X, Y, Z, float(thre), mask.data_ptr(), bbox.data_ptr(),
                                                 native.stream_ptr()), "alpha_pool")
        return mask, bbox
    a = alpha.clamp(0, 1).transpose(0, 2).contiguous()[None, None]
    mask = (torch.nn.functional.max_pool3d(a, kernel_size=3, padding=1, stride=1).view(Z, Y, X) >= thre).float()
    idx = mask.nonzero()
    if idx.numel() == 0:
        return mask, torch.tensor([X, Y, Z, -1, -1, -1], dtype=torch.int32, device=alpha.device)
    lo, hi = idx.amin(0), idx.amax(0)                       # (z, y, x) order
    return mask, torch.stack((lo[2], lo[1], lo[0], hi[2], hi[1], hi[0])).to(torch.int32)
