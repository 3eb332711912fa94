"""Python side of the tcgen05 fused-MLP kernels (see ``csrc/fused_mlp.cu``)."""
from __future__ import annotations

import torch


def fused_mlp_supported(decoder) -> bool:
    return False


def mlp_forward(decoder, features: torch.Tensor) -> torch.Tensor:
    raise NotImplementedError


def rgb_decoder_supported(decoder) -> bool:
    return False


def rgb_decoder_forward(decoder, dirs, feats):
    raise NotImplementedError


def anchor_heads_supported(decoder, *inputs) -> bool:
    return False


def anchor_heads_forward(decoder, *inputs):
    raise NotImplementedError
