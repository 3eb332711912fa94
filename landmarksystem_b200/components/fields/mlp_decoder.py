"""Small fully-connected decoders and the sin/cos positional encoding (reference:
landmark/nerf_components/model_components/fields/mlp_decoder.py:8-109).

``MLPDecoder`` keeps its weights in ordinary ``nn.Linear`` layers (so checkpoints carry the
reference's ``mlp.{i}.weight`` names).  On CUDA tensors, shapes supported by the tcgen05 fused-MLP
kernel run through it (see :mod:`landmarksystem_b200.ops.fused_mlp`); everything else, and every
CPU tensor, runs the plain layer-by-layer path.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..model.base_module import BaseModule


def positional_encoding(positions: torch.Tensor, freqs: int) -> torch.Tensor:
    """``[sin(x_d * 2^f) ...  cos(x_d * 2^f) ...]`` with index ``d * freqs + f`` inside each half."""
    bands = 2.0 ** torch.arange(freqs, device=positions.device, dtype=torch.float32)
    pts = (positions[..., None] * bands).reshape(*positions.shape[:-1], freqs * positions.shape[-1])
    return torch.cat((torch.sin(pts), torch.cos(pts)), dim=-1)


class MLPDecoder(BaseModule):
    def __init__(self, inChanel: int, layer_width: int = 128, num_layers: Optional[int] = None,
                 out_dim: Optional[int] = None, out_activation: Optional[torch.nn.Module] = None,
                 mlp_bias: bool = True):
        super().__init__()
        self.mlp_bias = mlp_bias
        self.in_dim, self.width, self.num_layers, self.out_dim = inChanel, layer_width, num_layers, out_dim
        layers = []
        dims = [inChanel] + [layer_width] * (num_layers - 1) + [out_dim]
        for i in range(num_layers):
            layers.append(torch.nn.Linear(dims[i], dims[i + 1], bias=mlp_bias))
            if i < num_layers - 1:
                layers.append(torch.nn.ReLU(inplace=True))
        if out_activation is not None:
            layers.append(out_activation)
        self.mlp = torch.nn.Sequential(*layers)
        self.out_activation = out_activation
        self.use_fused = False  # flipped by the runtime convertor / FusedMLPDecoder
        self.save_init_kwargs(locals())

    def linears(self):
        return [m for m in self.mlp if isinstance(m, torch.nn.Linear)]

    def forward(self, features, precomputed: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``features``: ``[N, K]`` or a sequence of ``[N, k_i]`` parts (concatenated along the last dimension; the
        fused path writes them straight into the kernel's bf16 input instead of materialising the concatenation)."""
        first = features[0] if isinstance(features, (tuple, list)) else features
        if self.use_fused and first.is_cuda:
            from ...ops.fused_mlp import fused_mlp_supported, mlp_forward

            if fused_mlp_supported(self):
                return mlp_forward(self, features, precomputed)
        if isinstance(features, (tuple, list)):
            features = torch.cat([f.to(first.dtype) for f in features], dim=-1)
        return self.mlp(features)
