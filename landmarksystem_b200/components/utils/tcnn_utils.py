"""A ``tcnn``-shaped front end over this package's own hash-grid, spherical-harmonics and fused-MLP kernels.

The reference imports tiny-cuda-nn lazily through a shim (landmark/nerf_components/utils/tcnn_utils.py:18-58) and
calls ``tcnn.Encoding(n_input_dims, encoding_config)`` / ``tcnn.Network(n_input_dims, n_output_dims,
network_config)`` (hash_encoding.py:97-107, sh_encoding.py:35-38, fused_mlp_decoder.py:86-90).  Code written against
those two calls runs here unchanged: ``from landmarksystem_b200.components.utils.tcnn_utils import tcnn``.

Supported descriptions
  * ``{"otype": "HashGrid", "n_levels", "n_features_per_level", "log2_hashmap_size", "base_resolution",
    "per_level_scale"}`` - inputs in [0, 1]^3, linear interpolation;
  * ``{"otype": "SphericalHarmonics", "degree": 1..5}`` - inputs are directions mapped to [0, 1]^3;
  * ``{"otype": "FullyFusedMLP" | "CutlassMLP", "activation", "output_activation", "n_neurons",
    "n_hidden_layers"}`` - no biases, as in tiny-cuda-nn.
Anything else raises ``ValueError`` with the list above.  Modules expose ``n_input_dims``, ``n_output_dims`` and a flat
``params`` parameter view like tiny-cuda-nn's.
"""
from __future__ import annotations

from types import SimpleNamespace
from typing import Mapping, Optional

import torch
from torch import nn

TCNN_EXISTS = True          # the compatible front end below is always importable
tcnn_import_exception = None

_ACTIVATIONS = {"relu": nn.ReLU, "sigmoid": nn.Sigmoid, "tanh": nn.Tanh, "softplus": nn.Softplus,
                "leaky relu": nn.LeakyReLU, "none": None}


def _activation(name: Optional[str]):
    key = (name or "None").strip().lower()
    if key not in _ACTIVATIONS:
        raise ValueError(f"activation '{name}' is not supported (supported: {sorted(_ACTIVATIONS)})")
    cls = _ACTIVATIONS[key]
    return None if cls is None else cls()


class Encoding(nn.Module):
    """``tcnn.Encoding``: a multiresolution hash grid or a spherical-harmonics basis."""

    def __init__(self, n_input_dims: int, encoding_config: Mapping, dtype: Optional[torch.dtype] = None,
                 device=None):
        super().__init__()
        cfg = dict(encoding_config)
        kind = str(cfg.get("otype", "")).lower()
        assert n_input_dims == 3, "three input dimensions (positions or directions)"
        self.n_input_dims, self.dtype = n_input_dims, dtype or torch.float32
        dev = device or ("cuda" if torch.cuda.is_available() else "cpu")
        if kind == "hashgrid":
            from ..fields.encodings.hash_encoding import HashEncoding

            levels, base = int(cfg.get("n_levels", 16)), int(cfg.get("base_resolution", 16))
            scale = float(cfg.get("per_level_scale", 2.0))
            assert str(cfg.get("interpolation", "Linear")) == "Linear", "only linear interpolation is implemented"
            self.inner = HashEncoding(levels, base, base * scale ** max(levels - 1, 0),
                                      int(cfg.get("log2_hashmap_size", 19)), int(cfg.get("n_features_per_level", 2)),
                                      device=dev)
            self.n_output_dims = self.inner.get_out_dim()
        elif kind == "sphericalharmonics":
            from ..fields.encodings.sh_encoding import SHEncoding

            self.inner = SHEncoding(levels=int(cfg.get("degree", 4)), unit_range=True)
            self.n_output_dims = self.inner.get_out_dim()
        else:
            raise ValueError(f"encoding '{cfg.get('otype')}' is not supported (supported: HashGrid, SphericalHarmonics)")
        self.encoding_config = cfg

    @property
    def params(self) -> torch.Tensor:
        own = list(self.inner.parameters())
        return own[0] if own else torch.zeros(0)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = self.inner(x.reshape(-1, 3).float())
        return out.to(self.dtype).reshape(*x.shape[:-1], self.n_output_dims)


class Network(nn.Module):
    """``tcnn.Network``: a bias-free MLP of ``n_hidden_layers`` hidden layers of ``n_neurons`` units; on a GPU it runs
    through the fused tensor-core kernels whenever the shape is one they cover."""

    def __init__(self, n_input_dims: int, n_output_dims: int, network_config: Mapping, device=None):
        super().__init__()
        from ..fields.mlp_decoder import MLPDecoder

        cfg = dict(network_config)
        kind = str(cfg.get("otype", "FullyFusedMLP")).lower()
        if kind not in ("fullyfusedmlp", "cutlassmlp"):
            raise ValueError(f"network '{cfg.get('otype')}' is not supported (supported: FullyFusedMLP, CutlassMLP)")
        if str(cfg.get("activation", "ReLU")).strip().lower() != "relu":
            raise ValueError("hidden activation must be ReLU")
        self.n_input_dims, self.n_output_dims = n_input_dims, n_output_dims
        dev = device or ("cuda" if torch.cuda.is_available() else "cpu")
        self.inner = MLPDecoder(n_input_dims, int(cfg.get("n_neurons", 64)), int(cfg.get("n_hidden_layers", 1)) + 1,
                                n_output_dims, _activation(cfg.get("output_activation")), mlp_bias=False).to(dev)
        self.inner.use_fused = True
        self.network_config = cfg

    @property
    def params(self) -> torch.Tensor:
        """All weights flattened into one vector (a copy: the layers keep their own storage)."""
        return torch.cat([p.reshape(-1) for p in self.inner.parameters()])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.inner(x.reshape(-1, self.n_input_dims)).reshape(*x.shape[:-1], self.n_output_dims)


class NetworkWithInputEncoding(nn.Module):
    """``tcnn.NetworkWithInputEncoding``: an :class:`Encoding` feeding a :class:`Network`."""

    def __init__(self, n_input_dims: int, n_output_dims: int, encoding_config: Mapping, network_config: Mapping,
                 device=None):
        super().__init__()
        self.encoding = Encoding(n_input_dims, encoding_config, device=device)
        self.network = Network(self.encoding.n_output_dims, n_output_dims, network_config, device=device)
        self.n_input_dims, self.n_output_dims = n_input_dims, n_output_dims

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.network(self.encoding(x))


tcnn = SimpleNamespace(Encoding=Encoding, Network=Network, NetworkWithInputEncoding=NetworkWithInputEncoding)
