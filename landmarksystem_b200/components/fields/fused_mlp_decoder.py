"""``MLPDecoder`` variant that always takes the tcgen05 fused-MLP kernel on GPU tensors.

The reference's counterpart swaps in tiny-cuda-nn networks and only supports bias-free layers
(landmark/nerf_components/model_components/fields/fused_mlp_decoder.py:37-105); this one keeps the
same parameters as ``MLPDecoder`` (biases included), so a checkpoint loads into either class.
"""
from .mlp_decoder import MLPDecoder


def activation_to_tcnn_string(activation) -> str:
    """Name of a ``torch.nn`` activation in tiny-cuda-nn's vocabulary (``"ReLU"``, ``"Leaky ReLU"``, ``"Sigmoid"``,
    ``"Softplus"``, ``"Tanh"``, ``"None"``), the vocabulary the reference's network descriptions use
    (fused_mlp_decoder.py:9-34)."""
    import torch

    names = ((torch.nn.ReLU, "ReLU"), (torch.nn.LeakyReLU, "Leaky ReLU"), (torch.nn.Sigmoid, "Sigmoid"),
             (torch.nn.Softplus, "Softplus"), (torch.nn.Tanh, "Tanh"), (type(None), "None"))
    for cls, name in names:
        if isinstance(activation, cls):
            return name
    raise ValueError(f"activation {activation} has no fused counterpart (supported: {[n for _, n in names]})")


class FusedMLPDecoder(MLPDecoder):
    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.use_fused = True
