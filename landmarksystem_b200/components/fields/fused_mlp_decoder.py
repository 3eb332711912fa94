"""``MLPDecoder`` variant that always takes the tcgen05 fused-MLP kernel on GPU tensors.

The reference's counterpart swaps in tiny-cuda-nn networks and only supports bias-free layers
(landmark/nerf_components/model_components/fields/fused_mlp_decoder.py:37-105); this one keeps the
same parameters as ``MLPDecoder`` (biases included), so a checkpoint loads into either class.
"""
from .mlp_decoder import MLPDecoder


class FusedMLPDecoder(MLPDecoder):
    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.use_fused = True
