"""Class-name swap tables used by the convertors (reference:
landmark/nerf_components/components_convertor/convert_maps.py:19-47)."""
from ..components.fields.anchor_decoder import AnchorDecoder, FusedAnchorDecoder
from ..components.fields.encodings.hash_encoding import BranchParallelHashEncoding, HashEncoding
from ..components.fields.encodings.tensor_vm_encoding import (BranchParallelTensorVMEncoding,
                                                              ChannelParallelTensorVMEncoding, TensorVMEncoding)
from ..components.fields.fused_mlp_decoder import FusedMLPDecoder
from ..components.fields.mlp_decoder import MLPDecoder
from ..components.ray_samplers.uniform_sampler import FusedUniformSampler, UniformSampler

CHANNEL_PARALLEL_MAP = {TensorVMEncoding: ChannelParallelTensorVMEncoding}
BRANCH_PARALLEL_MAP = {TensorVMEncoding: BranchParallelTensorVMEncoding, HashEncoding: BranchParallelHashEncoding}
ELEM_PARALLEL_MAP = {}
KERNEL_FUSION_MAP = {MLPDecoder: FusedMLPDecoder, UniformSampler: FusedUniformSampler,
                     AnchorDecoder: FusedAnchorDecoder}
PARALLEL_MAPS = {"ChannelParallel": CHANNEL_PARALLEL_MAP, "BranchParallel": BRANCH_PARALLEL_MAP,
                 "ElemParallel": ELEM_PARALLEL_MAP}
