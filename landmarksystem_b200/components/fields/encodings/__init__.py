from .base_encoding import BaseGaussianEncoding, VolumeEncoding
from .hash_encoding import BranchParallelHashEncoding, HashEncoding
from .sh_encoding import SHEncoding
from .tensor_vm_encoding import (BranchParallelTensorVMEncoding, ChannelParallelTensorVMEncoding,
                                 FusedChannelParallelTensorVMEncoding, FusedTensorVMEncoding, TensorVMEncoding)

__all__ = ["BaseGaussianEncoding", "VolumeEncoding", "BranchParallelHashEncoding", "HashEncoding", "SHEncoding",
           "BranchParallelTensorVMEncoding", "ChannelParallelTensorVMEncoding",
           "FusedChannelParallelTensorVMEncoding", "FusedTensorVMEncoding", "TensorVMEncoding"]
