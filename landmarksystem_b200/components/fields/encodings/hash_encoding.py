"""Multiresolution hash-grid encoding with one table per spatial block (reference:
landmark/nerf_components/model_components/fields/encodings/hash_encoding.py:15-223).

The reference delegates to tiny-cuda-nn and routes blocks with a python loop over boolean masks;
here each block's table is a slice of one parameter tensor per block (checkpoint keys
``tcnn_encoding.params`` / ``tcnn_encoding.{i}.params`` are kept) and block routing happens in a
sort-free way: samples are grouped by block index once and each group runs the hash-grid kernel.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch
from torch import nn
from typing_extensions import Literal

from ....ops.hashgrid import hashgrid_encode, make_meta
from ....render.types import MergeType
from .base_encoding import VolumeEncoding


class _Table(nn.Module):
    """Holder that gives the parameter the name ``params`` (as ``tcnn.Encoding`` does)."""

    def __init__(self, n_params: int, device, init: Optional[torch.Tensor] = None):
        super().__init__()
        data = init if init is not None else (torch.rand(n_params, device=device) * 2 - 1) * 1e-4
        self.params = nn.Parameter(data.to(device).float())


class HashEncoding(VolumeEncoding):
    def __init__(self, num_levels: int = 16, min_res: int = 16, max_res: int = 1024, log2_hashmap_size: int = 19,
                 features_per_level: int = 2,
                 interpolation: Optional[Literal["Nearest", "Linear", "Smoothstep"]] = None, device="cpu",
                 num_hash_table: int = 1):
        super().__init__()
        assert interpolation in (None, "Linear"), "only linear interpolation is implemented"
        self.in_dim = 3
        self.num_levels, self.features_per_level = num_levels, features_per_level
        self.log2_hashmap_size, self.hash_table_size = log2_hashmap_size, 2 ** log2_hashmap_size
        self.min_res, self.max_res, self.device = min_res, max_res, device
        self.num_hash_table = num_hash_table
        growth = float(np.exp((np.log(max_res) - np.log(min_res)) / (num_levels - 1))) if num_levels > 1 else 1.0
        self.meta = make_meta(num_levels, features_per_level, log2_hashmap_size, min_res, growth)
        self.init_hash_table()
        self.save_init_kwargs(locals())
        self.merge_config = {"merge_type": MergeType.List, "tcnn_encoding.*.params": 0}

    def init_hash_table(self):
        n = self.meta.n_params
        if self.num_hash_table > 1:
            self.tcnn_encoding = nn.ModuleList([_Table(n, self.device) for _ in range(self.num_hash_table)])
        else:
            self.tcnn_encoding = _Table(n, self.device)

    def tables(self):
        return list(self.tcnn_encoding) if isinstance(self.tcnn_encoding, nn.ModuleList) else [self.tcnn_encoding]

    def get_out_dim(self) -> int:
        return self.meta.out_dim

    def enable_table_shadow(self) -> None:
        """Give every table a persistent fp32 gradient accumulator and a bf16 copy for the lookup kernel to read (both
        maintained by the fused Adam kernel)."""
        from ....ops import FusedAdam

        for table in self.tables():
            if table.params.is_cuda and getattr(table.params, "_lmb_shadow", None) is None:
                FusedAdam.attach_sink(table.params, shadow=True)
                table.params._lmb_shadow_version = table.params._version

    def _encode(self, xyz: torch.Tensor, table: _Table, out_dtype=torch.float32, precomputed=None) -> torch.Tensor:
        p, F = table.params, self.features_per_level
        shadow, sink = getattr(p, "_lmb_shadow", None), getattr(p, "_lmb_grad_sink", None)
        if shadow is not None and xyz.is_cuda:
            if p._version != getattr(p, "_lmb_shadow_version", None):      # the master was written outside the optimiser
                shadow.copy_(p.detach())                                    # kernel (a checkpoint load): refresh the copy
                p._lmb_shadow_version = p._version
            return hashgrid_encode(xyz, p.view(-1, F), self.meta, out_dtype, shadow=shadow.view(-1, F),
                                   sink=None if sink is None else sink.view(-1, F), precomputed=precomputed)
        return hashgrid_encode(xyz, p.view(-1, F), self.meta, out_dtype, precomputed=precomputed)

    def forward(self, xyz: torch.Tensor, out_dtype=torch.float32, precomputed=None) -> torch.Tensor:
        """``xyz [N, 3]`` in ``[0, 1]`` or ``[N, 4]`` with the block index in the last column.  ``out_dtype`` /
        ``precomputed`` (single table only): see :func:`landmarksystem_b200.ops.hashgrid.hashgrid_encode`."""
        if xyz.shape[-1] == 3 or self.num_hash_table == 1:
            return self._encode(xyz[:, :3], self.tables()[0], out_dtype, precomputed)
        block = xyz[:, 3].long()
        out = torch.zeros(xyz.shape[0], self.meta.out_dim, device=xyz.device, dtype=torch.float32)
        for b, table in enumerate(self.tables()):
            if table.params.numel() == 0:        # not resident (dynamic loading): its samples are masked by the caller
                continue
            idx = (block == b).nonzero(as_tuple=True)[0]
            if idx.numel():
                out = out.index_put((idx,), self._encode(xyz[idx, :3], table))
        return out

    def merge_state_dicts(self, state_dicts, device="cpu"):
        """Per-rank single-table states -> one multi-table state (``tcnn_encoding.{i}.params``)."""
        merged = {}
        for i, sd in enumerate(state_dicts):
            for key, value in sd.items():
                merged[key.replace("tcnn_encoding.params", f"tcnn_encoding.{i}.params")] = value.to(device)
        return merged


class BranchParallelHashEncoding(HashEncoding):
    """One table per rank; the initial tables of all blocks are drawn on rank 0 and broadcast so the
    run starts from the same values as a single-process multi-table run."""

    def __init__(self, parallel_degree=1, parallel_part=0, group=None, init_state_dict=None, **kwargs):
        self.parallel_degree, self.parallel_part, self.group = parallel_degree, parallel_part, group
        self.init_state_dict = init_state_dict
        kwargs["num_hash_table"] = 1
        super().__init__(**kwargs)

    def init_hash_table(self):
        import torch.distributed as dist

        n = self.meta.n_params
        if self.init_state_dict is not None:
            key = f"tcnn_encoding.{self.parallel_part}.params"
            init = self.init_state_dict.get(key, self.init_state_dict.get("tcnn_encoding.params"))
            self.tcnn_encoding = _Table(n, self.device, init.clone())
            return
        full = (torch.rand(n, self.parallel_degree, device=self.device) * 2 - 1) * 1e-4
        if dist.is_initialized() and self.parallel_degree > 1:
            src = dist.get_global_rank(self.group, 0) if self.group is not None else 0
            dist.broadcast(full, src=src, group=self.group)
        self.tcnn_encoding = _Table(n, self.device, full[:, self.parallel_part].clone())
