"""VM-decomposed feature grid (planes x lines) with spatial-block, channel-parallel and
branch-parallel variants.

Behavioural counterpart of the reference's ``TensorVMEncoding`` family
(landmark/nerf_components/model_components/fields/encodings/tensor_vm_encoding.py:20-636).
Storage is re-designed for the memory system: planes live channels-last ``[B, H, W, C]`` and lines
``[B, Z, C]`` (fp32 masters, optional bf16 shadows read by the kernels), so one texel is one or a
few 32-byte sectors.  ``state_dict()`` / ``load_state_dict()`` still speak the reference layout
(``plane_coef.k [1, C, B, H, W]``, ``line_coef.k [1, C, Z, B]``), so checkpoints are interchangeable.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from ....ops import vm_encode
from ....render.types import MergeType
from .base_encoding import VolumeEncoding


def _plane_to_ref(p: torch.Tensor) -> torch.Tensor:      # [B,H,W,C] -> [1,C,B,H,W]
    return p.permute(3, 0, 1, 2).unsqueeze(0).contiguous()


def _plane_from_ref(p: torch.Tensor) -> torch.Tensor:    # [1,C,B,H,W] -> [B,H,W,C]
    return p[0].permute(1, 2, 3, 0).contiguous()


def _line_to_ref(l: torch.Tensor) -> torch.Tensor:       # [B,Z,C] -> [1,C,Z,B]
    return l.permute(2, 1, 0).unsqueeze(0).contiguous()


def _line_from_ref(l: torch.Tensor) -> torch.Tensor:     # [1,C,Z,B] -> [B,Z,C]
    return l[0].permute(2, 1, 0).contiguous()


def tv_term(plane: torch.Tensor) -> torch.Tensor:
    """Total-variation of channels-last planes ``[B, H, W, C]``; equals the reference ``TVLoss`` on
    ``[1, C, H, W]`` summed in the same normalisation (utils/loss_utils.py:64-82)."""
    B, H, W, C = plane.shape
    dh = (plane[:, 1:] - plane[:, :-1]).pow(2).sum()
    dw = (plane[:, :, 1:] - plane[:, :, :-1]).pow(2).sum()
    count_h = C * max(H - 1, 1) * W * B
    count_w = C * H * max(W - 1, 1) * B
    return 2.0 * (dh / count_h + dw / count_w)


class TensorVMEncoding(VolumeEncoding):
    """``ndims`` (plane, line) pairs x ``len(resolution_mode)`` levels; parameter index
    ``k = pair * n_levels + level``.  Only the XY-plane / Z-line pair (``ndims == 1``) is spatially
    partitioned into blocks, as in every shipped configuration of the reference."""

    _MATRIX_MODE = [[0, 1], [0, 2], [1, 2]]
    _VECTOR_MODE = [2, 1, 0]

    def __init__(self, ndims: int, resolution_mode: List[int], n_component, grid_size, device,
                 param_shape: Optional[Dict[str, Sequence[int]]] = None, n_blocks: int = 1, scale: float = 0.1):
        super().__init__()
        self.ndims = ndims
        self.matrix_mode = self._MATRIX_MODE[:ndims]
        self.vector_mode = self._VECTOR_MODE[:ndims]
        comps = list(n_component) if isinstance(n_component, (list, tuple)) else [n_component] * 3
        self.n_component = comps[:ndims]
        self.reso_mode = list(resolution_mode)
        self.device = device
        self.is_channel_last = True  # native layout; `channel_last()` is kept for API parity
        self.use_shadow = False
        grid = [int(v) for v in grid_size]
        planes, lines = [], []
        for i, (vec_id, (m0, m1)) in enumerate(zip(self.vector_mode, self.matrix_mode)):
            for idx, j in enumerate(self.reso_mode):
                if param_shape is not None:  # reference-layout shapes stored in kwargs.th
                    _, C, B, H, W = [int(v) for v in param_shape[f"plane_coef.{i * len(self.reso_mode) + idx}"]]
                    Z = int(param_shape[f"line_coef.{i * len(self.reso_mode) + idx}"][2])
                else:
                    C, B, H, W, Z = self.n_component[i], n_blocks, grid[m1] * j, grid[m0] * j, grid[vec_id] * j
                planes.append(torch.nn.Parameter(scale * torch.randn(B, H, W, C, device=device)))
                lines.append(torch.nn.Parameter(scale * torch.randn(B, Z, C, device=device)))
        self.plane_coef = torch.nn.ParameterList(planes)
        self.line_coef = torch.nn.ParameterList(lines)
        self.save_init_kwargs(locals())
        self.merge_config = {"merge_type": MergeType.Evenly}
        for k in range(3):
            self.merge_config[f"plane_coef.{k}"] = 2   # block dim in the reference layout [1,C,B,H,W]
            self.merge_config[f"line_coef.{k}"] = 3    # block dim in [1,C,Z,B]
        self._register_state_dict_hook(self._to_reference_layout)
        self._register_load_state_dict_pre_hook(self._from_reference_layout)

    # -- reference checkpoint layout --------------------------------------------------
    @staticmethod
    def _to_reference_layout(module, state, prefix, _local):
        for key in list(state.keys()):
            tail = key[len(prefix):]
            if tail.startswith("plane_coef."):
                state[key] = _plane_to_ref(state[key])
            elif tail.startswith("line_coef."):
                state[key] = _line_to_ref(state[key])
        return state

    def _from_reference_layout(self, state, prefix, *_):
        for key in list(state.keys()):
            tail = key[len(prefix):]
            if tail.startswith("plane_coef.") and state[key].dim() == 5:
                t = state[key]
                # accept both [1,C,B,H,W] and the reference's channel-last export [1,B,H,W,C]
                k = int(tail.split(".")[1])
                C = self.plane_coef[k].shape[-1] if k < len(self.plane_coef) else t.shape[1]
                state[key] = t[0].contiguous() if (t.shape[-1] == C and t.shape[1] != C) else _plane_from_ref(t)
            elif tail.startswith("line_coef.") and state[key].dim() == 4:
                state[key] = _line_from_ref(state[key])
        for k, (p, l) in enumerate(zip(self.plane_coef, self.line_coef)):
            for name, param in ((f"{prefix}plane_coef.{k}", p), (f"{prefix}line_coef.{k}", l)):
                if name in state and tuple(state[name].shape) != tuple(param.shape):
                    param.data = torch.empty_like(state[name], device=param.device)  # adopt checkpoint shape

    def param_shape(self) -> Dict[str, List[int]]:
        """Reference-layout parameter shapes (what ``kwargs.th`` stores under ``grid_shape``)."""
        shapes = {}
        for k, (p, l) in enumerate(zip(self.plane_coef, self.line_coef)):
            B, H, W, C = p.shape
            shapes[f"plane_coef.{k}"] = [1, C, B, H, W]
            shapes[f"line_coef.{k}"] = [1, C, l.shape[1], B]
        return shapes

    # -- bf16 shadows -----------------------------------------------------------------
    def enable_shadow(self, fused_optimizer: bool = True) -> None:
        """Keep bf16 copies of the grids for the lookup kernels (fp32 masters keep the gradients).
        With ``fused_optimizer`` the masters also get persistent gradient accumulators."""
        from ....ops import FusedAdam

        self.use_shadow = True
        for p in list(self.plane_coef) + list(self.line_coef):
            if fused_optimizer:
                FusedAdam.attach_sink(p, shadow=True)
            else:
                p._lmb_shadow = p.detach().to(torch.bfloat16)

    def refresh_shadow(self) -> None:
        for p in list(self.plane_coef) + list(self.line_coef):
            if getattr(p, "_lmb_shadow", None) is not None:
                p._lmb_shadow.copy_(p.detach())

    def channel_last(self) -> None:
        self.is_channel_last = True

    # -- forward ------------------------------------------------------------------------
    def _lookup(self, coords: torch.Tensor, ks: Sequence[int], count=None, out_dtype=torch.float32) -> torch.Tensor:
        planes = [self.plane_coef[k] for k in ks]
        lines = [self.line_coef[k] for k in ks]
        if self.use_shadow and coords.is_cuda:
            return vm_encode(coords, planes, lines, [p._lmb_shadow for p in planes], [l._lmb_shadow for l in lines],
                             count=count, out_dtype=out_dtype)
        return vm_encode(coords, planes, lines, count=count, out_dtype=out_dtype)

    def forward(self, xyzb: torch.Tensor, count=None, out_dtype=torch.float32) -> torch.Tensor:
        """``xyzb [N, 4]`` = block-local xyz in ``[-1, 1]`` + block index -> ``[N, sum(C) * n_levels]``."""
        n_levels = len(self.reso_mode)
        if self.ndims == 1:
            return self._lookup(xyzb, range(n_levels), count, out_dtype)
        outs = []
        for i, (vec_id, (m0, m1)) in enumerate(zip(self.vector_mode, self.matrix_mode)):
            coords = torch.stack((xyzb[..., m0], xyzb[..., m1], xyzb[..., vec_id], xyzb[..., 3]), dim=-1)
            outs.append(self._lookup(coords, range(i * n_levels, (i + 1) * n_levels), count, out_dtype))
        return torch.cat(outs, dim=-1)

    # -- schedule -----------------------------------------------------------------------
    @torch.no_grad()
    def upsample_volume_grid(self, grid_size) -> None:
        """Bilinear (align_corners) resize of every plane/line to ``grid_size * level``; parameters
        are replaced, so optimiser state must be rebuilt by the caller (as in the reference)."""
        grid = [int(v) for v in grid_size]
        n_levels = len(self.reso_mode)
        for i, (vec_id, (m0, m1)) in enumerate(zip(self.vector_mode, self.matrix_mode)):
            for idx, j in enumerate(self.reso_mode):
                k = i * n_levels + idx
                p = self.plane_coef[k].data.permute(0, 3, 1, 2)                        # [B,C,H,W]
                p = F.interpolate(p, size=(grid[m1] * j, grid[m0] * j), mode="bilinear", align_corners=True)
                l = self.line_coef[k].data.permute(0, 2, 1)                            # [B,C,Z]
                l = F.interpolate(l, size=grid[vec_id] * j, mode="linear", align_corners=True)
                self.plane_coef[k] = torch.nn.Parameter(p.permute(0, 2, 3, 1).contiguous())
                self.line_coef[k] = torch.nn.Parameter(l.permute(0, 2, 1).contiguous())
        if self.use_shadow:
            self.enable_shadow()

    # -- regularisers ---------------------------------------------------------------------
    def L1_loss(self) -> torch.Tensor:
        return sum(p.abs().mean() + l.abs().mean() for p, l in zip(self.plane_coef, self.line_coef))

    def TV_loss(self) -> torch.Tensor:
        return sum(tv_term(p) * 1e-2 for p in self.plane_coef)

    def vector_diffs(self) -> torch.Tensor:
        total = 0
        for line in self.line_coef:
            B, Z, C = line.shape
            v = line.permute(2, 1, 0).reshape(C, Z * B)
            dotp = v @ v.t()
            off = dotp.flatten()[1:].view(C - 1, C + 1)[:, :-1]
            total = total + off.abs().mean()
        return total

    # -- checkpoint merge -------------------------------------------------------------------
    def merge_state_dicts(self, state_dicts: List[Dict[str, torch.Tensor]], device="cpu") -> Dict[str, torch.Tensor]:
        """Stack per-block reference-layout state dicts: planes on dim 2, lines on dim 3."""
        merged = {}
        for key in sorted(state_dicts[0].keys()):
            parts = [sd[key].to(device) for sd in state_dicts]
            if "plane_coef" in key:
                merged[key] = torch.cat(parts, dim=2)
            elif "line_coef" in key:
                merged[key] = torch.cat(parts, dim=3)
            else:
                merged[key] = parts[0]
        return merged
