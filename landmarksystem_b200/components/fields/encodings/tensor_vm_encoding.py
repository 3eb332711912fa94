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
                 param_shape: Optional[Dict[str, Sequence[int]]] = None, n_blocks: int = 1, scale: float = 0.1,
                 random_init: bool = True):
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
                if random_init:
                    planes.append(torch.nn.Parameter(scale * torch.randn(B, H, W, C, device=device)))
                    lines.append(torch.nn.Parameter(scale * torch.randn(B, Z, C, device=device)))
                else:       # a checkpoint is loaded right after construction: skip the (slow, on the CPU) random fill
                    planes.append(torch.nn.Parameter(torch.zeros(B, H, W, C, device=device)))
                    lines.append(torch.nn.Parameter(torch.zeros(B, Z, C, device=device)))
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
        module.flush_lazy()
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

    def to_reference_layout(self, name: str, tensor: torch.Tensor) -> torch.Tensor:
        """A checkpoint tensor in the layout the block splitter expects: planes exported channels-last
        (``[1, B, H, W, C]``, the ``*_channel_last.th`` files) come back as ``[1, C, B, H, W]`` (a view)."""
        if name.startswith("plane_coef.") and tensor.dim() == 5:
            k = int(name.split(".")[1])
            C = self.plane_coef[k].shape[-1] if k < len(self.plane_coef) and self.plane_coef[k].dim() == 4 else None
            if C is not None and tensor.shape[-1] == C and tensor.shape[1] != C:
                return tensor.permute(0, 4, 1, 2, 3)
        return tensor

    @staticmethod
    def block_to_internal(name: str, piece: torch.Tensor) -> torch.Tensor:
        """One-block slice in checkpoint layout -> the in-memory (channels-last) layout, for dynamic loading."""
        if name.startswith("plane_coef") and piece.dim() == 5:
            return _plane_from_ref(piece)
        if name.startswith("line_coef") and piece.dim() == 4:
            return _line_from_ref(piece)
        return piece

    def param_shape(self) -> Dict[str, List[int]]:
        """Reference-layout parameter shapes (what ``kwargs.th`` stores under ``grid_shape``)."""
        shapes = {}
        for k, (p, l) in enumerate(zip(self.plane_coef, self.line_coef)):
            B, H, W, C = p.shape
            shapes[f"plane_coef.{k}"] = [1, C, B, H, W]
            shapes[f"line_coef.{k}"] = [1, C, l.shape[1], B]
        return shapes

    # -- bf16 shadows -----------------------------------------------------------------
    def enable_shadow(self, fused_optimizer: bool = True, lazy: bool = False) -> None:
        """Keep bf16 copies of the grids for the lookup kernels (fp32 masters keep the gradients).
        With ``fused_optimizer`` the masters also get persistent gradient accumulators; ``lazy`` turns on
        the deferred Adam update for the planes (lines are small and stay dense)."""
        from ....ops import FusedAdam

        self.use_shadow = True
        self.lazy = bool(lazy and fused_optimizer)
        for p in self.plane_coef:
            if fused_optimizer:
                FusedAdam.attach_sink(p, shadow=True, lazy=self.lazy)
            else:
                p._lmb_shadow = p.detach().to(torch.bfloat16)
        for p in self.line_coef:
            if fused_optimizer:
                FusedAdam.attach_sink(p, shadow=True)
            else:
                p._lmb_shadow = p.detach().to(torch.bfloat16)

    def flush_lazy(self) -> None:
        """Make every plane texel current (deferred Adam); no-op otherwise."""
        for p in self.plane_coef:
            state = getattr(p, "_lmb_lazy", None)
            if state is not None:
                state.flush(p)

    def refresh_shadow(self) -> None:
        for p in list(self.plane_coef) + list(self.line_coef):
            if getattr(p, "_lmb_shadow", None) is not None:
                p._lmb_shadow.copy_(p.detach())

    def channel_last(self) -> None:
        self.is_channel_last = True

    # -- forward ------------------------------------------------------------------------
    def _lookup(self, coords: torch.Tensor, ks: Sequence[int], count=None, out_dtype=torch.float32,
                out_width: int = 0, zero_fill: bool = True, tail=None) -> torch.Tensor:
        planes = [self.plane_coef[k] for k in ks]
        lines = [self.line_coef[k] for k in ks]
        if getattr(self, "lazy", False) and coords.is_cuda:
            coords = coords.contiguous().float()
            if self.training and torch.is_grad_enabled():
                for p in planes:
                    p._lmb_lazy.prepare(p, coords, count)
            else:
                self.flush_lazy()
        if self.use_shadow and coords.is_cuda:
            return vm_encode(coords, planes, lines, [p._lmb_shadow for p in planes], [l._lmb_shadow for l in lines],
                             count=count, out_dtype=out_dtype, out_width=out_width, zero_fill=zero_fill, tail=tail)
        return vm_encode(coords, planes, lines, count=count, out_dtype=out_dtype, out_width=out_width, zero_fill=zero_fill,
                         tail=tail)

    def fused_density_ok(self, xyzb: torch.Tensor) -> bool:
        from ....ops.vm import vm_density_supported

        return xyzb.is_cuda and self.ndims == 1 and type(self).forward is TensorVMEncoding.forward \
            and vm_density_supported(self.plane_coef)

    def density(self, xyzb: torch.Tensor, weight, inner_relu: bool, act: str, shift: float, count=None, route=None) -> torch.Tensor:
        """``sigma [N]`` straight from the lookup kernel: channel-weighted sum (``weight [1, L*C]`` or ``None``)
        and activation are applied in registers, the feature matrix is never written."""
        from ....ops.vm import vm_density

        ks = range(len(self.reso_mode))
        planes = [self.plane_coef[k] for k in ks]
        lines = [self.line_coef[k] for k in ks]
        coords = xyzb.contiguous().float()
        if getattr(self, "lazy", False):
            if self.training and torch.is_grad_enabled():
                for p in planes:
                    p._lmb_lazy.prepare(p, coords, count)
            else:
                self.flush_lazy()
        if self.use_shadow:
            return vm_density(coords, planes, lines, [p._lmb_shadow for p in planes], [l._lmb_shadow for l in lines],
                              weight, inner_relu, act, shift, count, route)
        return vm_density(coords, planes, lines, None, None, weight, inner_relu, act, shift, count, route)

    def forward(self, xyzb: torch.Tensor, count=None, out_dtype=torch.float32, out_width: int = 0,
                zero_fill: bool = True, tail=None) -> torch.Tensor:
        """``xyzb [N, 4]`` = block-local xyz in ``[-1, 1]`` + block index -> ``[N, sum(C) * n_levels]``
        (``out_width`` asks for wider zero-padded rows and ``tail`` for the rays' directions behind the features, see
        :func:`landmarksystem_b200.ops.vm_encode`)."""
        n_levels = len(self.reso_mode)
        if self.ndims == 1:
            return self._lookup(xyzb, range(n_levels), count, out_dtype, out_width, zero_fill, tail)
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
        self.flush_lazy()
        for i, (vec_id, (m0, m1)) in enumerate(zip(self.vector_mode, self.matrix_mode)):
            for idx, j in enumerate(self.reso_mode):
                k = i * n_levels + idx
                from ....ops.resize import resize_bilinear_nhwc, resize_linear_nlc   # channels-last, no transposes

                self.plane_coef[k] = torch.nn.Parameter(resize_bilinear_nhwc(self.plane_coef[k].data, grid[m1] * j, grid[m0] * j))
                self.line_coef[k] = torch.nn.Parameter(resize_linear_nlc(self.line_coef[k].data, grid[vec_id] * j))
        if self.use_shadow:
            self.enable_shadow(lazy=getattr(self, "lazy", False))

    # -- regularisers ---------------------------------------------------------------------
    def fused_regulariser_ok(self) -> bool:
        """The planes' TV / L1 terms can be folded into the optimiser's sweep: CUDA, bf16 shadows, fused dense Adam
        (gradient sinks, no deferred update), the unpartitioned encoding."""
        return (self.use_shadow and not getattr(self, "lazy", False) and type(self).L1_loss is TensorVMEncoding.L1_loss
                and all(p.is_cuda and getattr(p, "_lmb_grad_sink", None) is not None and p.shape[-1] % 4 == 0
                        for p in self.plane_coef))

    def set_plane_regulariser(self, tv_weight=None, tv_index: int = 0, l1_weight: float = 0.0, loss_scale: float = 1.0,
                              loss_out=None) -> None:
        """Ask the fused optimiser to apply ``tv_weight * TV_loss() + l1_weight * (plane part of L1_loss())`` inside its
        next steps (see ``FusedAdam.attach_plane_regulariser``)."""
        from ....ops import FusedAdam

        for p in self.plane_coef:
            FusedAdam.attach_plane_regulariser(p, tv_weight, tv_index, l1_weight, loss_scale, loss_out)

    def L1_loss_lines(self) -> torch.Tensor:
        """The line part of :meth:`L1_loss` (lines are a few KB: plain PyTorch ops)."""
        return sum(l.abs().mean() for l in self.line_coef)

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


class ChannelParallelTensorVMEncoding(TensorVMEncoding):
    """Feature channels split across the ranks of a group: each rank stores ``C / P`` channels of every
    plane and line, looks all samples up on its slice and the per-level ``plane * line`` products are
    all-gathered (reference: tensor_vm_encoding.py:335-551 gathers plane and line features separately,
    i.e. twice the bytes).  ``init_state_dict`` (reference layout, full channels) seeds the slices."""

    def __init__(self, ndims, resolution_mode, n_component, grid_size, device, param_shape=None, n_blocks=1,
                 scale=0.1, parallel_degree: int = 1, parallel_part: int = 0, group=None, init_state_dict=None,
                 random_init: bool = True):
        comps = list(n_component) if isinstance(n_component, (list, tuple)) else [n_component] * 3
        assert all(c % parallel_degree == 0 and (c // parallel_degree) % 8 == 0 for c in comps[:ndims]), \
            "channel-parallel slices must keep a multiple of 8 channels per rank"
        self.parallel_degree, self.parallel_part, self.group = parallel_degree, parallel_part, group
        self.full_component = comps[:ndims]
        local = [c // parallel_degree for c in comps]
        super().__init__(ndims, resolution_mode, local, grid_size, device, param_shape=None, n_blocks=n_blocks,
                         scale=scale, random_init=random_init and init_state_dict is None)
        if init_state_dict is not None:
            self.load_full_state(init_state_dict)
        self.merge_config = {}  # channel slices are not spatial blocks

    def load_full_state(self, state):
        """Take this rank's channel slice from a full (reference-layout) state dict."""
        lo = self.parallel_part
        for k in range(len(self.plane_coef)):
            p, l = state[f"plane_coef.{k}"], state[f"line_coef.{k}"]
            c = p.shape[1] // self.parallel_degree
            self.plane_coef[k].data = _plane_from_ref(p[:, lo * c:(lo + 1) * c]).to(self.plane_coef[k].device)
            self.line_coef[k].data = _line_from_ref(l[:, lo * c:(lo + 1) * c]).to(self.line_coef[k].device)
        if self.use_shadow:
            self.enable_shadow()

    def forward(self, xyzb, count=None, out_dtype=torch.float32):
        from ....comm.autograd import AllGather

        local = super().forward(xyzb, count, torch.float32)               # [N, L * C/P]
        if self.parallel_degree == 1:
            return local.to(out_dtype)
        N = local.shape[0]
        P = self.parallel_degree
        gathered = AllGather.apply(local, self.group)                     # [P*N, L * C/P]
        n_pairs, L = self.ndims, len(self.reso_mode)
        cl = local.shape[1] // (n_pairs * L)
        full = gathered.view(P, N, n_pairs * L, cl).permute(1, 2, 0, 3).reshape(N, n_pairs * L * P * cl)
        return full.to(out_dtype)

    def _gather_scalar(self, value: torch.Tensor) -> torch.Tensor:
        from ....comm.autograd import AllReduce

        return AllReduce.apply(value, self.group) / self.parallel_degree

    def L1_loss(self):
        return self._gather_scalar(super().L1_loss())

    def TV_loss(self):
        return self._gather_scalar(super().TV_loss())

    def vector_diffs(self):
        """Off-diagonal correlations need every channel: gather the (small) line tensors."""
        from ....comm.autograd import AllGather

        total = 0
        for line in self.line_coef:
            B, Z, C = line.shape
            v = line.permute(2, 1, 0).reshape(C, Z * B)
            full = AllGather.apply(v, self.group) if self.parallel_degree > 1 else v
            dotp = full @ full.t()
            n = full.shape[0]
            total = total + dotp.flatten()[1:].view(n - 1, n + 1)[:, :-1].abs().mean()
        return total

    def merge_state_dicts(self, state_dicts, device="cpu"):
        """Concatenate per-rank channel slices back on the channel dim (reference layout dim 1)."""
        return {k: torch.cat([sd[k].to(device) for sd in state_dicts], dim=1) if "_coef" in k else state_dicts[0][k]
                for k in sorted(state_dicts[0].keys())}


class BranchParallelTensorVMEncoding(TensorVMEncoding):
    """One spatial block per rank.  The initial values are drawn once for the whole scene (rank 0),
    broadcast, and each rank keeps its own block, so a branch-parallel run starts from the same field
    as a single-process run with the same seed (reference: tensor_vm_encoding.py:554-636)."""

    def __init__(self, ndims, resolution_mode, n_component, grid_size, device, param_shape=None, n_blocks=1,
                 scale=0.1, parallel_degree: int = 1, parallel_part: int = 0, group=None, init_state_dict=None,
                 random_init: bool = True):
        self.parallel_degree, self.parallel_part, self.group = parallel_degree, parallel_part, group
        super().__init__(ndims, resolution_mode, n_component, grid_size, device, param_shape=None, n_blocks=1,
                         scale=scale, random_init=random_init and init_state_dict is None)
        if init_state_dict is not None:
            self.load_full_state(init_state_dict)
        elif parallel_degree > 1 and torch.distributed.is_initialized():
            self._broadcast_init(scale)

    @torch.no_grad()
    def _broadcast_init(self, scale):
        import torch.distributed as dist

        src = dist.get_global_rank(self.group, 0) if self.group is not None else 0
        for params in (self.plane_coef, self.line_coef):
            for p in params:
                full = scale * torch.randn(self.parallel_degree, *p.shape[1:], device=p.device)
                dist.broadcast(full, src=src, group=self.group)
                p.data.copy_(full[self.parallel_part:self.parallel_part + 1])

    def load_full_state(self, state):
        """Keep this rank's block of a merged (block-stacked, reference-layout) state dict."""
        b = self.parallel_part
        for k in range(len(self.plane_coef)):
            p, l = state[f"plane_coef.{k}"], state[f"line_coef.{k}"]
            pb = p[:, :, b:b + 1] if p.shape[2] > 1 else p
            lb = l[..., b:b + 1] if l.shape[3] > 1 else l
            self.plane_coef[k].data = _plane_from_ref(pb).to(self.plane_coef[k].device)
            self.line_coef[k].data = _line_from_ref(lb).to(self.line_coef[k].device)
        if self.use_shadow:
            self.enable_shadow()


class FusedTensorVMEncoding(TensorVMEncoding):
    """Kernel-runtime name.  The reference's class raises ``NotImplementedError``
    (fields/encodings/fused_tensor_vm_encoding.py:6-53); here the base class already runs the fused
    channels-last lookup kernel, so the subclass only pins bf16 shadows on."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        if torch.device(self.device).type == "cuda":
            self.enable_shadow(fused_optimizer=False)


class FusedChannelParallelTensorVMEncoding(ChannelParallelTensorVMEncoding):
    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        if torch.device(self.device).type == "cuda":
            self.enable_shadow(fused_optimizer=False)


class CoefParam(torch.nn.Module):
    """A list of plane / line coefficient tensors as one module, so that a wrapper which only accepts modules
    (``DistributedDataParallel``) can hold them; ``forward`` samples one of them in the reference layout
    (reference: tensor_vm_encoding.py:639-677, unused there as well).

    ``coefs[k]``: ``[1, C, B, H, W]`` planes or ``[1, C, Z, B]`` lines; ``coordinates[idx_dim]``: a ``grid_sample``
    coordinate tensor for that layout."""

    def __init__(self, coefs: Sequence[torch.Tensor]) -> None:
        super().__init__()
        self.params = torch.nn.ParameterList([c if isinstance(c, torch.nn.Parameter) else torch.nn.Parameter(c)
                                              for c in coefs])

    def forward(self, coordinates: torch.Tensor, idx_plane: int, idx_dim: int, align_corners: bool = True):
        return F.grid_sample(self.params[idx_plane], coordinates[[idx_dim]], align_corners=align_corners)

    def __setitem__(self, idx: int, value):
        self.params[idx] = value

    def __getitem__(self, idx: int):
        return self.params[idx]

    def __len__(self) -> int:
        return len(self.params)
