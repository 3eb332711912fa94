"""Anchor-based Gaussian encodings: Scaffold-GS (reference:
landmark/nerf_components/model_components/fields/encodings/scaffoldgs_encoding.py:25-803).

Parameters per anchor: ``_anchor [N,3]``, ``_offset [N,k,3]``, ``_anchor_feat [N,F]``, ``_scaling [N,6]``
(log; 3 offset scales + 3 base sizes), ``_rotation [N,4]`` and ``_opacity [N,1]`` (both frozen).
Voxel de-duplication uses packed 64-bit voxel keys + ``torch.isin`` and the per-voxel feature
initialisation uses ``scatter_reduce(amax)`` where the reference loops over 4096-anchor chunks and
needs the external ``torch_scatter`` package.
"""
from __future__ import annotations

from typing import Dict

import numpy as np
import torch
from torch import nn

from ....ops.knn import distCUDA2
from ....render.types import MergeType
from ...utils.general_utils import inverse_sigmoid
from ...utils.ply_utils import read_ply, write_ply
from .base_encoding import BaseGaussianEncoding
from .gaussian_encoding import cat_tensors_to_optimizer, prune_optimizer

_ANCHOR_GROUPS = {"anchor": "_anchor", "offset": "_offset", "anchor_feat": "_anchor_feat", "opacity": "_opacity",
                  "scaling": "_scaling", "rotation": "_rotation"}
_KEY_OFF = 1 << 20


def voxel_keys(coords: torch.Tensor) -> torch.Tensor:
    """Pack integer voxel coordinates ``[M, 3]`` (|c| < 2^20) into one int64 key per voxel."""
    c = coords.long() + _KEY_OFF
    return (c[:, 0] << 42) | (c[:, 1] << 21) | c[:, 2]


def segment_amax(values: torch.Tensor, index: torch.Tensor, n_segments: int) -> torch.Tensor:
    """Per-segment maximum ``[n_segments, C]`` of ``values [N, C]`` grouped by ``index [N]`` (``-inf`` for empty
    segments); an atomic-max kernel on CUDA (``ops/csrc/gs_aux.cu``), ``scatter_reduce`` elsewhere."""
    out = torch.full((n_segments, values.shape[1]), -torch.inf, device=values.device, dtype=values.dtype)
    if values.is_cuda and values.dtype == torch.float32 and not values.requires_grad:
        from ctypes import c_int, c_longlong

        from ....ops import native

        if native.available():
            P = native.P
            native.register_signature("lmb_segment_amax", [P, P, c_longlong, c_int, c_longlong, P, P])
            v, ix = values.contiguous(), index.to(torch.int64).contiguous()
            native.check(native.lib().lmb_segment_amax(v.data_ptr(), ix.data_ptr(), v.shape[0], v.shape[1], n_segments,
                                                       out.data_ptr(), native.stream_ptr()), "segment_amax")
            return out
    out.scatter_reduce_(0, index[:, None].expand_as(values), values, reduce="amax", include_self=True)
    return out


class ScaffoldGSEncoding(BaseGaussianEncoding):
    def __init__(self, feat_dim: int = 32, n_offsets: int = 10, voxel_size: float = 0.01, update_depth: int = 3,
                 update_init_factor: int = 16, update_hierachy_factor: int = 4, percent_dense: float = 0.01,
                 device="cuda", use_feat_bank: bool = False):
        # ``use_feat_bank`` is accepted as in the reference (scaffoldgs_encoding.py, constructor); the feature bank
        # itself lives in the anchor decoder
        super().__init__()
        self.use_feat_bank = bool(use_feat_bank)
        dev = device if (torch.cuda.is_available() or str(device) == "cpu") else "cpu"
        self.device = torch.device(dev)
        self.feat_dim, self.n_offsets, self.voxel_size = feat_dim, n_offsets, voxel_size
        self.update_depth, self.update_init_factor = update_depth, update_init_factor
        self.update_hierachy_factor, self.percent_dense = update_hierachy_factor, percent_dense
        z = lambda *s: nn.Parameter(torch.zeros(*s, device=self.device))  # noqa: E731
        self._anchor, self._offset, self._anchor_feat = z(0, 3), z(0, n_offsets, 3), z(0, feat_dim)
        self._scaling = z(0, 6)
        self._rotation = nn.Parameter(torch.zeros(0, 4, device=self.device), requires_grad=False)
        self._opacity = nn.Parameter(torch.zeros(0, 1, device=self.device), requires_grad=False)
        self._reset_stats()
        self.save_init_kwargs(locals())
        self.merge_config = {"merge_type": MergeType.Unevenly, **{v: 0 for v in _ANCHOR_GROUPS.values()}}

    # -- accessors ------------------------------------------------------------------------------------
    @property
    def get_anchor(self):
        return self._anchor

    @property
    def get_scaling(self):
        return torch.exp(self._scaling)

    @property
    def get_rotation(self):
        return torch.nn.functional.normalize(self._rotation)

    @property
    def get_opacity(self):
        return torch.sigmoid(self._opacity)

    @property
    def get_anchor_feat(self):
        return self._anchor_feat

    @property
    def get_offset(self):
        return self._offset

    def set_anchor(self, new_anchor: torch.Tensor):
        assert new_anchor.shape == self._anchor.shape, "the new anchors must keep the shape of the old ones"
        self._anchor = nn.Parameter(new_anchor.to(self.device).float().contiguous(),
                                    requires_grad=self._anchor.requires_grad)

    def get_covariance(self, scaling_modifier: float = 1.0) -> torch.Tensor:
        """Upper triangle ``[N, 6]`` of the anchors' world-space covariance ``R S S^T R^T`` (first three scales)."""
        from ....components.utils.general_utils import build_scaling_rotation, strip_symmetric

        L = build_scaling_rotation(scaling_modifier * self.get_scaling[:, :3], self._rotation)
        return strip_symmetric(L @ L.transpose(1, 2))

    def construct_list_of_attributes(self):
        """Column names of the PLY file, in file order."""
        return list(self._ply_columns().keys())

    def __len__(self):
        return self._anchor.shape[0]

    def _reset_stats(self):
        n, dev = self._anchor.shape[0], self.device
        self.opacity_accum = torch.zeros(n, 1, device=dev)
        self.anchor_demon = torch.zeros(n, 1, device=dev)
        self.offset_gradient_accum = torch.zeros(n * self.n_offsets, 1, device=dev)
        self.offset_denom = torch.zeros(n * self.n_offsets, 1, device=dev)
        self.max_radii2D = torch.zeros(n, device=dev)

    def _set_params(self, anchor, offset, feat, scaling, rotation, opacity):
        dev = self.device
        self._anchor = nn.Parameter(anchor.to(dev).float().contiguous())
        self._offset = nn.Parameter(offset.to(dev).float().contiguous())
        self._anchor_feat = nn.Parameter(feat.to(dev).float().contiguous())
        self._scaling = nn.Parameter(scaling.to(dev).float().contiguous())
        self._rotation = nn.Parameter(rotation.to(dev).float().contiguous(), requires_grad=False)
        self._opacity = nn.Parameter(opacity.to(dev).float().contiguous(), requires_grad=False)
        self._reset_stats()

    # -- initialisation ----------------------------------------------------------------------------------
    def voxelize_sample(self, points: torch.Tensor, voxel_size: float) -> torch.Tensor:
        return torch.unique(torch.round(points / voxel_size), dim=0) * voxel_size

    def _init_from_positions(self, positions: torch.Tensor):
        n = positions.shape[0]
        dist2 = distCUDA2(positions).clamp_min(1e-7)
        scales = torch.log(torch.sqrt(dist2))[:, None].repeat(1, 6)
        rots = torch.zeros(n, 4, device=self.device)
        rots[:, 0] = 1
        self._set_params(positions, torch.zeros(n, self.n_offsets, 3), torch.zeros(n, self.feat_dim), scales, rots,
                         inverse_sigmoid(0.1 * torch.ones(n, 1, device=self.device)))

    def create_from_pcd(self, pcd, spatial_lr_scale: float = 1.0):
        pts = torch.as_tensor(np.asarray(pcd.points), dtype=torch.float32, device=self.device)
        if self.voxel_size <= 0:
            d = distCUDA2(pts)
            self.voxel_size = float(torch.kthvalue(d, max(int(d.shape[0] * 0.5), 1)).values)
        self._init_from_positions(self.voxelize_sample(pts, self.voxel_size))

    # -- PLY -------------------------------------------------------------------------------------------------
    def _ply_columns(self) -> Dict[str, np.ndarray]:
        a = self._anchor.detach().cpu().numpy()
        cols = {"x": a[:, 0], "y": a[:, 1], "z": a[:, 2], "nx": np.zeros(len(a), np.float32),
                "ny": np.zeros(len(a), np.float32), "nz": np.zeros(len(a), np.float32)}
        off = self._offset.detach().transpose(1, 2).flatten(1).cpu().numpy()
        for i in range(off.shape[1]):
            cols[f"f_offset_{i}"] = off[:, i]
        feat = self._anchor_feat.detach().cpu().numpy()
        for i in range(feat.shape[1]):
            cols[f"f_anchor_feat_{i}"] = feat[:, i]
        cols["opacity"] = self._opacity.detach().cpu().numpy()[:, 0]
        sc, rot = self._scaling.detach().cpu().numpy(), self._rotation.detach().cpu().numpy()
        for i in range(sc.shape[1]):
            cols[f"scale_{i}"] = sc[:, i]
        for i in range(rot.shape[1]):
            cols[f"rot_{i}"] = rot[:, i]
        return {k: np.ascontiguousarray(v, dtype=np.float32) for k, v in cols.items()}

    def save_ply(self, path: str):
        write_ply(path, self._ply_columns())

    @staticmethod
    def _cols(v, prefix):
        names = sorted([n for n in v.dtype.names if n.startswith(prefix)], key=lambda s: int(s.split("_")[-1]))
        return np.stack([v[k] for k in names], 1).astype(np.float32)

    def load_ply_to_state_dict(self, path: str, map_location="cpu") -> Dict[str, torch.Tensor]:
        v = read_ply(path)
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(map_location)  # noqa: E731
        off = self._cols(v, "f_offset_").reshape(len(v), 3, -1).transpose(0, 2, 1)
        return {"_anchor": t(np.stack((v["x"], v["y"], v["z"]), 1).astype(np.float32)), "_offset": t(off),
                "_anchor_feat": t(self._cols(v, "f_anchor_feat_")), "_opacity": t(np.asarray(v["opacity"], np.float32)[:, None]),
                "_scaling": t(self._cols(v, "scale_")), "_rotation": t(self._cols(v, "rot_"))}

    def load_encoding_state(self, state: Dict[str, torch.Tensor]):
        self._set_params(state["_anchor"], state["_offset"], state["_anchor_feat"], state["_scaling"],
                         state["_rotation"], state["_opacity"])

    def load_ply(self, path: str):
        self.load_encoding_state(self.load_ply_to_state_dict(path, self.device))

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        keys = [prefix + n for n in _ANCHOR_GROUPS.values()]
        if all(k in state_dict for k in keys):
            self.load_encoding_state({n: state_dict[prefix + n] for n in _ANCHOR_GROUPS.values()})
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    # -- statistics ----------------------------------------------------------------------------------------------
    @torch.no_grad()
    def training_statis(self, viewspace_point_tensor, opacity, update_filter, offset_selection_mask, anchor_visible_mask):
        """Accumulate per-anchor opacity / visit counts and per-offset screen-space gradient norms."""
        k = self.n_offsets
        op = opacity.detach().clone().view(-1).clamp_min(0).view(-1, k)
        self.opacity_accum[anchor_visible_mask] += op.sum(dim=1, keepdim=True)
        self.anchor_demon[anchor_visible_mask] += 1
        vis_off = anchor_visible_mask[:, None].expand(-1, k).reshape(-1)
        combined = torch.zeros_like(vis_off)
        combined[vis_off] = offset_selection_mask
        chosen = combined.clone()
        combined[chosen] = update_filter
        grad = viewspace_point_tensor.grad
        if grad is None:
            return
        self.offset_gradient_accum[combined] += torch.norm(grad[update_filter, :2], dim=-1, keepdim=True)
        self.offset_denom[combined] += 1

    # -- structural updates -----------------------------------------------------------------------------------------
    def _adopt(self, tensors: Dict[str, nn.Parameter]):
        for group, attr in _ANCHOR_GROUPS.items():
            if group in tensors:
                p = tensors[group]
                if group in ("rotation", "opacity"):
                    p.requires_grad_(False)
                setattr(self, attr, p)

    def prune_anchor(self, mask: torch.Tensor, optimizer):
        self._adopt(prune_optimizer(optimizer, ~mask, set(_ANCHOR_GROUPS)))

    def _append(self, new: Dict[str, torch.Tensor], optimizer):
        n_new = new["anchor"].shape[0]
        pad = torch.zeros(n_new, 1, device=self.device)
        self.anchor_demon = torch.cat((self.anchor_demon, pad), 0)
        self.opacity_accum = torch.cat((self.opacity_accum, pad), 0)
        self._adopt(cat_tensors_to_optimizer(optimizer, new))

    def _new_anchor_tensors(self, anchors: torch.Tensor, size: float, feats: torch.Tensor) -> Dict[str, torch.Tensor]:
        n = anchors.shape[0]
        rot = torch.zeros(n, 4, device=self.device)
        rot[:, 0] = 1.0
        return {"anchor": anchors, "scaling": torch.log(torch.ones(n, 6, device=self.device) * size), "rotation": rot,
                "anchor_feat": feats, "offset": torch.zeros(n, self.n_offsets, 3, device=self.device),
                "opacity": inverse_sigmoid(0.1 * torch.ones(n, 1, device=self.device))}

    @torch.no_grad()
    def anchor_growing(self, grads, threshold, offset_mask, optimizer):
        """Multi-resolution growing: neural Gaussians with a large accumulated gradient spawn new
        anchors at the centres of the (not yet occupied) voxels they fall into."""
        init_length = self._anchor.shape[0] * self.n_offsets
        k = self.n_offsets
        for i in range(self.update_depth):
            cur_threshold = threshold * ((self.update_hierachy_factor // 2) ** i)
            cand = (grads >= cur_threshold) & offset_mask
            cand = cand & (torch.rand_like(cand.float()) > (0.5 ** (i + 1)))
            length_inc = self._anchor.shape[0] * k - init_length
            if length_inc == 0:
                if i > 0:
                    continue
            else:
                cand = torch.cat((cand, torch.zeros(length_inc, dtype=torch.bool, device=self.device)))
            all_xyz = self._anchor[:, None] + self._offset * self.get_scaling[:, None, :3]
            cur_size = self.voxel_size * (self.update_init_factor // (self.update_hierachy_factor ** i))
            if cur_size <= 0:
                continue
            occupied = voxel_keys(torch.round(self._anchor / cur_size))
            sel = torch.round(all_xyz.view(-1, 3)[cand] / cur_size)
            if sel.shape[0] == 0:
                continue
            uniq, inverse = torch.unique(sel, return_inverse=True, dim=0)
            fresh = ~torch.isin(voxel_keys(uniq), occupied)
            if fresh.sum() == 0:
                continue
            feats = self._anchor_feat[:, None].expand(-1, k, -1).reshape(-1, self.feat_dim)[cand]
            new_feat = segment_amax(feats, inverse, uniq.shape[0])[fresh]
            self._append(self._new_anchor_tensors(uniq[fresh] * cur_size, cur_size, new_feat), optimizer)

    def _after_growing(self, offset_mask):
        k, n = self.n_offsets, self._anchor.shape[0]
        self.offset_denom[offset_mask] = 0
        self.offset_gradient_accum[offset_mask] = 0
        pad = n * k - self.offset_denom.shape[0]
        if pad > 0:
            z = torch.zeros(pad, 1, device=self.device)
            self.offset_denom = torch.cat((self.offset_denom, z), 0)
            self.offset_gradient_accum = torch.cat((self.offset_gradient_accum, z), 0)

    def _prune_by_opacity(self, check_interval, success_threshold, min_opacity, optimizer):
        k = self.n_offsets
        prune = (self.opacity_accum < min_opacity * self.anchor_demon).squeeze(1)
        seen = (self.anchor_demon > check_interval * success_threshold).squeeze(1)
        prune = prune & seen
        self.offset_denom = self.offset_denom.view(-1, k)[~prune].reshape(-1, 1)
        self.offset_gradient_accum = self.offset_gradient_accum.view(-1, k)[~prune].reshape(-1, 1)
        self.opacity_accum[seen] = 0
        self.anchor_demon[seen] = 0
        self.opacity_accum, self.anchor_demon = self.opacity_accum[~prune], self.anchor_demon[~prune]
        if prune.any():
            self.prune_anchor(prune, optimizer)
        return prune

    @torch.no_grad()
    def adjust_anchor(self, check_interval=100, success_threshold=0.8, grad_threshold=0.0002, min_opacity=0.005,
                      optimizer=None):
        grads = self.offset_gradient_accum / self.offset_denom
        grads[grads.isnan()] = 0.0
        offset_mask = (self.offset_denom > check_interval * success_threshold * 0.5).squeeze(1)
        self.anchor_growing(torch.norm(grads, dim=-1), grad_threshold, offset_mask, optimizer)
        self._after_growing(offset_mask)
        self._prune_by_opacity(check_interval, success_threshold, min_opacity, optimizer)
        self.max_radii2D = torch.zeros(self._anchor.shape[0], device=self.device)
