"""Anchor -> neural-Gaussian decoder of Scaffold-GS / Octree-GS (reference:
landmark/nerf_components/model_components/fields/anchor_decoder.py:10-242 and its fused variant
fused_anchor_decoder.py:16-244).

For each visible anchor: view direction and distance to the camera, an optional view-conditioned
blend of the feature at three strides ("feature bank"), then three 2-layer MLP heads -> per-offset
opacity (tanh), covariance (7 values: 3 scale gates + quaternion) and colour (sigmoid).  Offsets with
positive opacity become Gaussians: ``xyz = anchor + offset * scale[:3]``,
``scale = scale[3:] * sigmoid(cov[:3])``, ``rot = normalize(cov[3:7])``.

Two documented deviations from the reference: with ``add_level`` the reference overwrites the
distance-carrying input by the distance-free one (anchor_decoder.py:181-182) - here each head gets
the input its ``add_*_dist`` flag asks for; and an appearance code is an embedding vector, not a
raw camera index.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from ..model.base_module import BaseModule


class AnchorDecoder(BaseModule):
    def __init__(self, use_feat_bank: bool, add_opacity_dist: bool, add_color_dist: bool, add_cov_dist: bool,
                 view_dim: int, feat_dim: int, n_offsets: int, appearance_dim: int = 0, add_level: bool = False,
                 dist2level: Optional[str] = None):
        super().__init__()
        self.use_feat_bank, self.add_opacity_dist = use_feat_bank, add_opacity_dist
        self.add_color_dist, self.add_cov_dist = add_color_dist, add_cov_dist
        self.add_level, self.dist2level = add_level, dist2level
        self.view_dim, self.feat_dim, self.n_offsets, self.appearance_dim = view_dim, feat_dim, n_offsets, appearance_dim
        lvl = 1 if add_level else 0
        base = feat_dim + view_dim + lvl
        if use_feat_bank:
            self.mlp_feature_bank = nn.Sequential(nn.Linear(view_dim + lvl, feat_dim), nn.ReLU(True),
                                                  nn.Linear(feat_dim, 3), nn.Softmax(dim=1))
        self.mlp_opacity = nn.Sequential(nn.Linear(base + int(add_opacity_dist), feat_dim), nn.ReLU(True),
                                         nn.Linear(feat_dim, n_offsets), nn.Tanh())
        self.mlp_cov = nn.Sequential(nn.Linear(base + int(add_cov_dist), feat_dim), nn.ReLU(True),
                                     nn.Linear(feat_dim, 7 * n_offsets))
        self.mlp_color = nn.Sequential(nn.Linear(base + int(add_color_dist) + appearance_dim, feat_dim), nn.ReLU(True),
                                       nn.Linear(feat_dim, 3 * n_offsets), nn.Sigmoid())
        self.use_fused = False
        self.save_init_kwargs(locals())

    def _heads(self, feat, ob_view, ob_dist, level, appearance):
        parts = [feat, ob_view]
        tail = [level] if (self.add_level and level is not None) else []
        with_dist = torch.cat(parts + [ob_dist] + tail, dim=1)
        without = torch.cat(parts + tail, dim=1)
        op_in = with_dist if self.add_opacity_dist else without
        cov_in = with_dist if self.add_cov_dist else without
        col_in = with_dist if self.add_color_dist else without
        if self.appearance_dim > 0:
            if appearance is None:
                appearance = torch.zeros(feat.shape[0], self.appearance_dim, device=feat.device, dtype=feat.dtype)
            elif appearance.dim() == 1:
                appearance = appearance[None].expand(feat.shape[0], -1)
            col_in = torch.cat((col_in, appearance), dim=1)
        if self.use_fused and feat.is_cuda and not torch.is_grad_enabled():
            from ...ops.fused_mlp import anchor_heads_forward, anchor_heads_supported

            if anchor_heads_supported(self, op_in, cov_in, col_in):
                return anchor_heads_forward(self, op_in, cov_in, col_in)
        return self.mlp_opacity(op_in), self.mlp_cov(cov_in), self.mlp_color(col_in)

    def forward(self, camera_center, anchor, anchor_feat, offset, scaling, visible_mask=None, level=None,
                prog_ratio=None, transition_mask=None, appearance_code=None):
        if visible_mask is None:
            visible_mask = torch.ones(anchor.shape[0], dtype=torch.bool, device=anchor.device)
        anchor, feat = anchor[visible_mask], anchor_feat[visible_mask]
        grid_offsets, grid_scaling = offset[visible_mask], scaling[visible_mask]
        if self.add_level and level is not None:
            level = level[visible_mask].reshape(-1, 1).to(feat.dtype)
        ob_view = anchor - camera_center
        ob_dist = ob_view.norm(dim=1, keepdim=True)
        ob_view = ob_view / ob_dist
        if self.use_feat_bank:
            bank_in = torch.cat((ob_view, level), dim=1) if (self.add_level and level is not None) else ob_view
            w = self.mlp_feature_bank(bank_in)                                  # [n, 3]
            feat = (feat[:, ::4].repeat(1, 4) * w[:, 0:1] + feat[:, ::2].repeat(1, 2) * w[:, 1:2]
                    + feat * w[:, 2:3])
        neural_opacity, scale_rot, color = self._heads(feat, ob_view, ob_dist, level, appearance_code)
        if self.dist2level == "progressive" and prog_ratio is not None and transition_mask is not None:
            prog = prog_ratio[visible_mask].clone().reshape(-1, 1)
            prog[~transition_mask[visible_mask]] = 1.0
            neural_opacity = neural_opacity * prog
        k = self.n_offsets
        if not self.training and not torch.is_grad_enabled() and anchor.is_cuda and neural_opacity.dtype == torch.float32:
            from ...ops import native

            if native.available():
                return (*_decode_epilogue(anchor, grid_offsets, grid_scaling, neural_opacity, color, scale_rot, k), None, None)
        neural_opacity = neural_opacity.reshape(-1, 1)
        mask = (neural_opacity > 0.0).view(-1)
        opacity = neural_opacity[mask]
        color = color.reshape(-1, 3)[mask]
        scale_rot = scale_rot.reshape(-1, 7)[mask]
        offsets = grid_offsets.reshape(-1, 3)[mask]
        idx = torch.arange(anchor.shape[0], device=anchor.device).repeat_interleave(k)[mask]
        scaling_rep, anchor_rep = grid_scaling[idx], anchor[idx]
        out_scaling = scaling_rep[:, 3:] * torch.sigmoid(scale_rot[:, :3])
        rot = torch.nn.functional.normalize(scale_rot[:, 3:7])
        xyz = anchor_rep + offsets * scaling_rep[:, :3]
        if self.training:
            return xyz, color, opacity, out_scaling, rot, neural_opacity, mask
        return xyz, color, opacity, out_scaling, rot, None, None


def _decode_epilogue(anchor, offsets, scaling, opacity, color, scale_rot, k: int):
    """Render-time tail of the decoder as one flag / scan / scatter kernel sequence (``ops/csrc/gs_aux.cu``): opacity
    mask, order-preserving compaction and the Gaussian attributes of the kept candidates.  One host read (the count)."""
    from ctypes import c_int, c_longlong

    from ...ops import native

    P = native.P
    native.register_signature("lmb_anchor_epilogue", [P, P, P, P, P, P, c_longlong, c_int, P, P, P, P, P, P, P, P, P, P])
    lib, dev = native.lib(), anchor.device
    scratch_bytes = lib.lmb_scan_scratch_bytes
    scratch_bytes.restype, scratch_bytes.argtypes = c_longlong, [c_longlong]
    n = anchor.shape[0] * k
    f = lambda t: t.detach().contiguous().float()  # noqa: E731
    anchor, offsets, scaling, opacity, color, scale_rot = map(f, (anchor, offsets, scaling, opacity, color, scale_rot))
    work = torch.empty(2, max(n, 1), dtype=torch.int32, device=dev)
    scratch = torch.empty(max(int(scratch_bytes(max(n, 1))), 4), dtype=torch.uint8, device=dev)
    xyz, col, scl, rot, opa = (torch.empty(max(n, 1), w, dtype=torch.float32, device=dev) for w in (3, 3, 3, 4, 1))
    count = torch.zeros(1, dtype=torch.int32, device=dev)
    native.check(lib.lmb_anchor_epilogue(anchor.data_ptr(), offsets.data_ptr(), scaling.data_ptr(), opacity.data_ptr(),
                                         color.data_ptr(), scale_rot.data_ptr(), n, k, work[0].data_ptr(), work[1].data_ptr(),
                                         scratch.data_ptr(), xyz.data_ptr(), col.data_ptr(), opa.data_ptr(), scl.data_ptr(),
                                         rot.data_ptr(), count.data_ptr(), native.stream_ptr()), "anchor_epilogue")
    m = int(count.item())
    return xyz[:m], col[:m], opa[:m], scl[:m], rot[:m]


class FusedAnchorDecoder(AnchorDecoder):
    """Same decoder with the three heads evaluated by the fused MLP kernel at render time."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.use_fused = True
