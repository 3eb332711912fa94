"""Optional NeRF refinement branch of GridNeRF: an 8-layer-style MLP that consumes grid features
(reference: landmark/nerf_components/model_components/fields/nerf_branch.py:41-194)."""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from ...ops import composite_weights
from .mlp_decoder import positional_encoding


def raw2alpha(raw, dists, act_fn=F.relu):
    return 1.0 - torch.exp(-act_fn(raw) * dists)


def raw2outputs(raw: torch.Tensor, dists=1):
    """``raw [R, S, 4]`` (rgb logits + density) -> composite; dists broadcast to ``[R, S]``."""
    rgb = torch.sigmoid(raw[..., :3])
    sigma = F.relu(raw[..., 3])
    d = dists if torch.is_tensor(dists) else torch.full_like(sigma, float(dists))
    weights, _ = composite_weights(sigma, d.expand_as(sigma).contiguous())
    alpha = 1.0 - torch.exp(-sigma * d)
    return {"rgb_map": (weights[..., None] * rgb).sum(-2), "weights": weights, "rgb": rgb, "alpha": alpha}


class NeRF(nn.Module):
    def __init__(self, args, den_n_comp: int, app_n_comp: int, nfreqs=None):
        super().__init__()
        self.num_freq = args.nerf_freq if nfreqs is None else nfreqs
        self.den_n_comp, self.app_n_comp = den_n_comp, app_n_comp
        self.skips = [4]
        self.use_viewdirs = True
        self.D, self.D_a, self.W = args.nerf_D, args.nerf_D_a, args.nerf_W
        self.encode_app = args.encode_app
        W = self.W
        in_pts = 3 + 6 * self.num_freq + den_n_comp
        in_views = 3 + 24 + app_n_comp + W + (48 if self.encode_app else 0)
        self.pts_linears = nn.ModuleList(
            [nn.Linear(in_pts, W)] + [nn.Linear(W + in_pts if i in self.skips else W, W) for i in range(self.D - 1)])
        self.views_linears = nn.ModuleList(
            [nn.Linear(in_views, W // 2)] + [nn.Linear(W // 2, W // 2) for _ in range(self.D_a - 1)])
        self.feature_linear = nn.Linear(W, W)
        self.alpha_linear = nn.Linear(W, 1)
        self.rgb_linear = nn.Linear(W // 2, 3)

    def forward(self, pts, viewdir=None, den_feats=None, app_feats=None, app_latent=None):
        x = torch.cat((pts, positional_encoding(pts, self.num_freq), den_feats), dim=-1)
        h = x
        for i, layer in enumerate(self.pts_linears):
            h = F.relu(layer(h))
            if i in self.skips:
                h = torch.cat((x, h), dim=-1)
        alpha = self.alpha_linear(h)
        viewdir = viewdir.reshape(-1, 3)
        parts = [self.feature_linear(h), viewdir, positional_encoding(viewdir, 4), app_feats]
        if self.encode_app:
            parts.append(app_latent)
        h = torch.cat(parts, dim=-1)
        for layer in self.views_linears:
            h = F.relu(layer(h))
        return torch.cat((self.rgb_linear(h), alpha), dim=-1)
