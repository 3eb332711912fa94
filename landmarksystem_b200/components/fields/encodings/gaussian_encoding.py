"""Vanilla 3D Gaussian splatting parameter store (reference:
landmark/nerf_components/model_components/fields/encodings/gaussian_encoding.py:26-947).

Parameters (names as in the reference checkpoints): ``_xyz [N,3]``, ``_features_dc [N,1,3]``,
``_features_rest [N,15,3]``, ``_scaling [N,3]`` (log), ``_rotation [N,4]``, ``_opacity [N,1]`` (logit).
Provides activations, point-cloud initialisation, PLY I/O (standard and activation-cache variants),
densification (clone / split / prune, opacity reset) and the optimiser-state surgery that goes with it.
"""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np
import torch
from torch import nn

from ....ops.knn import distCUDA2
from ....render.types import MergeType
from ...utils.general_utils import build_rotation, build_scaling_rotation, inverse_sigmoid, strip_symmetric
from ...utils.ply_utils import read_ply, write_ply
from ...utils.sh_utils import RGB2SH
from .base_encoding import BaseGaussianEncoding

_GROUPS = {"xyz": "_xyz", "f_dc": "_features_dc", "f_rest": "_features_rest", "opacity": "_opacity",
           "scaling": "_scaling", "rotation": "_rotation"}


# -- optimiser-state surgery (shared with the anchor encodings) ---------------------------------------------
def _state_tensors(state: dict):
    return [k for k in ("exp_avg", "exp_avg_sq") if k in state]


def replace_tensor_to_optimizer(optimizer, tensor: torch.Tensor, name: str) -> Dict[str, nn.Parameter]:
    """Swap the tensor of group ``name`` for ``tensor`` and zero its Adam moments."""
    out = {}
    for group in optimizer.param_groups:
        if group.get("name") != name:
            continue
        old = group["params"][0]
        state = optimizer.state.pop(old, None)
        new = nn.Parameter(tensor.requires_grad_(True))
        if state:
            for k in _state_tensors(state):
                state[k] = torch.zeros_like(tensor)
            optimizer.state[new] = state
        group["params"][0] = new
        out[name] = new
    return out


def prune_optimizer(optimizer, keep_mask: torch.Tensor, names=None) -> Dict[str, nn.Parameter]:
    out = {}
    for group in optimizer.param_groups:
        name = group.get("name")
        if name is None or (names is not None and name not in names) or len(group["params"]) != 1:
            continue
        old = group["params"][0]
        if old.shape[0] != keep_mask.shape[0]:
            continue
        state = optimizer.state.pop(old, None)
        new = nn.Parameter(old.detach()[keep_mask].clone().requires_grad_(True))
        if state:
            for k in _state_tensors(state):
                state[k] = state[k][keep_mask].clone()
            optimizer.state[new] = state
        group["params"][0] = new
        out[name] = new
    return out


def cat_tensors_to_optimizer(optimizer, tensors: Dict[str, torch.Tensor]) -> Dict[str, nn.Parameter]:
    out = {}
    for group in optimizer.param_groups:
        name = group.get("name")
        if name not in tensors or len(group["params"]) != 1:
            continue
        ext = tensors[name]
        old = group["params"][0]
        state = optimizer.state.pop(old, None)
        new = nn.Parameter(torch.cat((old.detach(), ext), dim=0).requires_grad_(True))
        if state:
            for k in _state_tensors(state):
                state[k] = torch.cat((state[k], torch.zeros_like(ext)), dim=0)
            optimizer.state[new] = state
        group["params"][0] = new
        out[name] = new
    return out


def build_covariance_from_scaling_rotation(scaling: torch.Tensor, scaling_modifier: float, rotation: torch.Tensor):
    """Upper triangle ``[N, 6]`` of ``R S S^T R^T`` with ``S = diag(scaling_modifier * scaling)`` and ``R`` from the
    quaternions ``rotation`` (reference: gaussian_encoding.py:22-38)."""
    L = build_scaling_rotation(scaling_modifier * scaling, rotation)
    return strip_symmetric(L @ L.transpose(1, 2))


class GaussianEncoding(BaseGaussianEncoding):
    def __init__(self, sh_degree: int = 3, percent_dense: float = 0.01, act_cache: bool = False, device="cuda"):
        super().__init__()
        self.active_sh_degree = 0
        self.max_sh_degree = sh_degree
        self.percent_dense = percent_dense
        self.act_cache = act_cache
        dev = device if (torch.cuda.is_available() or str(device) == "cpu") else "cpu"
        self.device = torch.device(dev)
        n_rest = (sh_degree + 1) ** 2 - 1
        z = lambda *s: nn.Parameter(torch.zeros(*s, device=self.device))  # noqa: E731
        self._xyz, self._features_dc, self._features_rest = z(0, 3), z(0, 1, 3), z(0, n_rest, 3)
        self._scaling, self._rotation, self._opacity = z(0, 3), z(0, 4), z(0, 1)
        self.max_radii2D = torch.empty(0, device=self.device)
        self.xyz_gradient_accum = torch.empty(0, device=self.device)
        self.denom = torch.empty(0, device=self.device)
        self._cache: Dict[str, torch.Tensor] = {}
        self.save_init_kwargs(locals())
        self.merge_config = {"merge_type": MergeType.Unevenly, "_xyz": 0, "_features_dc": 0, "_features_rest": 0,
                             "_scaling": 0, "_rotation": 0, "_opacity": 0}

    # -- activations -----------------------------------------------------------------------------
    scaling_activation = staticmethod(torch.exp)
    scaling_inverse_activation = staticmethod(torch.log)
    opacity_activation = staticmethod(torch.sigmoid)
    inverse_opacity_activation = staticmethod(inverse_sigmoid)
    rotation_activation = staticmethod(torch.nn.functional.normalize)

    def _cached(self, name, fn):
        if self.act_cache and not self.training:
            if name not in self._cache:
                self._cache[name] = fn().detach()
            return self._cache[name]
        return fn()

    def clear_cache(self):
        self._cache = {}

    @property
    def get_scaling(self):
        return self._cached("scaling", lambda: self.scaling_activation(self._scaling))

    @property
    def get_rotation(self):
        return self._cached("rotation", lambda: self.rotation_activation(self._rotation))

    @property
    def get_xyz(self):
        return self._xyz

    @property
    def get_features(self):
        return self._cached("features", lambda: torch.cat((self._features_dc, self._features_rest), dim=1))

    @property
    def get_opacity(self):
        return self._cached("opacity", lambda: self.opacity_activation(self._opacity))

    covariance_activation = staticmethod(build_covariance_from_scaling_rotation)

    def get_covariance(self, scaling_modifier: float = 1.0):
        return build_covariance_from_scaling_rotation(self.get_scaling, scaling_modifier, self._rotation)

    # -- setters (reference: gaussian_encoding.py:855-925).  With ``act_cache`` outside training the value is the
    # ACTIVATED quantity and lands in the cache the getters read; otherwise it replaces the raw tensor. ---------
    def _set(self, cache_name: str, attr: str, value: torch.Tensor):
        if self.act_cache and not self.training:
            self._cache[cache_name] = value
        elif isinstance(getattr(self, attr), nn.Parameter):
            getattr(self, attr).data = value
        else:
            setattr(self, attr, value)

    def set_scaling(self, value: torch.Tensor):
        self._set("scaling", "_scaling", value)

    def set_rotation(self, value: torch.Tensor):
        self._set("rotation", "_rotation", value)

    def set_opacity(self, value: torch.Tensor):
        self._set("opacity", "_opacity", value)

    def set_features(self, value: torch.Tensor):
        if not (self.act_cache and not self.training):
            raise NotImplementedError("features are set as a whole only through the activation cache")
        self._cache["features"] = value

    def set_xyz(self, value: torch.Tensor):
        if isinstance(self._xyz, nn.Parameter):
            self._xyz.data = value
        else:
            self._xyz = value

    # -- optimiser surgery under the reference's method names (gaussian_encoding.py:429-496) ---------------------
    def cat_tensors_to_optimizer(self, tensors_dict: Dict[str, torch.Tensor], optimizer) -> Dict[str, nn.Parameter]:
        return cat_tensors_to_optimizer(optimizer, tensors_dict)

    def replace_tensor_to_optimizer(self, tensor: torch.Tensor, name: str, optimizer) -> Dict[str, nn.Parameter]:
        return replace_tensor_to_optimizer(optimizer, tensor, name)

    def oneupSHdegree(self):
        if self.active_sh_degree < self.max_sh_degree:
            self.active_sh_degree += 1

    def __len__(self):
        return self._xyz.shape[0]

    # -- initialisation ------------------------------------------------------------------------------
    def _set_params(self, xyz, f_dc, f_rest, scaling, rotation, opacity):
        dev = self.device
        self._xyz = nn.Parameter(xyz.to(dev).float().contiguous())
        self._features_dc = nn.Parameter(f_dc.to(dev).float().contiguous())
        self._features_rest = nn.Parameter(f_rest.to(dev).float().contiguous())
        self._scaling = nn.Parameter(scaling.to(dev).float().contiguous())
        self._rotation = nn.Parameter(rotation.to(dev).float().contiguous())
        self._opacity = nn.Parameter(opacity.to(dev).float().contiguous())
        n = self._xyz.shape[0]
        self.max_radii2D = torch.zeros(n, device=dev)
        self.xyz_gradient_accum = torch.zeros(n, 1, device=dev)
        self.denom = torch.zeros(n, 1, device=dev)
        self.clear_cache()

    def create_from_pcd(self, pcd, spatial_lr_scale: float = 1.0):
        pts = torch.as_tensor(np.asarray(pcd.points), dtype=torch.float32, device=self.device)
        col = RGB2SH(torch.as_tensor(np.asarray(pcd.colors), dtype=torch.float32, device=self.device))
        n, n_coef = pts.shape[0], (self.max_sh_degree + 1) ** 2
        feats = torch.zeros(n, n_coef, 3, device=self.device)
        feats[:, 0, :] = col
        dist2 = distCUDA2(pts).clamp_min(1e-7)
        scales = torch.log(torch.sqrt(dist2))[:, None].repeat(1, 3)
        rots = torch.zeros(n, 4, device=self.device)
        rots[:, 0] = 1
        opac = inverse_sigmoid(0.1 * torch.ones(n, 1, device=self.device))
        self._set_params(pts, feats[:, :1], feats[:, 1:], scales, rots, opac)

    # -- PLY -----------------------------------------------------------------------------------------------
    def construct_list_of_attributes(self):
        names = ["x", "y", "z", "nx", "ny", "nz"]
        names += [f"f_dc_{i}" for i in range(self._features_dc.shape[1] * self._features_dc.shape[2])]
        names += [f"f_rest_{i}" for i in range(self._features_rest.shape[1] * self._features_rest.shape[2])]
        names += ["opacity"] + [f"scale_{i}" for i in range(self._scaling.shape[1])]
        names += [f"rot_{i}" for i in range(self._rotation.shape[1])]
        return names

    def construct_list_of_cache_attributes(self):
        return [("cache_" + n if n not in ("x", "y", "z", "nx", "ny", "nz") else n)
                for n in self.construct_list_of_attributes()]

    def save_ply(self, path: str, cache: bool = False):
        """Standard PLY (raw parameters) or, with ``cache``, the activation-cache variant whose
        ``cache_*`` properties hold activated opacity / scale / rotation."""
        xyz = self._xyz.detach().cpu().numpy()
        f_dc = self._features_dc.detach().transpose(1, 2).flatten(1).cpu().numpy()
        f_rest = self._features_rest.detach().transpose(1, 2).flatten(1).cpu().numpy()
        if cache:
            op, sc, rot = self.get_opacity, self.get_scaling, self.get_rotation
        else:
            op, sc, rot = self._opacity, self._scaling, self._rotation
        op, sc, rot = (t.detach().cpu().numpy() for t in (op, sc, rot))
        data = np.concatenate((xyz, np.zeros_like(xyz), f_dc, f_rest, op, sc, rot), axis=1).astype(np.float32)
        names = self.construct_list_of_cache_attributes() if cache else self.construct_list_of_attributes()
        write_ply(path, {n: data[:, i] for i, n in enumerate(names)})

    def load_ply_to_state_dict(self, path: str, map_location="cpu") -> Dict[str, torch.Tensor]:
        v = read_ply(path)
        names = v.dtype.names
        cached = any(n.startswith("cache_") for n in names)
        pre = "cache_" if cached else ""

        def cols(prefix):
            keys = sorted([n for n in names if n.startswith(pre + prefix)], key=lambda s: int(s.split("_")[-1]))
            return np.stack([v[k] for k in keys], 1).astype(np.float32) if keys else np.zeros((len(v), 0), np.float32)

        xyz = np.stack((v["x"], v["y"], v["z"]), 1).astype(np.float32)
        f_dc = cols("f_dc_").reshape(len(v), 3, -1).transpose(0, 2, 1)
        f_rest = cols("f_rest_")
        n_rest = (self.max_sh_degree + 1) ** 2 - 1
        f_rest = f_rest.reshape(len(v), 3, n_rest).transpose(0, 2, 1) if f_rest.shape[1] else np.zeros((len(v), n_rest, 3), np.float32)
        opacity = np.asarray(v[pre + "opacity"], dtype=np.float32)[:, None]
        scaling, rotation = cols("scale_"), cols("rot_")
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(map_location)  # noqa: E731
        state = {"_xyz": t(xyz), "_features_dc": t(f_dc), "_features_rest": t(f_rest), "_opacity": t(opacity),
                 "_scaling": t(scaling), "_rotation": t(rotation)}
        if cached:  # stored activated: map back to raw parameters
            state["_opacity"] = inverse_sigmoid(state["_opacity"].clamp(1e-6, 1 - 1e-6))
            state["_scaling"] = torch.log(state["_scaling"].clamp_min(1e-12))
        return state

    def load_ply(self, path: str):
        self.load_encoding_state(self.load_ply_to_state_dict(path, self.device))
        self.active_sh_degree = self.max_sh_degree

    def load_encoding_state(self, state: Dict[str, torch.Tensor]):
        self._set_params(state["_xyz"], state["_features_dc"], state["_features_rest"], state["_scaling"],
                         state["_rotation"], state["_opacity"])
        self.active_sh_degree = self.max_sh_degree

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        keys = [prefix + n for n in _GROUPS.values()]
        if all(k in state_dict for k in keys):  # adopt checkpoint sizes before the strict copy
            self.load_encoding_state({n: state_dict[prefix + n] for n in _GROUPS.values()})
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    # -- densification -------------------------------------------------------------------------------------------
    def _adopt(self, tensors: Dict[str, nn.Parameter]):
        for group_name, attr in _GROUPS.items():
            if group_name in tensors:
                setattr(self, attr, tensors[group_name])
        self.clear_cache()

    def reset_opacity(self, optimizer):
        new = inverse_sigmoid(torch.min(self.get_opacity, torch.ones_like(self.get_opacity) * 0.01))
        self._adopt(replace_tensor_to_optimizer(optimizer, new.detach().clone(), "opacity"))

    def prune_points(self, mask: torch.Tensor, optimizer):
        keep = ~mask
        self._adopt(prune_optimizer(optimizer, keep, set(_GROUPS)))
        self.xyz_gradient_accum, self.denom = self.xyz_gradient_accum[keep], self.denom[keep]
        self.max_radii2D = self.max_radii2D[keep]

    def densification_postfix(self, new, *rest, optimizer=None):
        """Append new Gaussians: ``densification_postfix({"xyz": ..., "f_dc": ..., "f_rest": ..., "opacity": ...,
        "scaling": ..., "rotation": ...}, optimizer)``, or the reference's positional form ``(new_xyz, new_features_dc,
        new_features_rest, new_opacities, new_scaling, new_rotation, optimizer)`` (gaussian_encoding.py:498-542)."""
        if torch.is_tensor(new):
            tensors = (new,) + tuple(rest[:5])
            optimizer = rest[5] if len(rest) > 5 else optimizer
            new = dict(zip(("xyz", "f_dc", "f_rest", "opacity", "scaling", "rotation"), tensors))
        else:
            optimizer = rest[0] if rest else optimizer
        self._adopt(cat_tensors_to_optimizer(optimizer, new))
        n = self._xyz.shape[0]
        self.xyz_gradient_accum = torch.zeros(n, 1, device=self._xyz.device)
        self.denom = torch.zeros(n, 1, device=self._xyz.device)
        self.max_radii2D = torch.zeros(n, device=self._xyz.device)

    def _gather(self, mask, repeat: int = 1):
        rep = lambda t: t.detach()[mask].repeat(repeat, *([1] * (t.dim() - 1)))  # noqa: E731
        return {"f_dc": rep(self._features_dc), "f_rest": rep(self._features_rest), "opacity": rep(self._opacity),
                "rotation": rep(self._rotation)}

    def densify_and_split(self, grads, grad_threshold, scene_extent, optimizer, N: int = 2):
        n = self._xyz.shape[0]
        padded = torch.zeros(n, device=self._xyz.device)
        padded[: grads.shape[0]] = grads.squeeze()
        mask = (padded >= grad_threshold) & (self.get_scaling.max(dim=1).values > self.percent_dense * scene_extent)
        if mask.sum() == 0:
            return
        stds = self.get_scaling[mask].repeat(N, 1)
        samples = torch.normal(mean=torch.zeros_like(stds), std=stds)
        rots = build_rotation(self._rotation[mask]).repeat(N, 1, 1)
        new = self._gather(mask, N)
        new["xyz"] = (rots @ samples[..., None]).squeeze(-1) + self._xyz.detach()[mask].repeat(N, 1)
        new["scaling"] = self.scaling_inverse_activation(self.get_scaling[mask].repeat(N, 1) / (0.8 * N)).detach()
        self.densification_postfix(new, optimizer)
        prune = torch.cat((mask, torch.zeros(N * int(mask.sum()), dtype=torch.bool, device=mask.device)))
        self.prune_points(prune, optimizer)

    def densify_and_clone(self, grads, grad_threshold, scene_extent, optimizer):
        mask = (torch.norm(grads, dim=-1) >= grad_threshold) & \
               (self.get_scaling.max(dim=1).values <= self.percent_dense * scene_extent)
        if mask.sum() == 0:
            return
        new = self._gather(mask)
        new["xyz"] = self._xyz.detach()[mask]
        new["scaling"] = self._scaling.detach()[mask]
        self.densification_postfix(new, optimizer)

    def densify_and_prune(self, max_grad, min_opacity, extent, max_screen_size, optimizer):
        grads = self.xyz_gradient_accum / self.denom
        grads[grads.isnan()] = 0.0
        self.densify_and_clone(grads, max_grad, extent, optimizer)
        self.densify_and_split(grads, max_grad, extent, optimizer)
        prune = (self.get_opacity < min_opacity).squeeze()
        if max_screen_size:
            prune = prune | (self.max_radii2D > max_screen_size) | (self.get_scaling.max(dim=1).values > 0.1 * extent)
        self.prune_points(prune, optimizer)

    def add_densification_stats(self, viewspace_point_tensor, update_filter):
        grad = viewspace_point_tensor.grad
        if grad is None:
            return
        self.xyz_gradient_accum[update_filter] += torch.norm(grad[update_filter, :2], dim=-1, keepdim=True)
        self.denom[update_filter] += 1
