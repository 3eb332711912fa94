"""Model base classes and the on-disk checkpoint contract (reference:
landmark/nerf_components/model/base_model.py:13-372).

NeRF-type models save ``state_dict.th`` + ``kwargs.th`` (``-sub{rank}`` suffixes for per-rank
model-parallel shards).  Gaussian models save the point-based encoding as ``point_cloud.ply`` and
everything else as ``state_dict.th``.
"""
from __future__ import annotations

import os
from typing import Any, Dict, Mapping, Optional

import torch
from torch.nn.parallel import DistributedDataParallel as DDP

from .base_module import BaseModule


def _strip_wrappers(state: Dict[str, Any], model: torch.nn.Module, prefix: str) -> Dict[str, Any]:
    """Remove ``module.`` segments introduced by (nested) DDP wrappers from state-dict keys."""
    wrapped = [name for name, mod in model.named_modules() if isinstance(mod, DDP)]
    out: Dict[str, Any] = {}
    for key, value in state.items():
        if prefix == "module." and key.startswith(prefix):
            key = key[len(prefix):]
        for name in wrapped:
            head = f"{name}.module." if name else "module."
            if key.startswith(head):
                key = (f"{name}." if name else "") + key[len(head):]
        out[key] = value
    return out


def _tensors_to(obj, device):
    if isinstance(obj, dict):
        return {k: _tensors_to(v, device) for k, v in obj.items()}
    if torch.is_tensor(obj):
        return obj.to(device)
    return obj


class Model(BaseModule):
    """Holds ``config``, ``scene_manager`` and the constructor kwargs that go into ``kwargs.th``."""

    def __init__(self, config=None, scene_manager=None, **kwargs):
        super().__init__()
        self.config = config
        self.scene_manager = scene_manager
        self._kwargs_keys = list(kwargs.keys())
        for key, value in kwargs.items():
            setattr(self, key, value)

    def kwargs(self) -> Dict[str, Any]:
        return {key: getattr(self, key) for key in self._kwargs_keys}

    def state_dict(self, *args, destination=None, prefix="", keep_vars=False):
        state = super().state_dict(*args, destination=destination, prefix=prefix, keep_vars=keep_vars)
        cleaned = _strip_wrappers(dict(state), self, prefix)
        state.clear()
        state.update(cleaned)
        return state

    # -- saving -------------------------------------------------------------------
    def save_kwargs(self, file_path) -> None:
        kwargs = self.kwargs()
        assert len(kwargs) > 0, "model has no constructor kwargs to save"
        torch.save(kwargs, file_path)

    def save_state_dict(self, file_path) -> None:
        state = self.state_dict()
        assert len(state) > 0, "model has an empty state dict"
        torch.save(state, file_path)

    def save_model(self, dir_path, rank: Optional[int] = None) -> None:
        os.makedirs(dir_path, exist_ok=True)
        suffix = "" if rank is None else f"-sub{rank}"
        if self._kwargs_keys:
            self.save_kwargs(os.path.join(dir_path, f"kwargs{suffix}.th"))
        self.save_state_dict(os.path.join(dir_path, f"state_dict{suffix}.th"))

    # -- loading -------------------------------------------------------------------
    def get_state_dict_from_ckpt(self, file_path, map_location, prefix: str = "") -> Mapping[str, Any]:
        assert os.path.exists(file_path), f"checkpoint {file_path} not found"
        return torch.load(file_path, map_location=map_location, weights_only=False)

    @staticmethod
    def get_kwargs_from_ckpt(file_path, map_location) -> Dict[str, Any]:
        assert os.path.exists(file_path), f"kwargs file {file_path} not found"
        kwargs = torch.load(file_path, map_location=map_location, weights_only=False)
        if "device" in kwargs:
            kwargs["device"] = map_location
        return _tensors_to(kwargs, map_location)

    def load_from_state_dict(self, state_dict: Mapping[str, Any], strict: bool = True):
        return super().load_state_dict(state_dict, strict)


class BaseNeRF(Model):
    """Volume-rendered radiance field: sampler + field components + renderer."""

    def init_sampler(self):
        raise NotImplementedError

    def init_field_components(self):
        raise NotImplementedError

    def init_renderer(self):
        raise NotImplementedError

    @torch.no_grad()
    def render_all_rays(self, rays, chunk_size=None, N_samples=-1, idxs=None, app_code=None):
        """Render ``rays [N, 6|7]`` in chunks of ``chunk_size`` and concatenate the maps."""
        n_total = rays.shape[0]
        chunk_size = chunk_size or n_total
        if idxs is None:
            idxs = torch.zeros(n_total, device=rays.device, dtype=rays.dtype)
        rgb, depth = [], []
        for start in range(0, n_total, chunk_size):
            chunk = rays[start:start + chunk_size]
            if chunk.shape[-1] == 6:
                chunk = torch.cat((chunk, idxs[start:start + chunk_size, None].to(chunk.dtype)), dim=-1)
            out = self.forward(chunk)
            if isinstance(out, dict):
                rgb.append(out["rgb_map"]); depth.append(out["depth_map"])
            else:
                rgb.append(out[0]); depth.append(out[1])
        return {"rgb_map": torch.cat(rgb, 0), "depth_map": torch.cat(depth, 0)}


class BaseGaussian(Model):
    """Point-based model: a Gaussian encoding (saved as PLY) + neural parts (saved as ``state_dict.th``)."""

    def init_field_components(self):
        raise NotImplementedError

    def init_renderer(self):
        raise NotImplementedError

    def _find_gaussian_encoding(self):
        from ..fields.encodings.base_encoding import BaseGaussianEncoding

        found = [(name, mod) for name, mod in self.named_modules() if isinstance(mod, BaseGaussianEncoding)]
        assert found, "model has no Gaussian encoding"
        return found[-1]

    def save_ply(self, dir_path, rank: Optional[int] = None) -> None:
        """``point_cloud[-sub{rank}].ply`` of the Gaussian encoding (reference: base_model.py:266-281)."""
        os.makedirs(dir_path, exist_ok=True)
        suffix = "" if rank is None else f"-sub{rank}"
        self._find_gaussian_encoding()[1].save_ply(os.path.join(dir_path, f"point_cloud{suffix}.ply"))

    def save_state_dict(self, file_path) -> None:
        """Everything but the Gaussian encoding, which travels as PLY (reference: base_model.py:283-304)."""
        name, _ = self._find_gaussian_encoding()
        torch.save({k: v for k, v in self.state_dict().items() if not k.startswith(name + ".")}, file_path)

    def save_model(self, dir_path, rank: Optional[int] = None) -> None:
        suffix = "" if rank is None else f"-sub{rank}"
        self.save_ply(dir_path, rank)
        self.save_state_dict(os.path.join(dir_path, f"state_dict{suffix}.th"))
        if self._kwargs_keys:
            self.save_kwargs(os.path.join(dir_path, f"kwargs{suffix}.th"))

    def get_state_dict_from_ckpt(self, file_path, map_location, prefix: str = "") -> Mapping[str, Any]:
        """``file_path`` is the ``point_cloud*.ply``; the sibling ``state_dict*.th`` is merged in."""
        name, encoding = self._find_gaussian_encoding()
        state = {f"{name}.{k}": v for k, v in encoding.load_ply_to_state_dict(file_path, map_location).items()}
        sibling = os.path.join(os.path.dirname(file_path),
                               os.path.basename(file_path).replace("point_cloud", "state_dict").replace(".ply", ".th"))
        if os.path.exists(sibling):
            state.update(torch.load(sibling, map_location=map_location, weights_only=False))
        return state

    def load_from_state_dict(self, state_dict: Mapping[str, Any], strict: bool = True):
        name, encoding = self._find_gaussian_encoding()
        head = name + "."
        encoding.load_encoding_state({k[len(head):]: v for k, v in state_dict.items() if k.startswith(head)})
        rest = {k: v for k, v in state_dict.items() if not k.startswith(head)}
        return super().load_state_dict(rest, strict=False)
