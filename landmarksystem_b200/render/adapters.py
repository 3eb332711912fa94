"""Ready-made inference adapters: pose -> rays -> image for the ray models, camera -> image for the
Gaussian models (the reference keeps equivalent adapters in its test helpers, tests/utils.py:15-201)."""
from __future__ import annotations

import torch

from ..components.data.datasets.ray_utils import get_ray_directions_blender, get_rays_with_directions
from .inference_module import InferenceModule


class NeRFInferenceModule(InferenceModule):
    """``engine(pose [4,4] c2w, chunk_size, H, W, focal=None, app_code=0)`` -> ``uint8`` RGBA image
    ``[H, W, 4]`` (and the depth map as second output)."""

    model_cls = None

    def __init__(self, **kwargs):
        super().__init__(self.model_cls(**kwargs))
        self._shape = None

    def preprocess(self, pose, chunk_size=8192, H=1080, W=1920, focal=None, app_code=0, **_):
        dev = next(self.model.parameters()).device
        focal = focal if focal is not None else 2317.6450 * (W / 1920.0)
        # the per-pixel camera-space directions depend on the intrinsics only: built once per (H, W, focal) and kept on the
        # device, so a frame costs one small pose upload and a matrix product instead of ~25 ms of host tensor ops and a
        # 25 MB pageable copy (1080p)
        key = (int(H), int(W), tuple(focal) if isinstance(focal, (list, tuple)) else float(focal), str(dev))
        cache = getattr(self, "_dirs_cache", None)
        if cache is None or cache[0] != key:
            cache = self._dirs_cache = (key, get_ray_directions_blender(int(H), int(W), focal).to(dev))
        dirs = cache[1]
        o, d = get_rays_with_directions(dirs, torch.as_tensor(pose, dtype=torch.float32, device=dev))
        d = d / d.norm(dim=-1, keepdim=True) if getattr(self.model.config, "normalize_render_dirs", True) else d
        self._shape = (int(H), int(W))
        self._chunk = int(chunk_size)
        return (torch.cat((o, d), -1),), {}

    def forward(self, rays):
        mp = getattr(self.model, "_mp_renderer", None)
        if mp is not None:                       # block model parallel: partial composites merged across the GPUs
            rgb, depth, _ = mp.render(rays, chunk=self._chunk)
            return rgb, depth
        ret = self.model.render_all_rays(rays, chunk_size=self._chunk)
        return ret["rgb_map"], ret["depth_map"].reshape(rays.shape[0], -1)[:, 0]

    def postprocess(self, rgb, depth=None):
        H, W = self._shape
        img = (rgb.clamp(0, 1).reshape(H, W, 3) * 255).to(torch.uint8)
        alpha = torch.full((H, W, 1), 255, dtype=torch.uint8, device=img.device)
        out = torch.cat((img, alpha), dim=-1)
        return out if depth is None else (out, depth.reshape(H, W))


class GaussianInferenceModule(InferenceModule):
    """``engine(camera)`` -> ``uint8`` image ``[H, W, 3]``.  The camera is reduced to plain tensors /
    numbers before it is pickled for the other ranks."""

    model_cls = None

    def __init__(self, **kwargs):
        super().__init__(self.model_cls(**kwargs))

    def preprocess(self, camera, **_):
        camera.image = None
        return (camera,), {}

    def forward(self, camera):
        return self.model(camera)

    def postprocess(self, image):
        return (image.clamp(0, 1).permute(1, 2, 0) * 255).to(torch.uint8)


def make_adapter(model_cls, gaussian: bool = False):
    base = GaussianInferenceModule if gaussian else NeRFInferenceModule
    return type(f"{model_cls.__name__}InferenceModule", (base,), {"model_cls": model_cls})
