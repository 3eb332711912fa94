"""A model, its configuration block and its trainer written by a user of the framework from the shipped components
(the walk-through of docs/trainer.md): hash-grid field + two small heads + uniform samples + the composite renderer,
trained by ``RayModelTrainer`` and reloaded from its checkpoint."""
import os
import textwrap

import numpy as np
import torch

from landmarksystem_b200.components.fields.encodings.hash_encoding import HashEncoding
from landmarksystem_b200.components.fields.mlp_decoder import MLPDecoder
from landmarksystem_b200.components.model.base_model import BaseNeRF
from landmarksystem_b200.configs import BaseConfig, ConfigClass
from landmarksystem_b200.ops import composite_render, composite_weights
from landmarksystem_b200.train.ray_trainer import RayModelTrainer


class TinyFieldConfig(ConfigClass):
    num_levels: int = 4
    log2_hashmap_size: int = 12
    hidden_dim: int = 32
    n_samples: int = 32
    train_near_far: list = [1.2, 4.8]
    lr_init: float = 1e-2
    lr_final: float = 1e-3
    lr_decay_max_steps: int = 100
    eps: float = 1e-15

    def check_args(self):
        assert self.n_samples > 1


class TinyField(BaseNeRF):
    def __init__(self, aabb, device, near_far, scene_manager=None, config=None, group=None):
        super().__init__(config=config, scene_manager=scene_manager, aabb=aabb, device=device, near_far=list(near_far))
        self.aabb = torch.as_tensor(aabb, dtype=torch.float32, device=device)
        self.device, self.near_far = device, list(near_far)
        self.init_field_components()

    def init_field_components(self):
        c = self.config
        self.grid = HashEncoding(c.num_levels, 8, 64, c.log2_hashmap_size, 2, device=self.device)
        self.density_head = MLPDecoder(self.grid.get_out_dim(), c.hidden_dim, 2, 1, None, mlp_bias=False).to(self.device)
        self.colour_head = MLPDecoder(self.grid.get_out_dim() + 3, c.hidden_dim, 2, 3, torch.nn.Sigmoid(),
                                      mlp_bias=False).to(self.device)

    def init_sampler(self):
        pass

    def init_renderer(self):
        pass

    def forward(self, rays_chunk):
        o, d = rays_chunk[:, :3], rays_chunk[:, 3:6]
        near, far = self.near_far
        S = self.config.n_samples
        edges = torch.linspace(near, far, S + 1, device=o.device)
        z = 0.5 * (edges[1:] + edges[:-1]).expand(o.shape[0], S)
        if self.training:
            z = z + (torch.rand_like(z) - 0.5) * (far - near) / S
        pts = o[:, None] + d[:, None] * z[..., None]
        unit = ((pts - self.aabb[0]) / (self.aabb[1] - self.aabb[0])).reshape(-1, 3)
        inside = ((unit > 0) & (unit < 1)).all(-1)
        feats = self.grid(unit.clamp(0, 1))
        sigma = torch.nn.functional.softplus(self.density_head(feats)[:, 0] - 1.0) * inside
        rgb = self.colour_head(torch.cat((feats, d[:, None].expand(-1, S, -1).reshape(-1, 3)), -1))
        dists = torch.full_like(z, (far - near) / S)
        weights, _ = composite_weights(sigma.view(-1, S), dists)
        rgb_map, depth_map, _ = composite_render(weights, rgb.view(-1, S, 3), z, bg=0.0)
        return {"rgb_map": rgb_map, "depth_map": depth_map}

    def get_optparam_groups(self):
        return [{"params": list(self.parameters()), "lr": self.config.lr_init}]

    def kwargs(self):
        return {"aabb": self.aabb, "device": self.device, "near_far": self.near_far}


class TinyTrainer(RayModelTrainer):
    model_cls = TinyField


CONF = """
from landmarksystem_b200.configs import DatasetConfig, TrainConfig
from test_custom_model import TinyFieldConfig

config = [TrainConfig(model_name="TinyField", expname="tiny_field", basedir="{basedir}", n_iters=40, batch_size=512,
                      progress_refresh_rate=10, vis_every=100000, N_vis=1, random_seed=0, print_timestamp=False, device="cpu"),
          DatasetConfig(dataset_name="synthetic", datadir="ring:4:16x16:20:3", lb=[-1.0, -1.0, -1.0], ub=[1.0, 1.0, 1.0]),
          TinyFieldConfig()]
"""


def test_user_model_trains_saves_and_reloads(tmp_path):
    import sys

    sys.path.insert(0, os.path.dirname(__file__))            # lets the configuration file import this module's block
    conf = tmp_path / "tiny_conf.py"
    conf.write_text(textwrap.dedent(CONF.format(basedir=str(tmp_path))))
    trainer = TinyTrainer(BaseConfig.from_file(str(conf)))
    psnrs = trainer.train()
    assert len(psnrs) == 4 and psnrs[-1] > psnrs[0]           # the loss goes down on the analytic scene
    assert np.isfinite(trainer.eval())
    ckpt = os.path.join(trainer.logfolder, "state_dict.th")
    kwargs = TinyField.get_kwargs_from_ckpt(os.path.join(trainer.logfolder, "kwargs.th"), "cpu")
    kwargs.update(config=trainer.config, scene_manager=trainer.scene_mgr, device="cpu")
    fresh = TinyField(**kwargs)
    fresh.load_from_state_dict(fresh.get_state_dict_from_ckpt(ckpt, "cpu"))
    rays = trainer.data_mgr.test_dataset.all_rays[0][:64]
    trainer.model.eval()
    fresh.eval()
    with torch.no_grad():
        assert torch.allclose(fresh(rays)["rgb_map"], trainer.model(rays)["rgb_map"], atol=1e-6)
