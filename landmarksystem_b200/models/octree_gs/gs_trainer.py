"""Octree-GS trainer (reference: benchmarks/nerf/octree_gs/gs_trainer.py:24-310): Scaffold-GS training with the
level structure initialised from the training cameras and the current iteration fed to the LOD rule."""
import sys

from ...components.utils.ply_utils import get_pcd
from ...configs import BaseConfig, get_default_parser, parse_console_args
from ..scaffold_gs.gs_trainer import ScaffoldGSTrainer
from .gs_model import OctreeGS


class OctreeGSTrainer(ScaffoldGSTrainer):
    model_cls = OctreeGS

    def create_model(self):
        cfg = self.config
        model = self.build_model()
        if cfg.start_checkpoint:
            model.load_from_state_dict(model.get_state_dict_from_ckpt(cfg.start_checkpoint, cfg.device))
        else:
            model.create_from_pcd(get_pcd(cfg, self.aabb, dataset=self.data_mgr.full_train_dataset), self.spatial_lr_scale,
                                  cameras=self.data_mgr.full_train_dataset.cameras)
        return model

    def before_step(self, viewpoint_cam):
        self.model.iteration = self.iteration


def main(argv=None):
    args, unknown = get_default_parser().parse_known_args(argv)
    trainer = OctreeGSTrainer(BaseConfig.from_file(args.config, parse_console_args(unknown)))
    print(f"final test PSNR {trainer.train():.3f}", flush=True)


if __name__ == "__main__":
    main(sys.argv[1:])
