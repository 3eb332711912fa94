"""Vanilla 3DGS trainer (reference: benchmarks/nerf/origin_gs/gs_trainer.py:24-233).  Launch:
``python -m landmarksystem_b200.models.origin_gs.gs_trainer --config conf.py [--key value]``."""
import sys

from ...components.utils.general_utils import get_expon_lr_func
from ...configs import BaseConfig, get_default_parser, parse_console_args
from ...train.gaussian_trainer import GaussianTrainerBase
from .gs_model import GaussianModel


class Gaussian3DTrainer(GaussianTrainerBase):
    def build_model(self):
        return GaussianModel(config=self.config, scene_manager=self.scene_mgr, cam_extent=self.spatial_lr_scale)

    def create_optimizer(self):
        cfg = self.config
        self.xyz_scheduler_args = get_expon_lr_func(cfg.position_lr_init * self.spatial_lr_scale,
                                                    cfg.position_lr_final * self.spatial_lr_scale,
                                                    lr_delay_mult=cfg.position_lr_delay_mult,
                                                    max_steps=cfg.position_lr_max_steps)
        return super().create_optimizer()

    def update_learning_rate(self):
        for group in self.optimizer.param_groups:
            if group["name"] == "xyz":
                group["lr"] = self.xyz_scheduler_args(self.iteration)


def main(argv=None):
    args, unknown = get_default_parser().parse_known_args(argv)
    trainer = Gaussian3DTrainer(BaseConfig.from_file(args.config, parse_console_args(unknown)))
    print(f"final test PSNR {trainer.train():.3f}", flush=True)


if __name__ == "__main__":
    main(sys.argv[1:])
