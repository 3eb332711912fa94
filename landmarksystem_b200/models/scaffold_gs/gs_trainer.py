"""Scaffold-GS trainer (reference: benchmarks/nerf/scaffold_gs/gs_trainer.py:24-277): per-group exponential
learning-rate schedules and the ``0.01 * mean(prod(scale))`` volume regulariser."""
import sys

from ...components.utils.general_utils import get_expon_lr_func
from ...configs import BaseConfig, get_default_parser, parse_console_args
from ...train.gaussian_trainer import GaussianTrainerBase
from .gs_model import ScaffoldGS

_SCHEDULED = {"anchor": ("position", True), "offset": ("offset", True), "mlp_opacity": ("mlp_opacity", False),
              "mlp_cov": ("mlp_cov", False), "mlp_color": ("mlp_color", False),
              "mlp_featurebank": ("mlp_featurebank", False), "embedding_appearance": ("appearance", False)}


class ScaffoldGSTrainer(GaussianTrainerBase):
    model_cls = ScaffoldGS

    def build_model(self):
        model = self.model_cls(config=self.config, scene_manager=self.scene_mgr, cam_extent=self.spatial_lr_scale)
        model.set_appearance(len(self.data_mgr.full_train_dataset))
        return model

    def create_optimizer(self):
        cfg = self.config
        self.schedulers = {}
        for group, (prefix, spatial) in _SCHEDULED.items():
            mult = self.spatial_lr_scale if spatial else 1.0
            self.schedulers[group] = get_expon_lr_func(cfg[f"{prefix}_lr_init"] * mult, cfg[f"{prefix}_lr_final"] * mult,
                                                       lr_delay_mult=cfg[f"{prefix}_lr_delay_mult"],
                                                       max_steps=cfg[f"{prefix}_lr_max_steps"])
        return super().create_optimizer()

    def update_learning_rate(self):
        for group in self.optimizer.param_groups:
            fn = self.schedulers.get(group.get("name"))
            if fn is not None:
                group["lr"] = fn(self.iteration)

    def extra_loss(self, image, gt_image):
        return 0.01 * self.model.scaling.prod(dim=1).mean()


def main(argv=None):
    args, unknown = get_default_parser().parse_known_args(argv)
    trainer = ScaffoldGSTrainer(BaseConfig.from_file(args.config, parse_console_args(unknown)))
    print(f"final test PSNR {trainer.train():.3f}", flush=True)


if __name__ == "__main__":
    main(sys.argv[1:])
