"""InstantNGP trainer (reference: benchmarks/nerf/instant_ngp/instant_ngp_trainer.py:40-458).  Launch:
``torchrun ... -m landmarksystem_b200.models.instant_ngp.instant_ngp_trainer --config conf.py [--key value]``."""
import sys

from ...configs import BaseConfig, get_default_parser, parse_console_args
from ...train.ray_trainer import RayModelTrainer
from ...train.utils import is_main_rank
from .instant_ngp import InstantNGP


class NGPTrainer(RayModelTrainer):
    model_cls = InstantNGP

    def before_forward(self, it: int):
        self.module.update_occupancy_grid(it)


def main(argv=None):
    args, unknown = get_default_parser().parse_known_args(argv)
    trainer = NGPTrainer(BaseConfig.from_file(args.config, parse_console_args(unknown)))
    trainer.train()
    ps = trainer.evaluation(prefix="final_", n_vis=trainer.config.N_vis)
    if is_main_rank():
        print(f"final test PSNR {ps:.3f}", flush=True)


if __name__ == "__main__":
    main(sys.argv[1:])
