"""Nerfacto trainer (reference: benchmarks/nerf/nerfacto/nerfacto_trainer.py:40-460): RAdam, MSE +
0.002 distortion + 1.0 inter-level loss, log-linear learning-rate decay on every group."""
import sys

import torch

from ...components.utils.loss_utils import distortion_loss, interlevel_loss
from ...configs import BaseConfig, get_default_parser, parse_console_args
from ...train.ray_trainer import RayModelTrainer
from ...train.utils import is_main_rank
from .nerfacto import Nerfacto


class NerfactoTrainer(RayModelTrainer):
    model_cls = Nerfacto

    def make_optimizer(self, groups):
        if torch.device(self.config.device).type == "cuda" and bool(self.config.get("fused_optimizer", True)):
            from ...ops.optim import FusedRAdam

            return FusedRAdam(groups, eps=self.config.eps)     # one device pass per tensor, gradients cleared in it
        return torch.optim.RAdam(groups, eps=self.config.eps)

    def before_forward(self, it: int):
        self.module.sampler.step_cb(it)

    def compute_loss(self, ret, rgb_train):
        cfg = self.config
        loss = torch.mean((ret["rgb_map"] - rgb_train) ** 2)
        if "weights_list" in ret:
            starts = [s.spacing_starts for s in ret["ray_samples_list"]]
            ends = [s.spacing_ends for s in ret["ray_samples_list"]]
            loss = loss + cfg.interlevel_loss_mult * interlevel_loss(ret["weights_list"], starts, ends)
            loss = loss + cfg.distortion_loss_mult * distortion_loss(ret["weights_list"], starts, ends)
        return loss


def main(argv=None):
    args, unknown = get_default_parser().parse_known_args(argv)
    trainer = NerfactoTrainer(BaseConfig.from_file(args.config, parse_console_args(unknown)))
    trainer.train()
    ps = trainer.evaluation(prefix="final_", n_vis=trainer.config.N_vis)
    if is_main_rank():
        print(f"final test PSNR {ps:.3f}", flush=True)


if __name__ == "__main__":
    main(sys.argv[1:])
