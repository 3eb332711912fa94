"""Gaussian3DEvaluator: evaluation entry point of this model family (reference: benchmarks/nerf/origin_gs/gs_evaluator.py).  Launch:
``torchrun ... -m landmarksystem_b200.models.origin_gs.gs_evaluator --config <render conf.py> [--key value]``."""
import sys

from ...train.nerf_evaluator import GaussianEvaluator, evaluator_main
from ..origin_gs.gs_model import GaussianModel


class Gaussian3DEvaluator(GaussianEvaluator):
    model_cls = GaussianModel


def main(argv=None):
    return evaluator_main(Gaussian3DEvaluator, argv)


if __name__ == "__main__":
    main(sys.argv[1:])
