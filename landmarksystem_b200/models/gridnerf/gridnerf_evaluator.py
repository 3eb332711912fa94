"""GridNeRFEvaluator: evaluation entry point of this model family (reference: benchmarks/nerf/gridnerf/gridnerf_evaluator.py).  Launch:
``torchrun ... -m landmarksystem_b200.models.gridnerf.gridnerf_evaluator --config <render conf.py> [--key value]``."""
import sys

from ...configs import BaseConfig, get_default_parser, parse_console_args
from ...train.nerf_evaluator import RayModelEvaluator
from ..gridnerf.gridnerf import GridNeRF


class GridNeRFEvaluator(RayModelEvaluator):
    model_cls = GridNeRF


def main(argv=None):
    args, unknown = get_default_parser().parse_known_args(argv)
    config = BaseConfig.from_file(args.config, parse_console_args(unknown))
    config.is_train = False
    return GridNeRFEvaluator(config).eval()


if __name__ == "__main__":
    main(sys.argv[1:])
