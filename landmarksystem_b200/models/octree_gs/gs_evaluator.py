"""OctreeGSEvaluator: evaluation entry point of this model family (reference: benchmarks/nerf/octree_gs/gs_evaluator.py).  Launch:
``torchrun ... -m landmarksystem_b200.models.octree_gs.gs_evaluator --config <render conf.py> [--key value]``."""
import sys

from ...configs import BaseConfig, get_default_parser, parse_console_args
from ...train.nerf_evaluator import GaussianEvaluator
from ..octree_gs.gs_model import OctreeGS


class OctreeGSEvaluator(GaussianEvaluator):
    model_cls = OctreeGS


def main(argv=None):
    args, unknown = get_default_parser().parse_known_args(argv)
    config = BaseConfig.from_file(args.config, parse_console_args(unknown))
    config.is_train = False
    return OctreeGSEvaluator(config).eval()


if __name__ == "__main__":
    main(sys.argv[1:])
