"""OctreeGSEvaluator: evaluation entry point of this model family (reference: benchmarks/nerf/octree_gs/gs_evaluator.py).  Launch:
``torchrun ... -m landmarksystem_b200.models.octree_gs.gs_evaluator --config <render conf.py> [--key value]``."""
import sys

from ...train.nerf_evaluator import GaussianEvaluator, evaluator_main
from ..octree_gs.gs_model import OctreeGS


class OctreeGSEvaluator(GaussianEvaluator):
    model_cls = OctreeGS


def main(argv=None):
    return evaluator_main(OctreeGSEvaluator, argv)


if __name__ == "__main__":
    main(sys.argv[1:])
