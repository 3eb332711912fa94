"""GridNeRFEvaluator: evaluation entry point of this model family (reference: benchmarks/nerf/gridnerf/gridnerf_evaluator.py).  Launch:
``torchrun ... -m landmarksystem_b200.models.gridnerf.gridnerf_evaluator --config <render conf.py> [--key value]``."""
import sys

from ...train.nerf_evaluator import RayModelEvaluator, evaluator_main
from ..gridnerf.gridnerf import GridNeRF


class GridNeRFEvaluator(RayModelEvaluator):
    model_cls = GridNeRF


def main(argv=None):
    return evaluator_main(GridNeRFEvaluator, argv)


if __name__ == "__main__":
    main(sys.argv[1:])
