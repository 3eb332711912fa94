"""ScaffoldGSEvaluator: evaluation entry point of this model family (reference: benchmarks/nerf/scaffold_gs/gs_evaluator.py).  Launch:
``torchrun ... -m landmarksystem_b200.models.scaffold_gs.gs_evaluator --config <render conf.py> [--key value]``."""
import sys

from ...train.nerf_evaluator import GaussianEvaluator, evaluator_main
from ..scaffold_gs.gs_model import ScaffoldGS


class ScaffoldGSEvaluator(GaussianEvaluator):
    model_cls = ScaffoldGS


def main(argv=None):
    return evaluator_main(ScaffoldGSEvaluator, argv)


if __name__ == "__main__":
    main(sys.argv[1:])
