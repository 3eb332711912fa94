"""NerfactoEvaluator: evaluation entry point of this model family (reference: benchmarks/nerf/nerfacto/nerfacto_evaluator.py).  Launch:
``torchrun ... -m landmarksystem_b200.models.nerfacto.nerfacto_evaluator --config <render conf.py> [--key value]``."""
import sys

from ...train.nerf_evaluator import RayModelEvaluator, evaluator_main
from ..nerfacto.nerfacto import Nerfacto


class NerfactoEvaluator(RayModelEvaluator):
    def build_from_kwargs(self, kwargs):
        kwargs.pop("alphaMask", None)
        return self.model_cls(kwargs["aabb"], kwargs["device"], kwargs["near_far"], scene_manager=kwargs["scene_manager"],
                              config=kwargs["config"])

    model_cls = Nerfacto


def main(argv=None):
    return evaluator_main(NerfactoEvaluator, argv)


if __name__ == "__main__":
    main(sys.argv[1:])
