"""NGPEvaluator: evaluation entry point of this model family (reference: benchmarks/nerf/instant_ngp/instant_ngp_evaluator.py).  Launch:
``torchrun ... -m landmarksystem_b200.models.instant_ngp.instant_ngp_evaluator --config <render conf.py> [--key value]``."""
import sys

from ...train.nerf_evaluator import RayModelEvaluator, evaluator_main
from ..instant_ngp.instant_ngp import InstantNGP


class NGPEvaluator(RayModelEvaluator):
    def build_from_kwargs(self, kwargs):
        kwargs.pop("alphaMask", None)
        return self.model_cls(kwargs["aabb"], kwargs["device"], kwargs["near_far"], scene_manager=kwargs["scene_manager"],
                              config=kwargs["config"])

    model_cls = InstantNGP


def main(argv=None):
    return evaluator_main(NGPEvaluator, argv)


if __name__ == "__main__":
    main(sys.argv[1:])
