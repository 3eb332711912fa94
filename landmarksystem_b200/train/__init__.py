"""Training and evaluation engines (reference: landmark/train/__init__.py exports ``NeRFTrainer`` and
``NeRFEvaluator``); resolved on first access so that importing a helper of ``train.utils`` stays light."""


def __getattr__(name):
    if name == "NeRFTrainer":
        from .nerf_trainer import NeRFTrainer

        return NeRFTrainer
    if name == "NeRFEvaluator":
        from .nerf_evaluator import NeRFEvaluator

        return NeRFEvaluator
    raise AttributeError(name)


__all__ = ["NeRFTrainer", "NeRFEvaluator"]
