"""Nerfacto on MatrixCity: training variant ``allblock_huge`` (see ``_matrixcity.py``)."""
from landmarksystem_b200.models.nerfacto.confs._matrixcity import train

config = train("allblock_huge")
train_config, dataset_config, model_config = config        # the blocks by name, for files that import this one with *
