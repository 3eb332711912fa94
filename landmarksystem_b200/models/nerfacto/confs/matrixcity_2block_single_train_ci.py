"""Nerfacto on MatrixCity: training variant ``2block_single_train_ci`` (see ``_matrixcity.py``)."""
from landmarksystem_b200.models.nerfacto.confs._matrixcity import train

config = train("2block_single_train_ci")
train_config, dataset_config, model_config = config        # the blocks by name, for files that import this one with *
