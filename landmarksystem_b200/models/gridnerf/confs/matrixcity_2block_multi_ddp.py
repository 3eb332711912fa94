"""GridNeRF on MatrixCity block A: training variant ``multi_ddp`` (see ``_matrixcity.py``)."""
from landmarksystem_b200.models.gridnerf.confs._matrixcity import train

config = train("multi_ddp")
train_config, dataset_config, model_config = config        # the blocks by name, for files that import this one with *
