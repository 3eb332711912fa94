"""GridNeRF on MatrixCity block A: training variant ``multi_BranchParallel_10x5`` (see ``_matrixcity.py``)."""
from landmarksystem_b200.models.gridnerf.confs._matrixcity import train

config = train("multi_BranchParallel_10x5")
train_config, dataset_config, model_config = config        # the blocks by name, for files that import this one with *
