"""GridNeRF on MatrixCity block A: training variant ``lowquality_BranchParallel`` (see ``_matrixcity.py``)."""
from landmarksystem_b200.models.gridnerf.confs._matrixcity import train

config = train("lowquality_BranchParallel")
train_config, dataset_config, model_config = config        # the blocks by name, for files that import this one with *
