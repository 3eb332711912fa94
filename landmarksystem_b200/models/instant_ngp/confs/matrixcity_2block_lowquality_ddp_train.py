"""InstantNGP on MatrixCity block A: training variant ``lowquality_ddp_train`` (see ``_matrixcity.py``)."""
from landmarksystem_b200.models.instant_ngp.confs._matrixcity import train

config = train("lowquality_ddp_train")
train_config, dataset_config, model_config = config        # the blocks by name, for files that import this one with *
